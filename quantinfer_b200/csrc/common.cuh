// Shared helpers of the sm_100a kernels: element types, conversions, warp and
// block reductions, and the error channel of the C entry points.
//
// Every entry point is `extern "C" int qi_*(..., cudaStream_t)`; it returns 0
// on success and a non-zero code after storing a message that
// `qi_last_error()` returns. Entry points validate sizes and refuse what the
// kernel behind them does not cover; they never compute a wrong result.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace qi {

// Element type codes shared with the Python side.
enum DType : int { kF32 = 0, kBF16 = 1 };

// Bits of the device status word that kernels set instead of trapping.
enum Status : int {
    kStatusBadToken = 1,     // token id outside the vocabulary
    kStatusBadPage = 2,      // block table entry < 0 or >= pool size where a page was needed
    kStatusNonFinite = 4,    // logits held NaN or Inf where a sampler read them
    kStatusWaitTimeout = 8,  // a bounded mbarrier wait ran out
    kStatusBadRange = 16,    // a position beyond the rotation table, or keys beyond the ranges a launch covers
};

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` holds 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < nwarps; ++w) total += scratch[w];  // fixed order
    return total;
}

// Programmatic dependent launch: every kernel lets the next kernel of the stream be
// scheduled as soon as all of its own blocks have started (so that launch latency and
// the next kernel's set-up overlap this kernel's run), and waits for the previous kernel
// to have completed, with its writes visible, before it touches global memory. Both are
// no-ops for a kernel launched without the attribute.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_enter() {
    pdl_launch_dependents();
    pdl_wait();
}

bool pdl_enabled();   // host: false when QUANTINFER_B200_PDL=0

// Launches `kern` with the programmatic-serialization attribute (when enabled).
template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// Host side: error message channel.
void set_error(const char* fmt, ...);
int fail(const char* fmt, ...);   // stores the message, returns 1
int check_launch(const char* what);  // cudaGetLastError -> message

}  // namespace qi

#define QI_REQUIRE(cond, ...)                    \
    do {                                         \
        if (!(cond)) return qi::fail(__VA_ARGS__); \
    } while (0)

// Calls `body` with `T` bound to the element type that `code` names.
#define QI_DISPATCH_DTYPE(code, T, ...)                           \
    do {                                                          \
        if ((code) == qi::kF32) {                                 \
            typedef float T;                                      \
            __VA_ARGS__                                           \
        } else if ((code) == qi::kBF16) {                         \
            typedef qi::bf16 T;                                   \
            __VA_ARGS__                                           \
        } else {                                                  \
            return qi::fail("unknown element type code %d", (int)(code)); \
        }                                                         \
    } while (0)
