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

// ---- a timeline of a step in its place (built only with -DQI_TIMELINE) -------------------------
// Thread 0 of every CTA of the instrumented kernels leaves a record: the global timer at the
// CTA's start, when its wait for the kernel before it ended, when its first data had arrived, and
// at its end. Each source file keeps its own log (qi_timeline_<file>), the host sorts the
// records of a step into launches afterwards. Without the flag the macros are empty.
#ifdef QI_TIMELINE
struct QiStamp { unsigned long long t0, tw, td, t1; int kind, grid, cta, sm; };
#define QI_TL_CAP (1 << 19)
__device__ __forceinline__ unsigned long long qi_now() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
#define QI_TL_DEFINE(NAME)                                                                                       \
    __device__ QiStamp qi_tl_log[QI_TL_CAP];                                                                     \
    __device__ unsigned qi_tl_n;                                                                                 \
    __device__ __forceinline__ void qi_tl_put(int kind, unsigned long long t0, unsigned long long tw, unsigned long long td) { \
        const unsigned i = atomicAdd(&qi_tl_n, 1u);                                                              \
        if (i < QI_TL_CAP) {                                                                                     \
            unsigned sm; asm volatile("mov.u32 %0, %smid;" : "=r"(sm));                                          \
            QiStamp s; s.t0 = t0; s.tw = tw; s.td = td; s.t1 = qi_now(); s.kind = kind;                          \
            s.grid = gridDim.x * gridDim.y * gridDim.z; s.cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z); \
            s.sm = (int)sm; qi_tl_log[i] = s;                                                                    \
        }                                                                                                        \
    }                                                                                                            \
    int NAME##_impl(QiStamp* host, unsigned* n, int reset) {                                                     \
        cudaDeviceSynchronize();                                                                                 \
        cudaMemcpyFromSymbol(n, qi_tl_n, 4);                                                                     \
        if (host) cudaMemcpyFromSymbol(host, qi_tl_log, sizeof(QiStamp) * (*n < QI_TL_CAP ? *n : QI_TL_CAP));    \
        if (reset) { unsigned z = 0; cudaMemcpyToSymbol(qi_tl_n, &z, 4); }                                       \
        return 0;                                                                                                \
    }
#define QI_TL_EXPORT(NAME) extern "C" int NAME(QiStamp* host, unsigned* n, int reset) { return NAME##_impl(host, n, reset); }
#define QI_TL_BEGIN() const unsigned long long qi_tl_t0 = qi_now(); unsigned long long qi_tl_tw = 0, qi_tl_td = 0; (void)qi_tl_tw; (void)qi_tl_td
#define QI_TL_WAKE() qi_tl_tw = qi_now()
#define QI_TL_DATA() qi_tl_td = qi_now()
#define QI_TL_SHARED() __shared__ unsigned long long qi_tl_sh[2]
#define QI_TL_SHARED_WAKE() do { qi_tl_sh[0] = qi_now(); qi_tl_sh[1] = 0; } while (0)
#define QI_TL_SHARED_DATA() qi_tl_sh[1] = qi_now()
#define QI_TL_END(kind) do { if (threadIdx.x == 0) qi_tl_put(kind, qi_tl_t0, qi_tl_tw, qi_tl_td); } while (0)
#define QI_TL_END_SHARED(kind) do { if (threadIdx.x == 0) qi_tl_put(kind, qi_tl_t0, qi_tl_sh[0], qi_tl_sh[1]); } while (0)
#else
#define QI_TL_DEFINE(NAME)
#define QI_TL_EXPORT(NAME)
#define QI_TL_BEGIN() do { } while (0)
#define QI_TL_WAKE() do { } while (0)
#define QI_TL_DATA() do { } while (0)
#define QI_TL_SHARED() do { } while (0)
#define QI_TL_SHARED_WAKE() do { } while (0)
#define QI_TL_SHARED_DATA() do { } while (0)
#define QI_TL_END(kind) do { } while (0)
#define QI_TL_END_SHARED(kind) do { } while (0)
#endif

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
