// Fused residual add + RMSNorm.
//
// For each output row r (source row s = rows ? rows[r] : r):
//     x   = resid[s, :] + sum_k delta[k, s, :]      (32-bit, k ascending)
//     if write_resid: resid[s, :] = x
//     out[r, :] = (x * (1 / sqrt(mean(x^2) + eps))) * gain
// The residual stream is always 32-bit; `delta` is the previous part's output
// in the activation type (or 32-bit split-K partial sums, delta_splits > 1);
// `out` is in the activation type. The formula and its order are the
// reference's (backends/cpu/src/backend.rs:172-193: mean square :185-186,
// inverse :187, scale :189; the residual add is crates/quantinfer-runtime/src/linear.rs:129-142).
#include "common.cuh"

#include <cooperative_groups.h>

namespace {

template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const TD* __restrict__ delta,
                                   int delta_splits, size_t delta_split_stride,
                                   const float* __restrict__ gain, float eps,
                                   TO* __restrict__ out, const int* __restrict__ rows, int hidden,
                                   int write_resid) {
    __shared__ float scratch[32];
    qi::pdl_enter();
    const int r = blockIdx.x;
    const int s = rows ? rows[r] : r;
    float* xr = resid + (size_t)s * hidden;
    const TD* dr = delta ? delta + (size_t)s * hidden : nullptr;

    float sumsq = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float x = xr[i];
        if (dr) {
            for (int k = 0; k < delta_splits; ++k) x += qi::to_f32<TD>(dr[k * delta_split_stride + i]);
        }
        if (write_resid) xr[i] = x;
        sumsq += x * x;
    }
    const float total = qi::block_sum(sumsq, scratch);
    const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
    TO* orow = out + (size_t)r * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float x = xr[i];  // same thread wrote it in the first pass when write_resid
        if (dr && !write_resid) {
            for (int k = 0; k < delta_splits; ++k) x += qi::to_f32<TD>(dr[k * delta_split_stride + i]);
        }
        orow[i] = qi::from_f32<TO>(x * inv * gain[i]);
    }
}

// The same, eight elements per thread and step (hidden a multiple of 8, rows 16-byte
// aligned): 32-byte loads of the residual, 16-byte loads of a bfloat16 delta.
template <typename T> struct Vec8;
template <> struct Vec8<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
        const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
};
template <> struct Vec8<qi::bf16> {
    static __device__ __forceinline__ void load(const qi::bf16* p, float (&v)[8]) {
        const uint4 u = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void store(qi::bf16* p, const float (&v)[8]) {
        uint4 u;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = u;
    }
};

QI_TL_DEFINE(qi_timeline_norm)

template <typename TD, typename TO>
__global__ void __launch_bounds__(512, 3) add_rmsnorm_vec_kernel(float* __restrict__ resid, const TD* __restrict__ delta,
                                       int delta_splits, size_t delta_split_stride,
                                       const float* __restrict__ gain, float eps, TO* __restrict__ out,
                                       const int* __restrict__ rows, int hidden, int write_resid, int n_rows) {
    __shared__ float scratch[32];
    QI_TL_BEGIN();
    qi::pdl_enter();
    QI_TL_WAKE();
    // A CTA takes rows blockIdx.x, blockIdx.x + gridDim.x, ...: the grid is what is resident at once, three
    // CTAs of 512 threads an SM (the register bound above). A timeline of the prefill step showed this kernel
    // at 40 us for a prompt of 2,048 tokens where it moves 100 MB: one CTA a row, and so many registers (all
    // partial sums of a row held at once) that one CTA filled an SM. Now 24 us; four CTAs an SM spill and take 26.
    for (int r = blockIdx.x; r < n_rows; r += gridDim.x) {
    const int s = rows ? rows[r] : r;
    float* xr = resid + (size_t)s * hidden;
    const TD* dr = delta ? delta + (size_t)s * hidden : nullptr;
    TO* orow = out + (size_t)r * hidden;
    if (hidden <= (int)blockDim.x * 8) {
        // the whole row fits the block once: values stay in registers between the two passes and
        // the gain is fetched together with the inputs (one round of loads instead of three)
        const int i = threadIdx.x * 8;
        const bool active = i < hidden;
        float x[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, d[8], g[8];
        if (active) {
            Vec8<float>::load(xr + i, x);
            Vec8<float>::load(gain + i, g);
            if (dr) {
                // (few registers, so that four CTAs of 512 threads share an SM; the cluster kernel below, for few
                // rows, requests all partial sums at once instead)
#pragma unroll 4
                for (int k = 0; k < delta_splits; ++k) {
                    Vec8<TD>::load(dr + k * delta_split_stride + i, d);
#pragma unroll
                    for (int j = 0; j < 8; ++j) x[j] += d[j];
                }
            }
            if (write_resid) Vec8<float>::store(xr + i, x);
        }
        float sumsq = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) sumsq += x[j] * x[j];
        const float total = qi::block_sum(sumsq, scratch);
        const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
        if (active) {
#pragma unroll
            for (int j = 0; j < 8; ++j) x[j] = x[j] * inv * g[j];
            Vec8<TO>::store(orow + i, x);
        }
        continue;
    }
    float sumsq = 0.f;
    for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
        float x[8], d[8];
        Vec8<float>::load(xr + i, x);
        if (dr) {
            // the loads of four splits go out together; the sums stay in split order
#pragma unroll 4
            for (int k = 0; k < delta_splits; ++k) {
                Vec8<TD>::load(dr + k * delta_split_stride + i, d);
#pragma unroll
                for (int j = 0; j < 8; ++j) x[j] += d[j];
            }
        }
        if (write_resid) Vec8<float>::store(xr + i, x);
#pragma unroll
        for (int j = 0; j < 8; ++j) sumsq += x[j] * x[j];
    }
    const float total = qi::block_sum(sumsq, scratch);
    const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
    for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
        float x[8], d[8], g[8];
        Vec8<float>::load(xr + i, x);   // the same thread wrote it in the first pass when write_resid
        if (dr && !write_resid) {
            for (int k = 0; k < delta_splits; ++k) {
                Vec8<TD>::load(dr + k * delta_split_stride + i, d);
#pragma unroll
                for (int j = 0; j < 8; ++j) x[j] += d[j];
            }
        }
        Vec8<float>::load(gain + i, g);
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = x[j] * inv * g[j];
        Vec8<TO>::store(orow + i, x);
    }
    }
    QI_TL_END(10);
}

// The same for few rows (a decode step): a row is spread over a thread-block cluster of kRowCtas
// CTAs, so that as many SMs pull the row's partial sums as the row has parts (eight rows of
// eight partial sums are 1 MB: on eight SMs the loads alone took 1.9 us). Each CTA adds its part of
// the row, the sums of squares meet in distributed shared memory and are added in the order of
// the CTAs' ranks.
constexpr int kRowCtas = 4;

template <typename TD, typename TO>
__global__ void add_rmsnorm_cluster_kernel(float* __restrict__ resid, const TD* __restrict__ delta,
                                           int delta_splits, size_t delta_split_stride,
                                           const float* __restrict__ gain, float eps, TO* __restrict__ out,
                                           const int* __restrict__ rows, int hidden, int write_resid) {
    namespace cg = cooperative_groups;
    __shared__ float scratch[32];
    __shared__ float part_sum;
    cg::cluster_group cluster = cg::this_cluster();
    QI_TL_BEGIN();
    qi::pdl_enter();
    QI_TL_WAKE();
    const int r = blockIdx.x / kRowCtas, part = (int)cluster.block_rank();
    const int cols = hidden / kRowCtas;                 // of this CTA (the launch checked that it divides)
    const int s = rows ? rows[r] : r;
    float* xr = resid + (size_t)s * hidden + (size_t)part * cols;
    const TD* dr = delta ? delta + (size_t)s * hidden + (size_t)part * cols : nullptr;
    const float* gr = gain + (size_t)part * cols;
    TO* orow = out + (size_t)r * hidden + (size_t)part * cols;
    const int i = threadIdx.x * 8;
    const bool active = i < cols;
    float x[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, d[8], g[8];
    if (active) {
        Vec8<float>::load(xr + i, x);
        Vec8<float>::load(gr + i, g);
        if (dr && delta_splits <= 8) {
            float d8[8][8];
#pragma unroll
            for (int k = 0; k < 8; ++k)
                if (k < delta_splits) Vec8<TD>::load(dr + k * delta_split_stride + i, d8[k]);
#pragma unroll
            for (int k = 0; k < 8; ++k)
                if (k < delta_splits) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) x[j] += d8[k][j];
                }
        } else if (dr) {
#pragma unroll 4
            for (int k = 0; k < delta_splits; ++k) {
                Vec8<TD>::load(dr + k * delta_split_stride + i, d);
#pragma unroll
                for (int j = 0; j < 8; ++j) x[j] += d[j];
            }
        }
        if (write_resid) Vec8<float>::store(xr + i, x);
    }
    float sumsq = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) sumsq += x[j] * x[j];
    const float mine = qi::block_sum(sumsq, scratch);
    if (threadIdx.x == 0) part_sum = mine;
    cluster.sync();
    float total = 0.f;
#pragma unroll
    for (int c = 0; c < kRowCtas; ++c) total += *cluster.map_shared_rank(&part_sum, c);      // rank order
    cluster.sync();                                      // nobody leaves while its sum may still be read
    const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
    if (active) {
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = x[j] * inv * g[j];
        Vec8<TO>::store(orow + i, x);
    }
    QI_TL_END(11);
}

// Launch with a cluster of kRowCtas CTAs along x (and the programmatic-serialization attribute, as qi::launch).
template <typename... KArgs, typename... Args>
cudaError_t launch_cluster(void (*kern)(KArgs...), dim3 grid, dim3 block, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kRowCtas;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = qi::pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// Plain RMSNorm over the last dimension of a [rows, width] matrix of type T,
// used by tests of the norm alone and by parts that normalise activations.
template <typename T>
__global__ void rmsnorm_kernel(const T* __restrict__ x, const float* __restrict__ gain, float eps,
                               T* __restrict__ out, int width) {
    __shared__ float scratch[32];
    qi::pdl_enter();
    const T* xr = x + (size_t)blockIdx.x * width;
    float sumsq = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = qi::to_f32<T>(xr[i]);
        sumsq += v * v;
    }
    const float total = qi::block_sum(sumsq, scratch);
    const float inv = 1.0f / sqrtf(total / (float)width + eps);
    T* orow = out + (size_t)blockIdx.x * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        orow[i] = qi::from_f32<T>(qi::to_f32<T>(xr[i]) * inv * gain[i]);
}

int pick_threads(int hidden) { return hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : (hidden >= 128 ? 128 : 32)); }

}  // namespace

// delta may be null (no add). rows may be null (identity; n_rows rows).
// With rows given, write_resid must be 0 (the gather variant feeds the head).
extern "C" int qi_add_rmsnorm(float* resid, const void* delta, int delta_dtype, int delta_splits,
                              long long delta_split_stride, const float* gain, float eps,
                              void* out, int out_dtype, const int* rows, int n_rows, int hidden,
                              int write_resid, cudaStream_t stream) {
    QI_REQUIRE(n_rows >= 0 && hidden > 0, "add_rmsnorm: bad sizes rows=%d hidden=%d", n_rows, hidden);
    QI_REQUIRE(!(rows && write_resid), "add_rmsnorm: the row-gather form does not write the residual");
    QI_REQUIRE(delta_splits >= 1, "add_rmsnorm: delta_splits must be >= 1");
    QI_REQUIRE(eps > 0.f, "add_rmsnorm: eps must be positive");
    if (n_rows == 0) return 0;
    const int dd = delta ? delta_dtype : qi::kF32;
    const bool vec = hidden % 8 == 0 && ((uintptr_t)resid & 31) == 0 && ((uintptr_t)delta & 15) == 0 &&
                     ((uintptr_t)out & 15) == 0 && ((uintptr_t)gain & 15) == 0 && delta_split_stride % 8 == 0;
    // few rows (a decode step): a row over a cluster of CTAs, so that more SMs pull its partial sums
    if (vec && n_rows <= 64 && delta && delta_splits > 1 && hidden % (8 * kRowCtas) == 0 && hidden / (8 * kRowCtas) <= 1024 &&
        hidden / kRowCtas >= 256) {
        const int threads = (hidden / kRowCtas / 8 + 31) / 32 * 32;
        QI_DISPATCH_DTYPE(dd, TD, {
            QI_DISPATCH_DTYPE(out_dtype, TO, {
                launch_cluster(add_rmsnorm_cluster_kernel<TD, TO>, dim3(n_rows * kRowCtas), dim3(threads), stream, resid, (const TD*)delta,
                               delta_splits, (size_t)delta_split_stride, gain, eps, (TO*)out, rows, hidden, write_resid);
            });
        });
        return qi::check_launch("add_rmsnorm (clusters)");
    }
    if (vec) {
        int threads = (hidden / 8 + 31) / 32 * 32;
        if (threads > 512) threads = 512;
        static int sms = 0;
        if (!sms) {
            int dev = 0;
            cudaGetDevice(&dev);
            if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
        }
        const int resident = sms * (2048 / threads < 3 ? 2048 / threads : 3) * (threads < 512 ? 512 / threads : 1);
        const int grid = n_rows < resident ? n_rows : resident;
        QI_DISPATCH_DTYPE(dd, TD, {
            QI_DISPATCH_DTYPE(out_dtype, TO, {
                qi::launch(add_rmsnorm_vec_kernel<TD, TO>, dim3(grid), dim3(threads), 0, stream, resid, (const TD*)delta,
                           delta_splits, (size_t)delta_split_stride, gain, eps, (TO*)out, rows, hidden, write_resid, n_rows);
            });
        });
        return qi::check_launch("add_rmsnorm");
    }
    const int threads = pick_threads(hidden);
    QI_DISPATCH_DTYPE(dd, TD, {
        QI_DISPATCH_DTYPE(out_dtype, TO, {
            qi::launch(add_rmsnorm_kernel<TD, TO>, dim3(n_rows), dim3(threads), 0, stream, resid, (const TD*)delta,
                       delta_splits, (size_t)delta_split_stride, gain, eps, (TO*)out, rows, hidden, write_resid);
        });
    });
    return qi::check_launch("add_rmsnorm");
}

extern "C" int qi_rmsnorm(const void* x, const float* gain, float eps, void* out, int dtype,
                          int n_rows, int width, cudaStream_t stream) {
    QI_REQUIRE(n_rows >= 0 && width > 0, "rmsnorm: bad sizes rows=%d width=%d", n_rows, width);
    QI_REQUIRE(eps > 0.f, "rmsnorm: eps must be positive");
    if (n_rows == 0) return 0;
    const int threads = pick_threads(width);
    QI_DISPATCH_DTYPE(dtype, T, {
        qi::launch(rmsnorm_kernel<T>, dim3(n_rows), dim3(threads), 0, stream, (const T*)x, gain, eps, (T*)out, width);
    });
    return qi::check_launch("rmsnorm");
}

QI_TL_EXPORT(qi_timeline_norm)
