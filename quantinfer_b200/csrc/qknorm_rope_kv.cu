// Per-head RMSNorm of q and k, rotary position encoding, and the write of k
// and v into the request's cache pages, in one pass over the fused qkv rows.
//
// Order, as the reference runs it (crates/quantinfer-runtime/src/qwen3/mod.rs:182-183,
// batch.rs:30-55): q and k are normalised over head_dim with one gain vector
// shared by all heads (backends/cpu/src/backend.rs:195-203), then rotated
// (half-split pairs (p, p + rot/2); backends/cpu/src/backend.rs:270-275), then k
// (rotated) and v (raw) are appended to the cache (cache.rs:94-127).
// The pairing rule is a parameter: `interleaved` rotates adjacent elements (2p, 2p + 1)
// with the angle of pair p instead, the order the reference's converter produces for
// architectures it stores that way (crates/quantinfer-format/src/gguf/layout.rs:52-55).
// A position beyond the rotation table sets a status bit and uses the table's last row.
// Norm sums, angles and the rotation are 32-bit. cos/sin come from a table
// [max_positions, rot/2] built once by rope_table below from 32-bit inverse
// frequencies (attention.rs:29-32: angle = position * theta^(-2p/d)).
//
// Cache pages of one layer: [num_pages, kv_heads, page_size, head_dim]; the
// token at position p of request r lies in page table[r, p / page_size] at row
// p % page_size.
#include "common.cuh"

namespace {

constexpr int kWarpsPerBlock = 4;
constexpr int kMaxHeadDim = 512;

template <typename T>
__global__ void qk_norm_rope_kv_kernel(
    const T* __restrict__ qkv, T* __restrict__ q_out, const float* __restrict__ q_gain,
    const float* __restrict__ k_gain, float eps, const float* __restrict__ cos_t,
    const float* __restrict__ sin_t, int rot, int interleaved, int table_positions, const int* __restrict__ positions,
    const int* __restrict__ token_req, const int* __restrict__ block_table, int max_blocks,
    int page_size, int num_pages, T* __restrict__ k_pages, T* __restrict__ v_pages, int nq, int nkv,
    int d, int* __restrict__ status) {
    qi::pdl_enter();
    const int t = blockIdx.x;
    const int head = blockIdx.y * kWarpsPerBlock + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    const int total_heads = nq + 2 * nkv;
    if (head >= total_heads) return;
    const int row_width = total_heads * d;
    const T* src = qkv + (size_t)t * row_width + (size_t)head * d;
    const int pos = positions[t];
    if (pos < 0) {
        if (lane == 0 && status) atomicOr(status, qi::kStatusBadRange);
        return;
    }
    int table_row = pos;
    if (cos_t && pos >= table_positions) {
        if (lane == 0 && status) atomicOr(status, qi::kStatusBadRange);
        table_row = table_positions - 1;
    }

    // Destination row.
    T* dst = nullptr;
    const bool is_q = head < nq;
    const bool is_k = !is_q && head < nq + nkv;
    if (is_q) {
        dst = q_out + (size_t)t * nq * d + (size_t)head * d;
    } else {
        if (k_pages == nullptr) return;  // a layer that reads another layer's cache writes none
        const int hk = is_k ? head - nq : head - nq - nkv;
        const int r = token_req[t];
        const int page = block_table[(size_t)r * max_blocks + pos / page_size];
        if (page < 0 || page >= num_pages) {
            if (lane == 0 && status) atomicOr(status, qi::kStatusBadPage);
            return;
        }
        T* base = is_k ? k_pages : v_pages;
        dst = base + (((size_t)page * nkv + hk) * page_size + (pos % page_size)) * (size_t)d;
    }

    if (!is_q && !is_k) {  // v: raw copy
        for (int i = lane; i < d; i += 32) dst[i] = src[i];
        return;
    }

    const float* gain = is_q ? q_gain : k_gain;
    float inv = 1.f;
    if (gain) {
        float ss = 0.f;
        for (int i = lane; i < d; i += 32) {
            const float v = qi::to_f32<T>(src[i]);
            ss += v * v;
        }
        ss = qi::warp_sum(ss);
        inv = 1.0f / sqrtf(ss / (float)d + eps);
    }
    const int half = rot / 2;
    // Rotated pairs.
    for (int p = lane; p < half; p += 32) {
        const int ia = interleaved ? 2 * p : p, ib = interleaved ? 2 * p + 1 : p + half;
        float a = qi::to_f32<T>(src[ia]);
        float b = qi::to_f32<T>(src[ib]);
        if (gain) {
            a = a * inv * gain[ia];
            b = b * inv * gain[ib];  // stays 32-bit until after the rotation
        }
        float c = 1.f, s = 0.f;
        if (cos_t) {
            c = cos_t[(size_t)table_row * half + p];
            s = sin_t[(size_t)table_row * half + p];
        }
        dst[ia] = qi::from_f32<T>(a * c - b * s);
        dst[ib] = qi::from_f32<T>(a * s + b * c);
    }
    // Dimensions beyond the rotary part pass through (normalised).
    for (int i = rot + lane; i < d; i += 32) {
        float a = qi::to_f32<T>(src[i]);
        if (gain) a = a * inv * gain[i];
        dst[i] = qi::from_f32<T>(a);
    }
}

// Two adjacent elements per access (head_dim a multiple of 4, rotation over the whole head).
template <typename T> struct Pair;
template <> struct Pair<float> {
    static __device__ __forceinline__ float2 load(const float* p) { return *reinterpret_cast<const float2*>(p); }
    static __device__ __forceinline__ void store(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
};
template <> struct Pair<qi::bf16> {
    static __device__ __forceinline__ float2 load(const qi::bf16* p) {
        return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
    }
    static __device__ __forceinline__ void store(qi::bf16* p, float a, float b) {
        *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
    }
};

// Sum over the K splits of a product's 32-bit partial sums (one split: the value itself).
template <typename TIn>
__device__ __forceinline__ float2 load_pair(const TIn* p, int splits, size_t stride) {
    float2 v = Pair<TIn>::load(p);
#pragma unroll 4
    for (int k = 1; k < splits; ++k) {
        const float2 w = Pair<TIn>::load(p + k * stride);
        v.x += w.x;
        v.y += w.y;
    }
    return v;
}

// TIn = T: qkv is the projection's output. TIn = float with splits > 1: qkv holds the
// projection's K-split partial sums [splits, n, width], added here in split order.
template <typename TIn, typename T>
__global__ void qk_norm_rope_kv_vec_kernel(
    const TIn* __restrict__ qkv, int splits, size_t split_stride, T* __restrict__ q_out, const float* __restrict__ q_gain,
    const float* __restrict__ k_gain, float eps, const float* __restrict__ cos_t,
    const float* __restrict__ sin_t, int table_positions, const int* __restrict__ positions,
    const int* __restrict__ token_req, const int* __restrict__ block_table, int max_blocks,
    int page_size, int num_pages, T* __restrict__ k_pages, T* __restrict__ v_pages, int nq, int nkv,
    int d, int* __restrict__ status) {
    qi::pdl_enter();
    const int t = blockIdx.x;
    const int head = blockIdx.y * kWarpsPerBlock + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    const int total_heads = nq + 2 * nkv;
    if (head >= total_heads) return;
    const TIn* src = qkv + (size_t)t * total_heads * d + (size_t)head * d;
    const int pos = positions[t];
    if (pos < 0) {
        if (lane == 0 && status) atomicOr(status, qi::kStatusBadRange);
        return;
    }
    int table_row = pos;
    if (cos_t && pos >= table_positions) {
        if (lane == 0 && status) atomicOr(status, qi::kStatusBadRange);
        table_row = table_positions - 1;
    }
    const bool is_q = head < nq;
    const bool is_k = !is_q && head < nq + nkv;
    T* dst;
    if (is_q) {
        dst = q_out + (size_t)t * nq * d + (size_t)head * d;
    } else {
        if (k_pages == nullptr) return;
        const int hk = is_k ? head - nq : head - nq - nkv;
        const int page = block_table[(size_t)token_req[t] * max_blocks + pos / page_size];
        if (page < 0 || page >= num_pages) {
            if (lane == 0 && status) atomicOr(status, qi::kStatusBadPage);
            return;
        }
        dst = (is_k ? k_pages : v_pages) + (((size_t)page * nkv + hk) * page_size + (pos % page_size)) * (size_t)d;
    }
    if (!is_q && !is_k) {
        for (int i = 2 * lane; i < d; i += 64) {
            const float2 v = load_pair<TIn>(src + i, splits, split_stride);
            Pair<T>::store(dst + i, v.x, v.y);
        }
        return;
    }
    const int half = d / 2;
    const float* gain = is_q ? q_gain : k_gain;
    float inv = 1.f;
    if (gain) {
        float ss = 0.f;
        for (int i = 2 * lane; i < d; i += 64) {
            const float2 v = load_pair<TIn>(src + i, splits, split_stride);
            ss += v.x * v.x + v.y * v.y;
        }
        ss = qi::warp_sum(ss);
        inv = 1.0f / sqrtf(ss / (float)d + eps);
    }
    for (int p = 2 * lane; p < half; p += 64) {
        float2 a = load_pair<TIn>(src + p, splits, split_stride), b = load_pair<TIn>(src + p + half, splits, split_stride);
        if (gain) {
            const float2 ga = *reinterpret_cast<const float2*>(gain + p), gb = *reinterpret_cast<const float2*>(gain + p + half);
            a.x = a.x * inv * ga.x; a.y = a.y * inv * ga.y;
            b.x = b.x * inv * gb.x; b.y = b.y * inv * gb.y;
        }
        float2 c = make_float2(1.f, 1.f), sn = make_float2(0.f, 0.f);
        if (cos_t) {
            c = *reinterpret_cast<const float2*>(cos_t + (size_t)table_row * half + p);
            sn = *reinterpret_cast<const float2*>(sin_t + (size_t)table_row * half + p);
        }
        Pair<T>::store(dst + p, a.x * c.x - b.x * sn.x, a.y * c.y - b.y * sn.y);
        Pair<T>::store(dst + p + half, a.x * sn.x + b.x * c.x, a.y * sn.y + b.y * c.y);
    }
}

__global__ void rope_table_kernel(const float* __restrict__ inv_freq, float* __restrict__ cos_t,
                                  float* __restrict__ sin_t, int max_pos, int half) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)max_pos * half) return;
    const int pos = (int)(idx / half), p = (int)(idx % half);
    const float angle = (float)pos * inv_freq[p];
    cos_t[idx] = cosf(angle);
    sin_t[idx] = sinf(angle);
}

}  // namespace

extern "C" int qi_rope_table(const float* inv_freq, float* cos_t, float* sin_t, int max_pos,
                             int half, cudaStream_t stream) {
    QI_REQUIRE(max_pos > 0 && half > 0, "rope_table: bad sizes max_pos=%d half=%d", max_pos, half);
    const size_t n = (size_t)max_pos * half;
    rope_table_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(inv_freq, cos_t, sin_t, max_pos,
                                                                      half);
    return qi::check_launch("rope_table");
}

// q_gain/k_gain null: no norm. cos_t null: no rotation. k_pages null: no cache write.
// interleaved: pairs (2p, 2p + 1) instead of (p, p + rot/2).
// qkv_splits > 1: `qkv` holds float32 partial sums [qkv_splits, n_tokens, width] of the projection.
extern "C" int qi_qk_norm_rope_kv(const void* qkv, int qkv_splits, void* q_out, int dtype, const float* q_gain,
                                  const float* k_gain, float eps, const float* cos_t,
                                  const float* sin_t, int rot, int interleaved, int table_positions,
                                  const int* positions, const int* token_req,
                                  const int* block_table, int max_blocks, int page_size,
                                  int num_pages, void* k_pages, void* v_pages, int n_tokens, int nq,
                                  int nkv, int d, int* status, cudaStream_t stream) {
    QI_REQUIRE(n_tokens >= 0 && nq > 0 && nkv > 0 && d > 0, "qk_norm_rope_kv: bad sizes");
    QI_REQUIRE(d <= kMaxHeadDim, "qk_norm_rope_kv: head_dim %d is above the limit %d", d, kMaxHeadDim);
    QI_REQUIRE(rot >= 0 && rot <= d && rot % 2 == 0, "qk_norm_rope_kv: rotary size %d must be even and <= head_dim %d", rot, d);
    QI_REQUIRE(!cos_t || (sin_t && table_positions > 0), "qk_norm_rope_kv: incomplete rotation table");
    QI_REQUIRE((k_pages == nullptr) == (v_pages == nullptr), "qk_norm_rope_kv: k and v pages must come together");
    QI_REQUIRE(!k_pages || (page_size > 0 && max_blocks > 0 && num_pages > 0 && block_table && token_req),
               "qk_norm_rope_kv: incomplete page arguments");
    if (n_tokens == 0) return 0;
    const int heads = nq + 2 * nkv;
    dim3 grid(n_tokens, (heads + kWarpsPerBlock - 1) / kWarpsPerBlock);
    QI_REQUIRE(grid.y <= 65535, "qk_norm_rope_kv: too many heads");
    if (!cos_t) rot = 0;
    QI_REQUIRE(qkv_splits >= 1, "qk_norm_rope_kv: qkv_splits must be >= 1");
    const bool vec = d % 4 == 0 && (rot == d || rot == 0) && (!interleaved || rot == 0) && ((uintptr_t)qkv & 7) == 0 && ((uintptr_t)q_out & 7) == 0 &&
                     ((uintptr_t)k_pages & 7) == 0 && ((uintptr_t)v_pages & 7) == 0;
    if (qkv_splits > 1) {
        QI_REQUIRE(vec, "qk_norm_rope_kv: partial sums as input need head_dim %% 4 == 0 and a half-split rotation over the whole head");
        const size_t stride = (size_t)n_tokens * heads * d;
        QI_DISPATCH_DTYPE(dtype, T, {
            qi::launch(qk_norm_rope_kv_vec_kernel<float, T>, grid, dim3(kWarpsPerBlock * 32), 0, stream,
                (const float*)qkv, qkv_splits, stride, (T*)q_out, q_gain, k_gain, eps, cos_t, sin_t, table_positions, positions, token_req,
                block_table, max_blocks, page_size, num_pages, (T*)k_pages, (T*)v_pages, nq, nkv, d, status);
        });
        return qi::check_launch("qk_norm_rope_kv");
    }
    if (vec) {
        QI_DISPATCH_DTYPE(dtype, T, {
            qi::launch(qk_norm_rope_kv_vec_kernel<T, T>, grid, dim3(kWarpsPerBlock * 32), 0, stream,
                (const T*)qkv, 1, (size_t)0, (T*)q_out, q_gain, k_gain, eps, cos_t, sin_t, table_positions, positions, token_req,
                block_table, max_blocks, page_size, num_pages, (T*)k_pages, (T*)v_pages, nq, nkv, d, status);
        });
        return qi::check_launch("qk_norm_rope_kv");
    }
    QI_DISPATCH_DTYPE(dtype, T, {
        qi::launch(qk_norm_rope_kv_kernel<T>, grid, dim3(kWarpsPerBlock * 32), 0, stream,
            (const T*)qkv, (T*)q_out, q_gain, k_gain, eps, cos_t, sin_t, rot, interleaved, table_positions, positions, token_req,
            block_table, max_blocks, page_size, num_pages, (T*)k_pages, (T*)v_pages, nq, nkv, d,
            status);
    });
    return qi::check_launch("qk_norm_rope_kv");
}
