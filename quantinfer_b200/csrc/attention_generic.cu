// Causal grouped-query attention over the paged cache, for any span length,
// any head size up to 256 and any page size: the kernel of the true 32-bit
// path and the one that takes whatever the tensor-core kernels refuse.
//
// For the query of token t (request r, absolute position p) and query head h
// (kv head h / (nq / nkv): consecutive query heads share a kv head):
//     score_j = (sum_i q_i k_{j,i}) * scale          for lo <= j <= p
//     out     = sum_j softmax(score)_j * v_j
// with lo = 0, or p - window + 1 for a windowed layer. Scores, the maximum,
// the exponentials and the weighted sum are 32-bit. This is the reference's
// loop (crates/quantinfer-runtime/src/attention.rs:105-135; group :83,
// scale :84, causal bound :106,111) with the softmax evaluated online, one
// chunk of 32 keys at a time, so that no score row is stored.
//
// One block per (token, head); its four warps take chunks of keys in turn and
// their partial results are combined in warp order.
#include "common.cuh"

#include <math.h>

namespace {

constexpr int kWarps = 4;
constexpr int kMaxD = 256;
constexpr int kAccPerLane = kMaxD / 32;

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
attention_generic_kernel(const T* __restrict__ q, T* __restrict__ out, const T* __restrict__ k_pages,
                         const T* __restrict__ v_pages, const int* __restrict__ block_table,
                         int max_blocks, int page_size, int num_pages,
                         const int* __restrict__ positions, const int* __restrict__ token_req,
                         int nq, int nkv, int d, float scale, int window, int* __restrict__ status) {
    extern __shared__ float smem[];
    float* q_s = smem;                          // [d]
    float* part_acc = smem + d;                 // [kWarps][d]
    float* part_m = part_acc + kWarps * d;      // [kWarps]
    float* part_l = part_m + kWarps;            // [kWarps]

    qi::pdl_enter();
    const int t = blockIdx.y, h = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hk = h / (nq / nkv);
    const int pos = positions[t];
    const int r = token_req[t];
    const int* table = block_table + (size_t)r * max_blocks;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

    const T* qrow = q + ((size_t)t * nq + h) * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) q_s[i] = qi::to_f32<T>(qrow[i]);
    __syncthreads();

    float m = -INFINITY, l = 0.f;
    float acc[kAccPerLane];
#pragma unroll
    for (int i = 0; i < kAccPerLane; ++i) acc[i] = 0.f;

    bool bad_page = false;
    for (int base = lo + warp * 32; base <= pos; base += kWarps * 32) {
        const int j = base + lane;
        const bool valid = j <= pos;
        float s = -INFINITY;
        if (valid) {
            const int page = table[j / page_size];
            if (page < 0 || page >= num_pages) {
                bad_page = true;
            } else {
                const T* krow = k_pages + (((size_t)page * nkv + hk) * page_size + (j % page_size)) * (size_t)d;
                float dot = 0.f;
                for (int i = 0; i < d; ++i) dot = fmaf(q_s[i], qi::to_f32<T>(krow[i]), dot);
                s = dot * scale;
            }
        }
        const float cm = qi::warp_max(s);
        if (cm == -INFINITY) continue;  // only after a bad page
        const float m_new = fmaxf(m, cm);
        const float corr = expf(m - m_new);  // m = -inf on the first chunk gives 0
        const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
        l = l * corr + qi::warp_sum(p);
#pragma unroll
        for (int i = 0; i < kAccPerLane; ++i) acc[i] *= corr;
        const int count = min(32, pos - base + 1);
        for (int jj = 0; jj < count; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int key = base + jj;
            const int page = table[key / page_size];
            if (page < 0 || page >= num_pages) continue;
            const T* vrow = v_pages + (((size_t)page * nkv + hk) * page_size + (key % page_size)) * (size_t)d;
#pragma unroll
            for (int i = 0; i < kAccPerLane; ++i) {
                const int idx = lane + 32 * i;
                if (idx < d) acc[i] = fmaf(pj, qi::to_f32<T>(vrow[idx]), acc[i]);
            }
        }
        m = m_new;
    }
    if (bad_page && status) atomicOr(status, qi::kStatusBadPage);

    if (lane == 0) {
        part_m[warp] = m;
        part_l[warp] = l;
    }
#pragma unroll
    for (int i = 0; i < kAccPerLane; ++i) {
        const int idx = lane + 32 * i;
        if (idx < d) part_acc[warp * d + idx] = acc[i];
    }
    __syncthreads();

    float gm = -INFINITY;
    for (int w = 0; w < kWarps; ++w) gm = fmaxf(gm, part_m[w]);
    float gl = 0.f;
    float wscale[kWarps];
    for (int w = 0; w < kWarps; ++w) {
        wscale[w] = (part_m[w] == -INFINITY) ? 0.f : expf(part_m[w] - gm);
        gl += part_l[w] * wscale[w];
    }
    T* orow = out + ((size_t)t * nq + h) * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float o = 0.f;
        for (int w = 0; w < kWarps; ++w) o += part_acc[w * d + i] * wscale[w];
        orow[i] = qi::from_f32<T>(gl > 0.f ? o / gl : 0.f);
    }
}

}  // namespace

extern "C" int qi_attention_generic(const void* q, void* out, int dtype, const void* k_pages,
                                    const void* v_pages, const int* block_table, int max_blocks,
                                    int page_size, int num_pages, const int* positions,
                                    const int* token_req, int n_tokens, int nq, int nkv, int d,
                                    float scale, int window, int* status, cudaStream_t stream) {
    QI_REQUIRE(n_tokens >= 0 && nq > 0 && nkv > 0 && d > 0, "attention: bad sizes");
    QI_REQUIRE(nq % nkv == 0, "attention: %d query heads are not a multiple of %d kv heads", nq, nkv);
    QI_REQUIRE(d <= kMaxD, "attention: head_dim %d is above the limit %d of this kernel", d, kMaxD);
    QI_REQUIRE(page_size > 0 && max_blocks > 0 && num_pages > 0, "attention: bad page geometry");
    QI_REQUIRE(window >= 0, "attention: window must be >= 0 (0 = all keys)");
    QI_REQUIRE(n_tokens <= 65535 * 32768 && nq <= 65535, "attention: grid too large");
    if (n_tokens == 0) return 0;
    const size_t smem = sizeof(float) * ((size_t)d + kWarps * d + 2 * kWarps);
    // grid.y is limited to 65535: launch in slabs of tokens.
    for (int t0 = 0; t0 < n_tokens; t0 += 65535) {
        const int nt = n_tokens - t0 < 65535 ? n_tokens - t0 : 65535;
        dim3 grid(nq, nt);
        QI_DISPATCH_DTYPE(dtype, T, {
            qi::launch(attention_generic_kernel<T>, grid, dim3(kWarps * 32), smem, stream,
                (const T*)q + (size_t)t0 * nq * d, (T*)out + (size_t)t0 * nq * d, (const T*)k_pages,
                (const T*)v_pages, block_table, max_blocks, page_size, num_pages, positions + t0,
                token_req + t0, nq, nkv, d, scale, window, status);
        });
    }
    return qi::check_launch("attention_generic");
}
