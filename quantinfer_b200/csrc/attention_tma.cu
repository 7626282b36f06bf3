// The attention kernels of attention_mma.cu with their key/value tiles fetched by
// TMA instead of per-thread cp.async: one thread issues, per 64-key tile, a few
// cp.async.bulk.tensor copies (one per page piece and 64-column half) into a ring
// of shared-memory stages guarded by mbarriers, and every other thread only does
// tensor-core work. The page pool of a layer is seen as a matrix
// [num_pages * kv_heads * page_size, head_dim]; positions of one page and kv head
// are consecutive rows, so a box of min(page_size, 64) rows is one page piece.
// Needs a page size that is a power of two >= 8 (a box must be whole multiples
// of the 8-row swizzle pattern); other page sizes use the cp.async kernels.
//
// Rows of a page beyond a request's length hold older or zero data; they are
// finite (the pool is zeroed once and only finite values are written) and their
// scores are masked, so they contribute exactly zero.
//
// No load uses cluster multicast. Every mbarrier wait is bounded; when a bound
// runs out the kernel sets kStatusWaitTimeout and leaves.
#include "attention_frag.cuh"
#include "attention_noalloc.h"

#include <cuda.h>

namespace {

using namespace qi_attn;

constexpr int kTileKeys = 64;
constexpr uint32_t kSpinLimit = 1u << 21;
constexpr int kMaxTableEntries = 2048;   // block table entries one CTA keeps in shared memory

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kSpinLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}

// The same with a hint for the L2: in a decode step a key/value tile is read once, so it is the first
// to go when the L2 needs room (what the step's small kernels pass on stays there meanwhile).
__device__ __forceinline__ void tma_load_2d_once(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "l"(policy) : "memory");
}

// Issues the copies of keys [t0, t0 + 64) of kv head hk for K and V into one stage.
// `needed` = [lo, hi): a missing page inside it is an error; outside it any page will do.
// ONCE: the tile is read once in the step (decode), not by many CTAs (prefill).
template <int D, bool ONCE = false>
__device__ __forceinline__ void issue_kv_tile(uint32_t stage_smem, uint32_t bar, const CUtensorMap* map_k,
                                              const CUtensorMap* map_v, const int* table, int blk0,
                                              int n_blk, int page_size, int box_rows, int num_pages, int nkv,
                                              int hk, int t0, int lo, int hi, int* __restrict__ status) {
    constexpr int kHalfBytes = kTileKeys * 128;
    constexpr int kTileBytes = kTileKeys * D * 2;
    mbar_expect_tx(bar, 2 * kTileBytes);
    for (int r0 = 0; r0 < kTileKeys; r0 += box_rows) {
        const int key = t0 + r0;
        const int blk = key / page_size - blk0;     // `table` holds the entries blk0 .. blk0 + n_blk - 1
        int page = blk < n_blk ? table[blk] : -1;
        if (page < 0 || page >= num_pages) {
            if (key < hi && key + box_rows > lo && status) atomicOr(status, qi::kStatusBadPage);
            page = 0;
        }
        const int row = (page * nkv + hk) * page_size + (key % page_size);
#pragma unroll
        for (int h = 0; h < D / 64; ++h) {
            if (ONCE) {
                tma_load_2d_once(stage_smem + h * kHalfBytes + r0 * 128, map_k, bar, h * 64, row);
                tma_load_2d_once(stage_smem + kTileBytes + h * kHalfBytes + r0 * 128, map_v, bar, h * 64, row);
            } else {
                tma_load_2d(stage_smem + h * kHalfBytes + r0 * 128, map_k, bar, h * 64, row);
                tma_load_2d(stage_smem + kTileBytes + h * kHalfBytes + r0 * 128, map_v, bar, h * 64, row);
            }
        }
    }
}

// ------------------------------------------------------------------ prefill

constexpr int kPrefillRows = 128;
constexpr int kPrefillThreads = 256;
constexpr int kPrefillStages = 3;

template <int D>
__global__ void __launch_bounds__(kPrefillThreads, 1)
attention_prefill_tma_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                             const __grid_constant__ CUtensorMap map_v, qi::bf16* __restrict__ out,
                             const int* __restrict__ block_table, int max_blocks, int page_size, int box_rows,
                             int num_pages, const int* __restrict__ q_start, const int* __restrict__ start_pos,
                             const int* __restrict__ tile_req, const int* __restrict__ tile_q0, int nq, int nkv,
                             float scale_log2e, int window, int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    constexpr int kTileBytes = kTileKeys * D * 2;
    constexpr int kQBytes = kPrefillRows * D * 2;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_s = base, kv_s = base + kQBytes;
    const uint32_t bars = kv_s + kPrefillStages * 2 * kTileBytes;   // full[stages], q
    auto full_bar = [&](int s) { return bars + 8u * s; };
    const uint32_t q_bar = bars + 8u * kPrefillStages;
    int* s_table = reinterpret_cast<int*>(smem_raw + (bars + 64u - smem_u32(smem_raw)));   // block table entries of this tile's keys

    qi::pdl_enter();
    // blockIdx.x is the head, so that the tile list's order (most keys first) holds across all heads
    const int tile = blockIdx.y, h = blockIdx.x;
    const int hk = h / (nq / nkv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = tile_req[tile], q0 = tile_q0[tile];
    const int rows_valid = min(kPrefillRows, q_start[r + 1] - q0);
    const int pos0 = start_pos[r] + (q0 - q_start[r]);
    const int* table = block_table + (size_t)r * max_blocks;
    const int hi = pos0 + rows_valid;
    const int lo = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    const int t_begin = (lo / kTileKeys) * kTileKeys;
    const int n_tiles = (hi - t_begin + kTileKeys - 1) / kTileKeys;
    // all table entries the issuing thread will need, fetched by everybody at once (one
    // round trip instead of one per tile on the issuing thread's critical path)
    const int blk0 = t_begin / page_size;
    const int n_blk = min(min((t_begin + n_tiles * kTileKeys + page_size - 1) / page_size, max_blocks) - blk0, kMaxTableEntries);
    for (int i = threadIdx.x; i < n_blk; i += blockDim.x) s_table[i] = table[blk0 + i];

    if (threadIdx.x == 0) {
        for (int s = 0; s < kPrefillStages; ++s) mbar_init(full_bar(s), 1);
        mbar_init(q_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        mbar_expect_tx(q_bar, kQBytes);
#pragma unroll
        for (int hh = 0; hh < D / 64; ++hh)
            tma_load_2d(q_s + hh * (kPrefillRows * 128), &map_q, q_bar, h * D + hh * 64, q0);
        for (int i = 0; i < kPrefillStages && i < n_tiles; ++i)
            issue_kv_tile<D>(kv_s + i * 2 * kTileBytes, full_bar(i), &map_k, &map_v, s_table, blk0, n_blk, page_size, box_rows,
                             num_pages, nkv, hk, t_begin + i * kTileKeys, lo, hi, status);
    }

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
    uint32_t qa[D / 16][4];
    const int g = lane >> 2, t4 = lane & 3;
    const int row_pos[2] = {pos0 + warp * 16 + g, pos0 + warp * 16 + g + 8};
    const int warp_max_pos = pos0 + warp * 16 + 15, warp_min_pos = pos0 + warp * 16;
    const bool warp_active = warp * 16 < rows_valid;
    bool ok = mbar_wait(q_bar, 0);
    if (ok) load_q_frags<D, TmaSwizzle<kPrefillRows>>(qa, q_s, warp * 16, lane);

    for (int i = 0; i < n_tiles && ok; ++i) {
        const int stage = i % kPrefillStages;
        const int t0 = t_begin + i * kTileKeys;
        ok = mbar_wait(full_bar(stage), (uint32_t)(i / kPrefillStages) & 1u);
        if (!ok) break;
        if (warp_active && t0 <= warp_max_pos) {
            const uint32_t k_s = kv_s + stage * 2 * kTileBytes, v_s = k_s + kTileBytes;
            float s[8][4];
            qk_tile<D, 8, TmaSwizzle<kTileKeys>>(s, qa, k_s, 0, lane);
            // a tile that lies wholly inside every row's key range needs no mask
            const bool inner = t0 + kTileKeys - 1 <= warp_min_pos && t0 >= lo && t0 + kTileKeys <= hi &&
                               (window <= 0 || t0 > warp_max_pos - window);
            if (!inner) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = t0 + j * 8 + t4 * 2 + (e & 1);
                        const int pos = row_pos[e >> 1];
                        const bool valid = key <= pos && key >= lo && key < hi && (window <= 0 || key > pos - window);
                        if (!valid) s[j][e] = -INFINITY;
                    }
                }
            }
            softmax_tile<D, 8>(s, m, l, o, scale_log2e);
            pv_tile<D, 8, TmaSwizzle<kTileKeys>>(o, s, v_s, 0, lane);
        }
        __syncthreads();   // every warp is done with this stage
        if (threadIdx.x == 0 && i + kPrefillStages < n_tiles)
            issue_kv_tile<D>(kv_s + stage * 2 * kTileBytes, full_bar(stage), &map_k, &map_v, s_table, blk0, n_blk, page_size,
                             box_rows, num_pages, nkv, hk, t0 + kPrefillStages * kTileKeys, lo, hi, status);
    }
    if (!ok) {
        if (lane == 0 && status) atomicOr(status, qi::kStatusWaitTimeout);
        return;
    }
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 1);
        l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 2);
    }
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        const int row = warp * 16 + g + rr * 8;
        if (row >= rows_valid) continue;
        const float inv = l[rr] > 0.f ? 1.f / l[rr] : 0.f;
        qi::bf16* orow = out + ((size_t)(q0 + row) * nq + h) * D;
#pragma unroll
        for (int n = 0; n < D / 8; ++n)
            *reinterpret_cast<uint32_t*>(orow + n * 8 + t4 * 2) = pack_bf16(o[n][rr * 2] * inv, o[n][rr * 2 + 1] * inv);
    }
}

// ------------------------------------------------------------------ decode

constexpr int kDecodeThreads = 128;
constexpr int kDecodeStages = 3;

// What the decode kernel needs to make its own queries and the step's new key and value from the
// q/k/v projection (FUSED): the projection's output [tokens, width] in bfloat16, or its K-split
// partial sums [splits, tokens, width] in 32-bit (added here in split order); the q/k RMSNorm
// gains (null: none); the rotation table [positions, D / 2] (null: none); the cache pages to
// write the new key and value into (null: another layer wrote them, nothing is computed).
struct DecodeRope {
    const void* qkv;
    long long split_stride;     // elements between two splits
    const float* q_gain;
    const float* k_gain;
    const float* cos_t;
    const float* sin_t;
    qi::bf16* k_pages;
    qi::bf16* v_pages;
    float eps;
    int splits, width;
    int table_positions;        // rows of cos_t / sin_t
};

template <typename TIn> __device__ __forceinline__ float2 load2(const TIn* p);
template <> __device__ __forceinline__ float2 load2<float>(const float* p) { return *reinterpret_cast<const float2*>(p); }
template <> __device__ __forceinline__ float2 load2<qi::bf16>(const qi::bf16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}

// One warp, one head of D elements at `src` (plus the other splits): the sum of the splits, the
// RMSNorm with `gain` (null: none) and the half-split rotation by `pos` (cos_t null: none), in
// 32-bit, in the order of the stand-alone kernel (qknorm_rope_kv.cu). Lane l holds elements
// 2l, 2l + 1 (lo) and D/2 + 2l, D/2 + 2l + 1 (hi); lanes with 2l >= D/2 hold nothing.
template <int D, typename TIn>
__device__ __forceinline__ void head_norm_rope(const TIn* src, int splits, long long stride, const float* gain, float eps,
                                               const float* cos_t, const float* sin_t, int pos, int lane,
                                               float2& lo, float2& hi) {
    constexpr int kHalf = D / 2;
    const int p = 2 * lane;
    const bool has = p < kHalf;
    float2 a = make_float2(0.f, 0.f), b = make_float2(0.f, 0.f);
    // everything the head needs is requested at once (one round trip): its parts of up to eight
    // splits, the gain, the row of the rotation table
    float2 ga = make_float2(1.f, 1.f), gb = ga, c = make_float2(1.f, 1.f), sn = make_float2(0.f, 0.f);
    if (has) {
        float2 xs[8], ys[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            if (k < splits) {
                xs[k] = load2<TIn>(src + k * stride + p);
                ys[k] = load2<TIn>(src + k * stride + p + kHalf);
            }
        }
        if (gain) {
            ga = *reinterpret_cast<const float2*>(gain + p);
            gb = *reinterpret_cast<const float2*>(gain + p + kHalf);
        }
        if (cos_t) {
            c = *reinterpret_cast<const float2*>(cos_t + (size_t)pos * kHalf + p);
            sn = *reinterpret_cast<const float2*>(sin_t + (size_t)pos * kHalf + p);
        }
        a = xs[0];
        b = ys[0];
#pragma unroll
        for (int k = 1; k < 8; ++k) {
            if (k < splits) {
                a.x += xs[k].x; a.y += xs[k].y;
                b.x += ys[k].x; b.y += ys[k].y;
            }
        }
        for (int k = 8; k < splits; ++k) {
            const float2 x = load2<TIn>(src + k * stride + p), y = load2<TIn>(src + k * stride + p + kHalf);
            a.x += x.x; a.y += x.y;
            b.x += y.x; b.y += y.y;
        }
    }
    if (gain) {
        float ss = a.x * a.x + a.y * a.y;
        ss += b.x * b.x + b.y * b.y;
        ss = qi::warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)D + eps);
        if (has) {
            a.x = a.x * inv * ga.x; a.y = a.y * inv * ga.y;
            b.x = b.x * inv * gb.x; b.y = b.y * inv * gb.y;
        }
    }
    lo = a;
    hi = b;
    if (cos_t && has) {
        lo = make_float2(a.x * c.x - b.x * sn.x, a.y * c.y - b.y * sn.y);
        hi = make_float2(a.x * sn.x + b.x * c.x, a.y * sn.y + b.y * c.y);
    }
}

QI_TL_DEFINE(qi_timeline_attention)

// DIRECT: the request's keys are one range, and the CTA writes the attention output itself.
// FUSED: the queries and the step's new key and value are made here from the q/k/v projection
// (`rope`), not read from `q` and the cache; TIn is the projection's element type.
template <int D, bool DIRECT, bool FUSED, typename TIn>
__global__ void __launch_bounds__(kDecodeThreads)
attention_decode_tma_kernel(const qi::bf16* __restrict__ q, qi::bf16* __restrict__ out, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const int* __restrict__ block_table,
                            int max_blocks, int page_size, int box_rows, int num_pages,
                            const int* __restrict__ kv_len, const int* __restrict__ q_start,
                            float* __restrict__ ws_o, float* __restrict__ ws_ml, int nq, int nkv, float scale_log2e,
                            int window, int chunk, int* __restrict__ status, const DecodeRope rope) {
    extern __shared__ uint8_t smem_raw[];
    constexpr int kTileBytes = kTileKeys * D * 2;
    constexpr int kQBytes = 16 * D * 2;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t kv_s = base;                                       // stages x (K, V), later the merge buffers
    const uint32_t q_s = base + kDecodeStages * 2 * kTileBytes;       // [16, D], row swizzle
    uint8_t* q_tile = aligned + kDecodeStages * 2 * kTileBytes;
    const uint32_t bars = q_s + kQBytes;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    int* s_table = reinterpret_cast<int*>(aligned + kDecodeStages * 2 * kTileBytes + kQBytes + 64);
    qi::bf16* new_kv = reinterpret_cast<qi::bf16*>(s_table + kMaxTableEntries);   // [2][D]: this step's key and value (FUSED)

    // Lengths and block tables were copied before the step began, and keys and values of earlier
    // positions were written by earlier steps: only the newest key (position S - 1) and the
    // queries come from the kernel before this one. So the first tiles are requested before the
    // wait for that kernel, unless they hold the newest key.
    QI_TL_BEGIN();
    qi::pdl_launch_dependents();
    const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
    const int n_splits = gridDim.x;
    const int G = nq / nkv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t4 = lane & 3;
    const int S = kv_len[b];
    const int lo = (window > 0 && S - window > 0) ? S - window : 0;
    // The request's visible key tiles are dealt out evenly over the ranges (`chunk` is only the most a
    // range may hold, for which the launch was sized): a request that is shorter than the longest one the
    // launch allows for still keeps every CTA of its ranges equally busy.
    const int t_lo = lo / kTileKeys, t_hi = (S + kTileKeys - 1) / kTileKeys;
    const int per = (t_hi - t_lo + n_splits - 1) / n_splits;
    const int k0 = max((t_lo + split * per) * kTileKeys, lo);
    const int k1 = min(S, (t_lo + (split + 1) * per) * kTileKeys);
    const size_t part = ((size_t)b * nq + (size_t)hk * G) * n_splits + split;
    // the ranges of this launch must cover the request's keys; what lies beyond them is not read, so say so
    if (split == n_splits - 1 && hk == 0 && threadIdx.x == 0 && (long long)n_splits * chunk < S && status)
        atomicOr(status, qi::kStatusBadRange);

    const int tok = q_start[b];
    if (k0 >= k1) {   // nothing of this range belongs to the request: an empty partial
        qi::pdl_wait();
        QI_TL_WAKE();
        QI_TL_END(30);
        if (DIRECT) {
            for (int idx = threadIdx.x; idx < G * D; idx += kDecodeThreads)
                out[((size_t)tok * nq + (size_t)hk * G) * D + idx] = __float2bfloat16_rn(0.f);
            return;
        }
        if (threadIdx.x < G) {
            float* ml = ws_ml + (part + (size_t)threadIdx.x * n_splits) * 2;
            ml[0] = -INFINITY;
            ml[1] = 0.f;
        }
        return;
    }
    const int* table = block_table + (size_t)b * max_blocks;
    const int t_begin = (k0 / kTileKeys) * kTileKeys;
    const int n_tiles = (k1 - t_begin + kTileKeys - 1) / kTileKeys;
    const int blk0 = t_begin / page_size;
    const int n_blk = min(min((t_begin + n_tiles * kTileKeys + page_size - 1) / page_size, max_blocks) - blk0, kMaxTableEntries);
    for (int i = threadIdx.x; i < n_blk; i += blockDim.x) s_table[i] = table[blk0 + i];

    if (threadIdx.x == 0) {
        for (int s = 0; s < kDecodeStages; ++s) mbar_init(full_bar(s), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    int issued = 0;     // thread 0: tiles requested so far
    if (threadIdx.x == 0) {
        for (; issued < kDecodeStages && issued < n_tiles; ++issued) {
            if (t_begin + (issued + 1) * kTileKeys >= S) break;      // holds the newest key
            issue_kv_tile<D, true>(kv_s + issued * 2 * kTileBytes, full_bar(issued), &map_k, &map_v, s_table, blk0, n_blk, page_size,
                             box_rows, num_pages, nkv, hk, t_begin + issued * kTileKeys, k0, k1, status);
        }
    }
    qi::pdl_wait();
    QI_TL_WAKE();
    constexpr int kChunks = D / 8;
    // this CTA's range holds the step's own position: it makes the new key and value, writes them to
    // the cache and, since its copy of that cache row may be older than the write, into its tile
    const bool owns_new = FUSED && rope.k_pages != nullptr && k1 == S;
    if constexpr (FUSED) {
        const int pos = S - 1;
        int table_row = pos;
        if (rope.cos_t && pos >= rope.table_positions) {   // beyond the rotation table: flagged, the last row stands in
            if (threadIdx.x == 0 && status) atomicOr(status, qi::kStatusBadRange);
            table_row = rope.table_positions - 1;
        }
        const TIn* tok_row = reinterpret_cast<const TIn*>(rope.qkv) + (size_t)tok * rope.width;
        for (int row = warp; row < 16; row += kDecodeThreads / 32) {
            float2 lo = make_float2(0.f, 0.f), hi = lo;
            if (row < G)
                head_norm_rope<D, TIn>(tok_row + (size_t)(hk * G + row) * D, rope.splits, rope.split_stride, rope.q_gain, rope.eps,
                                       rope.cos_t, rope.sin_t, table_row, lane, lo, hi);
            const int p = 2 * lane;
            if (p < D / 2) {
                *reinterpret_cast<uint32_t*>(q_tile + RowSwizzle<D>::off(row, p >> 3) + (p & 7) * 2) = pack_bf16(lo.x, lo.y);
                const int ph = p + D / 2;
                *reinterpret_cast<uint32_t*>(q_tile + RowSwizzle<D>::off(row, ph >> 3) + (ph & 7) * 2) = pack_bf16(hi.x, hi.y);
            }
        }
        if (owns_new && warp < 2) {
            // warp 0: the key (norm, rotation); warp 1: the value (as it is)
            const TIn* src = tok_row + (size_t)(nq + (warp == 0 ? 0 : nkv) + hk) * D;
            float2 lo, hi;
            head_norm_rope<D, TIn>(src, rope.splits, rope.split_stride, warp == 0 ? rope.k_gain : nullptr, rope.eps,
                                   warp == 0 ? rope.cos_t : nullptr, rope.sin_t, table_row, lane, lo, hi);
            const int page = block_table[(size_t)b * max_blocks + pos / page_size];
            const int p = 2 * lane;
            if (page < 0 || page >= num_pages) {
                if (lane == 0 && status) atomicOr(status, qi::kStatusBadPage);
            } else if (p < D / 2) {
                qi::bf16* dst = (warp == 0 ? rope.k_pages : rope.v_pages) + (((size_t)page * nkv + hk) * page_size + (pos % page_size)) * (size_t)D;
                *reinterpret_cast<uint32_t*>(dst + p) = pack_bf16(lo.x, lo.y);
                *reinterpret_cast<uint32_t*>(dst + p + D / 2) = pack_bf16(hi.x, hi.y);
            }
            if (p < D / 2) {
                *reinterpret_cast<uint32_t*>(new_kv + warp * D + p) = pack_bf16(lo.x, lo.y);
                *reinterpret_cast<uint32_t*>(new_kv + warp * D + p + D / 2) = pack_bf16(hi.x, hi.y);
            }
        }
    } else {
        for (int idx = threadIdx.x; idx < 16 * kChunks; idx += kDecodeThreads) {
            const int row = idx / kChunks, c = idx % kChunks;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (row < G) v = *reinterpret_cast<const uint4*>(q + ((size_t)tok * nq + (size_t)hk * G + row) * D + c * 8);
            *reinterpret_cast<uint4*>(q_tile + RowSwizzle<D>::off(row, c)) = v;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = issued; i < kDecodeStages && i < n_tiles; ++i)
            issue_kv_tile<D, true>(kv_s + i * 2 * kTileBytes, full_bar(i), &map_k, &map_v, s_table, blk0, n_blk, page_size, box_rows,
                             num_pages, nkv, hk, t_begin + i * kTileKeys, k0, k1, status);
    }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
    uint32_t qa[D / 16][4];
    load_q_frags<D, RowSwizzle<D>>(qa, q_s, 0, lane);

    bool ok = true;
    for (int i = 0; i < n_tiles; ++i) {
        const int stage = i % kDecodeStages;
        const int t0 = t_begin + i * kTileKeys;
        ok = mbar_wait(full_bar(stage), (uint32_t)(i / kDecodeStages) & 1u);
        if (!ok) break;
        if (i == 0) QI_TL_DATA();
        if (owns_new && i == n_tiles - 1) {
            // the tile's row of position S - 1 is replaced by what this CTA computed
            const int r = S - 1 - t0;
            if (threadIdx.x < 2 * kChunks) {
                const int which = threadIdx.x / kChunks, c = threadIdx.x % kChunks;
                *reinterpret_cast<uint4*>(aligned + stage * 2 * kTileBytes + which * kTileBytes + TmaSwizzle<kTileKeys>::off(r, c)) =
                    *reinterpret_cast<const uint4*>(new_kv + which * D + c * 8);
            }
            __syncthreads();
        }
        const int wkey0 = t0 + warp * 16;   // each warp takes 16 of the tile's 64 keys
        if (wkey0 < k1 && wkey0 + 16 > k0) {
            const uint32_t k_s = kv_s + stage * 2 * kTileBytes, v_s = k_s + kTileBytes;
            float s[2][4];
            qk_tile<D, 2, TmaSwizzle<kTileKeys>>(s, qa, k_s, warp * 16, lane);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = wkey0 + j * 8 + t4 * 2 + (e & 1);
                    if (key < k0 || key >= k1) s[j][e] = -INFINITY;
                }
            }
            softmax_tile<D, 2>(s, m, l, o, scale_log2e);
            pv_tile<D, 2, TmaSwizzle<kTileKeys>>(o, s, v_s, warp * 16, lane);
        }
        __syncthreads();
        if (threadIdx.x == 0 && i + kDecodeStages < n_tiles)
            issue_kv_tile<D, true>(kv_s + stage * 2 * kTileBytes, full_bar(stage), &map_k, &map_v, s_table, blk0, n_blk, page_size,
                             box_rows, num_pages, nkv, hk, t0 + kDecodeStages * kTileKeys, k0, k1, status);
    }
    if (!ok) {
        if (lane == 0 && status) atomicOr(status, qi::kStatusWaitTimeout);
        return;
    }
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 1);
        l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 2);
    }
    // merge the four warps (each saw different keys) through shared memory, in warp order;
    // every copy into the stages has completed (each tile's barrier was waited for)
    float* sm_o = reinterpret_cast<float*>(aligned);             // [4][16][D]
    float* sm_m = sm_o + 4 * 16 * D;                             // [4][16]
    float* sm_l = sm_m + 4 * 16;                                 // [4][16]
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        const int row = g + rr * 8;
        if (t4 == 0) {
            sm_m[warp * 16 + row] = m[rr];
            sm_l[warp * 16 + row] = l[rr];
        }
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            sm_o[(warp * 16 + row) * D + n * 8 + t4 * 2] = o[n][rr * 2];
            sm_o[(warp * 16 + row) * D + n * 8 + t4 * 2 + 1] = o[n][rr * 2 + 1];
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * D; idx += kDecodeThreads) {
        const int row = idx / D, col = idx % D;
        float M = -INFINITY;
        for (int w = 0; w < 4; ++w) M = fmaxf(M, sm_m[w * 16 + row]);
        float L = 0.f, O = 0.f;
        for (int w = 0; w < 4; ++w) {
            const float mw = sm_m[w * 16 + row];
            if (mw == -INFINITY) continue;
            const float f = exp2f(mw - M);
            L += sm_l[w * 16 + row] * f;
            O += sm_o[(w * 16 + row) * D + col] * f;
        }
        if (DIRECT) {
            out[((size_t)tok * nq + (size_t)hk * G + row) * D + col] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
        } else {
            const size_t p = part + (size_t)row * n_splits;
            ws_o[p * D + col] = O;
            if (col == 0) {
                ws_ml[p * 2] = M;
                ws_ml[p * 2 + 1] = L;
            }
        }
    }
    QI_TL_END(30);
}

// out[b, h, :] = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M), key ranges in order. A separate
// kernel: merging inside the decode kernel (last CTA by ticket) was measured slower, the
// merge then sits on the tail of the slowest CTA; so was making the ranges of a (request, kv
// head) one thread-block cluster that merges through distributed shared memory (4.31 against
// 4.25 ms a step at batch 16, 7.39 against 7.25 at batch 64).
template <int D>
__global__ void attention_merge_kernel(const float* __restrict__ ws_o, const float* __restrict__ ws_ml,
                                       const int* __restrict__ q_start, qi::bf16* __restrict__ out, int nq,
                                       int n_splits) {
    QI_TL_BEGIN();
    qi::pdl_enter();
    QI_TL_WAKE();
    const int h = blockIdx.x, b = blockIdx.y;
    const size_t base = ((size_t)b * nq + h) * n_splits;
    const int tok = q_start[b];
    if (n_splits <= 8 && (int)threadIdx.x < D && (int)blockDim.x >= D) {
        // few ranges: everything a column needs is requested at once (one round trip), then merged in range order
        const int col = threadIdx.x;
        float ms[8], ls[8], ov[8];
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            if (s < n_splits) {
                ms[s] = ws_ml[(base + s) * 2];
                ls[s] = ws_ml[(base + s) * 2 + 1];
                ov[s] = ws_o[(base + s) * D + col];
            }
        }
        float M = -INFINITY;
#pragma unroll
        for (int s = 0; s < 8; ++s)
            if (s < n_splits) M = fmaxf(M, ms[s]);
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            if (s < n_splits) {
                const float f = (ms[s] == -INFINITY) ? 0.f : exp2f(ms[s] - M);
                L += ls[s] * f;
                O += (ms[s] == -INFINITY) ? 0.f : ov[s] * f;      // an empty range's slot holds no data
            }
        }
        out[((size_t)tok * nq + h) * D + col] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
        QI_TL_END(31);
        return;
    }
    if (n_splits <= 8 && (int)blockDim.x >= D) return;      // the threads beyond the head's columns
    float M = -INFINITY;
#pragma unroll 4
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, ws_ml[(base + s) * 2]);
    for (int col = threadIdx.x; col < D; col += blockDim.x) {
        float L = 0.f, O = 0.f;
#pragma unroll 4
        for (int s = 0; s < n_splits; ++s) {
            const float ms = ws_ml[(base + s) * 2];
            const float o = ws_o[(base + s) * D + col];
            const float f = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
            L += ws_ml[(base + s) * 2 + 1] * f;
            O += (ms == -INFINITY) ? 0.f : o * f;      // an empty range's slot holds no data
        }
        out[((size_t)tok * nq + h) * D + col] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
    }
    QI_TL_END(31);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// Map of a row-major bf16 matrix [rows, cols] with boxes of [box_rows, 64] and the 128-byte swizzle.
int make_map(CUtensorMap* map, const void* ptr, long long rows, int cols, int box_rows) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return qi::fail("attention: cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return qi::fail("attention: cuTensorMapEncodeTiled failed with code %d (rows=%lld cols=%d box=%d)", (int)r, rows, cols, box_rows);
    return 0;
}

template <int D> constexpr int prefill_smem() { return kPrefillRows * D * 2 + kPrefillStages * 2 * kTileKeys * D * 2 + 64 + 4 * kMaxTableEntries + 1024; }
template <int D> constexpr int decode_smem() { return kDecodeStages * 2 * kTileKeys * D * 2 + 16 * D * 2 + 64 + 4 * kMaxTableEntries + 2 * D * 2 + 1024; }

template <int D>
int launch_prefill(const void* q, void* out, const void* k_pages, const void* v_pages, const int* block_table,
                   int max_blocks, int page_size, int num_pages, const int* q_start, const int* start_pos,
                   const int* tile_req, const int* tile_q0, int n_tiles, int n_tokens, int nq, int nkv, float scale,
                   int window, int* status, cudaStream_t stream) {
    auto kern = attention_prefill_tma_kernel<D>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, prefill_smem<D>());
        if (e != cudaSuccess) return qi::fail("attention_prefill: cannot reserve shared memory: %s", cudaGetErrorString(e));
        configured = true;
    }
    const int box_rows = page_size < kTileKeys ? page_size : kTileKeys;
    CUtensorMap mq, mk, mv;
    if (make_map(&mq, q, n_tokens, nq * D, kPrefillRows)) return 1;
    if (make_map(&mk, k_pages, (long long)num_pages * nkv * page_size, D, box_rows)) return 1;
    if (make_map(&mv, v_pages, (long long)num_pages * nkv * page_size, D, box_rows)) return 1;
    dim3 grid(nq, n_tiles);
    qi::launch(kern, grid, dim3(kPrefillThreads), prefill_smem<D>(), stream,
        mq, mk, mv, (qi::bf16*)out, block_table, max_blocks, page_size, box_rows, num_pages, q_start, start_pos,
        tile_req, tile_q0, nq, nkv, scale * 1.4426950408889634f, window, status);
    return qi::check_launch("attention_prefill_tma");
}

template <int D, bool FUSED, typename TIn>
int launch_decode_as(const void* q, void* out, const void* k_pages, const void* v_pages, const int* block_table,
                     int max_blocks, int page_size, int num_pages, const int* kv_len, const int* q_start, int batch,
                     int nq, int nkv, float scale, int window, int chunk, int n_splits, float* ws_o, float* ws_ml,
                     int* status, cudaStream_t stream, const DecodeRope& rope) {
    auto kern = attention_decode_tma_kernel<D, false, FUSED, TIn>;
    auto kern_direct = attention_decode_tma_kernel<D, true, FUSED, TIn>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, decode_smem<D>());
        if (e == cudaSuccess) e = cudaFuncSetAttribute(kern_direct, cudaFuncAttributeMaxDynamicSharedMemorySize, decode_smem<D>());
        if (e != cudaSuccess) return qi::fail("attention_decode: cannot reserve shared memory: %s", cudaGetErrorString(e));
        configured = true;
    }
    const int box_rows = page_size < kTileKeys ? page_size : kTileKeys;
    CUtensorMap mk, mv;
    if (make_map(&mk, k_pages, (long long)num_pages * nkv * page_size, D, box_rows)) return 1;
    if (make_map(&mv, v_pages, (long long)num_pages * nkv * page_size, D, box_rows)) return 1;
    dim3 grid(n_splits, nkv, batch);
    if (n_splits == 1) {
        qi::launch(kern_direct, grid, dim3(kDecodeThreads), decode_smem<D>(), stream,
            (const qi::bf16*)q, (qi::bf16*)out, mk, mv, block_table, max_blocks, page_size, box_rows, num_pages, kv_len,
            q_start, ws_o, ws_ml, nq, nkv, scale * 1.4426950408889634f, window, chunk, status, rope);
        return qi::check_launch("attention_decode_tma");
    }
    qi::launch(kern, grid, dim3(kDecodeThreads), decode_smem<D>(), stream,
        (const qi::bf16*)q, (qi::bf16*)out, mk, mv, block_table, max_blocks, page_size, box_rows, num_pages, kv_len, q_start, ws_o,
        ws_ml, nq, nkv, scale * 1.4426950408889634f, window, chunk, status, rope);
    if (int rc = qi::check_launch("attention_decode_tma")) return rc;
    qi::launch(attention_merge_kernel<D>, dim3(nq, batch), dim3(D >= 128 ? 128 : 64), 0, stream, (const float*)ws_o,
               (const float*)ws_ml, q_start, (qi::bf16*)out, nq, n_splits);
    return qi::check_launch("attention_merge");
}

// rope null: the queries are in `q` and the cache holds every key. Else the kernel makes them from
// the projection (`rope_dtype` says whether that is bfloat16 or 32-bit partial sums).
template <int D>
int launch_decode(const void* q, void* out, const void* k_pages, const void* v_pages, const int* block_table,
                  int max_blocks, int page_size, int num_pages, const int* kv_len, const int* q_start, int batch,
                  int nq, int nkv, float scale, int window, int chunk, int n_splits, float* ws_o, float* ws_ml,
                  int* status, cudaStream_t stream, const DecodeRope* rope = nullptr, int rope_dtype = qi::kF32) {
    if (!rope)
        return launch_decode_as<D, false, float>(q, out, k_pages, v_pages, block_table, max_blocks, page_size, num_pages, kv_len,
                                                 q_start, batch, nq, nkv, scale, window, chunk, n_splits, ws_o, ws_ml, status,
                                                 stream, DecodeRope{});
    if (rope_dtype == qi::kF32)
        return launch_decode_as<D, true, float>(q, out, k_pages, v_pages, block_table, max_blocks, page_size, num_pages, kv_len,
                                                q_start, batch, nq, nkv, scale, window, chunk, n_splits, ws_o, ws_ml, status,
                                                stream, *rope);
    return launch_decode_as<D, true, qi::bf16>(q, out, k_pages, v_pages, block_table, max_blocks, page_size, num_pages, kv_len,
                                               q_start, batch, nq, nkv, scale, window, chunk, n_splits, ws_o, ws_ml, status,
                                               stream, *rope);
}

bool pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

}  // namespace

// 1 if the TMA-fed attention kernels take this geometry.
extern "C" int qi_attention_tma_supported(int nq, int nkv, int d, int page_size, int max_blocks) {
    return (d == 64 || d == 128) && nkv > 0 && nq % nkv == 0 && nq / nkv <= 16 && pow2(page_size) && page_size >= 8 &&
           max_blocks > 0 && max_blocks <= kMaxTableEntries;
}

// Query rows per CTA of qi_attention_prefill_tma: the tile lists must be cut to this.
extern "C" int qi_attention_prefill_tma_rows() { return kPrefillRows; }

extern "C" int qi_attention_prefill_tma(const void* q, void* out, const void* k_pages, const void* v_pages,
                                        const int* block_table, int max_blocks, int page_size, int num_pages,
                                        const int* q_start, const int* start_pos, const int* tile_req,
                                        const int* tile_q0, int n_tiles, int n_tokens, int nq, int nkv, int d,
                                        float scale, int window, int* status, cudaStream_t stream) {
    QI_REQUIRE(qi_attention_tma_supported(nq, nkv, d, page_size, max_blocks),
               "attention_prefill_tma: heads %d/%d of size %d with %d pages of %d per request are not covered", nq, nkv, d, max_blocks, page_size);
    QI_REQUIRE(max_blocks > 0 && num_pages > 0 && window >= 0 && n_tokens > 0, "attention_prefill_tma: bad sizes");
    QI_REQUIRE(((uintptr_t)q & 15) == 0 && ((uintptr_t)k_pages & 15) == 0 && ((uintptr_t)v_pages & 15) == 0,
               "attention_prefill_tma: tensors must be 16-byte aligned");
    QI_REQUIRE((long long)num_pages * nkv * page_size < 2147483647LL, "attention_prefill_tma: the page pool has too many rows");
    QI_REQUIRE(n_tiles >= 0 && n_tiles <= 65535, "attention_prefill_tma: more than 65535 query tiles in one step");
    if (n_tiles == 0) return 0;
    if (d == 64)
        return launch_prefill<64>(q, out, k_pages, v_pages, block_table, max_blocks, page_size, num_pages, q_start,
                                  start_pos, tile_req, tile_q0, n_tiles, n_tokens, nq, nkv, scale, window, status, stream);
    return launch_prefill<128>(q, out, k_pages, v_pages, block_table, max_blocks, page_size, num_pages, q_start,
                               start_pos, tile_req, tile_q0, n_tiles, n_tokens, nq, nkv, scale, window, status, stream);
}

// Workspace floats: ws_o = batch * nq * n_splits * d, ws_ml = batch * nq * n_splits * 2.
extern "C" int qi_attention_decode_tma(const void* q, void* out, const void* k_pages, const void* v_pages,
                                       const int* block_table, int max_blocks, int page_size, int num_pages,
                                       const int* kv_len, const int* q_start, int batch, int nq, int nkv, int d,
                                       float scale, int window, int chunk, int n_splits, float* ws_o, float* ws_ml,
                                       int* status, cudaStream_t stream) {
    QI_REQUIRE(qi_attention_tma_supported(nq, nkv, d, page_size, max_blocks),
               "attention_decode_tma: heads %d/%d of size %d with %d pages of %d per request are not covered", nq, nkv, d, max_blocks, page_size);
    QI_REQUIRE(max_blocks > 0 && num_pages > 0 && window >= 0, "attention_decode_tma: bad sizes");
    QI_REQUIRE(chunk > 0 && chunk % kTileKeys == 0, "attention_decode_tma: the key range per CTA (%d) must be a positive multiple of %d", chunk, kTileKeys);
    QI_REQUIRE(n_splits > 0 && n_splits <= 65535 && nkv <= 65535 && batch <= 65535, "attention_decode_tma: grid too large");
    QI_REQUIRE(ws_o && ws_ml, "attention_decode_tma: workspace missing");
    QI_REQUIRE(((uintptr_t)q & 15) == 0 && ((uintptr_t)k_pages & 15) == 0 && ((uintptr_t)v_pages & 15) == 0,
               "attention_decode_tma: tensors must be 16-byte aligned");
    QI_REQUIRE((long long)num_pages * nkv * page_size < 2147483647LL, "attention_decode_tma: the page pool has too many rows");
    if (batch == 0) return 0;
    if (d == 64)
        return launch_decode<64>(q, out, k_pages, v_pages, block_table, max_blocks, page_size, num_pages, kv_len,
                                 q_start, batch, nq, nkv, scale, window, chunk, n_splits, ws_o, ws_ml, status, stream);
    return launch_decode<128>(q, out, k_pages, v_pages, block_table, max_blocks, page_size, num_pages, kv_len,
                              q_start, batch, nq, nkv, scale, window, chunk, n_splits, ws_o, ws_ml, status, stream);
}

// The same for a decode step whose q/k/v projection has just run: the kernel sums the projection's
// K-split partial sums (qkv_splits > 1: `qkv` is float32 [qkv_splits, tokens, (nq + 2 nkv) d]) or
// reads its output (qkv_splits == 1, element type qkv_dtype, [tokens, (nq + 2 nkv) d]), applies the
// q/k RMSNorm (gains null: none) and the rotation over the whole head (cos_t null: none), and writes
// the step's key and value into the cache at position kv_len - 1 of each request (writes 0: another
// layer has written them; nothing is computed). One launch does what qi_qk_norm_rope_kv followed by
// qi_attention_decode_tma does. Request b's token is row q_start[b] of the projection.
extern "C" int qi_attention_decode_rope_tma(const void* qkv, int qkv_dtype, int qkv_splits, int n_tokens, const float* q_gain,
                                            const float* k_gain, float eps, const float* cos_t, const float* sin_t,
                                            int table_positions, int writes, void* out, void* k_pages, void* v_pages,
                                            const int* block_table, int max_blocks, int page_size, int num_pages,
                                            const int* kv_len, const int* q_start, int batch, int nq, int nkv, int d,
                                            float scale, int window, int chunk, int n_splits, float* ws_o, float* ws_ml,
                                            int* status, cudaStream_t stream) {
    QI_REQUIRE(qi_attention_tma_supported(nq, nkv, d, page_size, max_blocks),
               "attention_decode_rope_tma: heads %d/%d of size %d with %d pages of %d per request are not covered", nq, nkv, d, max_blocks, page_size);
    QI_REQUIRE(max_blocks > 0 && num_pages > 0 && window >= 0 && n_tokens >= batch, "attention_decode_rope_tma: bad sizes");
    QI_REQUIRE(chunk > 0 && chunk % kTileKeys == 0, "attention_decode_rope_tma: the key range per CTA (%d) must be a positive multiple of %d", chunk, kTileKeys);
    QI_REQUIRE(n_splits > 0 && n_splits <= 65535 && nkv <= 65535 && batch <= 65535, "attention_decode_rope_tma: grid too large");
    QI_REQUIRE(ws_o && ws_ml && qkv && out, "attention_decode_rope_tma: a buffer is missing");
    QI_REQUIRE(qkv_splits >= 1 && (qkv_splits == 1 || qkv_dtype == qi::kF32), "attention_decode_rope_tma: partial sums must be float32");
    QI_REQUIRE(qkv_dtype == qi::kF32 || qkv_dtype == qi::kBF16, "attention_decode_rope_tma: unknown element type");
    QI_REQUIRE((cos_t == nullptr) == (sin_t == nullptr) && (!cos_t || table_positions > 0), "attention_decode_rope_tma: incomplete rotation table");
    QI_REQUIRE(((uintptr_t)qkv & 15) == 0 && ((uintptr_t)k_pages & 15) == 0 && ((uintptr_t)v_pages & 15) == 0 &&
               ((uintptr_t)q_gain & 7) == 0 && ((uintptr_t)k_gain & 7) == 0 && ((uintptr_t)cos_t & 7) == 0 && ((uintptr_t)sin_t & 7) == 0,
               "attention_decode_rope_tma: tensors must be aligned (16 bytes; gains and tables 8)");
    QI_REQUIRE((long long)num_pages * nkv * page_size < 2147483647LL, "attention_decode_rope_tma: the page pool has too many rows");
    if (batch == 0) return 0;
    DecodeRope r;
    r.qkv = qkv;
    r.width = (nq + 2 * nkv) * d;
    r.split_stride = (long long)n_tokens * r.width;
    r.q_gain = q_gain; r.k_gain = k_gain; r.cos_t = cos_t; r.sin_t = sin_t; r.table_positions = table_positions;
    r.k_pages = writes ? (qi::bf16*)k_pages : nullptr;
    r.v_pages = writes ? (qi::bf16*)v_pages : nullptr;
    r.eps = eps; r.splits = qkv_splits;
    if (d == 64)
        return launch_decode<64>(nullptr, out, k_pages, v_pages, block_table, max_blocks, page_size, num_pages, kv_len, q_start,
                                 batch, nq, nkv, scale, window, chunk, n_splits, ws_o, ws_ml, status, stream, &r, qkv_dtype);
    return launch_decode<128>(nullptr, out, k_pages, v_pages, block_table, max_blocks, page_size, num_pages, kv_len, q_start,
                              batch, nq, nkv, scale, window, chunk, n_splits, ws_o, ws_ml, status, stream, &r, qkv_dtype);
}

// ------------------------------------------------------------------ the entry point that allocates nothing

namespace {

// Partial results of qi_attention_decode_tma_static. In host code this name is only a
// stand-in for the symbol, not a device address: the address comes from
// cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_decode_scratch[QI_DECODE_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
float* g_decode_scratch_ptr[kMaxDevices] = {};

// The array's address on the current device, looked up once per device.
int decode_scratch(float** ptr) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return qi::fail("attention_decode_tma_static: cudaGetDevice failed: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return qi::fail("attention_decode_tma_static: device index %d is not supported", dev);
    if (!g_decode_scratch_ptr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_decode_scratch);
        if (e != cudaSuccess || !p)
            return qi::fail("attention_decode_tma_static: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
        g_decode_scratch_ptr[dev] = static_cast<float*>(p);
    }
    *ptr = g_decode_scratch_ptr[dev];
    return 0;
}

}  // namespace

extern "C" unsigned long long qi_attention_decode_static_scratch_bytes(void) { return QI_DECODE_STATIC_SCRATCH_BYTES; }

extern "C" int qi_attention_decode_tma_static(const void* q, void* out, const void* k_pages, const void* v_pages,
                                              const int* block_table, int max_blocks, int page_size, int num_pages,
                                              const int* kv_len, const int* q_start, int batch, int nq, int nkv, int d,
                                              float scale, int window, int chunk, int n_splits, int* status,
                                              cudaStream_t stream) {
    QI_REQUIRE(batch >= 0 && nq > 0 && d > 0 && n_splits > 0, "attention_decode_tma_static: bad sizes");
    const unsigned long long need = 4ull * (unsigned long long)batch * nq * n_splits * (unsigned long long)(d + 2);
    QI_REQUIRE(need <= QI_DECODE_STATIC_SCRATCH_BYTES,
               "attention_decode_tma_static: %d requests x %d heads x %d key ranges of size %d need %llu bytes of scratch, "
               "the static array holds %u; use fewer key ranges, a smaller batch, or qi_attention_decode_tma with a workspace",
               batch, nq, n_splits, d, need, QI_DECODE_STATIC_SCRATCH_BYTES);
    float* scratch = nullptr;
    if (decode_scratch(&scratch)) return 1;
    float* ws_o = scratch;
    float* ws_ml = scratch + (size_t)batch * nq * n_splits * d;
    return qi_attention_decode_tma(q, out, k_pages, v_pages, block_table, max_blocks, page_size, num_pages, kv_len,
                                   q_start, batch, nq, nkv, d, scale, window, chunk, n_splits, ws_o, ws_ml, status, stream);
}

QI_TL_EXPORT(qi_timeline_attention)
