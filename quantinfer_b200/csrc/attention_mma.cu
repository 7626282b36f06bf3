// bfloat16 attention over the paged cache on the tensor cores (mma.sync
// m16n8k16, 32-bit scores, softmax and accumulation), for head sizes 64 and 128:
//
//  * attention_prefill: causal flash attention for spans of any length. One CTA
//    takes 64 query rows of one request (a part of a tile of the batch's tile
//    list) and one query head and walks the keys
//    0 .. position in tiles of 64, with the softmax evaluated online.
//  * attention_decode: one query token per request. One CTA takes one request,
//    one kv head (all query heads of its group share every key and value read)
//    and one contiguous range of keys; partial results (maximum, sum, weighted
//    values) go to a 32-bit workspace and a second kernel merges the ranges in
//    order. The key ranges are fixed multiples of 64 positions, so the grid
//    does not depend on the requests' lengths and the launch can sit in a CUDA
//    graph; a CTA whose range lies beyond its request's length writes an empty
//    partial.
//
// Formulas as the reference's loop (crates/quantinfer-runtime/src/attention.rs:105-135:
// score = dot * 1/sqrt(d), softmax with the maximum subtracted, weighted sum of
// values; kv head = query head / group, :83). exp is evaluated as
// exp2((s - m) * log2 e).
//
// Keys and values are fetched with cp.async through the request's block table
// (page = table[position / page_size]), so any page size works; rows are kept in
// shared memory with a 16-byte-chunk XOR swizzle and read with ldmatrix.
#include "attention_frag.cuh"

namespace {

constexpr int kTileKeys = 64;
constexpr int kThreads = 128;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

using namespace qi_attn;

template <int D> __device__ __forceinline__ uint32_t swz(int row, int chunk) { return RowSwizzle<D>::off(row, chunk); }

// Copies keys [t0, t0 + 64) of one kv head into a shared tile; rows outside [vlo, vhi) are zeroed.
template <int D>
__device__ __forceinline__ void load_kv_tile(uint32_t dst, const qi::bf16* __restrict__ pages,
                                             const int* __restrict__ table, int page_size, int num_pages, int nkv,
                                             int hk, int t0, int vlo, int vhi, uint8_t* dst_generic, bool& bad_page) {
    constexpr int kChunks = D / 8;
    for (int idx = threadIdx.x; idx < kTileKeys * kChunks; idx += kThreads) {
        const int row = idx / kChunks, chunk = idx % kChunks;
        const int key = t0 + row;
        const uint32_t off = swz<D>(row, chunk);
        bool ok = key >= vlo && key < vhi;
        int page = 0;
        if (ok) {
            page = table[key / page_size];
            if (page < 0 || page >= num_pages) { bad_page = true; ok = false; }
        }
        if (ok) {
            const qi::bf16* src = pages + (((size_t)page * nkv + hk) * page_size + (key % page_size)) * (size_t)D + chunk * 8;
            cp_async16(dst + off, src);
        } else {
            *reinterpret_cast<uint4*>(dst_generic + off) = make_uint4(0u, 0u, 0u, 0u);
        }
    }
}

// ------------------------------------------------------------------ prefill

template <int D>
__global__ void __launch_bounds__(kThreads)
attention_prefill_kernel(const qi::bf16* __restrict__ q, qi::bf16* __restrict__ out,
                         const qi::bf16* __restrict__ k_pages, const qi::bf16* __restrict__ v_pages,
                         const int* __restrict__ block_table, int max_blocks, int page_size, int num_pages,
                         const int* __restrict__ q_start, const int* __restrict__ start_pos,
                         const int* __restrict__ tile_req, const int* __restrict__ tile_q0, int nq, int nkv,
                         float scale_log2e, int window, int* __restrict__ status) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int kTileBytes = kTileKeys * D * 2;
    uint8_t* q_tile = smem;                               // [64, D]
    uint8_t* kv_tile = smem + kTileBytes;                 // 2 x (K, V)
    const uint32_t q_s = smem_u32(q_tile), kv_s = smem_u32(kv_tile);

    qi::pdl_enter();
    const int tile = blockIdx.x, h = blockIdx.y;
    const int hk = h / (nq / nkv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = tile_req[tile], q0 = tile_q0[tile] + blockIdx.z * kTileKeys;   // blockIdx.z: 64-row part of the tile
    if (q0 >= q_start[r + 1]) return;
    const int rows_valid = min(kTileKeys, q_start[r + 1] - q0);
    const int pos0 = start_pos[r] + (q0 - q_start[r]);
    const int* table = block_table + (size_t)r * max_blocks;
    const int hi = pos0 + rows_valid;                                   // keys < hi
    const int lo = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    bool bad_page = false;

    // query rows of this head
    constexpr int kChunks = D / 8;
    for (int idx = threadIdx.x; idx < kTileKeys * kChunks; idx += kThreads) {
        const int row = idx / kChunks, chunk = idx % kChunks;
        const uint32_t off = swz<D>(row, chunk);
        if (row < rows_valid) cp_async16(q_s + off, q + ((size_t)(q0 + row) * nq + h) * D + chunk * 8);
        else *reinterpret_cast<uint4*>(q_tile + off) = make_uint4(0u, 0u, 0u, 0u);
    }
    const int t_begin = (lo / kTileKeys) * kTileKeys;
    const int n_tiles = (hi - t_begin + kTileKeys - 1) / kTileKeys;
    load_kv_tile<D>(kv_s, k_pages, table, page_size, num_pages, nkv, hk, t_begin, lo, hi, kv_tile, bad_page);
    load_kv_tile<D>(kv_s + kTileBytes, v_pages, table, page_size, num_pages, nkv, hk, t_begin, lo, hi, kv_tile + kTileBytes, bad_page);
    cp_async_commit();

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

    for (int i = 0; i < n_tiles; ++i) {
        const int buf = i & 1;
        const int t0 = t_begin + i * kTileKeys;
        if (i + 1 < n_tiles) {
            const uint32_t nb = kv_s + (buf ^ 1) * 2 * kTileBytes;
            uint8_t* ng = kv_tile + (buf ^ 1) * 2 * kTileBytes;
            load_kv_tile<D>(nb, k_pages, table, page_size, num_pages, nkv, hk, t0 + kTileKeys, lo, hi, ng, bad_page);
            load_kv_tile<D>(nb + kTileBytes, v_pages, table, page_size, num_pages, nkv, hk, t0 + kTileKeys, lo, hi, ng + kTileBytes, bad_page);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (i == 0) {
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                const int row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                ldmatrix_x4(q_s + swz<D>(row, ks * 2 + (lane >> 4)), qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3]);
            }
        }
        if (t0 <= warp_max_pos) {   // this warp's rows see at least one key of the tile
            const uint32_t k_s = kv_s + buf * 2 * kTileBytes, v_s = k_s + kTileBytes;
            float s[8][4];
            qk_tile<D, 8, RowSwizzle<D>>(s, qa, k_s, 0, lane);
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
            pv_tile<D, 8, RowSwizzle<D>>(o, s, v_s, 0, lane);
        }
        __syncthreads();
    }
    if (bad_page && status) atomicOr(status, qi::kStatusBadPage);

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
        for (int n = 0; n < D / 8; ++n) {
            const uint32_t v = pack_bf16(o[n][rr * 2] * inv, o[n][rr * 2 + 1] * inv);
            *reinterpret_cast<uint32_t*>(orow + n * 8 + t4 * 2) = v;
        }
    }
}

// ------------------------------------------------------------------ decode

template <int D>
__global__ void __launch_bounds__(kThreads)
attention_decode_kernel(const qi::bf16* __restrict__ q, const qi::bf16* __restrict__ k_pages,
                        const qi::bf16* __restrict__ v_pages, const int* __restrict__ block_table, int max_blocks,
                        int page_size, int num_pages, const int* __restrict__ kv_len,
                        const int* __restrict__ q_start, float* __restrict__ ws_o, float* __restrict__ ws_ml,
                        int nq, int nkv, float scale_log2e, int window, int chunk, int* __restrict__ status) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int kTileBytes = kTileKeys * D * 2;
    constexpr int kQBytes = 16 * D * 2;
    uint8_t* q_tile = smem;                       // [16, D]
    uint8_t* kv_tile = smem + kQBytes;            // 2 x (K, V)
    const uint32_t q_s = smem_u32(q_tile), kv_s = smem_u32(kv_tile);

    qi::pdl_enter();
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
    const size_t part = ((size_t)b * nq + (size_t)hk * G) * n_splits + split;   // + g * n_splits per head
    // the ranges of this launch must cover the request's keys; what lies beyond them is not read, so say so
    if (split == n_splits - 1 && hk == 0 && threadIdx.x == 0 && (long long)n_splits * chunk < S && status)
        atomicOr(status, qi::kStatusBadRange);

    if (k0 >= k1) {   // nothing of this range belongs to the request
        if (threadIdx.x < G) {
            float* ml = ws_ml + (part + (size_t)threadIdx.x * n_splits) * 2;
            ml[0] = -INFINITY;
            ml[1] = 0.f;
        }
        return;
    }
    const int* table = block_table + (size_t)b * max_blocks;
    const int tok = q_start[b];
    bool bad_page = false;

    constexpr int kChunks = D / 8;
    for (int idx = threadIdx.x; idx < 16 * kChunks; idx += kThreads) {
        const int row = idx / kChunks, chunk_i = idx % kChunks;
        const uint32_t off = swz<D>(row, chunk_i);
        if (row < G) cp_async16(q_s + off, q + ((size_t)tok * nq + (size_t)hk * G + row) * D + chunk_i * 8);
        else *reinterpret_cast<uint4*>(q_tile + off) = make_uint4(0u, 0u, 0u, 0u);
    }
    const int t_begin = (k0 / kTileKeys) * kTileKeys;
    const int n_tiles = (k1 - t_begin + kTileKeys - 1) / kTileKeys;
    load_kv_tile<D>(kv_s, k_pages, table, page_size, num_pages, nkv, hk, t_begin, k0, k1, kv_tile, bad_page);
    load_kv_tile<D>(kv_s + kTileBytes, v_pages, table, page_size, num_pages, nkv, hk, t_begin, k0, k1, kv_tile + kTileBytes, bad_page);
    cp_async_commit();

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
    uint32_t qa[D / 16][4];

    for (int i = 0; i < n_tiles; ++i) {
        const int buf = i & 1;
        const int t0 = t_begin + i * kTileKeys;
        if (i + 1 < n_tiles) {
            const uint32_t nb = kv_s + (buf ^ 1) * 2 * kTileBytes;
            uint8_t* ng = kv_tile + (buf ^ 1) * 2 * kTileBytes;
            load_kv_tile<D>(nb, k_pages, table, page_size, num_pages, nkv, hk, t0 + kTileKeys, k0, k1, ng, bad_page);
            load_kv_tile<D>(nb + kTileBytes, v_pages, table, page_size, num_pages, nkv, hk, t0 + kTileKeys, k0, k1, ng + kTileBytes, bad_page);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (i == 0) {
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                const int row = (lane & 7) + ((lane >> 3) & 1) * 8;
                ldmatrix_x4(q_s + swz<D>(row, ks * 2 + (lane >> 4)), qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3]);
            }
        }
        // each warp takes 16 of the tile's 64 keys
        const int wkey0 = t0 + warp * 16;
        if (wkey0 < k1 && wkey0 + 16 > k0) {
            const uint32_t k_s = kv_s + buf * 2 * kTileBytes, v_s = k_s + kTileBytes;
            float s[2][4];
            qk_tile<D, 2, RowSwizzle<D>>(s, qa, k_s, warp * 16, lane);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = wkey0 + j * 8 + t4 * 2 + (e & 1);
                    if (key < k0 || key >= k1) s[j][e] = -INFINITY;
                }
            }
            softmax_tile<D, 2>(s, m, l, o, scale_log2e);
            pv_tile<D, 2, RowSwizzle<D>>(o, s, v_s, warp * 16, lane);
        }
        __syncthreads();
    }
    if (bad_page && status) atomicOr(status, qi::kStatusBadPage);

#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 1);
        l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 2);
    }
    // merge the four warps (each saw different keys) through shared memory, in warp order
    float* sm_o = reinterpret_cast<float*>(kv_tile);            // [4][16][D]
    float* sm_m = sm_o + 4 * 16 * D;                            // [4][16]
    float* sm_l = sm_m + 4 * 16;                                // [4][16]
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
    for (int idx = threadIdx.x; idx < G * D; idx += kThreads) {
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
        const size_t p = part + (size_t)row * n_splits;
        ws_o[p * D + col] = O;
        if (col == 0) {
            ws_ml[p * 2] = M;
            ws_ml[p * 2 + 1] = L;
        }
    }
}

// out[b, h, :] = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M), splits in order.
template <int D>
__global__ void attention_decode_merge_kernel(const float* __restrict__ ws_o, const float* __restrict__ ws_ml,
                                              const int* __restrict__ q_start, qi::bf16* __restrict__ out, int nq,
                                              int n_splits) {
    qi::pdl_enter();
    const int h = blockIdx.x, b = blockIdx.y;
    const size_t base = ((size_t)b * nq + h) * n_splits;
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, ws_ml[(base + s) * 2]);
    const int tok = q_start[b];
    for (int col = threadIdx.x; col < D; col += blockDim.x) {
        float L = 0.f, O = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float ms = ws_ml[(base + s) * 2];
            if (ms == -INFINITY) continue;
            const float f = exp2f(ms - M);
            L += ws_ml[(base + s) * 2 + 1] * f;
            O += ws_o[(base + s) * D + col] * f;
        }
        out[((size_t)tok * nq + h) * D + col] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
    }
}

template <int D> int prefill_smem() { return 5 * kTileKeys * D * 2; }
template <int D> int decode_smem() {
    const int tiles = 16 * D * 2 + 4 * kTileKeys * D * 2;
    const int merge = 16 * D * 2 + (4 * 16 * D + 2 * 4 * 16) * 4;
    return tiles > merge ? tiles : merge;
}

template <int D>
int launch_prefill(const void* q, void* out, const void* k_pages, const void* v_pages, const int* block_table,
                   int max_blocks, int page_size, int num_pages, const int* q_start, const int* start_pos,
                   const int* tile_req, const int* tile_q0, int n_tiles, int tile_rows, int nq, int nkv, float scale,
                   int window, int* status, cudaStream_t stream) {
    auto kern = attention_prefill_kernel<D>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, prefill_smem<D>());
        if (e != cudaSuccess) return qi::fail("attention_prefill: cannot reserve shared memory: %s", cudaGetErrorString(e));
        configured = true;
    }
    dim3 grid(n_tiles, nq, tile_rows / kTileKeys);
    qi::launch(kern, grid, dim3(kThreads), prefill_smem<D>(), stream,
        (const qi::bf16*)q, (qi::bf16*)out, (const qi::bf16*)k_pages, (const qi::bf16*)v_pages, block_table, max_blocks,
        page_size, num_pages, q_start, start_pos, tile_req, tile_q0, nq, nkv, scale * 1.4426950408889634f, window, status);
    return qi::check_launch("attention_prefill");
}

template <int D>
int launch_decode(const void* q, void* out, const void* k_pages, const void* v_pages, const int* block_table,
                  int max_blocks, int page_size, int num_pages, const int* kv_len, const int* q_start, int batch,
                  int nq, int nkv, float scale, int window, int chunk, int n_splits, float* ws_o, float* ws_ml,
                  int* status, cudaStream_t stream) {
    auto kern = attention_decode_kernel<D>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, decode_smem<D>());
        if (e != cudaSuccess) return qi::fail("attention_decode: cannot reserve shared memory: %s", cudaGetErrorString(e));
        configured = true;
    }
    dim3 grid(n_splits, nkv, batch);
    qi::launch(kern, grid, dim3(kThreads), decode_smem<D>(), stream,
        (const qi::bf16*)q, (const qi::bf16*)k_pages, (const qi::bf16*)v_pages, block_table, max_blocks, page_size,
        num_pages, kv_len, q_start, ws_o, ws_ml, nq, nkv, scale * 1.4426950408889634f, window, chunk, status);
    if (int rc = qi::check_launch("attention_decode")) return rc;
    qi::launch(attention_decode_merge_kernel<D>, dim3(nq, batch), dim3(D >= 128 ? 128 : 64), 0, stream,
        ws_o, ws_ml, q_start, (qi::bf16*)out, nq, n_splits);
    return qi::check_launch("attention_decode_merge");
}

}  // namespace

// 1 if the tensor-core attention kernels take this geometry (else use attention_generic).
extern "C" int qi_attention_mma_supported(int nq, int nkv, int d) {
    return (d == 64 || d == 128) && nkv > 0 && nq % nkv == 0 && nq / nkv <= 16;
}

extern "C" int qi_attention_prefill(const void* q, void* out, const void* k_pages, const void* v_pages,
                                    const int* block_table, int max_blocks, int page_size, int num_pages,
                                    const int* q_start, const int* start_pos, const int* tile_req,
                                    const int* tile_q0, int n_tiles, int tile_rows, int nq, int nkv, int d,
                                    float scale, int window, int* status, cudaStream_t stream) {
    QI_REQUIRE(qi_attention_mma_supported(nq, nkv, d), "attention_prefill: heads %d/%d of size %d are not covered (head size 64 or 128, group <= 16)", nq, nkv, d);
    QI_REQUIRE(page_size > 0 && max_blocks > 0 && num_pages > 0 && window >= 0, "attention_prefill: bad page geometry");
    QI_REQUIRE(n_tiles >= 0 && nq <= 65535, "attention_prefill: grid too large");
    QI_REQUIRE(tile_rows > 0 && tile_rows % kTileKeys == 0 && tile_rows / kTileKeys <= 64,
               "attention_prefill: the tile lists must be cut to a multiple of %d query rows", kTileKeys);
    if (n_tiles == 0) return 0;
    if (d == 64)
        return launch_prefill<64>(q, out, k_pages, v_pages, block_table, max_blocks, page_size, num_pages, q_start,
                                  start_pos, tile_req, tile_q0, n_tiles, tile_rows, nq, nkv, scale, window, status, stream);
    return launch_prefill<128>(q, out, k_pages, v_pages, block_table, max_blocks, page_size, num_pages, q_start,
                               start_pos, tile_req, tile_q0, n_tiles, tile_rows, nq, nkv, scale, window, status, stream);
}

// Workspace floats: ws_o = batch * nq * n_splits * d, ws_ml = batch * nq * n_splits * 2.
extern "C" int qi_attention_decode(const void* q, void* out, const void* k_pages, const void* v_pages,
                                   const int* block_table, int max_blocks, int page_size, int num_pages,
                                   const int* kv_len, const int* q_start, int batch, int nq, int nkv, int d,
                                   float scale, int window, int chunk, int n_splits, float* ws_o, float* ws_ml,
                                   int* status, cudaStream_t stream) {
    QI_REQUIRE(qi_attention_mma_supported(nq, nkv, d), "attention_decode: heads %d/%d of size %d are not covered (head size 64 or 128, group <= 16)", nq, nkv, d);
    QI_REQUIRE(page_size > 0 && max_blocks > 0 && num_pages > 0 && window >= 0, "attention_decode: bad page geometry");
    QI_REQUIRE(chunk > 0 && chunk % kTileKeys == 0, "attention_decode: the key range per CTA (%d) must be a positive multiple of %d", chunk, kTileKeys);
    QI_REQUIRE(n_splits > 0 && n_splits <= 65535 && nkv <= 65535 && batch <= 65535, "attention_decode: grid too large");
    QI_REQUIRE(ws_o && ws_ml, "attention_decode: workspace missing");
    if (batch == 0) return 0;
    if (d == 64)
        return launch_decode<64>(q, out, k_pages, v_pages, block_table, max_blocks, page_size, num_pages, kv_len,
                                 q_start, batch, nq, nkv, scale, window, chunk, n_splits, ws_o, ws_ml, status, stream);
    return launch_decode<128>(q, out, k_pages, v_pages, block_table, max_blocks, page_size, num_pages, kv_len,
                              q_start, batch, nq, nkv, scale, window, chunk, n_splits, ws_o, ws_ml, status, stream);
}
