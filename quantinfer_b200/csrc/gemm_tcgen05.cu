// bfloat16 matrix product on the 5th-generation tensor cores:
//     y[M, N] = x[M, K] . w[N, K]^T        (32-bit accumulation)
// Both operands are read along K ("K-major"), which is the checkpoint's
// [out, in] layout for w, so nothing is transposed at load.
//
// The output is cut into 128 x BN tiles of  D = A . B^T  where A and B are the two
// row-major operands; a CTA computes its share of the tiles one after the other. For many tokens A = x and B = w. For few tokens (decode)
// the operands are swapped: A = w, so the 128 rows of the MMA ride the weight's
// output dimension and the small token count rides the MMA's N (16..256); the
// epilogue then stores the tile transposed. A skinny product is bound by the
// weight stream from HBM, so the K dimension can be split over blockIdx.z to
// put enough CTAs in flight; partial sums go to a 32-bit workspace
// [splits, M, N] and are added in split order by a second kernel (or by the
// consumer: add_rmsnorm takes the partials directly).
//
// Roles inside a CTA (192 threads):
//   warp 0     one lane issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle)
//              into a ring of STAGES shared-memory buffers, each guarded by a
//              "full" mbarrier (expect-tx) and an "empty" mbarrier
//   warp 1     allocates tensor memory; one lane issues tcgen05.mma (kind::f16,
//              M = 128, N = BN, K = 16 per instruction, 4 per 64-wide k block) and
//              tcgen05.commit, which frees the stage and finally signals the
//              accumulator
//   warps 2-5  read the accumulator from tensor memory (tcgen05.ld, 32 lanes x
//              32 columns per warp) and store it
// No load uses cluster multicast. Every mbarrier wait is bounded: when a bound
// runs out the thread sets kStatusWaitTimeout in the status word and an abort
// flag in shared memory, all roles leave their loops, the producer waits (with
// a bound) for the copies it still has in flight, tensor memory is freed and
// the kernel returns.
//
// K must be a multiple of 8 (TMA wants row strides of whole 16 bytes); rows of
// A, B and K beyond the tensors are zero-filled by TMA and masked at the store.
#include "common.cuh"

#include <cuda.h>

namespace {

constexpr int BM = 128;       // rows of A per tile = MMA M
constexpr int BK = 64;        // bf16 elements per k block = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;
constexpr uint32_t kSpinLimit = 1u << 21;   // polls of try_wait before giving up (each poll may itself wait up to a few microseconds)

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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

// Waits for the phase with the given parity to complete; false when the bound ran out
// or another role already gave up.
// A timeout that any CTA recorded in the global status word ends the waits of all others early.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          const volatile int* status) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
        if ((i & 65535u) == 65535u && status && (*status & qi::kStatusWaitTimeout)) return false;
    }
    return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}

// The same with a hint for the L2: a weight tile of a product of few tokens is read once in a step,
// so it is the first to go when the L2 needs room, and what the step's small kernels pass on
// (partial sums, the residual stream, the attention's operands) stays there meanwhile.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "l"(policy) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0) : "memory");
}

// Arrives on the mbarrier when every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t addr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(addr));
}
__device__ __forceinline__ void tmem_ld16(uint32_t addr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(addr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile stored as rows of 128 bytes
// with the 128-byte swizzle (what TMA writes with CU_TENSOR_MAP_SWIZZLE_128B):
// start address >> 4 in bits 0-13, leading byte offset (unused for swizzled
// K-major, 1) in 16-29, stride byte offset = 8 rows x 128 B = 1024 >> 4 in
// 32-45, descriptor version 1 in 46-47, layout type 2 (128-byte swizzle) in 61-63.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor of kind::f16: D format F32 (1) in bits 4-5, A and B
// format BF16 (1) in 7-9 and 10-12, both K-major (0) in 15 and 16, N >> 3 in
// 17-22, M >> 4 in 24-28.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

template <typename TOut> __device__ __forceinline__ void store1(TOut* p, float v);
template <> __device__ __forceinline__ void store1<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store1<qi::bf16>(qi::bf16* p, float v) { *p = __float2bfloat16_rn(v); }

template <int BN, int STAGES>
struct Smem {
    static constexpr int kABytes = BM * BK * 2;
    static constexpr int kBBytes = BN * BK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kBarrierBytes = 8 * (2 * STAGES + 4) + 16;
    static constexpr int kTotal = STAGES * kStageBytes + kBarrierBytes + 1024;  // + alignment slack
};


__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.0f + expf(-g)) * u; }

// What the epilogue of the fused q/k/v projection needs (EPI = 2): the product's columns are
// heads of 128 (nq query heads, then nkv key heads, then nkv value heads); query and key heads
// get their RMSNorm (gain null: none) and the half-split rotation of the token's position (cos_t
// null: none), values pass through; queries go to q_out [tokens, nq * 128], keys and values to
// the token's place in the paged cache (k_pages null: nothing is written).
struct RopeEpilogue {
    qi::bf16* q_out;
    const float* q_gain;
    const float* k_gain;
    const float* cos_t;      // [positions, 64]
    const float* sin_t;
    const int* positions;    // [tokens]
    const int* token_req;    // [tokens]: row of the block table
    const int* block_table;  // [requests, max_blocks]
    qi::bf16* k_pages;       // [pages, nkv, page_size, 128]
    qi::bf16* v_pages;
    float eps;
    int max_blocks, page_size, num_pages, nq, nkv;
    int table_positions;     // rows of cos_t / sin_t
};

__device__ __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

// One accumulator tile [128 tokens, BN columns] of the q/k/v projection: this thread owns token
// `row` (TMEM lane) and walks the tile's heads. The norm's sum runs over the head's 128 columns
// in column order; everything is 32-bit until the store.
template <int BN>
__device__ __forceinline__ void rope_epilogue(uint32_t tmem_tile, int col_base, int row, bool row_ok, int n_cols,
                                              const RopeEpilogue& e, int* __restrict__ status) {
    constexpr int D = 128, HALF = 64;
    int pos = row_ok ? e.positions[row] : 0;
    if (pos < 0) {           // no such position: nothing of this token is written
        if (status) atomicOr(status, qi::kStatusBadRange);
        pos = 0;
        row_ok = false;
    }
    int table_row = pos;     // a position beyond the rotation table is flagged and takes the table's last row
    if (e.cos_t && pos >= e.table_positions) {
        if (status) atomicOr(status, qi::kStatusBadRange);
        table_row = e.table_positions - 1;
    }
    int page = -2;           // -2: not looked up yet
#pragma unroll 1
    for (int hh = 0; hh < BN / D; ++hh) {
        const int col0 = col_base + hh * D;
        if (col0 >= n_cols) break;                       // the same for every thread of the CTA
        const int head = col0 / D;
        const bool is_q = head < e.nq, is_k = !is_q && head < e.nq + e.nkv;
        const uint32_t t0 = tmem_tile + (uint32_t)(hh * D);
        const float* gain = is_q ? e.q_gain : is_k ? e.k_gain : nullptr;
        uint32_t lo[32], hi[32];
        float inv = 1.f;
        if (gain) {
            float ss = 0.f;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                tmem_ld32(t0 + 32u * c, lo);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) ss = fmaf(__uint_as_float(lo[i]), __uint_as_float(lo[i]), ss);
            }
            inv = 1.0f / sqrtf(ss / (float)D + e.eps);
        }
        qi::bf16* dst = nullptr;
        if (row_ok) {
            if (is_q) {
                dst = e.q_out + ((size_t)row * e.nq + head) * D;
            } else if (e.k_pages) {
                if (page == -2) {
                    page = e.block_table[(size_t)e.token_req[row] * e.max_blocks + pos / e.page_size];
                    if (page < 0 || page >= e.num_pages) {
                        if (status) atomicOr(status, qi::kStatusBadPage);
                        page = -1;
                    }
                }
                if (page >= 0) {
                    const int hk = is_k ? head - e.nq : head - e.nq - e.nkv;
                    dst = (is_k ? e.k_pages : e.v_pages) + (((size_t)page * e.nkv + hk) * e.page_size + (pos % e.page_size)) * (size_t)D;
                }
            }
        }
        const bool rotate = (is_q || is_k) && e.cos_t != nullptr;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
            tmem_ld32(t0 + 32u * c, lo);
            tmem_ld32(t0 + (uint32_t)HALF + 32u * c, hi);
            tmem_ld_wait();
            if (!dst) continue;
            float a[32], b[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                a[i] = __uint_as_float(lo[i]);
                b[i] = __uint_as_float(hi[i]);
            }
            if (gain) {
                const float4* ga = reinterpret_cast<const float4*>(gain + 32 * c);
                const float4* gb = reinterpret_cast<const float4*>(gain + HALF + 32 * c);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float4 x = ga[i], y = gb[i];
                    a[4 * i] = a[4 * i] * inv * x.x; a[4 * i + 1] = a[4 * i + 1] * inv * x.y;
                    a[4 * i + 2] = a[4 * i + 2] * inv * x.z; a[4 * i + 3] = a[4 * i + 3] * inv * x.w;
                    b[4 * i] = b[4 * i] * inv * y.x; b[4 * i + 1] = b[4 * i + 1] * inv * y.y;
                    b[4 * i + 2] = b[4 * i + 2] * inv * y.z; b[4 * i + 3] = b[4 * i + 3] * inv * y.w;
                }
            }
            if (rotate) {
                const float4* cs = reinterpret_cast<const float4*>(e.cos_t + (size_t)table_row * HALF + 32 * c);
                const float4* sn = reinterpret_cast<const float4*>(e.sin_t + (size_t)table_row * HALF + 32 * c);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float4 cc = cs[i], ss = sn[i];
                    const float cv[4] = {cc.x, cc.y, cc.z, cc.w}, sv[4] = {ss.x, ss.y, ss.z, ss.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float x = a[4 * i + j], y = b[4 * i + j];
                        a[4 * i + j] = x * cv[j] - y * sv[j];
                        b[4 * i + j] = x * sv[j] + y * cv[j];
                    }
                }
            }
            uint4* d_lo = reinterpret_cast<uint4*>(dst + 32 * c);
            uint4* d_hi = reinterpret_cast<uint4*>(dst + HALF + 32 * c);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                d_lo[i] = make_uint4(pack2(a[8 * i], a[8 * i + 1]), pack2(a[8 * i + 2], a[8 * i + 3]),
                                     pack2(a[8 * i + 4], a[8 * i + 5]), pack2(a[8 * i + 6], a[8 * i + 7]));
                d_hi[i] = make_uint4(pack2(b[8 * i], b[8 * i + 1]), pack2(b[8 * i + 2], b[8 * i + 3]),
                                     pack2(b[8 * i + 4], b[8 * i + 5]), pack2(b[8 * i + 6], b[8 * i + 7]));
            }
        }
    }
}

// EPI = 0: store the product. EPI = 1: the product's columns come in pairs (gate, up) and
// the kernel stores silu(gate) * up, half as wide (the feed-forward's activation fused in).
// EPI = 2 (operands not swapped): the product is the q/k/v projection and `rope` says where
// its heads go (q/k norm, rotation and the cache write fused in; `out` is not used).
//
// The kernel is persistent: CTA c takes tiles c, c + gridDim.x, ... of the linear tile
// list (A tiles fastest, then B tiles, then K splits, so CTAs that run together share a
// B tile in L2). The accumulator in tensor memory is double-buffered: while the
// epilogue warps drain one buffer, the MMA warp already fills the other with the next
// tile, and the TMA ring runs on across tile borders.
QI_TL_DEFINE(qi_timeline_gemm)

template <int BN, int STAGES, bool SWAP, typename TOut, int EPI>
__global__ void __launch_bounds__(kThreads)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    TOut* __restrict__ out, int rows_a, int rows_b, int K, long long ld_out,
                    int kb_per_split, int n_splits, long long split_stride, int* __restrict__ status,
                    const RopeEpilogue rope) {
    extern __shared__ uint8_t smem_raw[];
    using L = Smem<BN, STAGES>;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
    // barriers: full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]
    const uint32_t bars = base + STAGES * L::kStageBytes;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(aligned + STAGES * L::kStageBytes + 8 * (2 * STAGES + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto acc_full_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
    auto acc_empty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };

    QI_TL_BEGIN();
    QI_TL_SHARED();
    qi::pdl_launch_dependents();   // the next kernel may be scheduled while this one runs
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_a = (rows_a + BM - 1) / BM, tiles_b = (rows_b + BN - 1) / BN;
    const int total_tiles = tiles_a * tiles_b * n_splits;
    const int kb_total = (K + BK - 1) / BK;
    constexpr uint32_t kAccCols = BN < 32 ? 32 : BN;        // columns of one accumulator
    constexpr uint32_t kTmemCols = 2 * kAccCols;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(acc_full_bar(a), 1);
            mbar_init(acc_empty_bar(a), 4);     // one arrival per epilogue warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Set-up is done. Only the activations (and the output buffer) depend on the kernel before
    // this one: the producer fetches the first weight tiles before it waits for that kernel, the
    // epilogue warps wait before they write, and the MMA warp follows the producer's barriers.

    auto give_up = [&]() {
        if (!*abort_flag) {
            *abort_flag = 1;
            if (status) atomicOr(status, qi::kStatusWaitTimeout);
        }
    };

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            // The weights are the operand with the many rows: A when the operands are swapped
            // (few tokens), else B. They are never written on the device, so the first stages'
            // weight tiles of this CTA's first tile are requested before the wait.
            const uint64_t stream_once = l2_evict_first_policy();
            uint32_t early = 0;
            if (blockIdx.x < total_tiles) {
                const int tile = blockIdx.x;
                const int tile_a = tile % tiles_a, tile_b = (tile / tiles_a) % tiles_b, split = tile / (tiles_a * tiles_b);
                const int kb_begin = split * kb_per_split;
                const int n_kb = max(min(kb_total, kb_begin + kb_per_split) - kb_begin, 0);
                early = (uint32_t)min(n_kb, STAGES);
                for (uint32_t i = 0; i < early; ++i) {
                    mbar_expect_tx(full_bar(i), L::kStageBytes);
                    const uint32_t a_dst = base + i * L::kStageBytes;
                    const int k0 = (kb_begin + (int)i) * BK;
                    if (SWAP) tma_load_2d_hint(a_dst, &map_a, full_bar(i), k0, tile_a * BM, stream_once);
                    else tma_load_2d(a_dst + L::kABytes, &map_b, full_bar(i), k0, tile_b * BN);
                }
            }
            qi::pdl_wait();
            uint32_t it = 0;          // k blocks issued so far, over all tiles
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int tile_a = tile % tiles_a, tile_b = (tile / tiles_a) % tiles_b, split = tile / (tiles_a * tiles_b);
                const int kb_begin = split * kb_per_split;
                const int n_kb = max(min(kb_total, kb_begin + kb_per_split) - kb_begin, 0);
                for (int i = 0; i < n_kb; ++i, ++it) {
                    const int s = it % STAGES;
                    const uint32_t a_dst = base + s * L::kStageBytes;
                    const int k0 = (kb_begin + i) * BK;
                    if (it < early) {
                        // the weight tile of this stage is on its way already: add the activations
                        if (SWAP) tma_load_2d(a_dst + L::kABytes, &map_b, full_bar(s), k0, tile_b * BN);
                        else tma_load_2d(a_dst, &map_a, full_bar(s), k0, tile_a * BM);
                        continue;
                    }
                    if (!mbar_wait(empty_bar(s), ((it / STAGES) & 1u) ^ 1u, abort_flag, status)) {
                        give_up();
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(full_bar(s), L::kStageBytes);
                    if (SWAP) tma_load_2d_hint(a_dst, &map_a, full_bar(s), k0, tile_a * BM, stream_once);
                    else tma_load_2d(a_dst, &map_a, full_bar(s), k0, tile_a * BM);
                    tma_load_2d(a_dst + L::kABytes, &map_b, full_bar(s), k0, tile_b * BN);
                }
            }
            if (*abort_flag) {
                // Copies still in flight write into this CTA's shared memory: wait (bounded) for the
                // stages armed last before the CTA may exit.
                const uint32_t first = it > (uint32_t)STAGES ? it - STAGES : 0u;
                for (uint32_t i = first; i < it; ++i)
                    for (uint32_t t = 0; t < (1u << 20); ++t)
                        if (mbar_try_wait(full_bar(i % STAGES), (i / STAGES) & 1u)) break;
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            qi::pdl_wait();   // its operands come after the producer's wait: the polls below start counting from there
            QI_TL_SHARED_WAKE();
            constexpr uint32_t idesc = make_idesc(BM, BN);
            uint32_t it = 0;
            int j = 0;                // tiles this CTA has started
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++j) {
                const int split = tile / (tiles_a * tiles_b);
                const int kb_begin = split * kb_per_split;
                const int n_kb = max(min(kb_total, kb_begin + kb_per_split) - kb_begin, 0);
                const int acc = j & 1;
                // the epilogue must have drained this accumulator (first use of each passes at once)
                if (!mbar_wait(acc_empty_bar(acc), (((uint32_t)j >> 1) & 1u) ^ 1u, abort_flag, status)) {
                    give_up();
                    break;
                }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)acc * kAccCols;
                for (int i = 0; i < n_kb; ++i, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(full_bar(s), (it / STAGES) & 1u, abort_flag, status)) {
                        give_up();
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    if (it == 0) QI_TL_SHARED_DATA();
                    const uint32_t a_addr = base + s * L::kStageBytes;
                    const uint64_t adesc = make_smem_desc(a_addr);
                    const uint64_t bdesc = make_smem_desc(a_addr + L::kABytes);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // 16 bf16 = 32 bytes further along the swizzled row: +2 in units of 16 bytes
                        umma_bf16(tmem_d, adesc + 2u * k, bdesc + 2u * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(empty_bar(s));   // the stage is free once these MMAs have read it
                }
                if (ok) umma_commit(acc_full_bar(acc));  // the accumulator is complete
            }
        }
    } else {
        // ---------------- epilogue (warps 2..5) ----------------
        const int quarter = warp & 3;   // the 32 TMEM lanes this warp may read
        qi::pdl_wait();                 // the output buffer may still be read by the kernel before
        int j = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++j) {
            const int tile_a = tile % tiles_a, tile_b = (tile / tiles_a) % tiles_b, split = tile / (tiles_a * tiles_b);
            const int kb_begin = split * kb_per_split;
            const int n_kb = max(min(kb_total, kb_begin + kb_per_split) - kb_begin, 0);
            const int acc = j & 1;
            if (!mbar_wait(acc_full_bar(acc), ((uint32_t)j >> 1) & 1u, abort_flag, status)) {
                if (lane == 0) give_up();
                break;
            }
            tc_fence_after();
            const int a_row = tile_a * BM + quarter * 32 + lane;
            if constexpr (EPI == 2 && BN % 128 == 0) {
                rope_epilogue<BN>(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)acc * kAccCols, tile_b * BN, a_row,
                                  a_row < rows_a, rows_b, rope, status);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty_bar(acc));
                continue;
            }
            TOut* obase = out + (size_t)split * split_stride;
            constexpr int kChunk = BN >= 32 ? 32 : 16;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += kChunk) {
                uint32_t r[32];
                if (n_kb > 0) {
                    const uint32_t addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)acc * kAccCols + (uint32_t)c0;
                    if (kChunk == 32) tmem_ld32(addr, r); else tmem_ld16(addr, r);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int q = 0; q < 32; ++q) r[q] = 0u;   // an empty K range contributes zeros
                }
                if (c0 + kChunk >= BN) {
                    // everything of this accumulator is in registers: hand it back to the MMA warp
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty_bar(acc));
                }
                const int b0 = tile_b * BN + c0;
                if (SWAP && EPI == 1) {
                    // rows of A come in pairs (gate, up): even lanes hold gate, their neighbours up
#pragma unroll
                    for (int q = 0; q < kChunk; ++q) {
                        const float mine = __uint_as_float(r[q]);
                        const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
                        if ((lane & 1) == 0 && a_row + 1 < rows_a && b0 + q < rows_b)
                            store1<TOut>(obase + (size_t)(b0 + q) * ld_out + (a_row >> 1), silu_mul(mine, other));
                    }
                } else if (SWAP) {
                    // out[b, a]: for a fixed column the warp's lanes write consecutive addresses
                    if (a_row < rows_a) {
#pragma unroll
                        for (int q = 0; q < kChunk; ++q)
                            if (b0 + q < rows_b) store1<TOut>(obase + (size_t)(b0 + q) * ld_out + a_row, __uint_as_float(r[q]));
                    }
                } else if (EPI == 1) {
                    if (a_row < rows_a) {
                        TOut* orow = obase + (size_t)a_row * ld_out + (b0 >> 1);
                        const bool full = b0 + kChunk <= rows_b;
                        const bool aligned16 = ((reinterpret_cast<uintptr_t>(orow) & 15u) == 0);
                        if (full && aligned16 && sizeof(TOut) == 2) {
#pragma unroll
                            for (int q0 = 0; q0 < kChunk; q0 += 16) {
                                uint4 v;
                                uint32_t* vw = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
                                for (int q = 0; q < 4; ++q) {
                                    __nv_bfloat162 pr = __floats2bfloat162_rn(
                                        silu_mul(__uint_as_float(r[q0 + 4 * q]), __uint_as_float(r[q0 + 4 * q + 1])),
                                        silu_mul(__uint_as_float(r[q0 + 4 * q + 2]), __uint_as_float(r[q0 + 4 * q + 3])));
                                    vw[q] = *reinterpret_cast<uint32_t*>(&pr);
                                }
                                *reinterpret_cast<uint4*>(reinterpret_cast<qi::bf16*>(orow) + (q0 >> 1)) = v;
                            }
                        } else {
#pragma unroll
                            for (int q = 0; q < kChunk; q += 2)
                                if (b0 + q + 1 < rows_b)
                                    store1<TOut>(orow + (q >> 1), silu_mul(__uint_as_float(r[q]), __uint_as_float(r[q + 1])));
                        }
                    }
                } else {
                    if (a_row < rows_a) {
                        TOut* orow = obase + (size_t)a_row * ld_out + b0;
                        const bool full = b0 + kChunk <= rows_b;
                        const bool aligned16 = ((reinterpret_cast<uintptr_t>(orow) & 15u) == 0);
                        if (full && aligned16 && sizeof(TOut) == 2) {
#pragma unroll
                            for (int q = 0; q < kChunk; q += 8) {
                                uint4 v;
                                __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(r[q + 0]), __uint_as_float(r[q + 1]));
                                __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(r[q + 2]), __uint_as_float(r[q + 3]));
                                __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(r[q + 4]), __uint_as_float(r[q + 5]));
                                __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(r[q + 6]), __uint_as_float(r[q + 7]));
                                v.x = *reinterpret_cast<uint32_t*>(&p0);
                                v.y = *reinterpret_cast<uint32_t*>(&p1);
                                v.z = *reinterpret_cast<uint32_t*>(&p2);
                                v.w = *reinterpret_cast<uint32_t*>(&p3);
                                *reinterpret_cast<uint4*>(reinterpret_cast<qi::bf16*>(orow) + q) = v;
                            }
                        } else if (full && aligned16 && sizeof(TOut) == 4) {
#pragma unroll
                            for (int q = 0; q < kChunk; q += 4) {
                                uint4 v = make_uint4(r[q], r[q + 1], r[q + 2], r[q + 3]);
                                *reinterpret_cast<uint4*>(reinterpret_cast<float*>(orow) + q) = v;
                            }
                        } else {
#pragma unroll
                            for (int q = 0; q < kChunk; ++q)
                                if (b0 + q < rows_b) store1<TOut>(orow + q, __uint_as_float(r[q]));
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    QI_TL_END_SHARED(20 + EPI + (SWAP ? 0 : 5));
    if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

// Adds split-K partial sums in split order: out[i] = sum_s partial[s, i].
// ------------------------------------------------------------------ two CTAs on one tile
//
// For many tokens the single-CTA kernel is bound by what its 128 x 256 tiles draw from L2 and
// shared memory (48 KB per 64-wide k block for 512 cycles of tensor-core work) rather than
// by the tensor core. Here a pair of CTAs on neighbouring SMs (a cluster of two) computes one
// 256 x 256 tile with tcgen05.mma.cta_group::2: each CTA loads 128 rows of A and 128 rows of
// B (32 KB per k block, six stages instead of four), the tensor cores of both SMs read B
// from both CTAs' shared memory, and each CTA's tensor memory receives its 128 rows of the
// result. Only the even CTA of the pair issues MMAs. Barriers:
//   full[s]   in the even CTA: its producer announces the bytes of both CTAs' copies, and
//             both CTAs' TMA copies report there (cta_group::2 form of the copy)
//   empty[s]  in each CTA: the MMAs' commit arrives on both (multicast commit, not a load)
//   acc_full  in each CTA: the same at the end of a tile
//   acc_empty in the even CTA: the four epilogue warps of both CTAs arrive there
// No load uses cluster multicast. All waits are bounded as in the kernel above; a CTA that
// gave up is seen by its partner through the status word. Both CTAs pass a cluster barrier
// before they leave, so that neither frees shared or tensor memory its partner still uses.

constexpr int kPairStages = 6;
constexpr int kPairHalfBytes = BM * BK * 2;              // 128 rows x 64 bf16 = 16 KB
constexpr int kPairStageBytes = 2 * kPairHalfBytes;      // this CTA's rows of A, then its rows of B
constexpr int kPairSmem = kPairStages * kPairStageBytes + 8 * (2 * kPairStages + 4) + 16 + 1024;

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The copy of a CTA of a pair; its bytes are reported to the barrier at the same address in the even CTA.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar & 0xFEFFFFFFu), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8, %9, %10, %11, %12}, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0), "r"(0), "r"(0),
          "r"(0), "r"(0) : "memory");
}
// Arrives on the barrier at this address in both CTAs of the pair when every MMA issued so far has completed.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}
// Arrives on the barrier at this address in the even CTA of the pair.
__device__ __forceinline__ void mbar_arrive_leader(uint32_t bar) {
    asm volatile(
        "{\n\t.reg .b32 ra;\n\t"
        "mapa.shared::cluster.u32 ra, %0, 0;\n\t"
        "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n\t}"
        ::"r"(bar) : "memory");
}

// out[M, N] = A[M, K] . B[N, K]^T in tiles of 256 x 256, one per pair of CTAs at a time; A are the
// tokens, B the weights. EPI as in the kernel above (0: the product, 1: silu(gate) * up of column
// pairs, 2: the q/k/v projection's heads through `rope`).
template <typename TOut, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         TOut* __restrict__ out, int rows_a, int rows_b, int K, long long ld_out, int kb_per_split,
                         int n_splits, long long split_stride, int* __restrict__ status, const RopeEpilogue rope) {
    extern __shared__ uint8_t smem_raw[];
    constexpr int STAGES = kPairStages;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + STAGES * kPairStageBytes;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(aligned + STAGES * kPairStageBytes + 8 * (2 * STAGES + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto acc_full_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
    auto acc_empty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };

    QI_TL_BEGIN();
    qi::pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    constexpr int TM = 2 * BM, TN = 256;
    const int tiles_m = (rows_a + TM - 1) / TM, tiles_n = (rows_b + TN - 1) / TN;
    const int total_tiles = tiles_m * tiles_n * n_splits;     // K splits slowest: split s writes out + s * split_stride
    const int kb_total = (K + BK - 1) / BK;
    auto kb_range = [&](int tile, int& kb_begin) {
        kb_begin = (tile / (tiles_m * tiles_n)) * kb_per_split;
        return max(min(kb_total, kb_begin + kb_per_split) - kb_begin, 0);
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(acc_full_bar(a), 1);
            mbar_init(acc_empty_bar(a), 8);     // four epilogue warps in each CTA of the pair
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(tmem_slot), 512);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    cluster_sync_all();       // both CTAs' barriers and tensor memory exist before anything crosses over
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    auto give_up = [&]() {
        if (!*abort_flag) {
            *abort_flag = 1;
            if (status) atomicOr(status, qi::kStatusWaitTimeout);
        }
    };

    if (warp == 0) {
        // ---------------- TMA producer (in both CTAs) ----------------
        if (lane == 0) {
            // the first stages' weight rows are requested before the wait for the kernel before this one
            uint32_t early = 0;
            if (pair < total_tiles) {
                const int tile_n = (pair / tiles_m) % tiles_n;
                int kb_begin;
                const int n_kb = kb_range(pair, kb_begin);
                early = (uint32_t)min(n_kb, STAGES);
                for (uint32_t i = 0; i < early; ++i) {
                    if (rank == 0) mbar_expect_tx(full_bar(i), 2 * kPairStageBytes);
                    tma_load_2d_pair(base + i * kPairStageBytes + kPairHalfBytes, &map_b, full_bar(i), (kb_begin + (int)i) * BK,
                                     tile_n * TN + (int)rank * BM);
                }
            }
            qi::pdl_wait();
            QI_TL_WAKE();
            uint32_t it = 0;
            bool ok = true;
            for (int tile = pair; tile < total_tiles && ok; tile += n_pairs) {
                const int tile_m = tile % tiles_m, tile_n = (tile / tiles_m) % tiles_n;
                int kb_begin;
                const int n_kb = kb_range(tile, kb_begin);
                for (int i = 0; i < n_kb; ++i, ++it) {
                    const int s = it % STAGES;
                    const uint32_t dst = base + s * kPairStageBytes;
                    const int k0 = (kb_begin + i) * BK;
                    if (it < early) {
                        tma_load_2d_pair(dst, &map_a, full_bar(s), k0, tile_m * TM + (int)rank * BM);
                        continue;
                    }
                    if (!mbar_wait(empty_bar(s), ((it / STAGES) & 1u) ^ 1u, abort_flag, status)) {
                        give_up();
                        ok = false;
                        break;
                    }
                    if (rank == 0) mbar_expect_tx(full_bar(s), 2 * kPairStageBytes);
                    tma_load_2d_pair(dst, &map_a, full_bar(s), k0, tile_m * TM + (int)rank * BM);
                    tma_load_2d_pair(dst + kPairHalfBytes, &map_b, full_bar(s), k0, tile_n * TN + (int)rank * BM);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (the even CTA only) ----------------
        if (lane == 0 && rank == 0) {
            qi::pdl_wait();
            constexpr uint32_t idesc = make_idesc(TM, TN);
            uint32_t it = 0;
            int j = 0;
            bool ok = true;
            for (int tile = pair; tile < total_tiles && ok; tile += n_pairs, ++j) {
                const int acc = j & 1;
                int kb_begin;
                const int n_kb = kb_range(tile, kb_begin);
                if (!mbar_wait(acc_empty_bar(acc), (((uint32_t)j >> 1) & 1u) ^ 1u, abort_flag, status)) {
                    give_up();
                    break;
                }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)acc * TN;
                for (int i = 0; i < n_kb; ++i, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(full_bar(s), (it / STAGES) & 1u, abort_flag, status)) {
                        give_up();
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = base + s * kPairStageBytes;
                    const uint64_t adesc = make_smem_desc(a_addr);
                    const uint64_t bdesc = make_smem_desc(a_addr + kPairHalfBytes);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_bf16_pair(tmem_d, adesc + 2u * k, bdesc + 2u * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                    umma_commit_pair(empty_bar(s));
                }
                if (ok) umma_commit_pair(acc_full_bar(acc));
            }
        }
    } else {
        // ---------------- epilogue (warps 2..5 of both CTAs): this CTA's 128 rows of the tile ----------------
        const int quarter = warp & 3;
        qi::pdl_wait();
        int j = 0;
        for (int tile = pair; tile < total_tiles; tile += n_pairs, ++j) {
            const int tile_m = tile % tiles_m, tile_n = (tile / tiles_m) % tiles_n;
            TOut* obase = out + (size_t)(tile / (tiles_m * tiles_n)) * split_stride;
            const int acc = j & 1;
            if (!mbar_wait(acc_full_bar(acc), ((uint32_t)j >> 1) & 1u, abort_flag, status)) {
                if (lane == 0) give_up();
                break;
            }
            tc_fence_after();
            const int row = tile_m * TM + (int)rank * BM + quarter * 32 + lane;
            const uint32_t tmem_tile = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)acc * TN;
            if constexpr (EPI == 2) {
                rope_epilogue<TN>(tmem_tile, tile_n * TN, row, row < rows_a, rows_b, rope, status);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_leader(acc_empty_bar(acc));
                continue;
            }
#pragma unroll 1
            for (int c0 = 0; c0 < TN; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(tmem_tile + (uint32_t)c0, r);
                tmem_ld_wait();
                if (c0 + 32 >= TN) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_leader(acc_empty_bar(acc));
                }
                const int b0 = tile_n * TN + c0;
                if (row >= rows_a) continue;
                const bool full = b0 + 32 <= rows_b;
                if (EPI == 1) {
                    // columns come in pairs (gate, up): half as many outputs
                    TOut* orow = obase + (size_t)row * ld_out + (b0 >> 1);
                    if (full && ((reinterpret_cast<uintptr_t>(orow) & 15u) == 0) && sizeof(TOut) == 2) {
#pragma unroll
                        for (int q0 = 0; q0 < 32; q0 += 16) {
                            uint4 v;
                            v.x = pack2(silu_mul(__uint_as_float(r[q0 + 0]), __uint_as_float(r[q0 + 1])),
                                        silu_mul(__uint_as_float(r[q0 + 2]), __uint_as_float(r[q0 + 3])));
                            v.y = pack2(silu_mul(__uint_as_float(r[q0 + 4]), __uint_as_float(r[q0 + 5])),
                                        silu_mul(__uint_as_float(r[q0 + 6]), __uint_as_float(r[q0 + 7])));
                            v.z = pack2(silu_mul(__uint_as_float(r[q0 + 8]), __uint_as_float(r[q0 + 9])),
                                        silu_mul(__uint_as_float(r[q0 + 10]), __uint_as_float(r[q0 + 11])));
                            v.w = pack2(silu_mul(__uint_as_float(r[q0 + 12]), __uint_as_float(r[q0 + 13])),
                                        silu_mul(__uint_as_float(r[q0 + 14]), __uint_as_float(r[q0 + 15])));
                            *reinterpret_cast<uint4*>(reinterpret_cast<qi::bf16*>(orow) + (q0 >> 1)) = v;
                        }
                    } else {
#pragma unroll
                        for (int q = 0; q < 32; q += 2)
                            if (b0 + q + 1 < rows_b)
                                store1<TOut>(orow + (q >> 1), silu_mul(__uint_as_float(r[q]), __uint_as_float(r[q + 1])));
                    }
                } else {
                    TOut* orow = obase + (size_t)row * ld_out + b0;
                    if (full && ((reinterpret_cast<uintptr_t>(orow) & 15u) == 0) && sizeof(TOut) == 2) {
#pragma unroll
                        for (int q = 0; q < 32; q += 8) {
                            uint4 v;
                            v.x = pack2(__uint_as_float(r[q + 0]), __uint_as_float(r[q + 1]));
                            v.y = pack2(__uint_as_float(r[q + 2]), __uint_as_float(r[q + 3]));
                            v.z = pack2(__uint_as_float(r[q + 4]), __uint_as_float(r[q + 5]));
                            v.w = pack2(__uint_as_float(r[q + 6]), __uint_as_float(r[q + 7]));
                            *reinterpret_cast<uint4*>(reinterpret_cast<qi::bf16*>(orow) + q) = v;
                        }
                    } else if (full && ((reinterpret_cast<uintptr_t>(orow) & 15u) == 0) && sizeof(TOut) == 4) {
#pragma unroll
                        for (int q = 0; q < 32; q += 4)
                            *reinterpret_cast<uint4*>(reinterpret_cast<float*>(orow) + q) = make_uint4(r[q], r[q + 1], r[q + 2], r[q + 3]);
                    } else {
#pragma unroll
                        for (int q = 0; q < 32; ++q)
                            if (b0 + q < rows_b) store1<TOut>(orow + q, __uint_as_float(r[q]));
                    }
                }
            }
        }
    }
    tc_fence_before();
    cluster_sync_all();       // neither CTA goes before its partner is done with what it holds
    QI_TL_END(25 + EPI);
    if (warp == 1) tmem_dealloc_pair(tmem_base, 512);
}

template <typename TOut>
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, TOut* __restrict__ out, size_t n, int splits) {
    qi::pdl_enter();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float s = 0.f;
#pragma unroll 4
        for (int k = 0; k < splits; ++k) s += partial[(size_t)k * n + i];
        store1<TOut>(out + i, s);
    }
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

// Map of a row-major bf16 matrix [rows, K] with boxes of [box_rows, 64] and the 128-byte swizzle.
int make_map(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return qi::fail("gemm_bf16: cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return qi::fail("gemm_bf16: cuTensorMapEncodeTiled failed with code %d (rows=%d K=%d box=%d)", (int)r, rows, K, box_rows);
    return 0;
}

int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

template <int BN, int STAGES, bool SWAP, typename TOut, int EPI>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, TOut* out, int rows_a, int rows_b, int K, long long ld,
           int splits, int kb_per_split, long long split_stride, int* status, cudaStream_t stream,
           const RopeEpilogue& rope = RopeEpilogue{}) {
    auto kern = gemm_tcgen05_kernel<BN, STAGES, SWAP, TOut, EPI>;
    constexpr int smem = Smem<BN, STAGES>::kTotal;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return qi::fail("gemm_bf16: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    const long long tiles = (long long)((rows_a + BM - 1) / BM) * ((rows_b + BN - 1) / BN) * splits;
    // as many CTAs as fit on the GPU at once (by shared memory); each walks its share of the tiles
    const int per_sm = (227 * 1024) / smem > 0 ? (227 * 1024) / smem : 1;
    const long long resident = (long long)sm_count() * per_sm;
    const unsigned grid = (unsigned)(tiles < resident ? tiles : resident);
    qi::launch(kern, dim3(grid), dim3(kThreads), smem, stream, ma, mb, out, rows_a, rows_b, K, ld, kb_per_split, splits,
               split_stride, status, rope);
    return qi::check_launch("gemm_bf16");
}

template <typename TOut, int EPI>
int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, TOut* out, int M, int N, int K, long long ld, int* status,
                cudaStream_t stream, const RopeEpilogue& rope = RopeEpilogue{}, int splits = 1, long long split_stride = 0) {
    auto kern = gemm_tcgen05_pair_kernel<TOut, EPI>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmem);
        if (e != cudaSuccess) return qi::fail("gemm_bf16: cannot reserve %d bytes of shared memory: %s", kPairSmem, cudaGetErrorString(e));
        configured = true;
    }
    const long long tiles = (long long)((M + 2 * BM - 1) / (2 * BM)) * ((N + 255) / 256) * splits;
    const long long pairs = sm_count() / 2;
    const unsigned grid = 2u * (unsigned)(tiles < pairs ? tiles : pairs);
    const int kb_total = (K + BK - 1) / BK;
    qi::launch(kern, dim3(grid), dim3(kThreads), kPairSmem, stream, ma, mb, out, M, N, K, ld, (kb_total + splits - 1) / splits,
               splits, split_stride, status, rope);
    return qi::check_launch("gemm_bf16 (CTA pairs)");
}

// Pipeline stages by tile width: as many as let two CTAs stay resident on an SM for the narrow
// tiles (6 of 18 KB, 5 of 20 KB, 4 of 24 KB: the first stages' weight tiles are requested before
// the kernel waits for its predecessor, so deeper is better while two CTAs fit), 6 for the
// 128-wide tile and 4 for the widest, one CTA an SM.
constexpr int stages_of(int bn) { return bn <= 16 ? 6 : bn == 32 ? 5 : bn == 128 ? 6 : 4; }

template <bool SWAP, typename TOut, int EPI = 0>
int launch_bn(int bn, const CUtensorMap& ma, const CUtensorMap& mb, TOut* out, int rows_a, int rows_b, int K,
              long long ld, int splits, int kb_per_split, long long split_stride, int* status, cudaStream_t stream) {
    switch (bn) {
        case 16: return launch<16, stages_of(16), SWAP, TOut, EPI>(ma, mb, out, rows_a, rows_b, K, ld, splits, kb_per_split, split_stride, status, stream);
        case 32: return launch<32, stages_of(32), SWAP, TOut, EPI>(ma, mb, out, rows_a, rows_b, K, ld, splits, kb_per_split, split_stride, status, stream);
        case 64: return launch<64, stages_of(64), SWAP, TOut, EPI>(ma, mb, out, rows_a, rows_b, K, ld, splits, kb_per_split, split_stride, status, stream);
        case 128: return launch<128, stages_of(128), SWAP, TOut, EPI>(ma, mb, out, rows_a, rows_b, K, ld, splits, kb_per_split, split_stride, status, stream);
        case 256: return launch<256, stages_of(256), SWAP, TOut, EPI>(ma, mb, out, rows_a, rows_b, K, ld, splits, kb_per_split, split_stride, status, stream);
    }
    return qi::fail("gemm_bf16: no kernel for a tile width of %d", bn);
}

}  // namespace

// The orientation (0: tokens on the 128 rows, 1: weights on the 128 rows, 2: tokens on the rows of
// CTA pairs), tile width and K split `qi_gemm_bf16` uses when the caller does not say
// (allow_split 0: the caller needs the whole sum in one CTA, as the fused activation does).
//
// Up to 64 tokens the product is a weight stream: the weights are the 128-row operand, the
// tokens the narrow one, and K is split until about 148 CTAs pull weights.
// Above that, the candidates (tokens as the narrow operand in one tile of 128 or 256 while they
// fit; tokens as the 128-row operand with weight tiles of 256 or 128; K in 1 to 16 parts) are
// compared by a count of k blocks per SM: waves of CTAs x (k blocks of a CTA + 12 for its start
// and its epilogue) x the relative cost of a k block at that width, plus what the partial sums
// cost to write and to read again (at 5.5 TB/s, in units of a 128 x 256 k block = 0.27 us).
// Splitting K fills the SMs when there are few tiles (a 4096-wide product of 512 tokens has 64
// tiles of 128 x 256) and evens out a ragged last wave; its price grows with the tokens. The
// constants were fitted to a sweep of all candidates over 72 to 4,096 tokens at four layer
// shapes: the choice is within 1% of the best candidate on average, 10% at worst.
extern "C" int qi_gemm_bf16_plan(int M, int N, int K, int allow_split, int* swap, int* bn, int* splits) {
    const int kb_total = (K + BK - 1) / BK;
    int sw = 1, b = 256, sp = 1;
    if (M <= 64) {
        b = M <= 16 ? 16 : M <= 32 ? 32 : 64;
        const int tiles = (N + BM - 1) / BM;
        // enough CTAs to keep the weight stream busy on 148 SMs, at least 8 k blocks per split
        // (filling every resident slot with 6 or 9 splits was measured no faster than powers of two)
        while (allow_split && tiles * sp < 148 && sp * 2 <= 16 && kb_total / (sp * 2) >= 8) sp *= 2;
    } else {
        const int sms = sm_count();
        double best = 1e30;
        const int split_choices[8] = {1, 2, 3, 4, 6, 8, 12, 16};
        for (int cand = 0; cand < 3; ++cand) {
            // 0: tokens narrow, one tile; 1, 2: tokens in rows of 128, weight tiles of 256, 128
            if (cand == 0 && M > 256) continue;
            const int c_swap = cand == 0, c_bn = cand == 0 ? (M <= 128 ? 128 : 256) : cand == 1 ? 256 : 128;
            const int rows_a = c_swap ? N : M, rows_b = c_swap ? M : N;
            const double k_cost = (c_bn == 256 ? 1.0 : 0.65) * (c_swap ? 1.05 : 1.0);
            for (int si = 0; si < (allow_split ? 8 : 1); ++si) {
                const int s = split_choices[si];
                const int kbs = (kb_total + s - 1) / s;
                if (s > 1 && ((s - 1) * kbs >= kb_total || kbs < 8)) continue;
                const long long units = (long long)((rows_a + BM - 1) / BM) * ((rows_b + c_bn - 1) / c_bn) * s;
                const long long waves = (units + sms - 1) / sms;
                double cost = (double)waves * (kbs + 12) * k_cost;
                if (s > 1) cost += (double)s * M * N * 8.0 / 5.5e12 / 0.27e-6;
                if (cost < best * 0.999) {
                    best = cost;
                    sw = c_swap;
                    b = c_bn;
                    sp = s;
                }
            }
        }
        // pairs of CTAs on tiles of 256 x 256: a k block of a pair's tile takes what a k block
        // of a 128 x 256 tile takes on one SM, less the 13% the lighter load on L2 and shared memory gives
        const long long pair_tiles = (long long)((M + 2 * BM - 1) / (2 * BM)) * ((N + 255) / 256);
        for (int si = 0; si < (allow_split ? 8 : 1); ++si) {
            const int s = split_choices[si];
            const int kbs = (kb_total + s - 1) / s;
            if (s > 1 && ((s - 1) * kbs >= kb_total || kbs < 8)) continue;
            const long long waves = (pair_tiles * s + sms / 2 - 1) / (sms / 2);
            double cost = (double)waves * (kbs + 12) * 0.87;
            if (s > 1) cost += (double)s * M * N * 8.0 / 5.5e12 / 0.27e-6;
            if (cost < best * 0.999) {
                best = cost;
                sw = 2;
                b = 256;
                sp = s;
            }
        }
    }
    *swap = sw; *bn = b; *splits = sp;
    return 0;
}

// y[M, N] = x[M, K] . w[N, K]^T, bf16 operands, out bf16 or float32 (out_dtype).
// With splits > 1, `workspace` must hold splits * M * N floats.
// epilogue 1: w's rows come in (gate, up) pairs and out[M, N / 2] = silu(gate) * up (bf16, no split).
// out may be null with splits > 1: the partial sums stay in the workspace for the consumer.
extern "C" int qi_gemm_bf16(const void* x, const void* w, void* out, int out_dtype, int M, int N, int K,
                            int swap, int bn, int splits, int epilogue, void* workspace, int* status,
                            cudaStream_t stream) {
    QI_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_bf16: bad sizes M=%d N=%d K=%d", M, N, K);
    QI_REQUIRE(K % 8 == 0, "gemm_bf16: K=%d must be a multiple of 8 (16-byte rows for TMA)", K);
    QI_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0, "gemm_bf16: operands must be 16-byte aligned");
    QI_REQUIRE(splits >= 1 && (splits == 1 || workspace), "gemm_bf16: split-K needs a workspace");
    QI_REQUIRE(out_dtype == qi::kF32 || out_dtype == qi::kBF16, "gemm_bf16: output type must be float32 or bfloat16");
    QI_REQUIRE(epilogue == 0 || (epilogue == 1 && splits == 1 && out_dtype == qi::kBF16 && N % 2 == 0 && out),
               "gemm_bf16: the fused activation needs bfloat16 output, an even N and no K split");
    const int kb_total = (K + BK - 1) / BK;
    const int kb_per_split = (kb_total + splits - 1) / splits;
    QI_REQUIRE((splits - 1) * kb_per_split < kb_total, "gemm_bf16: %d splits leave one without work (K=%d)", splits, K);
    if (swap == 2) {
        // pairs of CTAs: tokens on the rows, no K split
        CUtensorMap pa, pb;
        if (make_map(&pa, x, M, K, BM)) return 1;
        if (make_map(&pb, w, N, K, BM)) return 1;
        if (splits > 1) {
            float* ws = (float*)workspace;
            if (int rc = launch_pair<float, 0>(pa, pb, ws, M, N, K, N, status, stream, RopeEpilogue{}, splits, (long long)M * N)) return rc;
            if (out) {
                const size_t n = (size_t)M * N;
                unsigned blocks = (unsigned)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
                if (out_dtype == qi::kF32) qi::launch(splitk_reduce_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)ws, (float*)out, n, splits);
                else qi::launch(splitk_reduce_kernel<qi::bf16>, dim3(blocks), dim3(256), 0, stream, (const float*)ws, (qi::bf16*)out, n, splits);
                return qi::check_launch("splitk_reduce");
            }
            return 0;
        }
        if (epilogue == 1) return launch_pair<qi::bf16, 1>(pa, pb, (qi::bf16*)out, M, N, K, N / 2, status, stream);
        if (out_dtype == qi::kF32) return launch_pair<float, 0>(pa, pb, (float*)out, M, N, K, N, status, stream);
        return launch_pair<qi::bf16, 0>(pa, pb, (qi::bf16*)out, M, N, K, N, status, stream);
    }
    const void* a = swap ? w : x;
    const void* b = swap ? x : w;
    const int rows_a = swap ? N : M, rows_b = swap ? M : N;
    QI_REQUIRE((long long)((rows_a + BM - 1) / BM) * ((rows_b + bn - 1) / bn) * splits < 2147483647LL, "gemm_bf16: too many tiles");
    CUtensorMap ma, mb;
    if (make_map(&ma, a, rows_a, K, BM)) return 1;
    if (make_map(&mb, b, rows_b, K, bn)) return 1;
    const long long split_stride = (long long)M * N;
    int rc;
    if (splits > 1) {
        float* ws = (float*)workspace;
        rc = swap ? launch_bn<true, float>(bn, ma, mb, ws, rows_a, rows_b, K, N, splits, kb_per_split, split_stride, status, stream)
                  : launch_bn<false, float>(bn, ma, mb, ws, rows_a, rows_b, K, N, splits, kb_per_split, split_stride, status, stream);
        if (rc) return rc;
        if (out) {
            const size_t n = (size_t)M * N;
            unsigned blocks = (unsigned)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
            if (out_dtype == qi::kF32) qi::launch(splitk_reduce_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)ws, (float*)out, n, splits);
            else qi::launch(splitk_reduce_kernel<qi::bf16>, dim3(blocks), dim3(256), 0, stream, (const float*)ws, (qi::bf16*)out, n, splits);
            return qi::check_launch("splitk_reduce");
        }
        return 0;
    }
    if (epilogue == 1)
        return swap ? launch_bn<true, qi::bf16, 1>(bn, ma, mb, (qi::bf16*)out, rows_a, rows_b, K, N / 2, 1, kb_per_split, 0, status, stream)
                    : launch_bn<false, qi::bf16, 1>(bn, ma, mb, (qi::bf16*)out, rows_a, rows_b, K, N / 2, 1, kb_per_split, 0, status, stream);
    if (out_dtype == qi::kF32)
        return swap ? launch_bn<true, float>(bn, ma, mb, (float*)out, rows_a, rows_b, K, N, 1, kb_per_split, 0, status, stream)
                    : launch_bn<false, float>(bn, ma, mb, (float*)out, rows_a, rows_b, K, N, 1, kb_per_split, 0, status, stream);
    return swap ? launch_bn<true, qi::bf16>(bn, ma, mb, (qi::bf16*)out, rows_a, rows_b, K, N, 1, kb_per_split, 0, status, stream)
                : launch_bn<false, qi::bf16>(bn, ma, mb, (qi::bf16*)out, rows_a, rows_b, K, N, 1, kb_per_split, 0, status, stream);
}

// The q/k/v projection of many tokens with what follows it fused into the epilogue:
// [q | k | v] = x[M, K] . w[(nq + 2 nkv) * 128, K]^T, then RMSNorm of every query and key head
// (gains null: none), the half-split rotation by the token's position (cos_t null: none), queries
// to q_out [M, nq * 128], keys and values to the paged cache (k_pages null: not written). Head size
// 128, rotation over the whole head, bfloat16 throughout. The operands are not swapped, so this is
// the path for prompts; few tokens go through qi_gemm_bf16 (K split) and qi_qk_norm_rope_kv.
extern "C" int qi_gemm_bf16_qkv_rope(const void* x, const void* w, int M, int K, void* q_out, const float* q_gain,
                                     const float* k_gain, float eps, const float* cos_t, const float* sin_t,
                                     int table_positions, const int* positions, const int* token_req,
                                     const int* block_table, int max_blocks, int page_size, int num_pages,
                                     void* k_pages, void* v_pages, int nq, int nkv, int* status, cudaStream_t stream) {
    QI_REQUIRE(M > 0 && K > 0 && nq > 0 && nkv > 0, "gemm_bf16_qkv_rope: bad sizes M=%d K=%d heads %d/%d", M, K, nq, nkv);
    QI_REQUIRE(K % 8 == 0, "gemm_bf16_qkv_rope: K=%d must be a multiple of 8 (16-byte rows for TMA)", K);
    QI_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0 && ((uintptr_t)q_out & 15) == 0 &&
               ((uintptr_t)k_pages & 15) == 0 && ((uintptr_t)v_pages & 15) == 0,
               "gemm_bf16_qkv_rope: operands, q_out and pages must be 16-byte aligned");
    QI_REQUIRE(q_out && positions, "gemm_bf16_qkv_rope: q_out and positions are needed");
    QI_REQUIRE((cos_t == nullptr) == (sin_t == nullptr) && (!cos_t || table_positions > 0), "gemm_bf16_qkv_rope: incomplete rotation table");
    QI_REQUIRE(((uintptr_t)cos_t & 15) == 0 && ((uintptr_t)sin_t & 15) == 0 && ((uintptr_t)q_gain & 15) == 0 && ((uintptr_t)k_gain & 15) == 0,
               "gemm_bf16_qkv_rope: gains and tables must be 16-byte aligned");
    QI_REQUIRE((k_pages == nullptr) == (v_pages == nullptr), "gemm_bf16_qkv_rope: k and v pages must come together");
    QI_REQUIRE(!k_pages || (page_size > 0 && max_blocks > 0 && num_pages > 0 && block_table && token_req),
               "gemm_bf16_qkv_rope: incomplete page arguments");
    const long long n_ll = (long long)(nq + 2 * nkv) * 128;
    QI_REQUIRE(n_ll < 2147483647LL, "gemm_bf16_qkv_rope: too many heads");
    const int N = (int)n_ll;
    int plan_mode, bn, plan_splits;
    qi_gemm_bf16_plan(M > 256 ? M : 257, N, K, 0, &plan_mode, &bn, &plan_splits);   // the width for operands that are not swapped
    if (bn < 128) bn = 128;                                                        // a tile holds whole heads
    const int kb_total = (K + BK - 1) / BK;
    QI_REQUIRE((long long)((M + BM - 1) / BM) * ((N + bn - 1) / bn) < 2147483647LL, "gemm_bf16_qkv_rope: too many tiles");
    CUtensorMap ma, mb;
    if (make_map(&ma, x, M, K, BM)) return 1;
    if (make_map(&mb, w, N, K, bn)) return 1;
    RopeEpilogue e;
    e.q_out = (qi::bf16*)q_out; e.q_gain = q_gain; e.k_gain = k_gain; e.cos_t = cos_t; e.sin_t = sin_t;
    e.positions = positions; e.token_req = token_req; e.block_table = block_table;
    e.k_pages = (qi::bf16*)k_pages; e.v_pages = (qi::bf16*)v_pages; e.eps = eps;
    e.max_blocks = max_blocks; e.page_size = page_size; e.num_pages = num_pages; e.nq = nq; e.nkv = nkv;
    e.table_positions = table_positions;
    if (plan_mode == 2) {
        CUtensorMap pb;
        if (make_map(&pb, w, N, K, BM)) return 1;
        return launch_pair<qi::bf16, 2>(ma, pb, (qi::bf16*)nullptr, M, N, K, N, status, stream, e);
    }
    if (bn == 256)
        return launch<256, stages_of(256), false, qi::bf16, 2>(ma, mb, (qi::bf16*)nullptr, M, N, K, N, 1, kb_total, 0, status, stream, e);
    return launch<128, stages_of(128), false, qi::bf16, 2>(ma, mb, (qi::bf16*)nullptr, M, N, K, N, 1, kb_total, 0, status, stream, e);
}


QI_TL_EXPORT(qi_timeline_gemm)
