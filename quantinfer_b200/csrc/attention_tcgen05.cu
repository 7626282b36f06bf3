// Causal paged GQA flash attention for prefill on the 5th-generation tensor cores
// (tcgen05.mma with accumulators in tensor memory), head size 128, bfloat16.
//
// One CTA takes 128 query rows of one request and one query head and walks the keys in
// tiles of 64. Per tile two products run on the tensor core:
//     S = Q . K^T      (128 x 64,  K = head size)    -> tensor memory, 32-bit
//     O += P . V       (128 x 128, K = 64 keys)      -> tensor memory, 32-bit
// 128 softmax threads, one per query row, read their row of S from tensor memory, update the
// row's running maximum and sum, and write the weights P as bfloat16 back into tensor memory
// (two to a 32-bit column), from where the tensor core takes them as the A operand and adds
// P . V to O; P never passes through shared memory. The exponent's reference m_ref is not the
// running maximum itself: it follows the maximum only when that has grown by more than 8 (in
// the base-2 scale), and only then is the row of O read back, scaled by
// 2^(m_ref_old - m_ref_new) and stored again, after the last product has finished. Weights
// therefore reach 2^8 at most, sum and accumulator share one reference, and their quotient is
// unchanged; after the first few tiles of a row the accumulator is hardly ever touched.
//
// Two such CTAs share an SM (192 threads, 256 columns of tensor memory: S 64, O 128, P twice
// 32; Q, two stages of K and two of V in shared memory): the softmax of one overlaps the
// products of the other, and so do one CTA's start (barriers, the copy of Q, the first tiles)
// and end (the last product, the normalised store) with its neighbour's steady state, which at
// a few thousand keys are as long as the work itself. (An earlier form had one CTA an SM with
// two softmax groups on alternating key tiles of the same query rows, merged at the end: 322,
// 626, 685 TFLOP/s at 2,048, 8,192 and 16,384 tokens.)
//
// What the steady state waits for, measured with the cycle counter around each wait and each
// piece of work, decided the rest. K and V have rings and barriers of their own: a K tile's
// slot is free as soon as its S has been computed, one softmax before P.V frees the V slot,
// so the load of K for tile j + 2 starts a whole tile earlier than it would behind a shared
// barrier (the MMA thread waited 1,400 cycles a tile for K before). P has two buffers, so the
// weights of tile j + 1 do not wait for P.V of tile j. The exponentials of a row's 64 columns
// are one block of straight code (the choice between the masked and the unmasked form is made
// once per tile and warp, outside it): with a branch inside the loop only eight exponentials
// were in flight at a time and the loop took 1,580 cycles a tile, now 890. Together: 526, 756,
// 777 TFLOP/s before, 736, 1,116, 1,171 now (2,048, 8,192 and 16,384 tokens).
//
// What bounds it now is the tensor pipe itself: a tcgen05.mma of M = 128, K = 16 takes about 70
// cycles whether N is 32, 64 or 128 (one thread issuing 4,096 of them back to back: 74, 74, 70
// cycles with A in shared memory, 67 with A in tensor memory; N = 256 takes 128). S = Q.K^T
// over 64 keys is eight such instructions at half the pipe's rate, P.V four at the full rate:
// 835 cycles a tile, and the two CTAs of an SM finish a tile every 830 to 930 cycles. Key
// tiles of 128 (S at the full rate) need 128 columns for S, so with O the weights must go
// over S and a CTA's products and its softmax take turns; that was built (one softmax thread a
// row, and two), was right, and ran at 1,105 and 1,030 TFLOP/s at 16,384 tokens: the two CTAs
// of an SM fall into step instead of filling each other's gaps, their softmax phases share
// the special-function unit and their products queue. Two heads of a KV group in one CTA of
// 352 threads, so that one copy of K and V serves both: 1,042 TFLOP/s.
//
// Roles: warps 0-3 are the softmax threads; warp 4 issues the TMA loads of Q and of the K/V
// tiles (page pieces through the block table, as in attention_tma.cu); warp 5 allocates tensor
// memory and issues the MMAs: S of tile j + 1 as soon as the softmax threads have taken S of
// tile j into registers, then P.V of tile j when its weights are ready. K is read as a
// K-major operand, V as an MN-major operand (its rows are keys, the product contracts over
// keys), Q as a K-major operand, P from tensor memory. (Computing part of the exponentials by a
// polynomial on the FMA pipe, to relieve the special-function unit, was measured slower here.)
//
// Formulas: as attention_mma.cu (reference: crates/quantinfer-runtime/src/attention.rs:105-135).
// No load uses cluster multicast. Every mbarrier wait is bounded; on expiry the kernel sets
// kStatusWaitTimeout and its roles leave their loops, tensor memory is freed and it returns.
#include "common.cuh"
#include "attention_frag.cuh"

#include <cuda.h>
#include <math.h>

namespace {

using qi_attn::smem_u32;

constexpr int BM = 128;          // query rows per CTA
constexpr int BN = 64;           // keys per tile
constexpr int D = 128;           // head size
constexpr int kHalfBytes = 128 * 128;             // Q: 128 rows x 128 bytes, one 64-column half
constexpr int kQBytes = 2 * kHalfBytes;           // 32 KB
constexpr int kKVHalfBytes = BN * 128;            // K or V: 64 keys x 128 bytes, one 64-column half
constexpr int kKVBytes = 2 * kKVHalfBytes;        // 16 KB
constexpr int kMaxTableEntries = 2048;
constexpr uint32_t kSpinLimit = 1u << 22;   // polls of a barrier before a role gives up (each poll may itself wait a little)
constexpr float kRescaleStep = 8.f;   // the exponent's reference follows the maximum when that has grown by more (base 2)

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
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    return false;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
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
// The same with the A operand in tensor memory (lane = row, two bfloat16 per 32-bit column, K ascending).
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0) : "memory");
}
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
__device__ __forceinline__ void tmem_st32(uint32_t addr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
using qi_attn::ex2;
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// K-major operand tile (rows of 128 bytes, 128-byte swizzle): see gemm_tcgen05.cu.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;                      // leading byte offset: unused for swizzled K-major
    d |= (uint64_t)(1024 >> 4) << 32;            // stride byte offset: 8 rows x 128 bytes
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;                      // 128-byte swizzle
    return d;
}
// MN-major operand (V: rows are keys = the contraction dimension, 64 head-dim elements per
// 128-byte row, two such halves side by side): leading byte offset = distance between the
// halves, stride byte offset = distance between groups of 8 keys.
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(kKVHalfBytes >> 4) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// kind::f16 instruction descriptor: D = F32, A = B = BF16, M = 128, N = n; bit 16 = B is MN-major.
constexpr uint32_t idesc(int n, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(BM >> 4) << 24);
}


// The largest score of a row's 64 columns, of those in [c_lo, c_hi) with kMasked.
template <bool kMasked>
__device__ __forceinline__ float row_max(const uint32_t (&sv)[BN], int c_lo, int c_hi) {
    float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
    for (int i = 0; i < BN; i += 8) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int c = i + 2 * e;
            float a = __uint_as_float(sv[c]), b = __uint_as_float(sv[c + 1]);
            if (kMasked) {
                a = (c >= c_lo && c < c_hi) ? a : -INFINITY;
                b = (c + 1 >= c_lo && c + 1 < c_hi) ? b : -INFINITY;
            }
            mx4[e] = max3(mx4[e], a, b);
        }
    }
    return fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
}
// p = 2^(s * scale - ms) for a row's 64 columns (0 outside [c_lo, c_hi) with kMasked), packed as
// bfloat16 pairs; returns their sum in 32-bit. One block of straight code, so that the
// exponentials of all columns can be in flight together.
template <bool kMasked>
__device__ __forceinline__ float row_weights(const uint32_t (&sv)[BN], uint32_t (&pk)[BN / 2], float scale_log2e, float ms,
                                             int c_lo, int c_hi) {
    float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int c = 0; c < BN; c += 2) {
        float p0 = ex2(fmaf(__uint_as_float(sv[c]), scale_log2e, -ms));
        float p1 = ex2(fmaf(__uint_as_float(sv[c + 1]), scale_log2e, -ms));
        if (kMasked) {
            p0 = (c >= c_lo && c < c_hi) ? p0 : 0.f;
            p1 = (c + 1 >= c_lo && c + 1 < c_hi) ? p1 : 0.f;
        }
        sum4[(c >> 1) & 3] += p0 + p1;
        pk[c >> 1] = qi_attn::pack_bf16(p0, p1);
    }
    return (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
}

constexpr int kStages = 2;       // stages of the K ring and of the V ring (a K slot is free after S, a V slot after P.V)
constexpr int kThreads = 192;    // four softmax warps, the TMA warp, the MMA warp
struct Bars {
    static constexpr int q_full = 0;
    static constexpr int k_full = 8;                         // [kStages]
    static constexpr int k_empty = k_full + 8 * kStages;     // [kStages]
    static constexpr int v_full = k_empty + 8 * kStages;     // [kStages]
    static constexpr int v_empty = v_full + 8 * kStages;     // [kStages]
    static constexpr int s_full = v_empty + 8 * kStages;
    static constexpr int s_free = s_full + 8;
    static constexpr int p_ready = s_free + 8;               // [2]: one per buffer of P
    static constexpr int p_free = p_ready + 16;              // [2]
    static constexpr int total = p_free + 16;
};
constexpr int kSmemBytes = kQBytes + kStages * 2 * kKVBytes + 256 /*barriers*/ + 4 * kMaxTableEntries + 1024 /*alignment*/;


QI_TL_DEFINE(qi_timeline_prefill_attention)

__global__ void __launch_bounds__(kThreads, 2)
attention_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                      const __grid_constant__ CUtensorMap map_v, qi::bf16* __restrict__ out,
                                      const int* __restrict__ block_table, int max_blocks, int page_size, int box_rows,
                                      int num_pages, const int* __restrict__ q_start, const int* __restrict__ start_pos,
                                      const int* __restrict__ tile_req, const int* __restrict__ tile_q0, int nq, int nkv,
                                      float scale_log2e, int window, int* __restrict__ status, int n_ranges,
                                      float* __restrict__ ws_o, float* __restrict__ ws_ml) {
    extern __shared__ uint8_t smem_raw[];
    using B = Bars;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t q_s = base;
    const uint32_t kv_s = q_s + kQBytes;
    const uint32_t bars = kv_s + kStages * 2 * kKVBytes;
    uint8_t* bar_mem = aligned + kQBytes + kStages * 2 * kKVBytes;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_mem + B::total);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_mem + B::total + 4);
    int* s_table = reinterpret_cast<int*>(bar_mem + 256);

    // The lists of the step (requests, query tiles, block tables) were copied before the step's first
    // kernel began: the CTA reads them, sets up its barriers and its tensor memory while the kernel
    // before this one still runs, and waits for it only before it touches Q, the cache or the output.
    QI_TL_BEGIN();
    qi::pdl_launch_dependents();
    const int tile = blockIdx.y, h = blockIdx.x;
    const int hk = h / (nq / nkv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = tile_req[tile], q0 = tile_q0[tile];
    const int rows_valid = min(BM, q_start[r + 1] - q0);
    const int pos0 = start_pos[r] + (q0 - q_start[r]);
    const int* table = block_table + (size_t)r * max_blocks;
    const int hi = pos0 + rows_valid;
    const int lo = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    // With n_ranges > 1 the key tiles of these query rows are cut into that many ranges, one CTA each
    // (blockIdx.z); every CTA leaves its rows' reference, sum and accumulator in the workspace and a
    // second kernel merges them. A long context then gives enough CTAs to fill the GPU's last round.
    int t_begin = (lo / BN) * BN;
    int n_tiles = (hi - t_begin + BN - 1) / BN;
    if (n_ranges > 1) {
        const int per = (n_tiles + n_ranges - 1) / n_ranges;
        const int first = (int)blockIdx.z * per;
        const int count = max(min(n_tiles - first, per), 0);
        t_begin += first * BN;
        n_tiles = count;
        if (count == 0) {    // nothing of the rows' keys falls into this range: an empty partial
            const int row = threadIdx.x;
            qi::pdl_wait();
            QI_TL_WAKE();
            QI_TL_END(32);
            if (row < rows_valid) {
                float* ml = ws_ml + (((size_t)(q0 + row) * nq + h) * n_ranges + blockIdx.z) * 2;
                ml[0] = -INFINITY;
                ml[1] = 0.f;
            }
            return;
        }
    }
    const int blk0 = t_begin / page_size;
    const int n_blk = min(min((t_begin + n_tiles * BN + page_size - 1) / page_size, max_blocks) - blk0, kMaxTableEntries);
    for (int i = threadIdx.x; i < n_blk; i += blockDim.x) s_table[i] = table[blk0 + i];

    if (threadIdx.x == 0) {
        mbar_init(bars + B::q_full, 1);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bars + B::k_full + 8 * s, 1);
            mbar_init(bars + B::k_empty + 8 * s, 1);
            mbar_init(bars + B::v_full + 8 * s, 1);
            mbar_init(bars + B::v_empty + 8 * s, 1);
        }
        mbar_init(bars + B::s_full, 1);
        mbar_init(bars + B::s_free, 4);      // one arrival per softmax warp
        for (int b = 0; b < 2; ++b) {
            mbar_init(bars + B::p_ready + 8 * b, 4);
            mbar_init(bars + B::p_free + 8 * b, 1);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 5) {
        tmem_alloc(smem_u32(tmem_slot), 256);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 64, tmem_p = tmem_base + 192;   // P: two buffers of 32 columns
    qi::pdl_wait();
    QI_TL_WAKE();

    auto give_up = [&]() {
        if (!*abort_flag) {
            *abort_flag = 1;
            if (status) atomicOr(status, qi::kStatusWaitTimeout);
        }
    };

    if (warp == 4) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            mbar_expect_tx(bars + B::q_full, kQBytes);
            tma_load_2d(q_s, &map_q, bars + B::q_full, h * D, q0);
            tma_load_2d(q_s + kHalfBytes, &map_q, bars + B::q_full, h * D + 64, q0);
            // K of tile j + 1 goes out before V of tile j: a K slot is free as soon as its S has been
            // computed, a V slot only after P.V, one softmax later.
            int issued_k = 0, issued_v = 0;
            auto load_tile = [&](int j, bool is_v) -> bool {
                const int s = j % kStages;
                const uint32_t empty = bars + (is_v ? B::v_empty : B::k_empty) + 8 * s;
                const uint32_t full = bars + (is_v ? B::v_full : B::k_full) + 8 * s;
                if (!mbar_wait(empty, (((uint32_t)j / kStages) & 1u) ^ 1u, abort_flag)) return false;
                const uint32_t dst = kv_s + s * 2 * kKVBytes + (is_v ? kKVBytes : 0);
                const CUtensorMap* map = is_v ? &map_v : &map_k;
                mbar_expect_tx(full, kKVBytes);
                const int t0 = t_begin + j * BN;
                for (int r0 = 0; r0 < BN; r0 += box_rows) {
                    const int key = t0 + r0;
                    const int blk = key / page_size - blk0;
                    int page = blk < n_blk ? s_table[blk] : -1;
                    if (page < 0 || page >= num_pages) {
                        if (!is_v && key < hi && key + box_rows > lo && status) atomicOr(status, qi::kStatusBadPage);
                        page = 0;
                    }
                    const int row = (page * nkv + hk) * page_size + (key % page_size);
                    tma_load_2d(dst + r0 * 128, map, full, 0, row);
                    tma_load_2d(dst + kKVHalfBytes + r0 * 128, map, full, 64, row);
                }
                return true;
            };
            bool ok = n_tiles == 0 || load_tile(0, false);
            if (ok && n_tiles > 0) issued_k = 1;
            for (int j = 0; j < n_tiles && ok; ++j) {
                if (j + 1 < n_tiles) {
                    ok = load_tile(j + 1, false);
                    if (!ok) break;
                    issued_k = j + 2;
                }
                ok = load_tile(j, true);
                if (ok) issued_v = j + 1;
            }
            if (!ok) give_up();
            if (*abort_flag) {   // copies in flight write into this CTA's shared memory: wait (bounded) for them
                for (int j = max(issued_k - kStages, 0); j < issued_k; ++j)
                    for (uint32_t t = 0; t < (1u << 20); ++t)
                        if (mbar_try_wait(bars + B::k_full + 8 * (j % kStages), ((uint32_t)j / kStages) & 1u)) break;
                for (int j = max(issued_v - kStages, 0); j < issued_v; ++j)
                    for (uint32_t t = 0; t < (1u << 20); ++t)
                        if (mbar_try_wait(bars + B::v_full + 8 * (j % kStages), ((uint32_t)j / kStages) & 1u)) break;
            }
        }
    } else if (warp == 5) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc_qk = idesc(BN, false), idesc_pv = idesc(D, true);
            bool ok = mbar_wait(bars + B::q_full, 0, abort_flag);
            auto issue_qk = [&](int j) -> bool {
                const int s = j % kStages;
                if (!mbar_wait(bars + B::k_full + 8 * s, ((uint32_t)j / kStages) & 1u, abort_flag)) return false;
                if (!mbar_wait(bars + B::s_free, ((uint32_t)j & 1u) ^ 1u, abort_flag)) return false;   // the group holds S of tile j - 1
                tc_fence_after();
                const uint32_t k_addr = kv_s + s * 2 * kKVBytes;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint64_t adesc = desc_k_major(q_s + (ks >> 2) * kHalfBytes) + 2u * (ks & 3);
                    const uint64_t bdesc = desc_k_major(k_addr + (ks >> 2) * kKVHalfBytes) + 2u * (ks & 3);
                    umma_bf16(tmem_s, adesc, bdesc, idesc_qk, ks > 0 ? 1u : 0u);
                }
                umma_commit(bars + B::s_full);
                umma_commit(bars + B::k_empty + 8 * s);
                return true;
            };
            if (ok && n_tiles > 0) ok = issue_qk(0);
            for (int j = 0; j < n_tiles && ok; ++j) {
                if (j + 1 < n_tiles && !issue_qk(j + 1)) {
                    ok = false;
                    break;
                }
                const int pb = j & 1;
                const int s = j % kStages;
                if (!mbar_wait(bars + B::p_ready + 8 * pb, ((uint32_t)j >> 1) & 1u, abort_flag) ||
                    !mbar_wait(bars + B::v_full + 8 * s, ((uint32_t)j / kStages) & 1u, abort_flag)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t v_addr = kv_s + s * 2 * kKVBytes + kKVBytes;
#pragma unroll
                for (int kk = 0; kk < BN / 16; ++kk) {
                    const uint64_t bdesc = desc_mn_major(v_addr + kk * 16 * 128);
                    umma_bf16_ts(tmem_o, tmem_p + pb * 32 + kk * 8, bdesc, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(bars + B::v_empty + 8 * s);
                umma_commit(bars + B::p_free + 8 * pb);
            }
            if (!ok) give_up();
        }
    } else {
        // ---------------- softmax threads: one query row each ----------------
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const int pos = pos0 + row;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_tiles && ok; ++j) {
            const uint32_t u = (uint32_t)j;
            const int t0 = t_begin + j * BN;
            if (!mbar_wait(bars + B::s_full, u & 1u, abort_flag)) { ok = false; break; }
            tc_fence_after();
            int c_hi = min(min(pos, hi - 1) - t0 + 1, BN);
            int c_lo = max(lo, window > 0 ? pos - window + 1 : 0) - t0;
            if (c_lo < 0) c_lo = 0;
            if (c_hi < 0) c_hi = 0;
            uint32_t sv[BN];
            tmem_ld32(tmem_s + lane_addr, *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
            tmem_ld32(tmem_s + lane_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[32]));
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bars + B::s_free);
            // a tile that lies wholly inside every row's span takes the code without the comparisons
            const bool interior = __all_sync(0xffffffffu, c_lo == 0 && c_hi == BN);
            const float mx = interior ? row_max<false>(sv, 0, BN) : row_max<true>(sv, c_lo, c_hi);
            const float m_top = fmaxf(m, mx * scale_log2e);
            const bool fresh = m == -INFINITY;
            const bool moves = !fresh && m_top - m > kRescaleStep;
            if (__any_sync(0xffffffffu, moves)) {
                // every product into O so far has finished: the one of tile j - 1 arrives on its buffer's barrier
                if (!mbar_wait(bars + B::p_free + 8 * ((u - 1) & 1u), ((u - 1) >> 1) & 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const float f = moves ? ex2(m - m_top) : 1.f;
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld32(tmem_o + lane_addr + c0, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * f);
                    tmem_st32(tmem_o + lane_addr + c0, v);
                }
                tmem_st_wait();
                tc_fence_before();
                l *= f;
            }
            if (fresh || moves) m = m_top;
            const float ms = (m == -INFINITY) ? 0.f : m;
            if (u > 1 && !mbar_wait(bars + B::p_free + 8 * (u & 1u), ((u >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }   // P.V of tile j - 2 has read this buffer
            uint32_t pk[BN / 2];
            const float sum = interior ? row_weights<false>(sv, pk, scale_log2e, ms, 0, BN)
                                       : row_weights<true>(sv, pk, scale_log2e, ms, c_lo, c_hi);
            l += sum;
            tmem_st32(tmem_p + (u & 1u) * 32 + lane_addr, pk);
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bars + B::p_ready + 8 * (u & 1u));
        }
        // the accumulator, once the last product has finished: normalise and store
        if (ok && n_tiles > 0) {
            const uint32_t last = (uint32_t)(n_tiles - 1);
            ok = mbar_wait(bars + B::p_free + 8 * (last & 1u), (last >> 1) & 1u, abort_flag);
        }
        if (!ok && lane == 0) give_up();
        if (ok && n_ranges > 1) {
            tc_fence_after();
            const size_t part = ((size_t)(q0 + row) * nq + h) * n_ranges + blockIdx.z;
            if (row < rows_valid) {
                ws_ml[part * 2] = m;
                ws_ml[part * 2 + 1] = l;
            }
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem_o + lane_addr + c0, v);
                tmem_ld_wait();
                if (row < rows_valid) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *reinterpret_cast<uint4*>(ws_o + part * D + c0 + i) = make_uint4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                }
            }
        } else if (ok) {
            tc_fence_after();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            qi::bf16* orow = out + ((size_t)(q0 + row) * nq + h) * D;
            // the row's 128 columns in two halves, each half's loads in flight together
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 64) {
                uint32_t v[64];
                tmem_ld32(tmem_o + lane_addr + c0, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
                tmem_ld32(tmem_o + lane_addr + c0 + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
                tmem_ld_wait();
                if (row < rows_valid && n_tiles > 0) {
#pragma unroll
                    for (int i = 0; i < 64; i += 8) {
                        uint4 w;
                        w.x = qi_attn::pack_bf16(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv);
                        w.y = qi_attn::pack_bf16(__uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv);
                        w.z = qi_attn::pack_bf16(__uint_as_float(v[i + 4]) * inv, __uint_as_float(v[i + 5]) * inv);
                        w.w = qi_attn::pack_bf16(__uint_as_float(v[i + 6]) * inv, __uint_as_float(v[i + 7]) * inv);
                        *reinterpret_cast<uint4*>(orow + c0 + i) = w;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    QI_TL_END(32);
    if (warp == 5) tmem_dealloc(tmem_base, 256);
}

// out[t, h, :] = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M) over the key ranges of a query row, in range order.
__global__ void attention_prefill_merge_kernel(const float* __restrict__ ws_o, const float* __restrict__ ws_ml,
                                               qi::bf16* __restrict__ out, int nq, int n_ranges) {
    qi::pdl_enter();
    const int h = blockIdx.x;
    const size_t t = blockIdx.y;
    const size_t base = (t * nq + h) * n_ranges;
    float M = -INFINITY;
    for (int s = 0; s < n_ranges; ++s) M = fmaxf(M, ws_ml[(base + s) * 2]);
    for (int col = threadIdx.x; col < D; col += blockDim.x) {
        float L = 0.f, O = 0.f;
        for (int s = 0; s < n_ranges; ++s) {
            const float ms = ws_ml[(base + s) * 2];
            if (ms == -INFINITY) continue;          // an empty range's slot holds no data
            const float f = exp2f(ms - M);
            L += ws_ml[(base + s) * 2 + 1] * f;
            O += ws_o[(base + s) * D + col] * f;
        }
        out[(t * nq + h) * D + col] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
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

int make_map(CUtensorMap* map, const void* ptr, long long rows, int cols, int box_rows) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return qi::fail("attention_prefill_tcgen05: cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return qi::fail("attention_prefill_tcgen05: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}

bool pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

}  // namespace

// 1 if the tcgen05 prefill attention takes this geometry.
extern "C" int qi_attention_prefill_tcgen05_supported(int nq, int nkv, int d, int page_size, int max_blocks) {
    return d == D && nkv > 0 && nq % nkv == 0 && pow2(page_size) && page_size >= 8 && max_blocks > 0 &&
           max_blocks <= kMaxTableEntries;
}

// The kernel reads q_start, start_pos, the tile lists and the block table before it waits for the
// kernel launched before it: they must be complete when this call is made (copied, or written by a
// kernel that has ended), not still being written by a kernel under programmatic dependent launch.
// Arguments as qi_attention_prefill_tma (the tile lists are cut to 128 query rows), and: n_ranges > 1
// cuts every query tile's keys into that many ranges over separate CTAs, merged by a second kernel;
// `workspace` must then hold n_tokens * nq * n_ranges * (128 + 2) floats.
extern "C" int qi_attention_prefill_tcgen05(const void* q, void* out, const void* k_pages, const void* v_pages,
                                            const int* block_table, int max_blocks, int page_size, int num_pages,
                                            const int* q_start, const int* start_pos, const int* tile_req,
                                            const int* tile_q0, int n_tiles, int n_tokens, int nq, int nkv, int d,
                                            float scale, int window, int n_ranges, float* workspace, int* status,
                                            cudaStream_t stream) {
    QI_REQUIRE(qi_attention_prefill_tcgen05_supported(nq, nkv, d, page_size, max_blocks),
               "attention_prefill_tcgen05: heads %d/%d of size %d with %d pages of %d per request are not covered", nq, nkv,
               d, max_blocks, page_size);
    QI_REQUIRE(num_pages > 0 && window >= 0 && n_tokens > 0, "attention_prefill_tcgen05: bad sizes");
    QI_REQUIRE(((uintptr_t)q & 15) == 0 && ((uintptr_t)k_pages & 15) == 0 && ((uintptr_t)v_pages & 15) == 0,
               "attention_prefill_tcgen05: tensors must be 16-byte aligned");
    QI_REQUIRE((long long)num_pages * nkv * page_size < 2147483647LL, "attention_prefill_tcgen05: the page pool has too many rows");
    QI_REQUIRE(n_tiles >= 0 && n_tiles <= 65535, "attention_prefill_tcgen05: more than 65535 query tiles in one step");
    QI_REQUIRE(n_ranges >= 1 && n_ranges <= 64 && (n_ranges == 1 || workspace), "attention_prefill_tcgen05: key ranges need a workspace (1 to 64 ranges)");
    QI_REQUIRE(n_ranges == 1 || n_tokens <= 65535, "attention_prefill_tcgen05: key ranges take at most 65535 tokens a step");
    if (n_tiles == 0) return 0;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return qi::fail("attention_prefill_tcgen05: cannot reserve %d bytes of shared memory: %s", kSmemBytes, cudaGetErrorString(e));
        configured = true;
    }
    const int box_rows = page_size < BN ? page_size : BN;
    CUtensorMap mq, mk, mv;
    if (make_map(&mq, q, n_tokens, nq * D, BM)) return 1;
    if (make_map(&mk, k_pages, (long long)num_pages * nkv * page_size, D, box_rows)) return 1;
    if (make_map(&mv, v_pages, (long long)num_pages * nkv * page_size, D, box_rows)) return 1;
    float* ws_o = workspace;
    float* ws_ml = workspace ? workspace + (size_t)n_tokens * nq * n_ranges * D : nullptr;
    qi::launch(attention_prefill_tcgen05_kernel, dim3(nq, n_tiles, n_ranges), dim3(kThreads), kSmemBytes, stream, mq, mk, mv,
               (qi::bf16*)out, block_table, max_blocks, page_size, box_rows, num_pages, q_start, start_pos, tile_req,
               tile_q0, nq, nkv, scale * 1.4426950408889634f, window, status, n_ranges, ws_o, ws_ml);
    if (n_ranges > 1) {
        if (int rc = qi::check_launch("attention_prefill_tcgen05")) return rc;
        qi::launch(attention_prefill_merge_kernel, dim3(nq, n_tokens), dim3(128), 0, stream, (const float*)ws_o,
                   (const float*)ws_ml, (qi::bf16*)out, nq, n_ranges);
        return qi::check_launch("attention_prefill_merge");
    }
    return qi::check_launch("attention_prefill_tcgen05");
}

QI_TL_EXPORT(qi_timeline_prefill_attention)
