// A chain of the skinny matrix products of a decode step, with the norms between them, in ONE
// persistent kernel, so that the weight stream from HBM does not stop where one product ends and
// the next begins.
//
// A decode step is a weight stream: with a few tokens every product y = x . W^T costs what W costs
// to read. As separate kernels (gemm_tcgen05.cu) each product fills its pipeline of shared-memory
// stages, streams, and drains it again; between two products nothing is in flight for the length of
// an HBM round trip and a launch. Here the products of one stretch of a layer,
//     o_proj -> add + RMSNorm -> gate_up (+ SiLU . up) -> down -> add + RMSNorm -> q/k/v of the next layer,
// are phases of one kernel. Every CTA keeps its ring of stages through all phases. The producer
// thread runs ahead: while the other CTAs still finish phase p, it already requests the weight tiles
// of its first tiles of phase p + 1 (weights never depend on the step's data) and adds the matching
// activation tiles as soon as phase p is complete everywhere. Only the attention, whose work is of
// another shape, stays a kernel of its own between two chains.
//
// A phase is complete when every CTA has written its share: the four epilogue warps of a CTA fence
// their stores and one of them adds 1 to the phase's counter in global memory; the phase is complete
// when its counter has reached the number of CTAs. Whoever needs phase p's results (the producer, before it
// requests activation tiles by TMA; the threads that run a norm phase) polls the counter with a
// bound, then passes a proxy fence, since what other SMs wrote with ordinary stores is now read by
// the TMA unit. All CTAs of the grid are resident together (the host sizes the grid by the
// occupancy the runtime reports), and the kernels before and after this one in the stream cannot
// keep a CTA of it from starting: the one before ends without it, the one after is only scheduled
// once every CTA of this one has started. Every wait is bounded: when a bound runs out the thread
// sets kStatusWaitTimeout and the CTA's abort flag, all roles leave their loops, the producer waits
// (bounded) for copies in flight, tensor memory is freed and the CTA returns; the other CTAs then
// run out of their own bounds the same way.
//
// A product is computed as in gemm_tcgen05.cu with the operands swapped (few tokens): the 128 rows
// of the MMA ride the weight's output dimension, the tokens ride its N (16, 32 or 64), K may be cut
// into splits whose 32-bit partial sums [splits, tokens, N] are added by the consumer (the norm
// phase here, the attention kernel for q/k/v), and the gate_up product applies silu(gate) * up to
// its interleaved rows in the epilogue. Roles inside a CTA (192 threads): warp 0 lane 0 TMA producer,
// warp 1 lane 0 MMA issuer, warps 2-5 epilogue and norm phases. No load uses cluster multicast.
//
// Formulas: the products y = x . W^T (backends/cpu/src/matmul.rs:50-59), silu(g) * u in the
// division form (backends/cpu/src/backend.rs:224-238), the residual add and RMSNorm as norm.cu
// (backends/cpu/src/backend.rs:172-193; crates/quantinfer-runtime/src/linear.rs:129-142).
#include "gemm_tcgen05.cuh"

#include <stdint.h>

namespace {

using namespace qi_gemm;

constexpr int kMaxPhases = 6;
constexpr uint32_t kPollLimit = 1u << 22;   // polls of the phase counter (each sleeps some tens of nanoseconds)

enum PhaseKind : int { kPhaseGemm = 0, kPhaseNorm = 1 };

struct Phase {
    int kind;
    // a product: weights [N, K] (tensor map map_w), activations [tokens, K] (map_x)
    int N, K, splits, kb_per_split;
    int epi;                    // 0: float32 partial sums [splits, tokens, N]; 1: silu(gate) * up as bfloat16 [tokens, N / 2]
    void* out;
    long long split_stride;     // elements between two splits of `out`
    // a norm: resid += sum of delta's splits; x_out = rmsnorm(resid) * gain
    float* resid;               // [tokens, hidden], updated in place
    const float* delta;         // [delta_splits, tokens, hidden] or null
    int delta_splits;
    long long delta_stride;
    const float* gain;
    float eps;
    qi::bf16* x_out;            // [tokens, hidden]
    int hidden;
};

struct ChainParams {
    CUtensorMap map_w[kMaxPhases];
    CUtensorMap map_x[kMaxPhases];
    Phase ph[kMaxPhases];
    int n_phases;
    int tokens;
    unsigned* counter;          // zero at launch; counts (CTA, phase) completions
    int* status;
};

__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_add(unsigned* p, unsigned v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Meeting point of the 128 epilogue threads, bounded like every other wait: an mbarrier that each
// thread arrives on and then polls. A thread that gave up never arrives; the others then leave by
// the abort flag instead of hanging, which a bar.sync would.
struct EpilogueSync {
    uint32_t bar;
    uint32_t uses;
    volatile int* abort_flag;
    const volatile int* status;
    __device__ __forceinline__ bool sync() {
        mbar_arrive(bar);
        const bool ok = mbar_wait(bar, uses & 1u, abort_flag, status);
        ++uses;
        return ok;
    }
};

// Waits until `count` phase completions have been counted; false when the bound ran out or the
// CTA has given up.
__device__ __forceinline__ bool wait_count(const unsigned* counter, unsigned count, volatile int* abort_flag) {
    for (uint32_t i = 0; i < kPollLimit; ++i) {
        if (ld_acquire(counter) >= count) return true;
        if ((i & 255u) == 255u && *abort_flag) return false;
        __nanosleep(40);
    }
    return false;
}

template <int BN, int STAGES>
struct ChainSmem {
    static constexpr int kABytes = BM * BK * 2;
    static constexpr int kBBytes = BN * BK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kBarrierBytes = 8 * (2 * STAGES + 5);    // full, empty, 2 x accumulator full and empty, the epilogue's meeting point
    static constexpr int kTotal = STAGES * kStageBytes + kBarrierBytes + 64 /* tensor-memory slot, abort flag, norm scratch */ + 1024;
};

// One token's add + RMSNorm by the 128 epilogue threads of a CTA (tid 0..127); hidden a multiple of 4.
__device__ __forceinline__ bool norm_token(const Phase& ph, int token, int tid, float* scratch, EpilogueSync& es) {
    const int hidden = ph.hidden;
    float* xr = ph.resid + (size_t)token * hidden;
    const float* dr = ph.delta ? ph.delta + (size_t)token * hidden : nullptr;
    float ss = 0.f;
    for (int c = tid * 4; c < hidden; c += 512) {
        float4 x = __ldcg(reinterpret_cast<const float4*>(xr + c));
        if (dr) {
            for (int k = 0; k < ph.delta_splits; ++k) {      // k ascending, as the stand-alone kernel adds them
                const float4 d = __ldcg(reinterpret_cast<const float4*>(dr + (size_t)k * ph.delta_stride + c));
                x.x += d.x; x.y += d.y; x.z += d.z; x.w += d.w;
            }
            __stcg(reinterpret_cast<float4*>(xr + c), x);
        }
        ss += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
    }
    ss = qi::warp_sum(ss);
    if ((tid & 31) == 0) scratch[tid >> 5] = ss;
    if (!es.sync()) return false;
    const float total = (scratch[0] + scratch[1]) + (scratch[2] + scratch[3]);
    const float inv = 1.0f / sqrtf(total / (float)hidden + ph.eps);
    qi::bf16* orow = ph.x_out + (size_t)token * hidden;
    for (int c = tid * 4; c < hidden; c += 512) {
        const float4 x = __ldcg(reinterpret_cast<const float4*>(xr + c));     // this thread wrote it above
        const float4 g = *reinterpret_cast<const float4*>(ph.gain + c);
        __nv_bfloat162 lo = __floats2bfloat162_rn(x.x * inv * g.x, x.y * inv * g.y);
        __nv_bfloat162 hi = __floats2bfloat162_rn(x.z * inv * g.z, x.w * inv * g.w);
        uint2 v;
        v.x = *reinterpret_cast<uint32_t*>(&lo);
        v.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(orow + c) = v;
    }
    return es.sync();      // the scratch may be used again
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(kThreads)
gemm_chain_kernel(const __grid_constant__ ChainParams p) {
    extern __shared__ uint8_t smem_raw[];
    using L = ChainSmem<BN, STAGES>;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + STAGES * L::kStageBytes;
    uint8_t* tail = aligned + STAGES * L::kStageBytes + L::kBarrierBytes;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 4);
    float* norm_scratch = reinterpret_cast<float*>(tail + 16);
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto acc_full_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
    auto acc_empty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };

    qi::pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned G = gridDim.x;
    constexpr uint32_t kAccCols = BN < 32 ? 32 : BN;
    constexpr uint32_t kTmemCols = 2 * kAccCols;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(acc_full_bar(a), 1);
            mbar_init(acc_empty_bar(a), 4);
        }
        mbar_init(bars + 8u * (2 * STAGES + 4), 128);
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
    int* status = p.status;

    auto give_up = [&]() {
        if (!*abort_flag) {
            *abort_flag = 1;
            if (status) atomicOr(status, qi::kStatusWaitTimeout);
        }
    };

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t it = 0;          // k blocks whose weight tile has been requested, over all phases
            bool ok = true;
            for (int q = 0; q < p.n_phases && ok; ++q) {
                const Phase& ph = p.ph[q];
                if (ph.kind != kPhaseGemm) continue;
                const int tiles_a = (ph.N + BM - 1) / BM, total_tiles = tiles_a * ph.splits;
                const int kb_total = (ph.K + BK - 1) / BK;
                // The weights of this phase may be requested at once. Its activations exist when the
                // phase before it is complete on every CTA (for the first phase: when the kernel before
                // this one has ended). Until then the k blocks of [pend_begin, it) wait for theirs.
                bool ready = false;
                uint32_t pend_begin = it;
                int pend_k0[STAGES];
                auto finish_ready = [&]() {
                    fence_proxy_async();     // what other SMs stored is now read by the TMA unit
                    for (uint32_t j = pend_begin; j < it; ++j) {
                        const int s = j % STAGES;
                        tma_load_2d(base + s * L::kStageBytes + L::kABytes, &p.map_x[q], full_bar(s), pend_k0[s], 0);
                    }
                    ready = true;
                };
                auto wait_ready = [&]() -> bool {
                    if (q == 0) qi::pdl_wait();
                    else if (!wait_count(p.counter + (q - 1), G, abort_flag)) return false;
                    finish_ready();
                    return true;
                };
                for (int tile = blockIdx.x; tile < total_tiles && ok; tile += (int)G) {
                    const int tile_a = tile % tiles_a, split = tile / tiles_a;
                    const int kb_begin = split * ph.kb_per_split;
                    const int n_kb = max(min(kb_total, kb_begin + ph.kb_per_split) - kb_begin, 0);
                    for (int i = 0; i < n_kb && ok; ++i) {
                        const int s = it % STAGES;
                        // every stage holds a k block that still waits for its activations: nothing can move before they exist
                        if (!ready && it - pend_begin >= (uint32_t)STAGES && !wait_ready()) { ok = false; break; }
                        const uint32_t parity = ((it / STAGES) & 1u) ^ 1u;
                        uint32_t spins = 0;
                        while (!mbar_try_wait(empty_bar(s), parity)) {
                            if (!ready && q > 0 && ld_acquire(p.counter + (q - 1)) >= G) finish_ready();
                            if (++spins >= kSpinLimit || ((spins & 1023u) == 0 && *abort_flag)) { ok = false; break; }
                        }
                        if (!ok) break;
                        const int k0 = (kb_begin + i) * BK;
                        const uint32_t dst = base + s * L::kStageBytes;
                        mbar_expect_tx(full_bar(s), L::kStageBytes);
                        tma_load_2d(dst, &p.map_w[q], full_bar(s), k0, tile_a * BM);
                        if (ready) tma_load_2d(dst + L::kABytes, &p.map_x[q], full_bar(s), k0, 0);
                        else pend_k0[s] = k0;
                        ++it;
                    }
                }
                if (ok && !ready && it > pend_begin && !wait_ready()) ok = false;
            }
            if (!ok) give_up();
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
            qi::pdl_wait();   // nothing can arrive before the kernel ahead has ended: the bounded polls start counting here
            constexpr uint32_t idesc = make_idesc(BM, BN);
            uint32_t it = 0;
            int j = 0;                // tiles this CTA has started, over all phases
            bool ok = true;
            for (int q = 0; q < p.n_phases && ok; ++q) {
                const Phase& ph = p.ph[q];
                if (ph.kind != kPhaseGemm) continue;
                const int tiles_a = (ph.N + BM - 1) / BM, total_tiles = tiles_a * ph.splits;
                const int kb_total = (ph.K + BK - 1) / BK;
                for (int tile = blockIdx.x; tile < total_tiles && ok; tile += (int)G, ++j) {
                    const int split = tile / tiles_a;
                    const int kb_begin = split * ph.kb_per_split;
                    const int n_kb = max(min(kb_total, kb_begin + ph.kb_per_split) - kb_begin, 0);
                    const int acc = j & 1;
                    if (!mbar_wait(acc_empty_bar(acc), (((uint32_t)j >> 1) & 1u) ^ 1u, abort_flag, status)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t tmem_d = tmem_base + (uint32_t)acc * kAccCols;
                    for (int i = 0; i < n_kb; ++i, ++it) {
                        const int s = it % STAGES;
                        if (!mbar_wait(full_bar(s), (it / STAGES) & 1u, abort_flag, status)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t a_addr = base + s * L::kStageBytes;
                        const uint64_t adesc = make_smem_desc(a_addr);
                        const uint64_t bdesc = make_smem_desc(a_addr + L::kABytes);
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k)
                            umma_bf16(tmem_d, adesc + 2u * k, bdesc + 2u * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                        umma_commit(empty_bar(s));
                    }
                    if (ok) umma_commit(acc_full_bar(acc));
                }
            }
            if (!ok) give_up();
        }
    } else {
        // ---------------- epilogue warps 2..5: the products' stores and the norm phases ----------------
        const int quarter = warp & 3;
        const int tid = (int)threadIdx.x - 64;
        qi::pdl_wait();                 // the buffers written here may still be read by the kernel before
        EpilogueSync es = {bars + 8u * (2 * STAGES + 4), 0u, abort_flag, status};
        int j = 0;
        bool ok = true;
        for (int q = 0; q < p.n_phases && ok; ++q) {
            const Phase& ph = p.ph[q];
            if (ph.kind == kPhaseNorm) {
                if ((int)blockIdx.x < p.tokens) {
                    if (q > 0 && !wait_count(p.counter + (q - 1), G, abort_flag)) { ok = false; break; }
                    if (!norm_token(ph, (int)blockIdx.x, tid, norm_scratch, es)) { ok = false; break; }
                }
            } else {
                const int tiles_a = (ph.N + BM - 1) / BM, total_tiles = tiles_a * ph.splits;
                const int kb_total = (ph.K + BK - 1) / BK;
                const long long ld_out = ph.epi == 1 ? ph.N / 2 : ph.N;
                for (int tile = blockIdx.x; tile < total_tiles && ok; tile += (int)G, ++j) {
                    const int tile_a = tile % tiles_a, split = tile / tiles_a;
                    const int kb_begin = split * ph.kb_per_split;
                    const int n_kb = max(min(kb_total, kb_begin + ph.kb_per_split) - kb_begin, 0);
                    const int acc = j & 1;
                    if (!mbar_wait(acc_full_bar(acc), ((uint32_t)j >> 1) & 1u, abort_flag, status)) { ok = false; break; }
                    tc_fence_after();
                    const int a_row = tile_a * BM + quarter * 32 + lane;
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
                            for (int e = 0; e < 32; ++e) r[e] = 0u;
                        }
                        if (c0 + kChunk >= BN) {
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(acc_empty_bar(acc));
                        }
                        if (ph.epi == 1) {
                            // rows of the weight come in pairs (gate, up): even lanes hold gate, their neighbours up
                            qi::bf16* obase = reinterpret_cast<qi::bf16*>(ph.out);
#pragma unroll
                            for (int e = 0; e < kChunk; ++e) {
                                const float mine = __uint_as_float(r[e]);
                                const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
                                if ((lane & 1) == 0 && a_row + 1 < ph.N && c0 + e < p.tokens)
                                    obase[(size_t)(c0 + e) * ld_out + (a_row >> 1)] = __float2bfloat16_rn(silu_mul(mine, other));
                            }
                        } else if (a_row < ph.N) {
                            float* obase = reinterpret_cast<float*>(ph.out) + (size_t)split * ph.split_stride;
#pragma unroll
                            for (int e = 0; e < kChunk; ++e)
                                if (c0 + e < p.tokens) obase[(size_t)(c0 + e) * ld_out + a_row] = __uint_as_float(r[e]);
                        }
                    }
                }
                if (!ok) break;
            }
            // this CTA's share of the phase is written: make it visible, to the TMA unit of other SMs too, and count it
            __threadfence();
            fence_proxy_async();
            if (!es.sync()) { ok = false; break; }
            if (tid == 0) red_release_add(p.counter + q, 1u);
        }
        if (!ok && lane == 0) give_up();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

template <int BN, int STAGES>
int launch_chain(const ChainParams& params, cudaStream_t stream) {
    auto kern = gemm_chain_kernel<BN, STAGES>;
    constexpr int smem = ChainSmem<BN, STAGES>::kTotal;
    static int per_sm = 0;
    if (!per_sm) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return qi::fail("gemm_chain: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
        int n = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, kThreads, smem);
        if (e != cudaSuccess || n <= 0) return qi::fail("gemm_chain: the runtime reports no resident CTA for this kernel: %s", cudaGetErrorString(e));
        per_sm = n > 2 ? 2 : n;      // two rings of stages an SM keep the weight stream full; more only thin them
    }
    // every CTA must be resident at once (CTAs wait for one another between phases)
    const unsigned grid = (unsigned)(sm_count() * per_sm);
    if ((int)grid <= params.tokens) return qi::fail("gemm_chain: %u CTAs cannot take %d tokens in a norm phase", grid, params.tokens);
    qi::launch(kern, dim3(grid), dim3(kThreads), smem, stream, params);
    return qi::check_launch("gemm_chain");
}

}  // namespace

// One phase as the caller describes it. kind 0, a product: out = x[tokens, K] . w[N, K]^T as float32
// partial sums [splits, tokens, N] (epi 0) or, for w's rows in (gate, up) pairs, silu(gate) * up as
// bfloat16 [tokens, N / 2] (epi 1, splits 1). kind 1, a norm: resid[tokens, hidden] += the sum of
// delta's delta_splits partial sums [delta_splits, tokens, hidden] (delta null: nothing is added);
// x_out = rmsnorm(resid) * gain as bfloat16.
struct QiChainPhase {
    int kind;
    int N, K, splits, epi;
    const void* w;
    const void* x;
    void* out;
    float* resid;
    const float* delta;
    int delta_splits;
    int hidden;
    const float* gain;
    float eps;
    void* x_out;
};

// Into how many parts the chain cuts K of a product [tokens <= 64] x [N, K]: as the stand-alone
// product does, until about one CTA an SM pulls weights and while a part keeps 8 k blocks.
extern "C" int qi_gemm_chain_splits(int N, int K, int allow_split) {
    const int kb_total = (K + BK - 1) / BK;
    const int tiles = (N + BM - 1) / BM;
    int sp = 1;
    while (allow_split && tiles * sp < 148 && sp * 2 <= 16 && kb_total / (sp * 2) >= 8) sp *= 2;
    return sp;
}

// Runs the phases in order in one kernel. tokens <= 64. `counters` holds n_phases zeros (the kernel
// counts completed phases there; zero them again before the next launch that uses them).
extern "C" int qi_gemm_chain(const QiChainPhase* phases, int n_phases, int tokens, unsigned* counters, int* status,
                             cudaStream_t stream) {
    QI_REQUIRE(n_phases >= 1 && n_phases <= kMaxPhases, "gemm_chain: %d phases, at most %d fit one launch", n_phases, kMaxPhases);
    QI_REQUIRE(tokens >= 1 && tokens <= 64, "gemm_chain: %d tokens; the chain takes 1 to 64", tokens);
    QI_REQUIRE(counters, "gemm_chain: the phase counters are missing");
    const int bn = tokens <= 16 ? 16 : tokens <= 32 ? 32 : 64;
    ChainParams cp = {};
    cp.n_phases = n_phases;
    cp.tokens = tokens;
    cp.counter = counters;
    cp.status = status;
    for (int q = 0; q < n_phases; ++q) {
        const QiChainPhase& in = phases[q];
        Phase& ph = cp.ph[q];
        ph.kind = in.kind;
        if (in.kind == kPhaseGemm) {
            QI_REQUIRE(in.N > 0 && in.K > 0 && in.K % 8 == 0, "gemm_chain: phase %d: bad sizes N=%d K=%d (K a multiple of 8)", q, in.N, in.K);
            QI_REQUIRE(in.w && in.x && in.out, "gemm_chain: phase %d: an operand is missing", q);
            QI_REQUIRE(((uintptr_t)in.w & 15) == 0 && ((uintptr_t)in.x & 15) == 0, "gemm_chain: phase %d: operands must be 16-byte aligned", q);
            QI_REQUIRE(in.epi == 0 || (in.epi == 1 && in.splits == 1 && in.N % 2 == 0), "gemm_chain: phase %d: the fused activation needs an even N and no K split", q);
            const int kb_total = (in.K + BK - 1) / BK;
            QI_REQUIRE(in.splits >= 1 && in.splits <= kb_total, "gemm_chain: phase %d: %d splits for %d k blocks", q, in.splits, kb_total);
            ph.N = in.N; ph.K = in.K; ph.splits = in.splits; ph.epi = in.epi;
            ph.kb_per_split = (kb_total + in.splits - 1) / in.splits;
            ph.out = in.out;
            ph.split_stride = (long long)tokens * in.N;
            if (make_map(&cp.map_w[q], in.w, in.N, in.K, BM)) return 1;
            if (make_map(&cp.map_x[q], in.x, tokens, in.K, bn)) return 1;
        } else if (in.kind == kPhaseNorm) {
            QI_REQUIRE(in.hidden > 0 && in.hidden % 4 == 0, "gemm_chain: phase %d: the norm's width %d must be a multiple of 4", q, in.hidden);
            QI_REQUIRE(in.resid && in.gain && in.x_out, "gemm_chain: phase %d: a buffer of the norm is missing", q);
            QI_REQUIRE(((uintptr_t)in.resid & 15) == 0 && ((uintptr_t)in.delta & 15) == 0 && ((uintptr_t)in.gain & 15) == 0 &&
                       ((uintptr_t)in.x_out & 7) == 0, "gemm_chain: phase %d: the norm's buffers must be 16-byte aligned", q);
            QI_REQUIRE(!in.delta || in.delta_splits >= 1, "gemm_chain: phase %d: delta needs its number of splits", q);
            ph.resid = in.resid; ph.delta = in.delta; ph.delta_splits = in.delta_splits;
            ph.delta_stride = (long long)tokens * in.hidden;
            ph.gain = in.gain; ph.eps = in.eps; ph.x_out = (qi::bf16*)in.x_out; ph.hidden = in.hidden;
        } else {
            return qi::fail("gemm_chain: phase %d has unknown kind %d", q, in.kind);
        }
    }
    switch (bn) {
        case 16: return launch_chain<16, 6>(cp, stream);
        case 32: return launch_chain<32, 5>(cp, stream);
        default: return launch_chain<64, 4>(cp, stream);
    }
}
