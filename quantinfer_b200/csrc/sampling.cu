// Token selection from 32-bit logits [rows, vocab], one block per row.
//
// temperature == 0: the first maximum (strict >, lowest index wins ties), as
// the reference's argmax (crates/quantinfer-runtime/src/generation.rs:58-77).
// Otherwise the reference's candidate rule (generation.rs:104-154): scale by
// 1/temperature, keep the top_k largest (ties: lowest index first, which is
// what its stable descending sort keeps), then the shortest prefix of the
// descending order whose mass reaches top_p of the kept mass, then draw from
// what is left. Two things differ from the reference on purpose. Its draw is a
// hash of the logits that never advances with the seed (generation.rs:219-230);
// here the uniform comes from Philox-4x32-10 keyed by the request's seed with
// the number of tokens already emitted as counter, so a request's samples do
// not depend on the batch it is in. And the inverse CDF runs over the kept
// candidates in index order, which needs no sort.
//
// Arithmetic: y = logit / temperature and w = exp(y - max y) in 32-bit; every
// sum of weights in 64-bit, warp by warp in index order.
#include "common.cuh"

#include <cooperative_groups.h>
#include <math.h>

namespace {

constexpr int kThreads = 1024;
constexpr int kNumWarps = kThreads / 32;

__device__ __forceinline__ uint32_t order_key(float v) {
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// Inverse of order_key.
__device__ __forceinline__ float key_value(uint32_t key) {
    return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}

__device__ __forceinline__ uint4 philox4x32_10(uint4 c, uint2 k) {
    const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
    for (int round = 0; round < 10; ++round) {
        if (round > 0) {
            k.x += W0;
            k.y += W1;
        }
        const uint32_t hi0 = __umulhi(M0, c.x), lo0 = M0 * c.x;
        const uint32_t hi1 = __umulhi(M1, c.z), lo1 = M1 * c.z;
        c = make_uint4(hi1 ^ c.y ^ k.x, lo1, hi0 ^ c.w ^ k.y, lo0);
    }
    return c;
}

__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Block sums in a fixed order; every thread gets the result.
__device__ double block_sum_d(double v, double* scratch) {
    v = warp_sum_d(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    double t = 0.0;
    for (int w = 0; w < kNumWarps; ++w) t += scratch[w];
    return t;
}

__device__ long long block_sum_ll(long long v, long long* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    long long t = 0;
    for (int w = 0; w < kNumWarps; ++w) t += scratch[w];
    return t;
}

// Where a row's options come from. Two forms:
//  * arrays with one entry per row of the logits (slot_ids null, stride 1);
//  * records of the per-request slots: the row's request is found through the step's own device
//    arrays (logit_rows: flat token of the row; token_req: its entry; slot_ids: the entry's slot), the
//    options lie `stride` 32-bit words apart (the record's size), and after the draw the kernel
//    advances the slot's counter itself (`bump`), so that the host uploads nothing per step.
struct SampleParams {
    const float* temperature;
    const int* top_k;
    const float* top_p;
    const long long* seed;
    int* counter;
    const int* logit_rows;
    const int* token_req;
    const int* slot_ids;
    int stride;
    int bump;
};

__device__ __forceinline__ size_t param_index(const SampleParams& sp, int row) {
    const int r = sp.slot_ids ? sp.slot_ids[sp.token_req[sp.logit_rows[row]]] : row;
    return (size_t)r * (size_t)sp.stride;
}
// seeds are 64-bit: in a record they lie stride / 2 of their own size apart
__device__ __forceinline__ size_t seed_index(const SampleParams& sp, size_t pi) { return sp.stride == 1 ? pi : pi / 2; }

__global__ void __launch_bounds__(kThreads)
sample_kernel(const float* __restrict__ logits, int vocab, const SampleParams sp,
              int* __restrict__ out_token, int* __restrict__ status) {
    __shared__ double sd[kNumWarps];
    __shared__ long long sl[kNumWarps];
    __shared__ float sbest_v[kNumWarps];
    __shared__ int sbest_i[kNumWarps];
    __shared__ double warp_mass[kNumWarps];
    __shared__ long long warp_eq[kNumWarps];
    __shared__ int result;

    qi::pdl_enter();
    const int row = blockIdx.x;
    const float* x = logits + (size_t)row * vocab;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    // Pass 0: first maximum and a finiteness check.
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    bool nonfinite = false;
    for (int i = tid; i < vocab; i += kThreads) {
        const float v = x[i];
        if (!isfinite(v)) nonfinite = true;
        if (v > bv || bi == 0x7fffffff) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { sbest_v[warp] = bv; sbest_i[warp] = bi; }
    if (nonfinite && status) atomicOr(status, qi::kStatusNonFinite);
    __syncthreads();
    float max_v = sbest_v[0];
    int max_i = sbest_i[0];
    for (int w = 1; w < kNumWarps; ++w) {
        if (sbest_v[w] > max_v || (sbest_v[w] == max_v && sbest_i[w] < max_i)) {
            max_v = sbest_v[w];
            max_i = sbest_i[w];
        }
    }
    const size_t pi = param_index(sp, row);
    const float temp = sp.temperature ? sp.temperature[pi] : 0.f;
    if (!(temp > 0.f)) {
        if (tid == 0) {
            out_token[row] = max_i;
            if (sp.bump && sp.counter) sp.counter[pi] += 1;
        }
        return;
    }

    const float max_y = max_v / temp;
    int k = sp.top_k ? sp.top_k[pi] : 0;
    if (k <= 0 || k > vocab) k = 0;  // 0: keep all
    float p_keep = sp.top_p ? sp.top_p[pi] : 0.f;
    if (!(p_keep > 0.f) || p_keep >= 1.f) p_keep = 0.f;  // 0: keep all

    // Threshold of the kept set: every y > thr_key is kept, and the first
    // n_eq (by index) of those equal to it. thr_key = 0 keeps everything.
    uint32_t thr_key = 0;
    long long n_eq = (long long)vocab + 1;

    if (k > 0) {
        uint32_t t = 0;
        for (int bit = 31; bit >= 0; --bit) {
            const uint32_t cand = t | (1u << bit);
            long long c = 0;
            for (int i = tid; i < vocab; i += kThreads) c += order_key(x[i] / temp) >= cand;
            if (block_sum_ll(c, sl) >= k) t = cand;
        }
        long long gt = 0;
        for (int i = tid; i < vocab; i += kThreads) gt += order_key(x[i] / temp) > t;
        gt = block_sum_ll(gt, sl);
        thr_key = t;
        n_eq = k - gt;
    }

    // Mass of the kept set after top-k: everything above the threshold, plus
    // n_eq times the weight of the threshold value itself.
    double total;
    {
        double s = 0.0;
        for (int i = tid; i < vocab; i += kThreads) {
            const float y = x[i] / temp;
            if (order_key(y) > thr_key) s += (double)expf(y - max_y);
        }
        total = block_sum_d(s, sd);
        if (thr_key != 0) total += (double)n_eq * (double)expf(key_value(thr_key) - max_y);
    }

    if (p_keep > 0.f) {
        const double need = (double)p_keep * total;
        // Largest t with mass(kept, key >= t) >= need.
        uint32_t t = 0;
        for (int bit = 31; bit >= 0; --bit) {
            const uint32_t cand = t | (1u << bit);
            double mass;
            if (cand <= thr_key) {
                mass = total;  // everything kept by top-k lies at or above the candidate
            } else {
                double s = 0.0;
                for (int i = tid; i < vocab; i += kThreads) {
                    const float y = x[i] / temp;
                    if (order_key(y) >= cand) s += (double)expf(y - max_y);
                }
                mass = block_sum_d(s, sd);
            }
            if (mass >= need) t = cand;
        }
        // Mass strictly above t and the number of equals available.
        double sgt = 0.0;
        long long ceq = 0;
        for (int i = tid; i < vocab; i += kThreads) {
            const float y = x[i] / temp;
            const uint32_t key = order_key(y);
            if (key > t) sgt += (double)expf(y - max_y);
            ceq += key == t;
        }
        sgt = block_sum_d(sgt, sd);
        ceq = block_sum_ll(ceq, sl);
        const long long avail = (t == thr_key) ? n_eq : ceq;
        const double wt = (double)expf(key_value(t) - max_y);
        long long want = 1;
        if (wt > 0.0) {
            const double rest = need - sgt;
            want = (long long)ceil(rest / wt);
            if (want < 1) want = 1;
        }
        if (want > avail) want = avail;
        thr_key = t;
        n_eq = want;
        total = sgt + (double)want * wt;
    }

    // Draw.
    const unsigned long long sd64 = sp.seed ? (unsigned long long)sp.seed[seed_index(sp, pi)] : 0ull;
    const uint32_t ctr = sp.counter ? (uint32_t)sp.counter[pi] : 0u;
    const uint4 rnd = philox4x32_10(make_uint4(ctr, 0u, 0u, 0u),
                                    make_uint2((uint32_t)sd64, (uint32_t)(sd64 >> 32)));
    const double target = (double)((float)(rnd.x >> 8) * (1.0f / 16777216.0f)) * total;

    // Ordered passes: each warp owns a contiguous range of indices.
    int per = (vocab + kNumWarps - 1) / kNumWarps;
    per = (per + 31) / 32 * 32;
    const int w_begin = min(vocab, warp * per), w_end = min(vocab, w_begin + per);

    // (1) equals to the threshold per warp -> how many equals precede each warp.
    {
        long long c = 0;
        for (int i = w_begin + lane; i < w_end; i += 32) c += order_key(x[i] / temp) == thr_key;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
        if (lane == 0) warp_eq[warp] = c;
    }
    __syncthreads();
    long long eq_base = 0;
    for (int w = 0; w < warp; ++w) eq_base += warp_eq[w];

    // (2) kept mass per warp, in index order.
    double my_mass = 0.0;
    {
        long long eq_seen = eq_base;
        for (int base = w_begin; base < w_end; base += 32) {
            const int i = base + lane;
            float y = 0.f;
            uint32_t key = 0;
            const bool in = i < w_end;
            if (in) { y = x[i] / temp; key = order_key(y); }
            const bool is_eq = in && key == thr_key;
            const unsigned eq_mask = __ballot_sync(0xffffffffu, is_eq);
            const long long rank = eq_seen + __popc(eq_mask & ((1u << lane) - 1u));
            const bool kept = in && (key > thr_key || (is_eq && rank < n_eq));
            if (kept) my_mass += (double)expf(y - max_y);
            eq_seen += __popc(eq_mask);
        }
        my_mass = warp_sum_d(my_mass);
        if (lane == 0) warp_mass[warp] = my_mass;
    }
    if (tid == 0) result = -1;
    __syncthreads();

    // (3) the warp whose range holds the target walks it.
    double mass_before = 0.0;
    for (int w = 0; w < warp; ++w) mass_before += warp_mass[w];
    int last_nonempty = -1;
    for (int w = 0; w < kNumWarps; ++w) if (warp_mass[w] > 0.0) last_nonempty = w;
    const bool holds = (warp_mass[warp] > 0.0) &&
                       ((target <= mass_before + warp_mass[warp] && target > mass_before) ||
                        (target <= mass_before && mass_before == 0.0 && target == 0.0) ||
                        (warp == last_nonempty && target > mass_before));
    // More than one warp can satisfy the first test only through rounding; the
    // lowest index wins below (atomicMin-like selection via ordered check).
    if (holds) {
        double cum = mass_before;
        long long eq_seen = eq_base;
        int found = -1, last_kept = -1;
        for (int base = w_begin; base < w_end && found < 0; base += 32) {
            const int i = base + lane;
            float y = 0.f;
            uint32_t key = 0;
            const bool in = i < w_end;
            if (in) { y = x[i] / temp; key = order_key(y); }
            const bool is_eq = in && key == thr_key;
            const unsigned eq_mask = __ballot_sync(0xffffffffu, is_eq);
            const long long rank = eq_seen + __popc(eq_mask & ((1u << lane) - 1u));
            const bool kept = in && (key > thr_key || (is_eq && rank < n_eq));
            double wv = kept ? (double)expf(y - max_y) : 0.0;
            // inclusive scan over lanes
            double inc = wv;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const double n = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += n;
            }
            const bool hit = kept && (cum + inc >= target);
            const unsigned hit_mask = __ballot_sync(0xffffffffu, hit);
            const unsigned kept_mask = __ballot_sync(0xffffffffu, kept);
            if (kept_mask) last_kept = base + 31 - __clz(kept_mask);
            if (hit_mask) found = base + __ffs(hit_mask) - 1;
            cum += __shfl_sync(0xffffffffu, inc, 31);
            eq_seen += __popc(eq_mask);
        }
        if (found < 0) found = last_kept;
        if (lane == 0 && found >= 0) atomicCAS(&result, -1, found);
    }
    __syncthreads();
    if (tid == 0) {
        out_token[row] = result >= 0 ? result : max_i;
        if (sp.bump && sp.counter) sp.counter[pi] += 1;      // every thread read the counter before the barrier above
    }
}

// ------------------------------------------------------------------ a row on a cluster of eight CTAs
//
// The kernel above passes over the whole row in global memory for every step of its two
// threshold searches, on one SM: 1 to 2 ms for a vocabulary of 150,000. Here a row belongs to
// a thread-block cluster of eight CTAs. Each keeps its eighth of the scaled logits y and of
// the weights w = exp(y - max y) in shared memory, so a pass costs a few dozen
// shared-memory reads a thread; sums and counts are added within the block and then over
// the cluster through distributed shared memory, in rank order (the results are the same
// numbers in every CTA). The rule is the one above, step for step: the top-k threshold is
// the k-th largest key (found by four rounds of 256-bin counting instead of 32 bisection
// passes: counts are integers, so the result is the same), the top-p threshold is found
// by the same bisection over 64-bit sums, and the draw walks the kept candidates in index
// order, CTA by CTA and warp by warp.

namespace cg = cooperative_groups;
constexpr int kClusterSize = 8;
constexpr int kMaxSlice = 24576;      // elements of y (and of w) a CTA can keep: 2 x 96 KB

struct ClusterScratch {
    double d[2][2];            // [turn][which]: this CTA's block totals of a cluster sum
    long long ll[2][2];
    float best_v[2];
    int best_i[2];
    int hist[2][256];
    int total_hist[256];
    int pick[2];               // chosen bin, count above it
};

// Sum over the block (fixed order), then over the cluster's CTAs in rank order. Two values at a time; `turn`
// alternates between calls so that one cluster barrier a call suffices (a slot is written again only
// after every CTA has passed the barrier of the call in between).
__device__ void cluster_sum_d2(cg::cluster_group& cluster, ClusterScratch* cs, int& turn, double a, double b, double* scratch,
                               double& out_a, double& out_b) {
    const double ta = block_sum_d(a, scratch), tb = block_sum_d(b, scratch);
    if (threadIdx.x == 0) {
        cs->d[turn][0] = ta;
        cs->d[turn][1] = tb;
    }
    cluster.sync();
    out_a = 0.0;
    out_b = 0.0;
    for (unsigned r = 0; r < kClusterSize; ++r) {
        const ClusterScratch* o = cluster.map_shared_rank(cs, r);
        out_a += o->d[turn][0];
        out_b += o->d[turn][1];
    }
    turn ^= 1;
}
__device__ void cluster_sum_ll2(cg::cluster_group& cluster, ClusterScratch* cs, int& turn, long long a, long long b,
                                long long* scratch, long long& out_a, long long& out_b) {
    const long long ta = block_sum_ll(a, scratch), tb = block_sum_ll(b, scratch);
    if (threadIdx.x == 0) {
        cs->ll[turn][0] = ta;
        cs->ll[turn][1] = tb;
    }
    cluster.sync();
    out_a = 0;
    out_b = 0;
    for (unsigned r = 0; r < kClusterSize; ++r) {
        const ClusterScratch* o = cluster.map_shared_rank(cs, r);
        out_a += o->ll[turn][0];
        out_b += o->ll[turn][1];
    }
    turn ^= 1;
}

__global__ void __cluster_dims__(kClusterSize, 1, 1) __launch_bounds__(kThreads, 1)
sample_cluster_kernel(const float* __restrict__ logits, int vocab, int per, const SampleParams sp,
                      int* __restrict__ out_token, int* __restrict__ status) {
    extern __shared__ float cache[];          // y[per], then w[per]
    __shared__ ClusterScratch cs;
    __shared__ double sd[kNumWarps];
    __shared__ long long sl[kNumWarps];
    __shared__ float sbest_v[kNumWarps];
    __shared__ int sbest_i[kNumWarps];
    __shared__ double warp_mass[kNumWarps];
    __shared__ long long warp_eq[kNumWarps];

    qi::pdl_enter();
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned rank = cluster.block_rank();
    const int row = blockIdx.x / kClusterSize;
    const float* x = logits + (size_t)row * vocab;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int begin = min(vocab, (int)rank * per), end = min(vocab, begin + per), n = end - begin;
    float* ys = cache;
    float* ws = cache + per;
    int turn = 0;

    const size_t pi = param_index(sp, row);
    const float temp = sp.temperature ? sp.temperature[pi] : 0.f;
    const bool greedy = !(temp > 0.f);

    // Pass 0: this CTA's first maximum, the finiteness check, and y into shared memory.
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    bool nonfinite = false;
    for (int j = tid; j < n; j += kThreads) {
        const float v = x[begin + j];
        if (!isfinite(v)) nonfinite = true;
        if (v > bv || bi == 0x7fffffff) { bv = v; bi = begin + j; }
        ys[j] = greedy ? v : v / temp;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { sbest_v[warp] = bv; sbest_i[warp] = bi; }
    if (nonfinite && status) atomicOr(status, qi::kStatusNonFinite);
    __syncthreads();
    if (tid == 0) {
        float mv = sbest_v[0];
        int mi = sbest_i[0];
        for (int w = 1; w < kNumWarps; ++w)
            if (sbest_v[w] > mv || (sbest_v[w] == mv && sbest_i[w] < mi)) { mv = sbest_v[w]; mi = sbest_i[w]; }
        cs.best_v[0] = mv;
        cs.best_i[0] = mi;
    }
    cluster.sync();
    float max_v = -INFINITY;
    int max_i = 0x7fffffff;
    for (unsigned r = 0; r < kClusterSize; ++r) {
        const ClusterScratch* o = cluster.map_shared_rank(&cs, r);
        const float v = o->best_v[0];
        const int i = o->best_i[0];
        if (i != 0x7fffffff && (max_i == 0x7fffffff || v > max_v || (v == max_v && i < max_i))) { max_v = v; max_i = i; }
    }
    if (greedy) {
        if (rank == 0 && tid == 0) {
            out_token[row] = max_i;
            if (sp.bump && sp.counter) sp.counter[pi] += 1;
        }
        cluster.sync();       // nobody leaves while a partner may still read its shared memory
        return;
    }

    const float max_y = max_v / temp;
    for (int j = tid; j < n; j += kThreads) ws[j] = expf(ys[j] - max_y);
    __syncthreads();

    int k = sp.top_k ? sp.top_k[pi] : 0;
    if (k <= 0 || k > vocab) k = 0;
    float p_keep = sp.top_p ? sp.top_p[pi] : 0.f;
    if (!(p_keep > 0.f) || p_keep >= 1.f) p_keep = 0.f;

    uint32_t thr_key = 0;
    long long n_eq = (long long)vocab + 1;

    if (k > 0) {
        // the k-th largest key, eight bits a round: counts of the keys that share the bits found so far
        uint32_t prefix = 0;
        long long above = 0;          // keys greater than every key with this prefix
        int hturn = 0;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int b = tid; b < 256; b += kThreads) cs.hist[hturn][b] = 0;
            __syncthreads();
            for (int j = tid; j < n; j += kThreads) {
                const uint32_t key = order_key(ys[j]);
                if (shift == 24 || (key >> (shift + 8)) == (prefix >> (shift + 8))) atomicAdd(&cs.hist[hturn][(key >> shift) & 255u], 1);
            }
            __syncthreads();
            cluster.sync();
            if (tid < 256) {
                int t = 0;
                for (unsigned r = 0; r < kClusterSize; ++r) t += cluster.map_shared_rank(&cs, r)->hist[hturn][tid];
                cs.total_hist[tid] = t;
            }
            __syncthreads();
            if (tid == 0) {
                long long cum = above;
                int b = 255;
                for (; b > 0; --b) {
                    if (cum + cs.total_hist[b] >= k) break;
                    cum += cs.total_hist[b];
                }
                cs.pick[0] = b;
                cs.pick[1] = (int)(cum - above);
            }
            __syncthreads();
            prefix |= (uint32_t)cs.pick[0] << shift;
            above += cs.pick[1];
            hturn ^= 1;
            __syncthreads();
        }
        thr_key = prefix;
        n_eq = k - above;
    }

    // Mass of the kept set after top-k.
    double total, unused_d;
    {
        double s = 0.0;
        for (int j = tid; j < n; j += kThreads)
            if (order_key(ys[j]) > thr_key) s += (double)ws[j];
        cluster_sum_d2(cluster, &cs, turn, s, 0.0, sd, total, unused_d);
        if (thr_key != 0) total += (double)n_eq * (double)expf(key_value(thr_key) - max_y);
    }

    if (p_keep > 0.f) {
        const double need = (double)p_keep * total;
        const uint32_t max_key = order_key(max_y);
        uint32_t t = 0;
        for (int bit = 31; bit >= 0; --bit) {
            const uint32_t cand = t | (1u << bit);
            double mass;
            if (cand <= thr_key) {
                mass = total;
            } else if (cand > max_key) {
                mass = 0.0;              // no key reaches the candidate
            } else {
                double s = 0.0;
                for (int j = tid; j < n; j += kThreads)
                    if (order_key(ys[j]) >= cand) s += (double)ws[j];
                cluster_sum_d2(cluster, &cs, turn, s, 0.0, sd, mass, unused_d);
            }
            if (mass >= need) t = cand;
        }
        double sgt = 0.0;
        long long ceq = 0, unused_ll;
        for (int j = tid; j < n; j += kThreads) {
            const uint32_t key = order_key(ys[j]);
            if (key > t) sgt += (double)ws[j];
            ceq += key == t;
        }
        cluster_sum_d2(cluster, &cs, turn, sgt, 0.0, sd, sgt, unused_d);
        cluster_sum_ll2(cluster, &cs, turn, ceq, 0, sl, ceq, unused_ll);
        const long long avail = (t == thr_key) ? n_eq : ceq;
        const double wt = (double)expf(key_value(t) - max_y);
        long long want = 1;
        if (wt > 0.0) {
            const double rest = need - sgt;
            want = (long long)ceil(rest / wt);
            if (want < 1) want = 1;
        }
        if (want > avail) want = avail;
        thr_key = t;
        n_eq = want;
        total = sgt + (double)want * wt;
    }

    // Draw.
    const unsigned long long sd64 = sp.seed ? (unsigned long long)sp.seed[seed_index(sp, pi)] : 0ull;
    const uint32_t ctr = sp.counter ? (uint32_t)sp.counter[pi] : 0u;
    const uint4 rnd = philox4x32_10(make_uint4(ctr, 0u, 0u, 0u), make_uint2((uint32_t)sd64, (uint32_t)(sd64 >> 32)));
    const double target = (double)((float)(rnd.x >> 8) * (1.0f / 16777216.0f)) * total;

    // Ordered passes: CTAs in rank order, inside a CTA each warp owns a contiguous range of indices.
    int pw = (n + kNumWarps - 1) / kNumWarps;
    pw = (pw + 31) / 32 * 32;
    const int w_begin = min(n, warp * pw), w_end = min(n, w_begin + pw);

    // (1) equals to the threshold: how many precede this CTA and this warp
    {
        long long c = 0;
        for (int j = w_begin + lane; j < w_end; j += 32) c += order_key(ys[j]) == thr_key;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
        if (lane == 0) warp_eq[warp] = c;
    }
    __syncthreads();
    long long eq_cta = 0, eq_base = 0;
    for (int w = 0; w < kNumWarps; ++w) {
        if (w < warp) eq_base += warp_eq[w];
        eq_cta += warp_eq[w];
    }
    if (tid == 0) cs.ll[turn][0] = eq_cta;
    cluster.sync();
    for (unsigned r = 0; r < rank; ++r) eq_base += cluster.map_shared_rank(&cs, r)->ll[turn][0];
    turn ^= 1;

    // (2) kept mass per warp, in index order
    double my_mass = 0.0;
    {
        long long eq_seen = eq_base;
        for (int base = w_begin; base < w_end; base += 32) {
            const int j = base + lane;
            const bool in = j < w_end;
            const uint32_t key = in ? order_key(ys[j]) : 0u;
            const bool is_eq = in && key == thr_key;
            const unsigned eq_mask = __ballot_sync(0xffffffffu, is_eq);
            const long long rk = eq_seen + __popc(eq_mask & ((1u << lane) - 1u));
            const bool kept = in && (key > thr_key || (is_eq && rk < n_eq));
            if (kept) my_mass += (double)ws[j];
            eq_seen += __popc(eq_mask);
        }
        my_mass = warp_sum_d(my_mass);
        if (lane == 0) warp_mass[warp] = my_mass;
    }
    __syncthreads();
    double mass_cta = 0.0, mass_before = 0.0;
    int last_warp = -1;
    for (int w = 0; w < kNumWarps; ++w) {
        if (w < warp) mass_before += warp_mass[w];
        mass_cta += warp_mass[w];
        if (warp_mass[w] > 0.0) last_warp = w;
    }
    if (tid == 0) cs.d[turn][0] = mass_cta;
    if (rank == 0 && tid == 0) out_token[row] = 0x7fffffff;
    cluster.sync();
    int last_cta = -1;
    for (unsigned r = 0; r < kClusterSize; ++r) {
        const double mr = cluster.map_shared_rank(&cs, r)->d[turn][0];
        if (r < rank) mass_before += mr;
        if (mr > 0.0) last_cta = (int)r;
    }
    turn ^= 1;

    // (3) the warp whose range holds the target walks it
    const bool last_nonempty = (int)rank == last_cta && warp == last_warp;
    const bool holds = (warp_mass[warp] > 0.0) &&
                       ((target <= mass_before + warp_mass[warp] && target > mass_before) ||
                        (target <= mass_before && mass_before == 0.0 && target == 0.0) ||
                        (last_nonempty && target > mass_before));
    if (holds) {
        double cum = mass_before;
        long long eq_seen = eq_base;
        int found = -1, last_kept = -1;
        for (int base = w_begin; base < w_end && found < 0; base += 32) {
            const int j = base + lane;
            const bool in = j < w_end;
            const uint32_t key = in ? order_key(ys[j]) : 0u;
            const bool is_eq = in && key == thr_key;
            const unsigned eq_mask = __ballot_sync(0xffffffffu, is_eq);
            const long long rk = eq_seen + __popc(eq_mask & ((1u << lane) - 1u));
            const bool kept = in && (key > thr_key || (is_eq && rk < n_eq));
            double inc = kept ? (double)ws[j] : 0.0;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const double nb = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += nb;
            }
            const bool hit = kept && (cum + inc >= target);
            const unsigned hit_mask = __ballot_sync(0xffffffffu, hit);
            const unsigned kept_mask = __ballot_sync(0xffffffffu, kept);
            if (kept_mask) last_kept = base + 31 - __clz(kept_mask);
            if (hit_mask) found = base + __ffs(hit_mask) - 1;
            cum += __shfl_sync(0xffffffffu, inc, 31);
            eq_seen += __popc(eq_mask);
        }
        if (found < 0) found = last_kept;
        // more than one warp can hold the target only through rounding: the lowest index wins
        if (lane == 0 && found >= 0) atomicMin(&out_token[row], begin + found);
    }
    __threadfence();
    cluster.sync();
    if (rank == 0 && tid == 0) {
        if (out_token[row] == 0x7fffffff) out_token[row] = max_i;
        if (sp.bump && sp.counter) sp.counter[pi] += 1;      // every CTA of the cluster read the counter before the barrier above
    }
}

// After a decode step that ran wholly on the device: the sampled tokens become the
// next step's input, every request moves one position on, and its draw counter advances.
// It writes the lengths that the next step's kernels read before their own wait for their
// predecessor, so it does not release its successor early (no launch_dependents).
__global__ void advance_decode_kernel(int* __restrict__ token_ids, int* __restrict__ positions,
                                      int* __restrict__ start_pos, int* __restrict__ kv_len,
                                      int* __restrict__ counter, const int* __restrict__ sampled,
                                      int* __restrict__ history, int b) {
    qi::pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= b) return;
    const int t = sampled[i];
    token_ids[i] = t;
    positions[i] += 1;
    start_pos[i] += 1;
    kv_len[i] += 1;
    if (counter) counter[i] += 1;
    if (history) history[i] = t;
}

}  // namespace

extern "C" int qi_advance_decode(int* token_ids, int* positions, int* start_pos, int* kv_len, int* counter,
                                 const int* sampled, int* history, int b, cudaStream_t stream) {
    QI_REQUIRE(b >= 0, "advance_decode: bad batch size %d", b);
    if (b == 0) return 0;
    qi::launch(advance_decode_kernel, dim3((b + 127) / 128), dim3(128), 0, stream, token_ids, positions, start_pos, kv_len,
               counter, sampled, history, b);
    return qi::check_launch("advance_decode");
}

namespace {

int launch_sample(const float* logits, int rows, int vocab, const SampleParams& sp, int* out_token, int* status,
                  cudaStream_t stream) {
    // rows that draw go to clusters of eight CTAs that keep the row in shared memory; all-greedy batches
    // (temperature null) and vocabularies too large for that keep the one-block kernel
    int per = (vocab + kClusterSize - 1) / kClusterSize;
    per = (per + 31) / 32 * 32;
    if (sp.temperature && per <= kMaxSlice && rows <= 65535 / kClusterSize) {
        const size_t smem = (size_t)per * 2 * sizeof(float);
        static size_t configured = 0;
        if (smem > configured) {
            cudaError_t e = cudaFuncSetAttribute(sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(2 * kMaxSlice * sizeof(float)));
            if (e != cudaSuccess) return qi::fail("sample: cannot reserve shared memory: %s", cudaGetErrorString(e));
            configured = 2 * kMaxSlice * sizeof(float);
        }
        qi::launch(sample_cluster_kernel, dim3(rows * kClusterSize), dim3(kThreads), smem, stream, logits, vocab, per, sp,
                   out_token, status);
        return qi::check_launch("sample (cluster)");
    }
    qi::launch(sample_kernel, dim3(rows), dim3(kThreads), 0, stream, logits, vocab, sp, out_token, status);
    return qi::check_launch("sample");
}

}  // namespace

// One token per row of float32 logits [rows, vocab]. The options are arrays with one entry per row; any
// of them may be null (greedy / no truncation / seed 0 / counter 0).
extern "C" int qi_sample(const float* logits, int rows, int vocab, const float* temperature,
                         const int* top_k, const float* top_p, const long long* seed,
                         const int* counter, int* out_token, int* status, cudaStream_t stream) {
    QI_REQUIRE(rows >= 0 && vocab > 0, "sample: bad sizes rows=%d vocab=%d", rows, vocab);
    if (rows == 0) return 0;
    SampleParams sp = {};
    sp.temperature = temperature; sp.top_k = top_k; sp.top_p = top_p; sp.seed = seed;
    sp.counter = const_cast<int*>(counter);
    sp.stride = 1;
    return launch_sample(logits, rows, vocab, sp, out_token, status, stream);
}

// The same with the options taken from the per-request slot records: `slots` is int32
// [num_slots, QI_SLOT_WORDS] on the device, one record a slot: temperature (float bits), top_k, top_p
// (float bits), tokens emitted (the counter of the request's random stream), seed low and high word,
// max_new_tokens, eos token id (-1: none). Row r of the logits belongs to the request in slot
// slot_ids[token_req[logit_rows[r]]], the step's own arrays. After a row's token is chosen the kernel
// adds one to the record's count of emitted tokens, so the host writes a record once, when the request
// is admitted, and nothing per step.
extern "C" int qi_sample_slots(const float* logits, int rows, int vocab, const int* logit_rows, const int* token_req,
                               const int* slot_ids, int* slots, int slot_words, int all_greedy, int* out_token,
                               int* status, cudaStream_t stream) {
    QI_REQUIRE(rows >= 0 && vocab > 0, "sample_slots: bad sizes rows=%d vocab=%d", rows, vocab);
    QI_REQUIRE(slot_words == 8, "sample_slots: a slot record has 8 words, got %d", slot_words);
    QI_REQUIRE(logit_rows && token_req && slot_ids && slots, "sample_slots: a step array or the slot records are missing");
    QI_REQUIRE(((uintptr_t)slots & 31) == 0, "sample_slots: the slot records must be 32-byte aligned");
    if (rows == 0) return 0;
    SampleParams sp = {};
    // a step whose rows are all greedy takes the one-block kernel (temperature null), as with arrays
    sp.temperature = all_greedy ? nullptr : reinterpret_cast<const float*>(slots);
    sp.top_k = slots + 1;
    sp.top_p = reinterpret_cast<const float*>(slots + 2);
    sp.counter = slots + 3;
    sp.seed = reinterpret_cast<const long long*>(slots + 4);
    sp.logit_rows = logit_rows; sp.token_req = token_req; sp.slot_ids = slot_ids;
    sp.stride = slot_words;
    sp.bump = 1;
    return launch_sample(logits, rows, vocab, sp, out_token, status, stream);
}
