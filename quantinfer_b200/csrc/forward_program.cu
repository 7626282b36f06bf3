// The forward pass of a step, driven from C++.
//
// A step is a few hundred kernel launches. Issued one by one from Python each costs some fifteen
// microseconds of interpreter, argument conversion and allocator time, which is more than many of
// the kernels take: a step that is not replayed from a CUDA graph (a prompt portion, a mixed
// batch) then waits for its host. qi_forward runs the whole sequence
//     embedding, blocks in the run order, add + norm on the wanted rows, head
// in one call: it chooses each kernel by the same rules as the Python parts
// (parts/linear.py, parts/attention.py, parts/ffn.py, parts/norm.py, parts/embedding.py), takes
// its temporaries from one workspace the caller provides (qi_forward_workspace_bytes says how
// large), and launches through the library's own entry points. It knows one arrangement of parts,
// the pre-norm block of RMSNorm, paged attention with an optional q/k norm and rotation, RMSNorm and
// a gated feed-forward; the host describes a model of such blocks once (QiModelDesc) and falls
// back to the parts themselves for any model that has another kind of block.
//
// The order of operations is the reference's layer (crates/quantinfer-runtime/src/qwen3/mod.rs:117-209,
// 345-378); the reference drives it from Rust, one backend call per operation (mod.rs:158-209).
#include "common.cuh"

#include <stdint.h>

extern "C" {
int qi_embedding(const void* table, int table_dtype, const int* ids, float* out, int n_tokens, int hidden, int vocab,
                 int* status, cudaStream_t stream);
int qi_add_rmsnorm(float* resid, const void* delta, int delta_dtype, int delta_splits, long long delta_split_stride,
                   const float* gain, float eps, void* out, int out_dtype, const int* rows, int n_rows, int hidden,
                   int write_resid, cudaStream_t stream);
int qi_gemm_simt(const void* x, int x_dtype, const void* w, int w_dtype, void* y, int y_dtype, int M, int N, int K,
                 long long ldx, long long ldw, long long ldy, cudaStream_t stream);
int qi_gemm_bf16_plan(int M, int N, int K, int allow_split, int* swap, int* bn, int* splits);
int qi_gemm_bf16(const void* x, const void* w, void* out, int out_dtype, int M, int N, int K, int swap, int bn, int splits,
                 int epilogue, void* workspace, int* status, cudaStream_t stream);
int qi_gemm_bf16_qkv_rope(const void* x, const void* w, int M, int K, void* q_out, const float* q_gain, const float* k_gain,
                          float eps, const float* cos_t, const float* sin_t, int table_positions, const int* positions,
                          const int* token_req, const int* block_table, int max_blocks, int page_size, int num_pages,
                          void* k_pages, void* v_pages, int nq, int nkv, int* status, cudaStream_t stream);
int qi_qk_norm_rope_kv(const void* qkv, int qkv_splits, void* q_out, int dtype, const float* q_gain, const float* k_gain,
                       float eps, const float* cos_t, const float* sin_t, int rot, int interleaved, int table_positions,
                       const int* positions, const int* token_req, const int* block_table, int max_blocks, int page_size,
                       int num_pages, void* k_pages, void* v_pages, int n_tokens, int nq, int nkv, int d, int* status,
                       cudaStream_t stream);
int qi_act_mul(const void* gate_up, void* out, int dtype, int n_tokens, int inter, int interleaved, int activation,
               cudaStream_t stream);
int qi_attention_generic(const void* q, void* out, int dtype, const void* k_pages, const void* v_pages,
                         const int* block_table, int max_blocks, int page_size, int num_pages, const int* positions,
                         const int* token_req, int n_tokens, int nq, int nkv, int d, float scale, int window, int* status,
                         cudaStream_t stream);
int qi_attention_mma_supported(int nq, int nkv, int d);
int qi_attention_tma_supported(int nq, int nkv, int d, int page_size, int max_blocks);
int qi_attention_prefill_tcgen05_supported(int nq, int nkv, int d, int page_size, int max_blocks);
int qi_attention_prefill(const void* q, void* out, const void* k_pages, const void* v_pages, const int* block_table,
                         int max_blocks, int page_size, int num_pages, const int* q_start, const int* start_pos,
                         const int* tile_req, const int* tile_q0, int n_tiles, int tile_rows, int nq, int nkv, int d,
                         float scale, int window, int* status, cudaStream_t stream);
int qi_attention_prefill_tma(const void* q, void* out, const void* k_pages, const void* v_pages, const int* block_table,
                             int max_blocks, int page_size, int num_pages, const int* q_start, const int* start_pos,
                             const int* tile_req, const int* tile_q0, int n_tiles, int n_tokens, int nq, int nkv, int d,
                             float scale, int window, int* status, cudaStream_t stream);
int qi_attention_prefill_tcgen05(const void* q, void* out, const void* k_pages, const void* v_pages, const int* block_table,
                                 int max_blocks, int page_size, int num_pages, const int* q_start, const int* start_pos,
                                 const int* tile_req, const int* tile_q0, int n_tiles, int n_tokens, int nq, int nkv, int d,
                                 float scale, int window, int n_ranges, float* workspace, int* status, cudaStream_t stream);
int qi_attention_decode(const void* q, void* out, const void* k_pages, const void* v_pages, const int* block_table,
                        int max_blocks, int page_size, int num_pages, const int* kv_len, const int* q_start, int batch,
                        int nq, int nkv, int d, float scale, int window, int chunk, int n_splits, float* ws_o, float* ws_ml,
                        int* status, cudaStream_t stream);
int qi_attention_decode_tma(const void* q, void* out, const void* k_pages, const void* v_pages, const int* block_table,
                            int max_blocks, int page_size, int num_pages, const int* kv_len, const int* q_start, int batch,
                            int nq, int nkv, int d, float scale, int window, int chunk, int n_splits, float* ws_o,
                            float* ws_ml, int* status, cudaStream_t stream);
int qi_attention_decode_rope_tma(const void* qkv, int qkv_dtype, int qkv_splits, int n_tokens, const float* q_gain,
                                 const float* k_gain, float eps, const float* cos_t, const float* sin_t, int table_positions,
                                 int writes, void* out, void* k_pages, void* v_pages, const int* block_table, int max_blocks,
                                 int page_size, int num_pages, const int* kv_len, const int* q_start, int batch, int nq,
                                 int nkv, int d, float scale, int window, int chunk, int n_splits, float* ws_o, float* ws_ml,
                                 int* status, cudaStream_t stream);
}

// ---- what the host describes once per model -----------------------------------------------------

struct QiLinear {
    const void* w;          // [out_features, in_features]
    int w_dtype;
    int out_features, in_features;
};

struct QiBlock {
    const float* norm1_gain;
    const float* norm2_gain;
    float norm1_eps, norm2_eps;
    QiLinear qkv, o, gate_up, down;      // gate_up's rows are (gate, up) pairs
    const float* q_gain;                 // null: no q/k norm
    const float* k_gain;
    const float* cos_t;                  // null: no rotation
    const float* sin_t;
    float qk_eps, scale;
    int nq, nkv, d, window, rotary_dim, table_positions, interleaved;
    int activation;                      // of the feed-forward's gate: 0 silu, 1 gelu, 2 gelu_tanh, 3 relu
};

struct QiCall {               // one entry of the run order
    int block;
    int group;                // which block table of the step
    int writes;               // 0: the call reads a cache entry that an earlier call wrote
    int page_size, num_pages;
    void* k_pages;            // [num_pages, nkv, page_size, d]
    void* v_pages;
};

struct QiModelDesc {
    const QiBlock* blocks;
    const QiCall* calls;
    int n_blocks, n_calls;
    int act_dtype;            // the activation type: float32 or bfloat16
    int hidden, vocab;
    const void* embedding;
    int embedding_dtype;
    float final_eps;
    const float* final_gain;
    QiLinear head;
    int* status;
};

constexpr int kMaxGroups = 8;

struct QiStep {               // one step's batch (engine/batch.py): counts and device arrays
    int n_tokens, n_requests, n_logit_rows, all_decode, max_kv_len, n_tiles;
    int n_lead_decode;        // mixed steps: entries of one token at the front, which the tile lists leave out
    int reserved;
    const int* token_ids;
    const int* positions;
    const int* token_req;
    const int* q_start;
    const int* start_pos;
    const int* kv_len;
    const int* logit_rows;
    const int* tile_req;
    const int* tile_q0;
    const int* block_tables[kMaxGroups];
    int max_blocks[kMaxGroups];
};

namespace {

// Temporaries come from one workspace, handed out front to back. A dry run (no base address, nothing
// launched) walks the same path and reports how far it got: that is the size the real run needs.
struct Arena {
    uint8_t* base;
    long long size, off, peak;
    bool dry;
    void* take(long long bytes) {
        off = (off + 255) & ~255LL;
        const long long at = off;
        off += bytes;
        if (off > peak) peak = off;
        return dry ? nullptr : base + at;
    }
};

struct Run {
    const QiModelDesc* m;
    const QiStep* b;
    Arena arena;
    cudaStream_t stream;
    int launches;
    int failed;
    // runs an entry point unless this is a dry run or an earlier one failed
    template <typename F> void call(F&& f) {
        if (arena.dry || failed) return;
        if (f()) failed = 1;
        else ++launches;
    }
};

inline long long esize(int dtype) { return dtype == qi::kF32 ? 4 : 2; }

// What a projection hands on: its output [tokens, out] in `dtype`, or (splits > 1) the float32
// partial sums [splits, tokens, out] of a product cut along K, for a consumer that adds them.
struct Tensor {
    void* p;
    int dtype;
    int splits;
};

// y = x . W^T; the kernel is chosen as parts/linear.py chooses it.
Tensor linear(Run& r, const QiLinear& L, const void* x, int x_dtype, int M, int out_dtype, bool keep_partials, void* out_given = nullptr) {
    const int N = L.out_features, K = L.in_features;
    const bool tensor_core = x_dtype == qi::kBF16 && L.w_dtype == qi::kBF16 && M > 0 && K % 8 == 0;
    if (tensor_core) {
        int swap = 0, bn = 0, splits = 1;
        qi_gemm_bf16_plan(M, N, K, 1, &swap, &bn, &splits);
        const bool partial_only = keep_partials && splits > 1;
        void* out = partial_only ? nullptr : (out_given ? out_given : r.arena.take((long long)M * N * esize(out_dtype)));
        void* ws = splits > 1 ? r.arena.take((long long)splits * M * N * 4) : nullptr;
        r.call([&] { return qi_gemm_bf16(x, L.w, out, partial_only ? qi::kBF16 : out_dtype, M, N, K, swap, bn, splits, 0, ws, r.m->status, r.stream); });
        return partial_only ? Tensor{ws, qi::kF32, splits} : Tensor{out, out_dtype, 1};
    }
    void* out = out_given ? out_given : r.arena.take((long long)M * N * esize(out_dtype));
    r.call([&] { return qi_gemm_simt(x, x_dtype, L.w, L.w_dtype, out, out_dtype, M, N, K, K, K, N, r.stream); });
    return Tensor{out, out_dtype, 1};
}

// act(gate) * up of a projection whose weight rows are (gate, up) pairs: [tokens, out / 2] (parts/linear.py):
// silu in the tensor-core product's epilogue, anything else by the activation kernel over the product's output.
void* linear_act_mul(Run& r, const QiLinear& L, const void* x, int dtype, int M, int activation) {
    const int N = L.out_features, K = L.in_features, half = N / 2;
    void* act = r.arena.take((long long)M * half * esize(dtype));
    if (activation == 0 && dtype == qi::kBF16 && L.w_dtype == qi::kBF16 && K % 8 == 0) {
        int swap = 0, bn = 0, splits = 1;
        qi_gemm_bf16_plan(M, N, K, 0, &swap, &bn, &splits);
        r.call([&] { return qi_gemm_bf16(x, L.w, act, qi::kBF16, M, N, K, swap, bn, 1, 1, nullptr, r.m->status, r.stream); });
        return act;
    }
    Tensor gu = linear(r, L, x, dtype, M, dtype, false);
    r.call([&] { return qi_act_mul(gu.p, act, dtype, M, half, 1, activation, r.stream); });
    return act;
}

// Fused residual add and RMSNorm (parts/norm.py): resid += delta; out = rmsnorm(resid) * gain.
void* add_norm(Run& r, float* resid, const Tensor* delta, const float* gain, float eps, const int* rows, int n_out, int n_tokens) {
    const int h = r.m->hidden;
    void* out = r.arena.take((long long)n_out * h * esize(r.m->act_dtype));
    const void* dp = delta ? delta->p : nullptr;
    const int dcode = delta ? delta->dtype : qi::kF32;
    const int splits = delta ? delta->splits : 1;
    const long long stride = splits > 1 ? (long long)n_tokens * h : 0;
    r.call([&] { return qi_add_rmsnorm(resid, dp, dcode, splits, stride, gain, eps, out, r.m->act_dtype, rows, n_out, h, rows ? 0 : 1, r.stream); });
    return out;
}

// Into how many key ranges the tcgen05 prefill attention cuts every query tile (kernels/__init__.py,
// attention_prefill_ranges: the same estimate of both times).
int prefill_ranges(long long n_ctas, int max_kv_len) {
    const int choices[6] = {1, 2, 3, 4, 6, 8};
    int best = 1;
    double best_time = -1.0;
    for (int i = 0; i < 6; ++i) {
        const int ranges = choices[i];
        if (ranges > 1 && max_kv_len < 2048 * ranges) break;
        const long long units = n_ctas * ranges;
        const long long rounds = (units + 295) / 296;
        double time = (double)rounds * ((double)max_kv_len / ranges) * (units <= 148 ? 0.0132 : 0.0154);
        if (ranges > 1) time += (double)n_ctas * 128 * ranges * 0.0009;
        if (best_time < 0 || time < best_time * 0.97) {
            best = ranges;
            best_time = time;
        }
    }
    return best;
}

// (keys per CTA, key ranges) of a decode batch (kernels/__init__.py, attention_decode_plan).
void decode_plan(int batch, int nkv, int max_kv_len, int* chunk, int* splits) {
    const int bk = batch * nkv > 1 ? batch * nkv : 1;
    const int target = 296 / bk > 1 ? 296 / bk : 1;
    int c = (max_kv_len + target - 1) / target;
    c = (c + 63) / 64 * 64;
    if (c < 64) c = 64;
    *chunk = c;
    *splits = (max_kv_len + c - 1) / c;
}

// Attention over the cache for queries `q` (parts/attention.py, Attention.attend).
void attend(Run& r, const QiBlock& B, const QiCall& c, const void* q, void* out) {
    const QiStep& b = *r.b;
    const QiModelDesc& m = *r.m;
    const int* table = b.block_tables[c.group];
    const int max_blocks = b.max_blocks[c.group];
    if (m.act_dtype == qi::kBF16 && qi_attention_mma_supported(B.nq, B.nkv, B.d)) {
        if (b.all_decode) {
            int chunk = 0, splits = 0;
            decode_plan(b.n_requests, B.nkv, b.max_kv_len, &chunk, &splits);
            const long long n_o = (long long)b.n_requests * B.nq * splits * B.d;
            float* ws = (float*)r.arena.take((n_o + (long long)b.n_requests * B.nq * splits * 2) * 4);
            const bool tma = qi_attention_tma_supported(B.nq, B.nkv, B.d, c.page_size, max_blocks);
            r.call([&] {
                return (tma ? qi_attention_decode_tma : qi_attention_decode)(
                    q, out, c.k_pages, c.v_pages, table, max_blocks, c.page_size, c.num_pages, b.kv_len, b.q_start, b.n_requests,
                    B.nq, B.nkv, B.d, B.scale, B.window, chunk, splits, ws, ws + n_o, m.status, r.stream);
            });
            return;
        }
        // a mixed step: the entries of one token at its front go to the decode kernel (their rows of q and out
        // are the first rows), the others, which the tile lists hold, to the flash kernel
        if (b.n_lead_decode > 0) {
            const int lead = b.n_lead_decode;
            int chunk = 0, splits = 0;
            decode_plan(lead, B.nkv, b.max_kv_len, &chunk, &splits);
            const long long n_o = (long long)lead * B.nq * splits * B.d;
            float* ws = (float*)r.arena.take((n_o + (long long)lead * B.nq * splits * 2) * 4);
            const bool tma = qi_attention_tma_supported(B.nq, B.nkv, B.d, c.page_size, max_blocks);
            r.call([&] {
                return (tma ? qi_attention_decode_tma : qi_attention_decode)(
                    q, out, c.k_pages, c.v_pages, table, max_blocks, c.page_size, c.num_pages, b.kv_len, b.q_start, lead, B.nq,
                    B.nkv, B.d, B.scale, B.window, chunk, splits, ws, ws + n_o, m.status, r.stream);
            });
        }
        if (b.n_tiles == 0) return;
        if (qi_attention_prefill_tcgen05_supported(B.nq, B.nkv, B.d, c.page_size, max_blocks)) {
            int ranges = prefill_ranges((long long)B.nq * b.n_tiles, b.max_kv_len);
            if (b.n_tokens > 65535) ranges = 1;
            float* ws = ranges > 1 ? (float*)r.arena.take((long long)b.n_tokens * B.nq * ranges * (B.d + 2) * 4) : nullptr;
            r.call([&] {
                return qi_attention_prefill_tcgen05(q, out, c.k_pages, c.v_pages, table, max_blocks, c.page_size, c.num_pages,
                                                    b.q_start, b.start_pos, b.tile_req, b.tile_q0, b.n_tiles, b.n_tokens, B.nq,
                                                    B.nkv, B.d, B.scale, B.window, ranges, ws, m.status, r.stream);
            });
        } else if (qi_attention_tma_supported(B.nq, B.nkv, B.d, c.page_size, max_blocks)) {
            r.call([&] {
                return qi_attention_prefill_tma(q, out, c.k_pages, c.v_pages, table, max_blocks, c.page_size, c.num_pages,
                                                b.q_start, b.start_pos, b.tile_req, b.tile_q0, b.n_tiles, b.n_tokens, B.nq, B.nkv,
                                                B.d, B.scale, B.window, m.status, r.stream);
            });
        } else {
            r.call([&] {
                return qi_attention_prefill(q, out, c.k_pages, c.v_pages, table, max_blocks, c.page_size, c.num_pages, b.q_start,
                                            b.start_pos, b.tile_req, b.tile_q0, b.n_tiles, 128, B.nq, B.nkv, B.d, B.scale,
                                            B.window, m.status, r.stream);
            });
        }
        return;
    }
    r.call([&] {
        return qi_attention_generic(q, out, m.act_dtype, c.k_pages, c.v_pages, table, max_blocks, c.page_size, c.num_pages,
                                    b.positions, b.token_req, b.n_tokens, B.nq, B.nkv, B.d, B.scale, B.window, m.status, r.stream);
    });
}

// The mixer (parts/attention.py, Attention.forward): projections, q/k norm, rotation, cache write,
// attention, output projection; returns the output projection's result (partial sums where K was cut).
Tensor attention(Run& r, const QiBlock& B, const QiCall& c, const void* x) {
    const QiStep& b = *r.b;
    const QiModelDesc& m = *r.m;
    const int n = b.n_tokens, dt = m.act_dtype;
    const int* table = b.block_tables[c.group];
    const int max_blocks = b.max_blocks[c.group];
    const long long q_bytes = (long long)n * B.nq * B.d * esize(dt);
    // the two fused kernels rotate whole heads in half-split pairs; any other rule takes the stand-alone kernel
    const bool whole_head = !B.cos_t || (B.rotary_dim == B.d && !B.interleaved);
    void* kp = c.writes ? c.k_pages : nullptr;
    void* vp = c.writes ? c.v_pages : nullptr;
    if (whole_head && n > 256 && B.qkv.in_features % 8 == 0 && B.d == 128 && dt == qi::kBF16 && B.qkv.w_dtype == qi::kBF16) {
        // many tokens: norm, rotation and the cache write ride in the projection's epilogue
        void* q = r.arena.take(q_bytes);
        r.call([&] {
            return qi_gemm_bf16_qkv_rope(x, B.qkv.w, n, B.qkv.in_features, q, B.q_gain, B.k_gain, B.qk_eps, B.cos_t, B.sin_t,
                                         B.cos_t ? B.table_positions : 0, b.positions, b.token_req, table, kp ? max_blocks : 0,
                                         c.page_size, kp ? c.num_pages : 0, kp, vp, B.nq, B.nkv, m.status, r.stream);
        });
        void* out = r.arena.take(q_bytes);
        attend(r, B, c, q, out);
        return linear(r, B.o, out, dt, n, dt, true);
    }
    // K-split partial sums of the projection are added by the next kernel where it can take them
    Tensor qkv = linear(r, B.qkv, x, dt, n, dt, B.d % 4 == 0 && whole_head);
    if (b.all_decode && dt == qi::kBF16 && whole_head && (qkv.splits > 1 || qkv.dtype == qi::kBF16) &&
        qi_attention_tma_supported(B.nq, B.nkv, B.d, c.page_size, max_blocks)) {
        // one token per request: the attention kernel makes its queries and the new key and value itself
        void* out = r.arena.take(q_bytes);
        int chunk = 0, splits = 0;
        decode_plan(b.n_requests, B.nkv, b.max_kv_len, &chunk, &splits);
        const long long n_o = (long long)b.n_requests * B.nq * splits * B.d;
        float* ws = (float*)r.arena.take((n_o + (long long)b.n_requests * B.nq * splits * 2) * 4);
        r.call([&] {
            return qi_attention_decode_rope_tma(qkv.p, qkv.dtype, qkv.splits, n, B.q_gain, B.k_gain, B.qk_eps, B.cos_t, B.sin_t,
                                                B.cos_t ? B.table_positions : 0, c.writes, out, c.k_pages, c.v_pages, table,
                                                max_blocks, c.page_size, c.num_pages, b.kv_len, b.q_start, b.n_requests, B.nq,
                                                B.nkv, B.d, B.scale, B.window, chunk, splits, ws, ws + n_o, m.status, r.stream);
        });
        return linear(r, B.o, out, dt, n, dt, true);
    }
    void* q = r.arena.take(q_bytes);
    r.call([&] {
        return qi_qk_norm_rope_kv(qkv.p, qkv.splits, q, dt, B.q_gain, B.k_gain, B.qk_eps, B.cos_t, B.sin_t,
                                  B.cos_t ? B.rotary_dim : 0, B.interleaved, B.cos_t ? B.table_positions : 0, b.positions,
                                  b.token_req, table, kp ? max_blocks : 0, c.page_size, kp ? c.num_pages : 0, kp, vp, n, B.nq,
                                  B.nkv, B.d, m.status, r.stream);
    });
    void* out = r.arena.take(q_bytes);
    attend(r, B, c, q, out);
    return linear(r, B.o, out, dt, n, dt, true);
}

// The whole pass. `logits`: float32 [n_logit_rows, vocab]. Temporaries of a layer are given back when
// the layer is done; what crosses layers (the residual stream and the last part's output, which the
// next norm adds) lives at the front of the workspace, the output in two places used in turn.
void forward(Run& r, float* logits) {
    const QiModelDesc& m = *r.m;
    const QiStep& b = *r.b;
    const int n = b.n_tokens, h = m.hidden, dt = m.act_dtype;
    float* resid = (float*)r.arena.take((long long)n * h * 4);
    r.call([&] { return qi_embedding(m.embedding, m.embedding_dtype, b.token_ids, resid, n, h, m.vocab, m.status, r.stream); });
    // room for a feed-forward's output: its whole sum in the activation type or up to 16 partial sums
    const long long delta_bytes = (long long)16 * n * h * 4;
    void* delta_room[2] = {r.arena.take(delta_bytes), r.arena.take(delta_bytes)};
    const long long layer_base = r.arena.off;
    Tensor delta = {nullptr, dt, 1};
    bool have_delta = false;
    for (int i = 0; i < m.n_calls; ++i) {
        const QiCall& c = m.calls[i];
        const QiBlock& B = m.blocks[c.block];
        r.arena.off = layer_base;
        void* x = add_norm(r, resid, have_delta ? &delta : nullptr, B.norm1_gain, B.norm1_eps, nullptr, n, n);
        Tensor a = attention(r, B, c, x);
        void* x2 = add_norm(r, resid, &a, B.norm2_gain, B.norm2_eps, nullptr, n, n);
        void* act = linear_act_mul(r, B.gate_up, x2, dt, n, B.activation);
        // the down projection writes into this layer's place for what crosses to the next layer
        QiLinear down = B.down;
        const long long keep = r.arena.off;
        Arena saved = r.arena;
        r.arena.base = r.arena.dry ? nullptr : (uint8_t*)delta_room[i & 1];
        r.arena.off = 0;
        r.arena.size = delta_bytes;
        delta = linear(r, down, act, dt, n, dt, true);
        const long long used = r.arena.off;
        r.arena = saved;
        r.arena.off = keep;
        if (used > delta_bytes) r.failed = 1;      // cannot happen: at most 16 splits, or one whole sum
        have_delta = true;
    }
    if (b.n_logit_rows == 0) return;
    r.arena.off = layer_base;
    void* normed = add_norm(r, resid, have_delta ? &delta : nullptr, m.final_gain, m.final_eps, b.logit_rows, b.n_logit_rows, n);
    linear(r, m.head, normed, dt, b.n_logit_rows, qi::kF32, false, logits);
}

}  // namespace

namespace {

int check_desc(const QiModelDesc* m, const QiStep* b) {
    QI_REQUIRE(m && b, "forward: the model or the step is missing");
    QI_REQUIRE(m->n_blocks > 0 && m->n_calls > 0 && m->blocks && m->calls, "forward: a model needs blocks and a run order");
    QI_REQUIRE(m->act_dtype == qi::kF32 || m->act_dtype == qi::kBF16, "forward: unknown activation type %d", m->act_dtype);
    QI_REQUIRE(m->hidden > 0 && m->vocab > 0 && m->embedding && m->final_gain && m->head.w && m->status, "forward: the model is incomplete");
    QI_REQUIRE(b->n_tokens > 0 && b->n_requests > 0 && b->n_logit_rows >= 0, "forward: bad counts (%d tokens, %d requests, %d rows)",
               b->n_tokens, b->n_requests, b->n_logit_rows);
    for (int i = 0; i < m->n_calls; ++i) {
        const QiCall& c = m->calls[i];
        QI_REQUIRE(c.block >= 0 && c.block < m->n_blocks, "forward: run order entry %d names block %d of %d", i, c.block, m->n_blocks);
        QI_REQUIRE(c.group >= 0 && c.group < kMaxGroups && b->block_tables[c.group] && b->max_blocks[c.group] > 0,
                   "forward: run order entry %d uses block table %d, which the step does not bring", i, c.group);
        QI_REQUIRE(c.k_pages && c.v_pages && c.page_size > 0 && c.num_pages > 0, "forward: run order entry %d has no cache pages", i);
    }
    return 0;
}

}  // namespace

// Bytes of workspace that qi_forward needs for this step (a walk over the same path that launches nothing).
extern "C" long long qi_forward_workspace_bytes(const QiModelDesc* m, const QiStep* b) {
    if (check_desc(m, b)) return -1;
    Run r = {m, b, Arena{nullptr, 0, 0, 0, true}, nullptr, 0, 0};
    forward(r, nullptr);
    return r.failed ? -1 : r.arena.peak + 256;
}

// Runs the step. `logits`: float32 [n_logit_rows, vocab] (may be null when no row is wanted). `launches`
// receives the number of entry points that launched. Returns non-zero, with a message for
// qi_last_error, as soon as an entry point refuses; nothing after it is launched.
extern "C" int qi_forward(const QiModelDesc* m, const QiStep* b, void* workspace, long long workspace_bytes, float* logits,
                          int* launches, cudaStream_t stream) {
    if (check_desc(m, b)) return 1;
    QI_REQUIRE(workspace && ((uintptr_t)workspace & 255) == 0, "forward: the workspace must be 256-byte aligned");
    QI_REQUIRE(b->n_logit_rows == 0 || logits, "forward: %d rows are wanted and there is no place for them", b->n_logit_rows);
    const long long need = qi_forward_workspace_bytes(m, b);
    QI_REQUIRE(need >= 0 && need <= workspace_bytes, "forward: the step needs %lld bytes of workspace, %lld were given", need, workspace_bytes);
    Run r = {m, b, Arena{(uint8_t*)workspace, workspace_bytes, 0, 0, false}, stream, 0, 0};
    forward(r, logits);
    if (launches) *launches = r.launches;
    return r.failed;
}
