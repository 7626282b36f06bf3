"""A plain, slow implementation of Qwen3 dense on the CPU: whole sequences, no
cache, one function per part. It is the yardstick the engine is compared with
and shares no code with it: it reads config.json as a dictionary and the
weights through the `safetensors` package.

It rests on the reference's formulas, not on running the reference: the
reference is a Rust workspace and neither `cargo` nor `rustc` exists here, so
its model code cannot be compiled or imported; there is therefore no golden
output from it. Each function cites the file:line it restates; the two literal
test vectors the reference's own unit tests give (a rotation and a matrix
product) are checked in tests/test_plain.py.

Arithmetic is float32 by default, like the reference (every tensor there is
f32); `dtype=torch.float64` gives a higher-precision answer to judge which of
two float32 results is nearer the truth.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


# ---------------------------------------------------------------- parts


def plain_embedding(table: torch.Tensor, ids) -> torch.Tensor:
    """Row gather; an id outside the table is an error.
    backends/cpu/src/backend.rs:282-298."""
    vocab = table.shape[0]
    for i in ids:
        if not 0 <= int(i) < vocab:
            raise ValueError(f"token id {i} is outside vocabulary size {vocab}")
    return torch.stack([table[int(i)] for i in ids])


def plain_rms_norm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """mean square over the last dim; inverse = 1/sqrt(ms + eps); y = x * inverse * gain.
    backends/cpu/src/backend.rs:172-193 (mean square :185-186, inverse :187, output :189)."""
    ms = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    inverse = 1.0 / torch.sqrt(ms + torch.tensor(eps, dtype=x.dtype))
    return x * inverse * gain


def plain_linear(x: torch.Tensor, w_out_in: torch.Tensor) -> torch.Tensor:
    """out[c] = sum_k x[k] * W[k, c] with W = checkpoint weight transposed.
    backends/cpu/src/matmul.rs:50-59; the transpose of the checkpoint's [out, in]
    layout is crates/quantinfer-format/src/dense.rs:80-106."""
    return x @ w_out_in.t()


_rope_rows = {}   # (theta, head_dim, dtype) -> {position: (cos row, sin row)}: a row depends on nothing else


def plain_rope_tables(theta: float, head_dim: int, positions, dtype=torch.float32):
    """exponent = 2p / d; angle = position * theta^(-exponent); cos and sin; all in `dtype`.
    crates/quantinfer-runtime/src/attention.rs:7-36 (the three lines :29-32). Rows are kept
    between calls (every layer and every request asks for the same ones)."""
    rows = _rope_rows.setdefault((float(theta), int(head_dim), dtype), {})
    missing = [p for p in positions if p not in rows]
    if missing:
        cos, sin = _plain_rope_rows(theta, head_dim, missing, dtype)
        for i, p in enumerate(missing):
            rows[p] = (cos[i], sin[i])
    return torch.stack([rows[p][0] for p in positions]), torch.stack([rows[p][1] for p in positions])


def _plain_rope_rows(theta: float, head_dim: int, positions, dtype):
    pairs = head_dim // 2
    cos = torch.empty((len(positions), pairs), dtype=dtype)
    sin = torch.empty((len(positions), pairs), dtype=dtype)
    th = torch.tensor(theta, dtype=dtype)
    for r, position in enumerate(positions):
        for p in range(pairs):
            exponent = torch.tensor(2.0 * p, dtype=dtype) / torch.tensor(float(head_dim), dtype=dtype)
            angle = torch.tensor(float(position), dtype=dtype) * torch.pow(th, -exponent)
            cos[r, p] = torch.cos(angle)
            sin[r, p] = torch.sin(angle)
    return cos, sin


def plain_apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [tokens, heads, d]; pairs (p, p + d/2): first*cos - second*sin, first*sin + second*cos.
    backends/cpu/src/backend.rs:240-280 (the rotation :270-275)."""
    half = x.shape[-1] // 2
    first, second = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([first * c - second * s, first * s + second * c], dim=-1)


def plain_gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window=None) -> torch.Tensor:
    """q [T, nq, d], k and v [T, nkv, d] of one whole sequence from position 0.
    For each token and query head: scores over keys 0..t (inclusive), times
    1/sqrt(d) after the dot product, softmax with the maximum subtracted,
    weighted sum of values in key order. Query head h uses kv head h // (nq // nkv).
    crates/quantinfer-runtime/src/attention.rs:39-141 (group :83, scale :84,
    bound :106,111, score :113-118, max :121, denominator :122-125, weight :128,
    sum :130-133). `window` (not in the reference, which rejects it) limits the
    keys to the last `window` positions."""
    T, nq, d = q.shape
    nkv = k.shape[1]
    group = nq // nkv
    scale = 1.0 / math.sqrt(d) if q.dtype == torch.float64 else float(torch.tensor(float(d), dtype=q.dtype).sqrt().reciprocal())
    out = torch.zeros_like(q)
    for t in range(T):
        lo = 0 if window is None else max(0, t - window + 1)
        for h in range(nq):
            hk = h // group
            scores = (k[lo:t + 1, hk, :] @ q[t, h, :]) * scale
            m = scores.max()
            e = torch.exp(scores - m)
            w = e / e.sum()
            out[t, h, :] = (w[:, None] * v[lo:t + 1, hk, :]).sum(dim=0)
    return out


def plain_silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """gate / (1 + exp(-gate)) * up. backends/cpu/src/backend.rs:224-238 (:235)."""
    return gate / (1.0 + torch.exp(-gate)) * up


def plain_attention_block(x, w, prefix, cfg, positions, window=None):
    """Three projections, per-head q/k norm, rotation of q and k, attention, output projection.
    crates/quantinfer-runtime/src/qwen3/mod.rs:140-192 (:158-181 projections,
    :182-183 norms, :186-191 output); crates/quantinfer-runtime/src/batch.rs:30-65."""
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    T = x.shape[0]
    q = plain_linear(x, w[prefix + "q_proj.weight"]).reshape(T, nq, d)
    k = plain_linear(x, w[prefix + "k_proj.weight"]).reshape(T, nkv, d)
    v = plain_linear(x, w[prefix + "v_proj.weight"]).reshape(T, nkv, d)
    q = plain_rms_norm(q, w[prefix + "q_norm.weight"], cfg["rms_norm_eps"])
    k = plain_rms_norm(k, w[prefix + "k_norm.weight"], cfg["rms_norm_eps"])
    cos, sin = plain_rope_tables(cfg["rope_theta"], d, positions, dtype=x.dtype)
    q, k = plain_apply_rope(q, cos, sin), plain_apply_rope(k, cos, sin)
    a = plain_gqa_attention(q, k, v, window).reshape(T, nq * d)
    return plain_linear(a, w[prefix + "o_proj.weight"])


def plain_feed_forward(x, w, prefix):
    """down(silu(gate(x)) * up(x)). crates/quantinfer-runtime/src/qwen3/mod.rs:194-209."""
    g = plain_linear(x, w[prefix + "gate_proj.weight"])
    u = plain_linear(x, w[prefix + "up_proj.weight"])
    return plain_linear(plain_silu_mul(g, u), w[prefix + "down_proj.weight"])


def plain_decoder_layer(h, w, i, cfg, positions):
    """residual; norm; attention; add; norm; feed-forward; add.
    crates/quantinfer-runtime/src/qwen3/mod.rs:117-138."""
    p = f"model.layers.{i}."
    n = plain_rms_norm(h, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
    h = h + plain_attention_block(n, w, p + "self_attn.", cfg, positions)
    n = plain_rms_norm(h, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
    return h + plain_feed_forward(n, w, p + "mlp.")


def plain_forward(w: dict, cfg: dict, ids) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence. Embedding, layers, final norm, head
    (the embedding table when tied). crates/quantinfer-runtime/src/qwen3/mod.rs:345-378;
    tied head crates/quantinfer-runtime/src/qwen3/loader.rs:59."""
    h = plain_embedding(w["model.embed_tokens.weight"], ids)
    positions = list(range(len(ids)))
    for i in range(cfg["num_hidden_layers"]):
        h = plain_decoder_layer(h, w, i, cfg, positions)
    h = plain_rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return plain_linear(h, head)


# ---------------------------------------------------------------- loading


def plain_load(folder, dtype=torch.float32):
    """config.json as a dictionary (defaults filled as the reference does,
    crates/quantinfer-model/src/qwen3.rs:39-55) and the weights widened to `dtype`."""
    from safetensors.torch import load_file

    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    cfg.setdefault("rms_norm_eps", 1e-6)
    cfg.setdefault("rope_theta", 1_000_000.0)
    if cfg.get("head_dim") is None:
        cfg["head_dim"] = cfg["hidden_size"] // cfg["num_attention_heads"]
    w = {k: v.to(dtype) for k, v in load_file(str(folder / "model.safetensors")).items()}
    return cfg, w


# ---------------------------------------------------------------- sampling


def plain_argmax(logits) -> int:
    """First maximum: strict >, so the lowest index wins ties.
    crates/quantinfer-runtime/src/generation.rs:58-77."""
    best = 0
    for i in range(1, len(logits)):
        if logits[i] > logits[best]:
            best = i
    return best


_M0, _M1, _W0, _W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
_MASK = 0xFFFFFFFF


def plain_philox4x32_10(counter, key):
    """Philox-4x32 with 10 rounds (Salmon et al., 'Parallel random numbers: as easy as 1, 2, 3')."""
    c = list(counter)
    k = list(key)
    for r in range(10):
        if r > 0:
            k[0] = (k[0] + _W0) & _MASK
            k[1] = (k[1] + _W1) & _MASK
        p0, p1 = _M0 * c[0], _M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k[0]) & _MASK, p1 & _MASK, ((p0 >> 32) ^ c[3] ^ k[1]) & _MASK, p0 & _MASK]
    return c


def plain_uniform(seed: int, counter: int) -> float:
    """The engine's draw: Philox keyed by the 64-bit seed, counter = tokens emitted so far;
    the top 24 bits of the first word give a float32 in [0, 1)."""
    out = plain_philox4x32_10((counter & _MASK, 0, 0, 0), (seed & _MASK, (seed >> 32) & _MASK))
    return (out[0] >> 8) / 16777216.0


def plain_sample(logits, temperature: float, top_k=None, top_p=None, seed: int = 0, counter: int = 0) -> int:
    """Candidate rule of crates/quantinfer-runtime/src/generation.rs:79-155: greedy when
    temperature is 0; else scale by 1/temperature, sort descending (stable), keep
    top_k, keep the shortest prefix whose share of the kept mass reaches top_p,
    and draw. The draw differs from the reference on purpose (see the engine's
    sampling kernel): the uniform is `plain_uniform(seed, counter)` and the
    inverse CDF runs over the kept candidates in index order. Scaled logits and
    weights are float32, sums float64, like the kernel."""
    x = torch.as_tensor(logits, dtype=torch.float32)
    if not torch.isfinite(x).all():
        raise ValueError("logits must contain only finite values")
    if temperature == 0.0:
        return plain_argmax(x.tolist())
    y = x / torch.tensor(temperature, dtype=torch.float32)
    wts = torch.exp(y - y.max()).to(torch.float64)
    order = sorted(range(len(y)), key=lambda i: -float(y[i]))  # stable: ties keep index order
    if top_k is not None:
        order = order[:min(top_k, len(order))]
    if top_p is not None and top_p < 1.0:
        total = float(sum(wts[i] for i in order))
        need = float(torch.tensor(top_p, dtype=torch.float32)) * total
        cum, kept = 0.0, 0
        for i in order:
            cum += float(wts[i])
            kept += 1
            if cum >= need:
                break
        order = order[:max(kept, 1)]
    kept_sorted = sorted(order)
    total = float(sum(wts[i] for i in kept_sorted))
    target = plain_uniform(seed, counter) * total
    cum = 0.0
    for i in kept_sorted:
        cum += float(wts[i])
        if target <= cum:
            return i
    return kept_sorted[-1]


def plain_generate(w, cfg, prompt, max_new_tokens, temperature=0.0, top_k=None, top_p=None, seed=0, eos=None):
    """Whole-sequence recompute per token (no cache); stops after emitting `eos`.
    The loop is crates/quantinfer-runtime/src/session.rs:136-164."""
    ids = list(prompt)
    out = []
    for n in range(max_new_tokens):
        logits = plain_forward(w, cfg, ids)[-1]
        t = plain_sample(logits, temperature, top_k, top_p, seed, counter=n)
        out.append(t)
        ids.append(t)
        if eos is not None and t == eos:
            break
    return out
