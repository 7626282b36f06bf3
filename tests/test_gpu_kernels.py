"""Each kernel alone against a plain float32/float64 reference of the same operation, at
sizes other than the engine's: widths that are no power of two, odd row counts, head
sizes in steps of 16, several page sizes. Inputs are built so that faults show: a far
key that dominates a softmax, a window's edge, values in unused pages that would
poison a result if read."""


import pytest
import torch

from kernel_refs import build_pages, ref_paged_attention
from plain.plain_qwen3 import plain_sample

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _k():
    from quantinfer_b200 import kernels
    return kernels


def _status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def I(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


# ------------------------------------------------------------------ embedding, norms

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("vocab, hidden", [(37, 20), (300, 168), (1000, 4096)])
def test_embedding(dtype, vocab, hidden):
    torch.manual_seed(0)
    table = torch.randn(vocab, hidden).to(dtype).to(DEV)
    ids = torch.randint(0, vocab, (13,), dtype=torch.int32)
    out = torch.empty(13, hidden, dtype=torch.float32, device=DEV)
    st = _status()
    _k().embedding(table, ids.to(DEV), out, st)
    assert torch.equal(out.cpu(), table.float().cpu()[ids.long()]) and st.item() == 0
    bad = ids.clone()
    bad[3] = vocab
    _k().embedding(table, bad.to(DEV), out, st)
    assert st.item() == _k().STATUS_BAD_TOKEN and float(out[3].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows, hidden", [(1, 20), (7, 168), (5, 4096), (3, 1000)])
def test_add_rmsnorm(dtype, rows, hidden):
    torch.manual_seed(1)
    resid = torch.randn(rows, hidden)
    delta = torch.randn(rows, hidden).to(dtype)
    gain = 1 + 0.1 * torch.randn(hidden)
    eps = 3e-6
    x = resid.double() + delta.double()
    ref = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * gain.double()
    r = resid.to(DEV)
    out = torch.empty(rows, hidden, dtype=dtype, device=DEV)
    _k().add_rmsnorm(r, delta.to(DEV), gain.to(DEV), eps, out)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert float((out.double().cpu() - ref).abs().max()) < tol
    assert float((r.double().cpu() - x).abs().max()) < 1e-6           # the residual stream was updated
    # no delta, row gather, residual untouched
    r2 = resid.to(DEV)
    pick = I([rows - 1, 0])
    out2 = torch.empty(2, hidden, dtype=dtype, device=DEV)
    _k().add_rmsnorm(r2, None, gain.to(DEV), eps, out2, rows=pick)
    x2 = resid.double()[[rows - 1, 0]]
    ref2 = x2 * torch.rsqrt((x2 * x2).mean(-1, keepdim=True) + eps) * gain.double()
    assert float((out2.double().cpu() - ref2).abs().max()) < tol and torch.equal(r2.cpu(), resid)


@pytest.mark.parametrize("rows, hidden, splits", [
    (6, 264, 3),          # one CTA a row
    (8, 4096, 8),         # few rows of a wide model: a row over a cluster of four CTAs, all partial sums at once
    (64, 1024, 2),        # the most rows and the narrowest rows that take the clusters
    (3, 5120, 16),        # more partial sums than are requested at once
    (65, 4096, 4),        # one row too many for the clusters
    (1500, 2048, 2),      # more rows than CTAs that stay: each walks several rows
])
def test_add_rmsnorm_takes_split_partials(rows, hidden, splits):
    torch.manual_seed(2)
    resid, parts = torch.randn(rows, hidden), torch.randn(splits, rows, hidden)
    gain = 1 + 0.1 * torch.randn(hidden)
    x = resid.double() + parts.double().sum(0)
    ref = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-6) * gain.double()
    out = torch.empty(rows, hidden, dtype=torch.bfloat16, device=DEV)
    r = resid.to(DEV)
    _k().add_rmsnorm(r, parts.to(DEV), gain.to(DEV), 1e-6, out)
    assert float((out.double().cpu() - ref).abs().max()) < 3e-2 and float((r.double().cpu() - x).abs().max()) < 1e-5
    # the same sums for picked rows only (what the head's norm does): the residual stays as it was
    r2 = resid.to(DEV)
    pick = [rows - 1, 0]
    out2 = torch.empty(2, hidden, dtype=torch.float32, device=DEV)
    _k().add_rmsnorm(r2, parts.to(DEV), gain.to(DEV), 1e-6, out2, rows=I(pick))
    assert float((out2.double().cpu() - ref[pick]).abs().max()) < 2e-5 and torch.equal(r2.cpu(), resid)


# ------------------------------------------------------------------ matrix products

@pytest.mark.parametrize("tx, tw, ty", [(torch.float32,) * 3, (torch.bfloat16,) * 3,
                                        (torch.bfloat16, torch.float32, torch.bfloat16),
                                        (torch.bfloat16, torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("M, N, K", [(1, 7, 5), (65, 130, 33), (200, 517, 168)])
def test_gemm_simt(tx, tw, ty, M, N, K):
    torch.manual_seed(3)
    x, w = torch.randn(M, K).to(tx), torch.randn(N, K).to(tw)
    out = torch.empty(M, N, dtype=ty, device=DEV)
    _k().gemm_simt(x.to(DEV), w.to(DEV), out)
    ref = x.double() @ w.double().t()
    tol = 1e-4 if ty == torch.float32 else 0.15
    assert float((out.double().cpu() - ref).abs().max()) < tol


@pytest.mark.parametrize("M, N, K, plan", [
    (128, 128, 64, (False, 128, 1)), (100, 72, 136, (False, 64, 1)), (300, 520, 264, None),
    (4, 128, 64, (True, 16, 1)), (1, 384, 96, None), (33, 517, 168, (True, 64, 2)),
    (64, 1000, 2048, None), (200, 300, 4096, None), (700, 328, 168, (False, 256, 1)), (17, 264, 1032, (True, 32, 4)),
    # pairs of CTAs on tiles of 256 x 256: one tile, ragged edges in both directions, many k blocks, more tiles than pairs
    (256, 256, 64, (2, 256, 1)), (300, 400, 136, (2, 256, 1)), (129, 130, 1032, (2, 256, 1)), (2560, 2304, 320, (2, 256, 1)),
    (512, 300, 2048, (2, 256, 3)), (700, 1100, 1600, (2, 256, 2)),      # the same with K split: partial sums, then added
])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_tcgen05(M, N, K, plan, out_dtype):
    torch.manual_seed(4)
    x, w = (torch.randn(M, K) * 0.5).bfloat16(), (torch.randn(N, K) * 0.5).bfloat16()
    out = torch.full((M, N), 7.0, dtype=out_dtype, device=DEV)
    st = _status()
    _k().gemm_bf16(x.to(DEV), w.to(DEV), out, plan=plan, status=st)
    ref = x.double() @ w.double().t()
    err = float((out.double().cpu() - ref).abs().max())
    scale = float(ref.abs().max())
    assert st.item() == 0
    assert err < (2e-4 if out_dtype == torch.float32 else scale * 2 ** -7), (err, scale)


@pytest.mark.parametrize("M, N, K", [(5, 256, 136), (130, 328, 264), (64, 4096, 512)])
def test_gemm_tcgen05_silu_epilogue_and_partials(M, N, K):
    torch.manual_seed(5)
    x, w = (torch.randn(M, K) * 0.3).bfloat16(), (torch.randn(N, K) * 0.3).bfloat16()
    act = torch.empty(M, N // 2, dtype=torch.bfloat16, device=DEV)
    _k().gemm_bf16(x.to(DEV), w.to(DEV), act, epilogue="silu_mul")
    y = x.double() @ w.double().t()
    g, u = y[:, 0::2], y[:, 1::2]
    ref = g / (1 + torch.exp(-g)) * u
    assert float((act.double().cpu() - ref).abs().max()) < max(0.05, float(ref.abs().max()) * 2 ** -7)
    parts = _k().gemm_bf16(x.to(DEV), w.to(DEV), None, plan=(True if M <= 256 else False, 16 if M <= 16 else 256 if M > 64 else 64, 2),
                           keep_partials=True)
    assert parts.shape == (2, M, N) and float((parts.double().sum(0).cpu() - y).abs().max()) < 2e-4
    parts = _k().gemm_bf16(x.to(DEV), w.to(DEV), None, plan=(2, 256, 2), keep_partials=True)     # on pairs of CTAs
    assert parts.shape == (2, M, N) and float((parts.double().sum(0).cpu() - y).abs().max()) < 2e-4
    # the same activation from the kernel that runs on pairs of CTAs
    act2 = torch.empty_like(act)
    _k().gemm_bf16(x.to(DEV), w.to(DEV), act2, plan=(2, 256, 1), epilogue="silu_mul")
    assert float((act2.double().cpu() - ref).abs().max()) < max(0.05, float(ref.abs().max()) * 2 ** -7)


def test_gemm_plan_takes_cta_pairs_for_many_tokens():
    k = _k()
    assert k.gemm_bf16_plan(2048, 4096, 4096)[0] == 2 and k.gemm_bf16_plan(2048, 24576, 4096, allow_split=False)[0] == 2
    assert k.gemm_bf16_plan(8, 4096, 4096)[0] == 1 and k.gemm_bf16_plan(64, 24576, 4096)[0] == 1


# ------------------------------------------------------------------ q/k norm, rotation, cache write

@pytest.mark.parametrize("M, K, nq, nkv, ps, norm, rope, write", [
    (300, 64, 2, 1, 16, True, True, True),      # 4 heads: two tiles of 256 columns; a ragged last row tile
    (257, 136, 3, 1, 8, True, True, True),      # 5 heads: the last tile is half empty; K no multiple of 64
    (513, 256, 1, 1, 64, False, True, True),    # 3 heads: one tile of 256 and a half; no norm
    (384, 72, 1, 2, 32, True, False, True),     # no rotation
    (260, 64, 2, 1, 16, True, True, False),     # reads another layer's cache: queries only
    (1300, 64, 12, 4, 16, True, True, True),    # 20 heads, many tokens: the kernel on pairs of CTAs
    (1100, 136, 9, 3, 64, True, True, True),    # 15 heads: the pair's last tile holds one head only
])
def test_gemm_qkv_rope(M, K, nq, nkv, ps, norm, rope, write):
    """The q/k/v projection with norm, rotation and cache write in its epilogue, against a 64-bit
    product followed by the formulas; heads that straddle tile borders, rows past the last token."""
    torch.manual_seed(M + K)
    d, eps, theta, max_pos = 128, 1e-5, 1e4, 1400
    k = _k()
    assert k.gemm_qkv_rope_supported(M, K, d, d if rope else 0, torch.bfloat16, torch.bfloat16)
    assert not k.gemm_qkv_rope_supported(200, K, d, d, torch.bfloat16, torch.bfloat16)
    assert not k.gemm_qkv_rope_supported(M, K, 64, 64, torch.bfloat16, torch.bfloat16)
    x = torch.randn(M, K).bfloat16()
    w = (torch.randn((nq + 2 * nkv) * d, K) / K ** 0.5).bfloat16()
    qg, kg = (1 + 0.1 * torch.randn(d), 1 + 0.1 * torch.randn(d)) if norm else (None, None)
    inv_freq = torch.pow(torch.tensor(theta), -(2.0 * torch.arange(d // 2)) / d)
    cos, sin = k.rope_table(inv_freq.to(DEV), max_pos) if rope else (None, None)
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv_freq.double()[None, :]
    # two requests: the first holds 40 earlier positions, the second starts at 0
    n0 = M // 3
    positions = list(range(40, 40 + n0)) + list(range(0, M - n0))
    token_req = [0] * n0 + [1] * (M - n0)
    max_blocks = -(-max_pos // ps)
    num_pages = 2 * max_blocks + 3
    perm = torch.randperm(num_pages).tolist()
    table = torch.tensor([[perm.pop() for _ in range(max_blocks)] for _ in range(2)], dtype=torch.int32)
    kp = torch.zeros(num_pages, nkv, ps, d, dtype=torch.bfloat16, device=DEV)
    vp = torch.zeros_like(kp)
    q_out = torch.empty(M, nq * d, dtype=torch.bfloat16, device=DEV)
    st = _status()
    k.gemm_qkv_rope(x.to(DEV), w.to(DEV), q_out, qg.to(DEV) if norm else None, kg.to(DEV) if norm else None, eps, cos, sin,
                    I(positions), I(token_req), table.to(DEV), ps, kp if write else None, vp if write else None, nq, nkv, st)
    assert st.item() == 0
    y = (x.double() @ w.double().T).reshape(M, nq + 2 * nkv, d)

    def norm_rot(h, gain, pos):
        if gain is not None:
            h = h * torch.rsqrt((h * h).mean(-1, keepdim=True) + eps) * gain.double()
        if not rope:
            return h
        c, s = torch.cos(ang[pos])[:, None, :], torch.sin(ang[pos])[:, None, :]
        a, b = h[..., :d // 2], h[..., d // 2:]
        return torch.cat([a * c - b * s, a * s + b * c], dim=-1)

    pos_t = torch.tensor(positions)
    ref_q = norm_rot(y[:, :nq], qg, pos_t)
    ref_k = norm_rot(y[:, nq:nq + nkv], kg, pos_t)
    ref_v = y[:, nq + nkv:]
    tol = 2e-2    # bfloat16 output of values up to about 4
    assert float((q_out.double().cpu().reshape(M, nq, d) - ref_q).abs().max()) < tol
    if not write:
        assert float(kp.abs().sum()) == 0 and float(vp.abs().sum()) == 0
        return
    pages = table[torch.tensor(token_req), pos_t // ps].long()
    rows = pos_t % ps
    assert float((kp.cpu()[pages, :, rows].double() - ref_k).abs().max()) < tol
    assert float((vp.cpu()[pages, :, rows].double() - ref_v).abs().max()) < tol
    assert int((kp.abs().sum(dim=(1, 3)) > 0).sum()) == M            # nothing else was touched


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq, nkv, d, rot, ps", [(4, 2, 16, 16, 4), (6, 3, 48, 48, 32), (8, 1, 128, 128, 64),
                                                (3, 3, 34, 34, 5), (4, 2, 32, 16, 8)])
def test_qk_norm_rope_kv(dtype, nq, nkv, d, rot, ps):
    torch.manual_seed(6)
    n, theta, eps = 9, 5e4, 1e-5
    positions = [3, 4, 5, 0, 17, 18, 19, 20, 63]
    token_req = [0, 0, 0, 1, 2, 2, 2, 2, 2]
    qkv = torch.randn(n, (nq + 2 * nkv) * d).to(dtype)
    qg, kg = 1 + 0.1 * torch.randn(d), 1 + 0.1 * torch.randn(d)
    inv_freq = torch.pow(torch.tensor(theta), -(2.0 * torch.arange(rot // 2)) / rot)
    cos, sin = _k().rope_table(inv_freq.to(DEV), 64)
    ang = torch.arange(64, dtype=torch.float32)[:, None] * inv_freq[None, :]
    assert float((cos.cpu() - torch.cos(ang)).abs().max()) < 2e-6 and float((sin.cpu() - torch.sin(ang)).abs().max()) < 2e-6
    max_blocks = -(-64 // ps)
    num_pages = 3 * max_blocks + 2
    table = torch.full((3, max_blocks), -1, dtype=torch.int32)
    perm = torch.randperm(num_pages).tolist()
    for r in range(3):
        for b in range(max_blocks):
            table[r, b] = perm.pop()
    kp = torch.zeros(num_pages, nkv, ps, d, dtype=dtype, device=DEV)
    vp = torch.zeros_like(kp)
    q_out = torch.empty(n, nq * d, dtype=dtype, device=DEV)
    st = _status()
    _k().qk_norm_rope_kv(qkv.to(DEV), q_out, qg.to(DEV), kg.to(DEV), eps, cos, sin, rot, I(positions), I(token_req),
                         table.to(DEV), ps, kp, vp, nq, nkv, d, st)
    assert st.item() == 0

    def norm_rot(x, gain, pos):
        x = x.double()
        x = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * gain.double()
        half = rot // 2
        c, s = torch.cos(ang[pos].double()), torch.sin(ang[pos].double())
        a, b = x[..., :half], x[..., half:rot]
        return torch.cat([a * c - b * s, a * s + b * c, x[..., rot:]], dim=-1)

    tol = 1e-5 if dtype == torch.float32 else 3e-2
    x = qkv.reshape(n, nq + 2 * nkv, d)
    for t in range(n):
        ref_q = norm_rot(x[t, :nq], qg, positions[t])
        assert float((q_out[t].double().cpu().reshape(nq, d) - ref_q).abs().max()) < tol
        page, row = int(table[token_req[t], positions[t] // ps]), positions[t] % ps
        ref_k = norm_rot(x[t, nq:nq + nkv], kg, positions[t])
        assert float((kp[page, :, row].double().cpu() - ref_k).abs().max()) < tol
        assert torch.equal(vp[page, :, row].cpu(), x[t, nq + nkv:])          # values are stored as they are
    written = {(int(table[token_req[t], positions[t] // ps]), positions[t] % ps) for t in range(n)}
    assert int((kp.abs().sum(dim=(1, 3)) > 0).sum()) == len(written)          # nothing else was touched


# ------------------------------------------------------------------ attention

def _attention_case(nq, nkv, d, ctx, new, ps, window, dtype, mode, decode_chunk=0, key_ranges=None, in_ulps=False):
    """ctx[r] cached positions and new[r] query tokens per request. One query per request
    has a far key that dominates its softmax, so a missed or misplaced key changes the result.
    Returns the largest absolute error, or with `in_ulps` the largest error in units of
    (6e-3 + half a bfloat16 step of the value), which does not grow with the value."""
    torch.manual_seed(7)
    k = _k()
    R = len(ctx)
    tot = [c + n for c, n in zip(ctx, new)]
    k_seq = [torch.randn(t, nkv, d).to(dtype).float() for t in tot]
    v_seq = [torch.randn(t, nkv, d).to(dtype).float() for t in tot]
    n = sum(new)
    q = (torch.randn(n, nq * d) * 1.5).to(dtype).float()
    positions, token_req, q_start = [], [], [0]
    for r in range(R):
        positions += list(range(ctx[r], tot[r]))
        token_req += [r] * new[r]
        q_start.append(q_start[-1] + new[r])
    for r in range(R):
        t = q_start[r + 1] - 1
        far = max(0, tot[r] - window) if window else min(1, tot[r] - 1)   # the window's far edge, or nearly the first key
        q[t, :d] = 0
        q[t, 0] = 8.0
        k_seq[r][far, 0, :] = 0
        k_seq[r][far, 0, 0] = 8.0
    num_pages = sum(-(-t // ps) for t in tot) + 3
    kp, vp, table = build_pages(k_seq, v_seq, ps, num_pages, nkv, d, dtype, DEV)
    scale = d ** -0.5
    ref = ref_paged_attention(q, k_seq, v_seq, positions, token_req, nq, nkv, d, scale, window)
    qd = q.to(dtype).to(DEV)
    out = torch.zeros_like(qd)
    st = _status()
    if mode == "generic":
        k.attention_generic(qd, out, kp, vp, table, I(positions), I(token_req), nq, nkv, d, scale, window, st)
    elif mode.startswith("decode"):
        chunk, splits = k.attention_decode_plan(R, nkv, max(tot) + 70)
        if decode_chunk:
            chunk, splits = decode_chunk, -(-(max(tot) + 70) // decode_chunk)
        k.attention_decode(qd, out, kp, vp, table, I(tot), I(q_start), nq, nkv, d, scale, window, chunk, splits, st,
                           use_tma=mode.endswith("tma"))
    else:
        tiles = [(r, q_start[r] + t0) for r in range(R) for t0 in range(0, new[r], k.QUERY_TILE)]
        impl = {"prefill": "cpasync", "prefill_tma": "tma", "prefill_tcgen05": "tcgen05"}[mode]
        k.attention_prefill(qd, out, kp, vp, table, I(q_start), I(ctx), I([t[0] for t in tiles]),
                            I([t[1] for t in tiles]), nq, nkv, d, scale, window, st, impl=impl, key_ranges=key_ranges)
    assert st.item() == 0
    err = (out.double().cpu() - ref).abs()
    if in_ulps:
        return float((err / (6e-3 + ref.abs() * 2.0 ** -8)).max())
    return float(err.max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq, nkv, d, ctx, new, ps, window", [
    (4, 2, 16, [0, 5], [33, 1], 4, 0), (6, 3, 48, [40, 0], [7, 100], 32, 0), (8, 1, 32, [300], [3], 8, 0),
    (4, 4, 80, [0], [70], 16, 0), (8, 2, 128, [200, 0], [2, 130], 64, 0), (2, 1, 256, [30], [10], 16, 0),
    (6, 3, 64, [40, 0], [90, 150], 32, 50), (4, 2, 16, [100], [1], 7, 9),
])
def test_attention_generic(dtype, nq, nkv, d, ctx, new, ps, window):
    err = _attention_case(nq, nkv, d, ctx, new, ps, window, dtype, "generic")
    assert err < (2e-5 if dtype == torch.float32 else 1.2e-2)


@pytest.mark.parametrize("mode", ["prefill", "prefill_tma"])
@pytest.mark.parametrize("nq, nkv, d, ctx, new, ps, window", [
    (4, 2, 64, [0], [64], 16, 0), (4, 2, 64, [0, 0], [100, 3], 16, 0), (8, 2, 128, [0, 37, 200], [130, 64, 1], 64, 0),
    (8, 1, 128, [5, 300], [70, 2], 8, 0), (6, 3, 64, [40, 0], [90, 150], 32, 50), (8, 2, 128, [100, 0], [300, 257], 128, 0),
    (16, 1, 64, [129], [127], 32, 0),
])
def test_attention_prefill_kernels(mode, nq, nkv, d, ctx, new, ps, window):
    assert _attention_case(nq, nkv, d, ctx, new, ps, window, torch.bfloat16, mode) < 1.2e-2


@pytest.mark.parametrize("nq, nkv, ctx, new, ps, window", [
    (8, 2, [0], [128], 64, 0), (8, 2, [0], [17], 64, 0), (8, 2, [0, 37, 200], [130, 64, 1], 64, 0), (8, 1, [5, 300], [70, 2], 8, 0),
    (8, 2, [100, 0], [300, 257], 128, 0), (4, 4, [40, 0], [90, 150], 32, 50), (32, 8, [0], [1024], 64, 0), (2, 1, [700], [129], 16, 100),
])
def test_attention_prefill_tcgen05(nq, nkv, ctx, new, ps, window):
    """The tensor-memory kernel (head size 128): spans that end inside a tile, several requests, page
    pieces smaller and larger than a tile, a window, an odd number of key tiles (the two softmax groups
    then hold different numbers of tiles)."""
    assert _attention_case(nq, nkv, 128, ctx, new, ps, window, torch.bfloat16, "prefill_tcgen05") < 1.2e-2


@pytest.mark.parametrize("ranges, ctx, new, ps, window", [
    (2, [0], [300], 64, 0), (3, [1000, 0], [130, 257], 64, 0), (4, [40], [64], 16, 0),   # the last: more ranges than key tiles
    (8, [2100], [200], 128, 0), (3, [700], [129], 32, 500), (2, [0, 37, 200], [130, 64, 1], 8, 0),
])
def test_attention_prefill_tcgen05_key_ranges(ranges, ctx, new, ps, window):
    """The keys of every query tile cut into ranges over separate CTAs and merged by a second kernel:
    ranges that are empty for short rows, a window that leaves the first ranges without keys."""
    assert _attention_case(8, 2, 128, ctx, new, ps, window, torch.bfloat16, "prefill_tcgen05", key_ranges=ranges) < 1.2e-2
    k = _k()
    # a launch that fills its rounds stays whole; one of few CTAs and many keys is cut
    assert k.attention_prefill_ranges(512, 2048) == 1 and k.attention_prefill_ranges(512, 8192) == 1 and k.attention_prefill_ranges(512, 32768) == 1
    assert k.attention_prefill_ranges(296, 30000) == 1
    assert k.attention_prefill_ranges(128, 2560) == 1 and k.attention_prefill_ranges(128, 6656) == 2 and k.attention_prefill_ranges(128, 31232) == 2
    assert k.attention_prefill_ranges(32, 32768) == 8


@pytest.mark.parametrize("seed", [11, 12])
def test_attention_prefill_tcgen05_random_cases(seed):
    """Twenty drawn cases a seed: heads and groups, several requests with and without earlier
    context, spans of one token to several query tiles, every page size, windows, key ranges."""
    import random

    rng = random.Random(seed)
    for case in range(20):
        nkv = rng.choice([1, 2, 4, 8])
        nq = nkv * rng.choice([1, 2, 4, 5, 8])
        n_req = rng.choice([1, 1, 2, 3, 4])
        ps = rng.choice([8, 16, 32, 64, 128, 256])
        ctx = [rng.choice([0, 0, rng.randint(1, 200), rng.randint(200, 3000)]) for _ in range(n_req)]
        new = [rng.choice([1, 2, rng.randint(3, 130), rng.randint(130, 700)]) for _ in range(n_req)]
        window = rng.choice([0, 0, 0, rng.randint(1, 600)])
        ranges = rng.choice([None, None, 1, 2, 3, 4, 8])
        err = _attention_case(nq, nkv, 128, ctx, new, ps, window, torch.bfloat16, "prefill_tcgen05", key_ranges=ranges, in_ulps=True)
        assert err < 1.0, (case, nq, nkv, ctx, new, ps, window, ranges, err)      # measured: 0.73 at most


def test_attention_prefill_without_tma_takes_any_page_size():
    assert _attention_case(4, 2, 64, [10, 0], [90, 31], 24, 0, torch.bfloat16, "prefill") < 1.2e-2
    assert _attention_case(4, 2, 64, [10, 77], [1, 1], 24, 0, torch.bfloat16, "decode") < 1.2e-2


@pytest.mark.parametrize("mode", ["decode", "decode_tma"])
@pytest.mark.parametrize("nq, nkv, d, ctx, ps, window", [
    (4, 2, 64, [63], 16, 0), (4, 2, 64, [10, 200, 64], 16, 0), (32, 8, 128, [2047, 100, 513, 0], 64, 0),
    (8, 1, 128, [700, 3], 8, 0), (8, 2, 128, [300, 90], 32, 64), (8, 2, 128, [1000, 90], 256, 0),
])
def test_attention_decode_kernels(mode, nq, nkv, d, ctx, ps, window):
    assert _attention_case(nq, nkv, d, ctx, [1] * len(ctx), ps, window, torch.bfloat16, mode) < 1.2e-2


@pytest.mark.parametrize("chunk, ctx, window", [
    (2048, [2047, 100, 513, 0], 0),     # one range: the CTA writes the result itself
    (2048, [2047, 100, 513, 0], 300),   # the same with a window
    (1024, [1500, 100, 1023, 1024], 0), # two ranges; a request of two key tiles has one in each
    (512, [1999, 64, 700, 0], 0),       # five ranges
    (256, [1700, 300, 255, 256], 200),  # a window: its tiles are dealt out over the ranges, the rest are empty
    (192, [1700, 300, 255, 256], 0),    # ten ranges
])
def test_attention_decode_key_ranges(chunk, ctx, window):
    """One key range per request (the kernel writes the output itself) and several (partial results,
    merged by a second kernel). A request's key tiles are dealt out evenly over the ranges, so a request
    with fewer tiles than ranges leaves the last ranges empty."""
    assert _attention_case(8, 2, 128, ctx, [1] * len(ctx), 64, window, torch.bfloat16, "decode_tma", decode_chunk=chunk) < 1.2e-2
    assert _attention_case(4, 1, 64, ctx[:2], [1, 1], 16, window, torch.bfloat16, "decode_tma", decode_chunk=chunk) < 1.2e-2


@pytest.mark.parametrize("nq, nkv, d, lens, ps, window, chunk, partial, writes", [
    (8, 2, 128, [1, 64, 65, 300, 513], 64, 0, 0, True, True),      # the new key opens a page, ends one, lies inside
    (8, 2, 128, [1, 64, 65, 300, 513], 16, 0, 128, False, True),   # several ranges: only the last one holds the new key
    (4, 4, 64, [33, 200], 8, 0, 64, True, True),
    (6, 1, 64, [90, 7, 129], 32, 50, 0, False, True),              # a window
    (8, 2, 128, [10, 140], 64, 0, 0, True, False),                 # the cache is another layer's: nothing is written
    (32, 8, 128, [2049] * 3, 64, 0, 0, True, True),
])
def test_attention_decode_with_rope_equals_the_two_kernels(nq, nkv, d, lens, ps, window, chunk, partial, writes):
    """One launch that makes the queries and the new key and value from the q/k/v projection against
    qk_norm_rope_kv followed by attention_decode (each checked against its formulas above): the same
    output, the same cache rows, nothing else touched."""
    torch.manual_seed(len(lens) * 7 + d)
    k = _k()
    B, eps = len(lens), 1e-6
    width = (nq + 2 * nkv) * d
    y = torch.randn(B, width, device=DEV)
    if partial:
        parts = torch.randn(3, B, width, device=DEV)
        parts[2] = y - parts[0] - parts[1]
        qkv = parts.contiguous()
    else:
        qkv = y.bfloat16()
    qg, kg = (1 + 0.1 * torch.randn(d)).to(DEV), (1 + 0.1 * torch.randn(d)).to(DEV)
    inv_freq = torch.pow(torch.tensor(1e4), -(2.0 * torch.arange(d // 2)) / d)
    cos, sin = k.rope_table(inv_freq.to(DEV), max(lens) + 1)
    max_blocks = -(-max(lens) // ps) + 1
    num_pages = B * max_blocks + 2
    perm = torch.randperm(num_pages).tolist()
    table = torch.tensor([[perm.pop() for _ in range(max_blocks)] for _ in range(B)], dtype=torch.int32, device=DEV)
    pages = [(torch.randn(num_pages, nkv, ps, d, device=DEV) * 0.7).bfloat16() for _ in range(2)]
    kv_len, q_start = I(lens), I(list(range(B + 1)))
    positions, token_req = I([n - 1 for n in lens]), I(list(range(B)))
    plan = k.attention_decode_plan(B, nkv, max(lens) + 40)
    if chunk:
        plan = (chunk, -(-(max(lens) + 40) // chunk))
    # the two kernels
    kp1, vp1 = pages[0].clone(), pages[1].clone()
    q = torch.empty(B, nq * d, dtype=torch.bfloat16, device=DEV)
    st = _status()
    if writes:
        k.qk_norm_rope_kv(qkv, q, qg, kg, eps, cos, sin, d, positions, token_req, table, ps, kp1, vp1, nq, nkv, d, st)
    else:
        k.qk_norm_rope_kv(qkv, q, qg, kg, eps, cos, sin, d, positions, token_req, table, ps, None, None, nq, nkv, d, st)
    out1 = torch.empty_like(q)
    k.attention_decode(q, out1, kp1, vp1, table, kv_len, q_start, nq, nkv, d, d ** -0.5, window, plan[0], plan[1], st, use_tma=True)
    # the one kernel
    kp2, vp2 = pages[0].clone(), pages[1].clone()
    out2 = torch.empty_like(q)
    k.attention_decode_rope(qkv, out2, qg, kg, eps, cos, sin, kp2, vp2, writes, table, kv_len, q_start, nq, nkv, d, d ** -0.5,
                            window, plan[0], plan[1], st)
    assert st.item() == 0
    assert float((out1.float() - out2.float()).abs().max()) < 4e-3
    assert float((kp1.float() - kp2.float()).abs().max()) < 2e-2 and float((vp1.float() - vp2.float()).abs().max()) < 2e-2
    changed = int(((kp2 != pages[0]).sum(dim=3) > 0).sum())
    assert changed == (B * nkv if writes else 0)


def test_attention_kernels_refuse_what_they_do_not_cover():
    from quantinfer_b200.errors import KernelError

    k = _k()
    assert not k.attention_mma_supported(4, 2, 48) and not k.attention_tma_supported(4, 2, 64, 24)
    q = torch.zeros(1, 4 * 48, dtype=torch.bfloat16, device=DEV)
    pages = torch.zeros(2, 2, 16, 48, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(KernelError, match="not covered"):
        k.attention_prefill(q, torch.empty_like(q), pages, pages, I([[0]]), I([0, 1]), I([0]), I([0]), I([0]), 4, 2, 48,
                            1.0, 0, _status(), use_tma=False)
    with pytest.raises(KernelError, match="limit"):
        big = torch.zeros(1, 2 * 272, dtype=torch.float32, device=DEV)
        k.attention_generic(big, torch.empty_like(big), torch.zeros(1, 2, 4, 272, device=DEV),
                            torch.zeros(1, 2, 4, 272, device=DEV), I([[0]]), I([0]), I([0]), 2, 2, 272, 1.0, 0, _status())


# ------------------------------------------------------------------ activation, sampling

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("interleaved", [False, True])
def test_silu_mul(dtype, interleaved):
    torch.manual_seed(8)
    g, u = torch.randn(5, 57).to(dtype) * 3, torch.randn(5, 57).to(dtype)
    gu = torch.stack([g, u], dim=2).reshape(5, 114) if interleaved else torch.cat([g, u], dim=1)
    out = torch.empty(5, 57, dtype=dtype, device=DEV)
    _k().silu_mul(gu.contiguous().to(DEV), out, interleaved=interleaved)
    ref = g.double() / (1 + torch.exp(-g.double())) * u.double()
    assert float((out.double().cpu() - ref).abs().max()) < (1e-6 if dtype == torch.float32 else 3e-2)


def _sample(logits, temperature=None, top_k=None, top_p=None, seed=None, counter=None):
    rows = logits.shape[0]
    st = _status()
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    f = lambda v, dt: None if v is None else torch.tensor(v, dtype=dt, device=DEV)
    _k().sample(logits.to(DEV), f(temperature, torch.float32), f(top_k, torch.int32), f(top_p, torch.float32),
                f(seed, torch.int64), f(counter, torch.int32), out, st)
    return out.cpu().tolist(), st.item()


def test_sample_greedy_first_maximum():
    x = torch.randn(4, 1000)
    x[1, 17] = x[1, 900] = 50.0          # a tie: the lowest index wins
    x[2, 999] = 60.0
    toks, st = _sample(x)
    assert st == 0 and toks == [int(x[0].argmax()), 17, 999, int(x[3].argmax())]
    x[3, 5] = float("nan")
    assert _sample(x)[1] == _k().STATUS_NON_FINITE


@pytest.mark.parametrize("vocab", [50, 517, 4099])
def test_sample_matches_the_plain_sampler(vocab):
    torch.manual_seed(9)
    rows = 24
    x = torch.randn(rows, vocab) * 2
    x[:, 3] = x[:, 11]                    # ties inside the candidate set
    temps = [0.0, 0.8, 1.3, 0.5] * 6
    ks = [0, 0, 5, 20, 0, 1] * 4
    ps = [0.0, 0.0, 0.0, 0.0, 0.9, 0.5, 0.3, 1.0] * 3
    seeds = [7 + (r << 33) for r in range(rows)]
    counters = list(range(rows))
    toks, st = _sample(x, temps, ks, ps, seeds, counters)
    assert st == 0
    for r in range(rows):
        expect = plain_sample(x[r], temps[r], ks[r] or None, ps[r] or None, seeds[r], counters[r])
        assert toks[r] == expect, (r, temps[r], ks[r], ps[r])


def test_sample_follows_the_distribution_and_the_counter():
    x = torch.tensor([[0.0, 2.0, 1.0, -1.0, 2.0]]).repeat(4000, 1)
    toks, _ = _sample(x, [1.0] * 4000, None, None, [12345] * 4000, list(range(4000)))
    p = torch.softmax(x[0], 0)
    freq = torch.bincount(torch.tensor(toks), minlength=5).double() / 4000
    assert float((freq - p.double()).abs().max()) < 0.03
    again, _ = _sample(x[:50], [1.0] * 50, None, None, [12345] * 50, list(range(50)))
    assert again == toks[:50]            # same seed and counter, same token
    other, _ = _sample(x[:50], [1.0] * 50, None, None, [12346] * 50, list(range(50)))
    assert other != toks[:50]


@pytest.mark.parametrize("vocab", [517, 4099])
def test_sample_from_slot_records(vocab):
    """The options of a row come from its request's slot record, found through the step's arrays
    (row -> flat token -> entry -> slot), and the kernel advances the record's counter: three draws in a
    row equal the plain sampler's with counters c, c + 1, c + 2, for requests that sit in other slots
    than their place in the batch, greedy rows among them."""
    from quantinfer_b200.sampling import GenerationConfig, RequestSlots

    torch.manual_seed(3)
    slots = RequestSlots(8, DEV)
    cfgs = {5: GenerationConfig(temperature=0.8, seed=11), 2: GenerationConfig(temperature=1.2, top_k=20, seed=(1 << 40) + 5),
            7: GenerationConfig(), 0: GenerationConfig(temperature=0.6, top_p=0.7, seed=3)}
    start = {5: 0, 2: 9, 7: 4, 0: 100}
    for slot, cfg in cfgs.items():
        slots.assign(slot, cfg, start[slot])
    # a step of four entries with 3, 1, 2 and 1 tokens; the rows wanted are the last token of each
    slot_ids, token_req, logit_rows = I([5, 2, 7, 0]), I([0, 0, 0, 1, 2, 2, 3]), I([2, 3, 5, 6])
    order = [5, 2, 7, 0]
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    for draw in range(3):
        x = torch.randn(4, vocab) * 2
        out = torch.empty(4, dtype=torch.int32, device=DEV)
        _k().sample_slots(x.to(DEV), logit_rows, token_req, slot_ids, slots.table, False, out, st)
        for r, slot in enumerate(order):
            c = cfgs[slot]
            assert int(out[r]) == plain_sample(x[r], c.temperature, c.top_k, c.top_p, c.seed, start[slot] + draw), (draw, slot)
    assert int(st) == 0
    assert slots.table[:, 3].tolist() == [103, 0, 12, 0, 0, 3, 0, 7]        # every record's counter moved by three
    # a step that the host knows to be all greedy takes the other kernel; the counter still moves
    slots.assign(1, GenerationConfig(), 0)
    x = torch.randn(1, vocab)
    out = torch.empty(1, dtype=torch.int32, device=DEV)
    _k().sample_slots(x.to(DEV), I([0]), I([0]), I([1]), slots.table, True, out, st)
    assert int(out[0]) == int(x[0].argmax()) and int(slots.table[1, 3]) == 1
    assert slots.table[1].tolist()[6:] == [128, -1]                          # max_new_tokens, no eos


def test_advance_decode():
    tok, pos, sp, kv, ctr = I([5, 6]), I([10, 20]), I([10, 20]), I([11, 21]), I([0, 3])
    hist = torch.zeros(2, dtype=torch.int32, device=DEV)
    _k().advance_decode(tok, pos, sp, kv, ctr, I([77, 88]), hist)
    assert tok.tolist() == [77, 88] and pos.tolist() == [11, 21] and sp.tolist() == [11, 21]
    assert kv.tolist() == [12, 22] and ctr.tolist() == [1, 4] and hist.tolist() == [77, 88]


# ------------------------------------------------------------------ lengths that a launch does not cover are flagged


def test_lengths_beyond_what_a_launch_covers_set_a_status_bit():
    """A position beyond the rotation table, and keys beyond the key ranges of a decode launch: the
    kernels read nothing out of range and drop nothing silently, they set STATUS_BAD_RANGE (the engine
    never passes such lengths; an embedder of the C symbols might)."""
    k = _k()
    torch.manual_seed(1)
    nq, nkv, d, ps = 4, 2, 64, 16
    # (1) the rotation table has 32 rows, one token stands at position 40
    inv_freq = torch.pow(torch.tensor(1e4), -(2.0 * torch.arange(d // 2)) / d)
    cos, sin = k.rope_table(inv_freq.to(DEV), 32)
    qkv = torch.randn(2, (nq + 2 * nkv) * d, device=DEV)
    q_out = torch.empty(2, nq * d, device=DEV)
    table = I([[0, 1, 2, 3]])
    kp = torch.zeros(4, nkv, ps, d, device=DEV)
    vp = torch.zeros_like(kp)
    for positions, want in (([3, 31], 0), ([3, 40], k.STATUS_BAD_RANGE)):
        st = _status()
        k.qk_norm_rope_kv(qkv, q_out, None, None, 1e-6, cos, sin, d, I(positions), I([0, 0]), table, ps, kp, vp, nq, nkv, d, st)
        assert st.item() == want, positions
    assert torch.isfinite(q_out).all()
    # (2) two key ranges of 64 keys cover 128 positions; one request holds 200
    ctx = [100, 200]
    max_blocks = -(-max(ctx) // ps)
    pages = torch.randn(2 * max_blocks, nkv, ps, d, device=DEV).bfloat16()
    tbl = torch.arange(2 * max_blocks, dtype=torch.int32, device=DEV).view(2, max_blocks)
    q = torch.randn(2, nq * d, device=DEV).bfloat16()
    out = torch.empty_like(q)
    for use_tma in (True, False):
        for n_splits, want in ((4, 0), (2, k.STATUS_BAD_RANGE)):
            st = _status()
            k.attention_decode(q, out, pages, pages, tbl, I(ctx), I([0, 1, 2]), nq, nkv, d, d ** -0.5, 0, 64, n_splits, st,
                               use_tma=use_tma)
            assert st.item() == want, (use_tma, n_splits)
    assert k.status_names(k.STATUS_BAD_RANGE) and "rotation table" in k.status_names(k.STATUS_BAD_RANGE)[0]
