"""The decode-attention entry point that allocates nothing (`qi_attention_decode_tma_static`).

Some embedders of the kernel library cannot call cudaMalloc where they call us: a plugin
invoked while its host has frozen the memory pool, a process whose device memory belongs
to its own arena, a loop with a latency bound that an allocation would break. For them
the library keeps the kernel's scratch space (partial results per key range) in a fixed
16 MiB device array of its own. This test calls the entry point through its exported C
symbol, twice in a row with different problems (the array is shared and keeps the last
call's contents, so stale data would show in the second call), and compares each result
with the ordinary entry point, which takes a caller-allocated workspace. It also checks
that a problem larger than the array is refused with an error instead of being run.

The file sorts last on purpose: a run that stops at the first failure has then already
run every other test.
"""

import ctypes as C

import pytest
import torch

from kernel_refs import build_pages, ref_paged_attention

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 1.2e-2     # the tolerance of the other bfloat16 attention tests


def _case(seed, nq, nkv, d, ctx, ps):
    torch.manual_seed(seed)
    R = len(ctx)
    tot = [c + 1 for c in ctx]
    k_seq = [torch.randn(t, nkv, d).bfloat16().float() for t in tot]
    v_seq = [torch.randn(t, nkv, d).bfloat16().float() for t in tot]
    q = (torch.randn(R, nq * d) * 1.5).bfloat16()
    kp, vp, table = build_pages(k_seq, v_seq, ps, sum(-(-t // ps) for t in tot) + 2, nkv, d, torch.bfloat16, DEV, seed)
    I = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    ref = ref_paged_attention(q.float(), k_seq, v_seq, ctx, list(range(R)), nq, nkv, d, d ** -0.5)
    return dict(q=q.to(DEV), kp=kp, vp=vp, table=table, kv_len=I(tot), q_start=I(list(range(R + 1))), R=R, ref=ref,
                max_len=max(tot))


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def test_static_scratch_entry_point_matches_the_ordinary_one():
    from quantinfer_b200 import kernels

    lib = C.CDLL(kernels.library_file())          # the exported C symbols, nothing of the Python wrappers
    lib.qi_last_error.restype = C.c_char_p
    lib.qi_attention_decode_static_scratch_bytes.restype = C.c_ulonglong
    assert lib.qi_attention_decode_static_scratch_bytes() == 16 * 1024 * 1024
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)

    # two calls in a row: a larger problem first, then a smaller one with other data
    for seed, (nq, nkv, d, ctx, ps) in enumerate([(32, 8, 128, [700, 64, 1500, 0, 333], 64), (8, 2, 64, [90, 257], 16)]):
        c = _case(seed, nq, nkv, d, ctx, ps)
        chunk, splits = kernels.attention_decode_plan(c["R"], nkv, c["max_len"])
        expect = torch.zeros_like(c["q"])
        kernels.attention_decode(c["q"], expect, c["kp"], c["vp"], c["table"], c["kv_len"], c["q_start"], nq, nkv, d,
                                 d ** -0.5, 0, chunk, splits, status, use_tma=True)
        got = torch.zeros_like(c["q"])
        rc = lib.qi_attention_decode_tma_static(
            _ptr(c["q"]), _ptr(got), _ptr(c["kp"]), _ptr(c["vp"]), _ptr(c["table"]), c["table"].shape[1], ps,
            c["kp"].shape[0], _ptr(c["kv_len"]), _ptr(c["q_start"]), c["R"], nq, nkv, d, C.c_float(d ** -0.5), 0, chunk,
            splits, _ptr(status), stream)
        assert rc == 0, lib.qi_last_error().decode()
        torch.cuda.synchronize()
        assert status.item() == 0
        assert float((got.float() - expect.float()).abs().max()) <= TOL
        assert float((got.double().cpu() - c["ref"]).abs().max()) <= TOL

    # a problem whose partial results do not fit the array is refused, and nothing runs
    c = _case(5, 8, 2, 64, [10], 16)
    untouched = torch.full_like(c["q"], 3.0)
    rc = lib.qi_attention_decode_tma_static(
        _ptr(c["q"]), _ptr(untouched), _ptr(c["kp"]), _ptr(c["vp"]), _ptr(c["table"]), c["table"].shape[1], 16,
        c["kp"].shape[0], _ptr(c["kv_len"]), _ptr(c["q_start"]), 60000, 8, 2, 64, C.c_float(0.125), 0, 64, 64,
        _ptr(status), stream)
    assert rc != 0 and b"static array holds" in lib.qi_last_error()
    torch.cuda.synchronize()
    assert float((untouched - 3.0).abs().max()) == 0.0
