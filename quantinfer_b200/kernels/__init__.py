"""Python face of the hand-written sm_100a kernels.

Each function checks its tensors (device, type, layout, sizes), passes raw
pointers and the current CUDA stream to the C entry point of the same name and
raises :class:`KernelError` with the library's message when the entry point
refuses. There is no fallback: without a CUDA device or without the compiled
library every call raises.
"""

from __future__ import annotations

import ctypes as C
import threading

import torch

from ..errors import KernelError

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}

STATUS_BAD_TOKEN = 1
STATUS_BAD_PAGE = 2
STATUS_NON_FINITE = 4
STATUS_WAIT_TIMEOUT = 8
STATUS_BAD_RANGE = 16

ABI_VERSION = 6


def status_names(code: int) -> list:
    """What the bits of a device status word mean."""
    return [name for bit, name in ((STATUS_BAD_TOKEN, "a token id outside the vocabulary"),
                                   (STATUS_BAD_PAGE, "a position without a cache page"),
                                   (STATUS_NON_FINITE, "non-finite logits"),
                                   (STATUS_WAIT_TIMEOUT, "a bounded wait inside a kernel ran out"),
                                   (STATUS_BAD_RANGE, "a position beyond the rotation table or the key ranges of a launch")) if code & bit]

_lib = None
_lib_lock = threading.Lock()


def library() -> C.CDLL:
    """The compiled kernel library; built at the first call if needed."""
    global _lib
    if _lib is not None:
        return _lib
    with _lib_lock:
        if _lib is not None:
            return _lib
        if not torch.cuda.is_available():
            raise KernelError(
                "no CUDA device is visible: the engine runs only on the GPU (there is no CPU path)"
            )
        from ..csrc.build import library_path

        try:
            path = library_path()
        except Exception as exc:  # the build failed or nvcc is missing
            raise KernelError(f"the sm_100a kernel library could not be built: {exc}") from exc
        lib = C.CDLL(str(path))
        lib.qi_last_error.restype = C.c_char_p
        lib.qi_abi_version.restype = C.c_int
        if lib.qi_abi_version() != ABI_VERSION:
            raise KernelError(
                f"{path} has ABI version {lib.qi_abi_version()}, expected {ABI_VERSION}; rebuild it"
            )
        _lib = lib
    return _lib


def library_file() -> str:
    return library()._name


def _stream() -> C.c_void_p:
    """The current CUDA stream of the current device, as the raw handle the entry points take. (Through
    torch's C binding: `torch.cuda.current_stream()` builds a Python object and costs about as much as
    a whole launch; a step of a few hundred launches asks this a few hundred times.)"""
    return C.c_void_p(_raw_stream(_current_device()))


try:
    _raw_stream = torch._C._cuda_getCurrentRawStream
    _current_device = torch._C._cuda_getDevice
except AttributeError:      # another torch: the public, slower way
    def _raw_stream(index):
        return torch.cuda.current_stream(index).cuda_stream

    _current_device = torch.cuda.current_device


launches = 0   # entry points called so far (each launches at least one kernel)


def _check(rc: int, name: str) -> None:
    global launches
    launches += 1
    if rc != 0:
        raise KernelError(f"{name}: {library().qi_last_error().decode()}")


knock_out = frozenset()   # kernel classes ("gemm", "attention", "norm", "rope", "other") whose launches are left out


def _call(cls, name: str, fn, *args) -> None:
    """Calls an entry point and raises with the library's message if it refuses. A class named in
    `knock_out` is not launched at all: a measurement leaves one class out at a time and times the
    rest of the step (the results of such a step mean nothing)."""
    if cls is not None and cls in knock_out:
        return
    _check(fn(*args), name)


def _code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise KernelError(f"element type {t.dtype} is not supported (float32 or bfloat16)") from None


def _req(t: torch.Tensor, name: str, dtype=None, ndim=None) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{name} must have {ndim} dimensions, got shape {tuple(t.shape)}")


def _ptr(t) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


# --------------------------------------------------------------------------
# embedding


def embedding(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, status: torch.Tensor) -> None:
    """out[t, :] = table[ids[t], :] as float32. ids int32 [n]; out float32 [n, hidden]."""
    _req(table, "table", ndim=2)
    _req(ids, "ids", torch.int32, 1)
    _req(out, "out", torch.float32, 2)
    _req(status, "status", torch.int32)
    n, hidden = out.shape
    if ids.numel() != n or table.shape[1] != hidden:
        raise KernelError(f"embedding: shapes do not agree: table {tuple(table.shape)}, ids {tuple(ids.shape)}, out {tuple(out.shape)}")
    _call('other', "embedding", library().qi_embedding,
          _ptr(table), _code(table), _ptr(ids), _ptr(out), n, hidden,
                                table.shape[0], _ptr(status), _stream())


# --------------------------------------------------------------------------
# norms


def add_rmsnorm(resid: torch.Tensor, delta, gain: torch.Tensor, eps: float, out: torch.Tensor,
                rows=None, write_resid: bool = True) -> None:
    """Fused residual add and RMSNorm.

    resid float32 [n, h] (updated in place when write_resid); delta None, [n, h]
    or [splits, n, h] (partial sums added in order); gain float32 [h]; out
    [n, h], or [len(rows), h] when `rows` (int32) selects source rows.
    """
    _req(resid, "resid", torch.float32, 2)
    _req(gain, "gain", torch.float32, 1)
    _req(out, "out", ndim=2)
    n, h = resid.shape
    splits, stride = 1, 0
    if delta is not None:
        _req(delta, "delta")
        if delta.dim() == 3:
            splits, stride = delta.shape[0], delta.shape[1] * delta.shape[2]
            if tuple(delta.shape[1:]) != (n, h):
                raise KernelError(f"add_rmsnorm: delta {tuple(delta.shape)} does not match resid {tuple(resid.shape)}")
        elif tuple(delta.shape) != (n, h):
            raise KernelError(f"add_rmsnorm: delta {tuple(delta.shape)} does not match resid {tuple(resid.shape)}")
    if gain.numel() != h:
        raise KernelError(f"add_rmsnorm: gain has {gain.numel()} elements, rows have {h}")
    n_out = n
    if rows is not None:
        _req(rows, "rows", torch.int32, 1)
        n_out = rows.numel()
        write_resid = False
    if tuple(out.shape) != (n_out, h):
        raise KernelError(f"add_rmsnorm: out is {tuple(out.shape)}, expected {(n_out, h)}")
    _call('norm', "add_rmsnorm", library().qi_add_rmsnorm,
          _ptr(resid), _ptr(delta), _code(delta) if delta is not None else F32, splits,
        C.c_longlong(stride), _ptr(gain), C.c_float(eps), _ptr(out), _code(out), _ptr(rows), n_out, h,
        int(bool(write_resid)), _stream())


def rmsnorm(x: torch.Tensor, gain: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """out = rmsnorm(x) * gain over the last dimension; x and out of one type."""
    _req(x, "x")
    _req(out, "out", x.dtype)
    _req(gain, "gain", torch.float32, 1)
    width = x.shape[-1]
    if gain.numel() != width or out.shape != x.shape:
        raise KernelError("rmsnorm: shapes do not agree")
    _call('norm', "rmsnorm", library().qi_rmsnorm,
          _ptr(x), _ptr(gain), C.c_float(eps), _ptr(out), _code(x),
                              x.numel() // width, width, _stream())


# --------------------------------------------------------------------------
# matrix products


def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = x[M, K] @ w[N, K]^T with 32-bit products and sums (no tensor cores)."""
    _req(x, "x", ndim=2)
    _req(w, "w", ndim=2)
    _req(out, "out", ndim=2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"gemm: shapes do not agree: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    _call('gemm', "gemm_simt", library().qi_gemm_simt,
          _ptr(x), _code(x), _ptr(w), _code(w), _ptr(out), _code(out), M, N, K,
                                C.c_longlong(K), C.c_longlong(K), C.c_longlong(N), _stream())


# --------------------------------------------------------------------------
# position encoding, q/k norm, cache write


def rope_table(inv_freq: torch.Tensor, max_positions: int):
    """cos and sin tables [max_positions, len(inv_freq)] in float32 from 32-bit angles."""
    _req(inv_freq, "inv_freq", torch.float32, 1)
    half = inv_freq.numel()
    cos = torch.empty((max_positions, half), dtype=torch.float32, device=inv_freq.device)
    sin = torch.empty_like(cos)
    _call(None, "rope_table", library().qi_rope_table,
          _ptr(inv_freq), _ptr(cos), _ptr(sin), max_positions, half, _stream())
    return cos, sin


def qk_norm_rope_kv(qkv, q_out, q_gain, k_gain, eps, cos, sin, rotary_dim, positions, token_req,
                    block_table, page_size, k_pages, v_pages, nq, nkv, d, status, interleaved: bool = False) -> None:
    """Per-head q/k RMSNorm, rotation, and the write of k and v into cache pages. Pairs of the
    rotation are (p, p + rotary_dim / 2), or (2p, 2p + 1) when `interleaved`.

    qkv [n, (nq + 2 nkv) d], or float32 [splits, n, (nq + 2 nkv) d] partial sums of a
    K-split projection (added here); q_out [n, nq d]; gains float32 [d] or None; cos/sin
    float32 [positions, rotary_dim / 2] or None; k_pages/v_pages
    [num_pages, nkv, page_size, d] or None (no write); block_table int32
    [requests, max_blocks].
    """
    _req(qkv, "qkv")
    _req(q_out, "q_out", ndim=2)
    splits = 1
    if qkv.dim() == 3:
        splits = qkv.shape[0]
        if qkv.dtype != torch.float32:
            raise KernelError("qk_norm_rope_kv: partial sums must be float32")
    elif qkv.dim() != 2 or qkv.dtype != q_out.dtype:
        raise KernelError(f"qk_norm_rope_kv: qkv {tuple(qkv.shape)} {qkv.dtype} does not fit q_out {q_out.dtype}")
    n = qkv.shape[-2]
    if qkv.shape[-1] != (nq + 2 * nkv) * d or tuple(q_out.shape) != (n, nq * d):
        raise KernelError(f"qk_norm_rope_kv: qkv {tuple(qkv.shape)} / q_out {tuple(q_out.shape)} do not match heads {nq}+2*{nkv} of {d}")
    for g, name in ((q_gain, "q_gain"), (k_gain, "k_gain")):
        if g is not None:
            _req(g, name, torch.float32, 1)
            if g.numel() != d:
                raise KernelError(f"{name} has {g.numel()} elements, head_dim is {d}")
    table_positions = 0
    if cos is not None:
        _req(cos, "cos", torch.float32, 2)
        _req(sin, "sin", torch.float32, 2)
        if cos.shape != sin.shape or cos.shape[1] * 2 != rotary_dim:
            raise KernelError("qk_norm_rope_kv: rotation tables do not match rotary_dim")
        table_positions = cos.shape[0]
    _req(positions, "positions", torch.int32, 1)
    _req(token_req, "token_req", torch.int32, 1)
    num_pages, max_blocks = 0, 0
    if k_pages is not None:
        _req(k_pages, "k_pages", q_out.dtype, 4)
        _req(v_pages, "v_pages", q_out.dtype, 4)
        _req(block_table, "block_table", torch.int32, 2)
        if tuple(k_pages.shape[1:]) != (nkv, page_size, d) or k_pages.shape != v_pages.shape:
            raise KernelError(f"qk_norm_rope_kv: pages {tuple(k_pages.shape)} do not match (pages, {nkv}, {page_size}, {d})")
        num_pages, max_blocks = k_pages.shape[0], block_table.shape[1]
    _call('rope', "qk_norm_rope_kv", library().qi_qk_norm_rope_kv,
          _ptr(qkv), splits, _ptr(q_out), _code(q_out), _ptr(q_gain), _ptr(k_gain), C.c_float(eps), _ptr(cos),
        _ptr(sin), rotary_dim, int(bool(interleaved)), table_positions, _ptr(positions), _ptr(token_req), _ptr(block_table),
        max_blocks, page_size, num_pages, _ptr(k_pages), _ptr(v_pages), n, nq, nkv, d, _ptr(status),
        _stream())


# --------------------------------------------------------------------------
# attention


def attention_generic(q, out, k_pages, v_pages, block_table, positions, token_req, nq, nkv, d,
                      scale: float, window: int, status) -> None:
    """Causal paged GQA attention, 32-bit arithmetic, any span length and page size."""
    _req(q, "q", ndim=2)
    _req(out, "out", q.dtype, 2)
    _req(k_pages, "k_pages", q.dtype, 4)
    _req(v_pages, "v_pages", q.dtype, 4)
    _req(block_table, "block_table", torch.int32, 2)
    _req(positions, "positions", torch.int32, 1)
    _req(token_req, "token_req", torch.int32, 1)
    n = q.shape[0]
    if q.shape[1] != nq * d or out.shape != q.shape:
        raise KernelError(f"attention: q {tuple(q.shape)} does not match {nq} heads of {d}")
    if k_pages.shape[1] != nkv or k_pages.shape[3] != d or k_pages.shape != v_pages.shape:
        raise KernelError(f"attention: pages {tuple(k_pages.shape)} do not match {nkv} kv heads of {d}")
    _call('attention', "attention_generic", library().qi_attention_generic,
          _ptr(q), _ptr(out), _code(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
        block_table.shape[1], k_pages.shape[2], k_pages.shape[0], _ptr(positions), _ptr(token_req), n,
        nq, nkv, d, C.c_float(scale), int(window or 0), _ptr(status), _stream())


def attention_mma_supported(nq: int, nkv: int, d: int) -> bool:
    """Whether the tensor-core attention kernels take this geometry (bfloat16 only)."""
    return bool(library().qi_attention_mma_supported(nq, nkv, d))


QUERY_TILE = 128   # query rows per entry of a batch's tile lists


def attention_tma_supported(nq: int, nkv: int, d: int, page_size: int, max_blocks: int = 1) -> bool:
    """Whether the TMA-fed attention kernels take this geometry (bfloat16 only)."""
    return bool(library().qi_attention_tma_supported(nq, nkv, d, page_size, max_blocks))


def attention_prefill_tcgen05_supported(nq: int, nkv: int, d: int, page_size: int, max_blocks: int = 1) -> bool:
    """Whether the tcgen05 prefill attention takes this geometry (bfloat16, head size 128)."""
    return bool(library().qi_attention_prefill_tcgen05_supported(nq, nkv, d, page_size, max_blocks))


def attention_prefill_ranges(n_ctas: int, max_kv_len: int) -> int:
    """Into how many key ranges the tcgen05 prefill attention cuts every query tile, given the CTAs
    it would launch uncut (heads x query tiles) and the longest context of the step. 296 CTAs are
    resident at once; cutting makes more and shorter ones, which fills the GPU when a step has few
    query tiles (a portion of 512 tokens of 32 heads is 128 CTAs: after 30,000 tokens 402 us uncut,
    268 in two ranges), and costs the partial results' trip through memory and a merge kernel, so
    it does not pay where the uncut launch already fills its rounds (2,048 tokens after 30,000:
    1,007 us uncut, 1,120 in four ranges). Estimated times, fitted to measurements at the 8B sizes
    (microseconds): rounds x keys of a CTA x 0.0154 (0.0132 while every CTA has an SM to itself),
    plus 0.0009 for every (query row, head, range) when cut."""
    best, best_time = 1, None
    for ranges in (1, 2, 3, 4, 6, 8):
        if ranges > 1 and max_kv_len < 2048 * ranges:
            break
        units = n_ctas * ranges
        rounds = -(-units // 296)
        time = rounds * (max_kv_len / ranges) * (0.0132 if units <= 148 else 0.0154)
        if ranges > 1:
            time += n_ctas * 128 * ranges * 0.0009
        if best_time is None or time < best_time * 0.97:
            best, best_time = ranges, time
    return best


def attention_prefill(q, out, k_pages, v_pages, block_table, q_start, start_pos, tile_req, tile_q0,
                      nq, nkv, d, scale: float, window: int, status, use_tma: bool | None = None,
                      impl: str | None = None, max_kv_len: int = 0, key_ranges: int | None = None) -> None:
    """Causal paged GQA flash attention (bfloat16, head size 64 or 128) for spans of any
    length. `tile_req[i]`, `tile_q0[i]`: request index and first flat token of the i-th
    block of up to QUERY_TILE query rows.

    Three kernels: "tcgen05" (head size 128, page size a power of two >= 8: tcgen05.mma with
    accumulators in tensor memory, TMA loads), "tma" (mma.sync with TMA loads, same page
    sizes, head size 64 or 128) and "cpasync" (mma.sync, any page size). `impl` forces one;
    the default is the first that takes the geometry. `use_tma` is the older switch between
    the last two. `max_kv_len` (the longest context of the step) lets the tcgen05 kernel cut long
    contexts into key ranges over more CTAs (`key_ranges` forces a number)."""
    if impl is None and use_tma is not None:
        impl = "tma" if use_tma else "cpasync"
    _req(q, "q", torch.bfloat16, 2)
    _req(out, "out", torch.bfloat16, 2)
    _req(k_pages, "k_pages", torch.bfloat16, 4)
    _req(v_pages, "v_pages", torch.bfloat16, 4)
    for t, name in ((block_table, "block_table"), (q_start, "q_start"), (start_pos, "start_pos"),
                    (tile_req, "tile_req"), (tile_q0, "tile_q0")):
        _req(t, name, torch.int32)
    if q.shape[1] != nq * d or out.shape != q.shape:
        raise KernelError(f"attention_prefill: q {tuple(q.shape)} does not match {nq} heads of {d}")
    if k_pages.shape[1] != nkv or k_pages.shape[3] != d or k_pages.shape != v_pages.shape:
        raise KernelError(f"attention_prefill: pages {tuple(k_pages.shape)} do not match {nkv} kv heads of {d}")
    if tile_req.numel() != tile_q0.numel():
        raise KernelError("attention_prefill: tile lists differ in length")
    if impl is None:
        if attention_prefill_tcgen05_supported(nq, nkv, d, k_pages.shape[2], block_table.shape[1]):
            impl = "tcgen05"
        elif attention_tma_supported(nq, nkv, d, k_pages.shape[2], block_table.shape[1]):
            impl = "tma"
        else:
            impl = "cpasync"
    if impl == "tcgen05":
        ranges = key_ranges or attention_prefill_ranges(nq * tile_req.numel(), max_kv_len)
        if q.shape[0] > 65535:
            ranges = 1
        ws = torch.empty(q.shape[0] * nq * ranges * (d + 2), dtype=torch.float32, device=q.device) if ranges > 1 else None
        _call('attention', "attention_prefill_tcgen05", library().qi_attention_prefill_tcgen05,
              _ptr(q), _ptr(out), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
            k_pages.shape[2], k_pages.shape[0], _ptr(q_start), _ptr(start_pos), _ptr(tile_req), _ptr(tile_q0),
            tile_req.numel(), q.shape[0], nq, nkv, d, C.c_float(scale), int(window or 0), ranges, _ptr(ws),
            _ptr(status), _stream())
        return
    if impl not in ("tma", "cpasync"):
        raise KernelError(f"attention_prefill: unknown kernel {impl!r}")
    if impl == "tma":
        _call('attention', "attention_prefill_tma", library().qi_attention_prefill_tma,
              _ptr(q), _ptr(out), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
            k_pages.shape[2], k_pages.shape[0], _ptr(q_start), _ptr(start_pos), _ptr(tile_req), _ptr(tile_q0),
            tile_req.numel(), q.shape[0], nq, nkv, d, C.c_float(scale), int(window or 0), _ptr(status), _stream())
        return
    _call('attention', "attention_prefill", library().qi_attention_prefill,
          _ptr(q), _ptr(out), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
        k_pages.shape[2], k_pages.shape[0], _ptr(q_start), _ptr(start_pos), _ptr(tile_req), _ptr(tile_q0),
        tile_req.numel(), QUERY_TILE, nq, nkv, d, C.c_float(scale), int(window or 0), _ptr(status), _stream())


def attention_decode_plan(batch: int, nkv: int, max_kv_len: int):
    """(keys per CTA, number of key ranges) for a decode batch: as many CTAs as are resident
    at once (two on each of 148 SMs) and no more, so that each requests its first tiles while
    the kernel before it still runs; ranges a multiple of 64 keys, independent of the
    requests' actual lengths."""
    target = max(1, 296 // max(batch * nkv, 1))
    chunk = max(64, -(-(-(-max_kv_len // target)) // 64) * 64)
    return chunk, -(-max_kv_len // chunk)


def attention_decode(q, out, k_pages, v_pages, block_table, kv_len, q_start, nq, nkv, d, scale: float,
                     window: int, chunk: int, n_splits: int, status, workspace=None,
                     use_tma: bool | None = None) -> None:
    """Paged GQA attention for one query token per request (bfloat16, head size 64 or
    128), a request's key tiles dealt out evenly over `n_splits` ranges of at most `chunk` positions
    (`n_splits * chunk` must cover the longest request). `workspace`: float32,
    at least batch * nq * n_splits * (d + 2) elements (allocated when None)."""
    _req(q, "q", torch.bfloat16, 2)
    _req(out, "out", torch.bfloat16, 2)
    _req(k_pages, "k_pages", torch.bfloat16, 4)
    _req(v_pages, "v_pages", torch.bfloat16, 4)
    for t, name in ((block_table, "block_table"), (kv_len, "kv_len"), (q_start, "q_start")):
        _req(t, name, torch.int32)
    batch = kv_len.numel()
    if q.shape[1] != nq * d or out.shape != q.shape or q.shape[0] < batch:
        raise KernelError(f"attention_decode: q {tuple(q.shape)} does not match {batch} requests, {nq} heads of {d}")
    if k_pages.shape[1] != nkv or k_pages.shape[3] != d or k_pages.shape != v_pages.shape:
        raise KernelError(f"attention_decode: pages {tuple(k_pages.shape)} do not match {nkv} kv heads of {d}")
    need = batch * nq * n_splits * (d + 2)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.float32, device=q.device)
    _req(workspace, "workspace", torch.float32, 1)
    if workspace.numel() < need:
        raise KernelError(f"attention_decode: workspace has {workspace.numel()} floats, {need} are needed")
    ws_o = workspace
    ws_ml = workspace[batch * nq * n_splits * d:]
    if use_tma is None:
        use_tma = attention_tma_supported(nq, nkv, d, k_pages.shape[2], block_table.shape[1])
    fn = library().qi_attention_decode_tma if use_tma else library().qi_attention_decode
    _call('attention', "attention_decode", fn,
          _ptr(q), _ptr(out), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
        k_pages.shape[2], k_pages.shape[0], _ptr(kv_len), _ptr(q_start), batch, nq, nkv, d, C.c_float(scale),
        int(window or 0), chunk, n_splits, _ptr(ws_o), _ptr(ws_ml), _ptr(status), _stream())


def attention_decode_rope(qkv, out, q_gain, k_gain, eps, cos, sin, k_pages, v_pages, writes: bool, block_table, kv_len,
                          q_start, nq, nkv, d, scale: float, window: int, chunk: int, n_splits: int, status,
                          workspace=None) -> None:
    """`qk_norm_rope_kv` and `attention_decode` in one launch, for a decode step: qkv is the
    q/k/v projection's output, bfloat16 [tokens, (nq + 2 nkv) d], or its float32 K-split partial
    sums [splits, tokens, (nq + 2 nkv) d]. The kernel makes each request's queries from it, and
    its new key and value, which it writes to the cache at position kv_len - 1 (`writes` False:
    another layer wrote them). Rotation over the whole head or none (cos None)."""
    _req(qkv, "qkv")
    if qkv.dim() == 3:
        if qkv.dtype != torch.float32:
            raise KernelError("attention_decode_rope: partial sums must be float32")
        splits, n_tokens, width = qkv.shape
    elif qkv.dim() == 2 and qkv.dtype in (torch.bfloat16, torch.float32):
        splits, (n_tokens, width) = 1, qkv.shape
    else:
        raise KernelError(f"attention_decode_rope: qkv {tuple(qkv.shape)} {qkv.dtype} is neither an output nor partial sums")
    _req(out, "out", torch.bfloat16, 2)
    _req(k_pages, "k_pages", torch.bfloat16, 4)
    _req(v_pages, "v_pages", torch.bfloat16, 4)
    for t, name in ((block_table, "block_table"), (kv_len, "kv_len"), (q_start, "q_start")):
        _req(t, name, torch.int32)
    batch = kv_len.numel()
    if width != (nq + 2 * nkv) * d or tuple(out.shape) != (n_tokens, nq * d) or n_tokens < batch:
        raise KernelError(f"attention_decode_rope: qkv {tuple(qkv.shape)} / out {tuple(out.shape)} do not match {batch} requests, heads {nq}+2*{nkv} of {d}")
    if k_pages.shape[1] != nkv or k_pages.shape[3] != d or k_pages.shape != v_pages.shape:
        raise KernelError(f"attention_decode_rope: pages {tuple(k_pages.shape)} do not match {nkv} kv heads of {d}")
    for g, name in ((q_gain, "q_gain"), (k_gain, "k_gain")):
        if g is not None:
            _req(g, name, torch.float32, 1)
            if g.numel() != d:
                raise KernelError(f"{name} has {g.numel()} elements, head_dim is {d}")
    table_positions = 0
    if cos is not None:
        _req(cos, "cos", torch.float32, 2)
        _req(sin, "sin", torch.float32, 2)
        if cos.shape != sin.shape or cos.shape[1] * 2 != d:
            raise KernelError("attention_decode_rope: rotation tables must cover the whole head")
        table_positions = cos.shape[0]
    need = batch * nq * n_splits * (d + 2)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.float32, device=out.device)
    _req(workspace, "workspace", torch.float32, 1)
    if workspace.numel() < need:
        raise KernelError(f"attention_decode_rope: workspace has {workspace.numel()} floats, {need} are needed")
    _call('attention', "attention_decode_rope", library().qi_attention_decode_rope_tma,
          _ptr(qkv), _code(qkv), splits, n_tokens, _ptr(q_gain), _ptr(k_gain), C.c_float(eps), _ptr(cos), _ptr(sin),
        table_positions, int(bool(writes)), _ptr(out), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
        block_table.shape[1], k_pages.shape[2], k_pages.shape[0], _ptr(kv_len), _ptr(q_start), batch, nq, nkv, d,
        C.c_float(scale), int(window or 0), chunk, n_splits, _ptr(workspace), _ptr(workspace[batch * nq * n_splits * d:]),
        _ptr(status), _stream())


# --------------------------------------------------------------------------
# feed-forward


ACTIVATIONS = {"silu": 0, "gelu": 1, "gelu_tanh": 2, "relu": 3}


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> None:
    """`act_mul` with the activation silu."""
    act_mul(gate_up, out, "silu", interleaved)


def act_mul(gate_up: torch.Tensor, out: torch.Tensor, activation: str = "silu", interleaved: bool = False) -> None:
    """out[t, i] = act(gate[t, i]) * up[t, i]; gate, up = gate_up[t, i], gate_up[t, I + i],
    or gate_up[t, 2i], gate_up[t, 2i + 1] when `interleaved`. `activation`: one of ACTIVATIONS."""
    if activation not in ACTIVATIONS:
        raise KernelError(f"act_mul: activation {activation!r} has no kernel (one of {sorted(ACTIVATIONS)})")
    _req(gate_up, "gate_up", ndim=2)
    _req(out, "out", gate_up.dtype, 2)
    n, two_i = gate_up.shape
    if two_i % 2 or tuple(out.shape) != (n, two_i // 2):
        raise KernelError(f"act_mul: gate_up {tuple(gate_up.shape)} / out {tuple(out.shape)} do not agree")
    _call("other", "act_mul", library().qi_act_mul,
          _ptr(gate_up), _ptr(out), _code(out), n, two_i // 2, int(bool(interleaved)), ACTIVATIONS[activation], _stream())


# --------------------------------------------------------------------------
# sampling


def sample(logits, temperature, top_k, top_p, seed, counter, out_token, status) -> None:
    """Token per row of float32 logits [rows, vocab]; temperature 0 = first maximum.

    temperature/top_p float32 [rows], top_k/counter int32 [rows], seed int64
    [rows]; any of them may be None (greedy / no truncation / seed 0 / counter 0).
    """
    _req(logits, "logits", torch.float32, 2)
    _req(out_token, "out_token", torch.int32, 1)
    rows, vocab = logits.shape
    for t, name, dt in ((temperature, "temperature", torch.float32), (top_k, "top_k", torch.int32),
                        (top_p, "top_p", torch.float32), (seed, "seed", torch.int64),
                        (counter, "counter", torch.int32)):
        if t is not None:
            _req(t, name, dt, 1)
            if t.numel() < rows:
                raise KernelError(f"sample: {name} has {t.numel()} entries for {rows} rows")
    if out_token.numel() < rows:
        raise KernelError("sample: out_token is too short")
    _call('other', "sample", library().qi_sample,
          _ptr(logits), rows, vocab, _ptr(temperature), _ptr(top_k), _ptr(top_p),
                             _ptr(seed), _ptr(counter), _ptr(out_token), _ptr(status), _stream())


def sample_slots(logits, logit_rows, token_req, slot_ids, slots, all_greedy: bool, out_token, status) -> None:
    """Token per row of float32 logits [rows, vocab] with the options of the row's request, read from
    the slot records `slots` (int32 [num_slots, 8], sampling/slots.py). The request of row r is the one
    in slot slot_ids[token_req[logit_rows[r]]] (the step's device arrays). The kernel adds one to the
    record's count of emitted tokens after the draw. `all_greedy`: no row draws (the host knows)."""
    _req(logits, "logits", torch.float32, 2)
    _req(out_token, "out_token", torch.int32, 1)
    _req(slots, "slots", torch.int32, 2)
    rows, vocab = logits.shape
    for t, name in ((logit_rows, "logit_rows"), (token_req, "token_req"), (slot_ids, "slot_ids")):
        _req(t, name, torch.int32, 1)
    if logit_rows.numel() < rows or out_token.numel() < rows:
        raise KernelError(f"sample_slots: {rows} rows of logits, {logit_rows.numel()} wanted rows, {out_token.numel()} places for tokens")
    _call("other", "sample_slots", library().qi_sample_slots,
          _ptr(logits), rows, vocab, _ptr(logit_rows), _ptr(token_req), _ptr(slot_ids), _ptr(slots), slots.shape[1],
          int(bool(all_greedy)), _ptr(out_token), _ptr(status), _stream())


def advance_decode(token_ids, positions, start_pos, kv_len, counter, sampled, history) -> None:
    """In place, for a decode batch kept on the device: token_ids = sampled, positions,
    start_pos and kv_len + 1, counter + 1 (may be None), history = sampled (may be None)."""
    for t, name in ((token_ids, "token_ids"), (positions, "positions"), (start_pos, "start_pos"),
                    (kv_len, "kv_len"), (sampled, "sampled")):
        _req(t, name, torch.int32, 1)
    b = token_ids.numel()
    _call(None, "advance_decode", library().qi_advance_decode,
          _ptr(token_ids), _ptr(positions), _ptr(start_pos), _ptr(kv_len),
                                     _ptr(counter), _ptr(sampled), _ptr(history), b, _stream())


def gemm_qkv_rope_supported(M: int, K: int, d: int, rotary_dim: int, dtype, weight_dtype) -> bool:
    """Whether `gemm_qkv_rope` takes this problem: many tokens (the operands are not swapped),
    bfloat16, heads of 128, rotation over the whole head or none."""
    return (M > 256 and K % 8 == 0 and d == 128 and rotary_dim in (0, d)
            and dtype == torch.bfloat16 and weight_dtype == torch.bfloat16)


def gemm_qkv_rope(x, w, q_out, q_gain, k_gain, eps, cos, sin, positions, token_req, block_table, page_size,
                  k_pages, v_pages, nq, nkv, status) -> None:
    """The q/k/v projection x[M, K] @ w[(nq + 2 nkv) 128, K]^T on the tcgen05 tensor cores with
    the q/k RMSNorm, the rotation and the cache write in its epilogue: what `gemm_bf16` followed
    by `qk_norm_rope_kv` computes, without the projection's output crossing memory.
    Arguments as for `qk_norm_rope_kv`."""
    d = 128
    _req(x, "x", torch.bfloat16, 2)
    _req(w, "w", torch.bfloat16, 2)
    _req(q_out, "q_out", torch.bfloat16, 2)
    M, K = x.shape
    if tuple(w.shape) != ((nq + 2 * nkv) * d, K) or tuple(q_out.shape) != (M, nq * d):
        raise KernelError(f"gemm_qkv_rope: x {tuple(x.shape)}, w {tuple(w.shape)}, q_out {tuple(q_out.shape)} do not match heads {nq}+2*{nkv} of {d}")
    for g, name in ((q_gain, "q_gain"), (k_gain, "k_gain")):
        if g is not None:
            _req(g, name, torch.float32, 1)
            if g.numel() != d:
                raise KernelError(f"{name} has {g.numel()} elements, head_dim is {d}")
    table_positions = 0
    if cos is not None:
        _req(cos, "cos", torch.float32, 2)
        _req(sin, "sin", torch.float32, 2)
        if cos.shape != sin.shape or cos.shape[1] * 2 != d:
            raise KernelError("gemm_qkv_rope: rotation tables must cover the whole head")
        table_positions = cos.shape[0]
    _req(positions, "positions", torch.int32, 1)
    _req(token_req, "token_req", torch.int32, 1)
    if positions.numel() != M or token_req.numel() != M:
        raise KernelError("gemm_qkv_rope: positions and token_req must have one entry per token")
    num_pages, max_blocks = 0, 0
    if k_pages is not None:
        _req(k_pages, "k_pages", torch.bfloat16, 4)
        _req(v_pages, "v_pages", torch.bfloat16, 4)
        _req(block_table, "block_table", torch.int32, 2)
        if tuple(k_pages.shape[1:]) != (nkv, page_size, d) or k_pages.shape != v_pages.shape:
            raise KernelError(f"gemm_qkv_rope: pages {tuple(k_pages.shape)} do not match (pages, {nkv}, {page_size}, {d})")
        num_pages, max_blocks = k_pages.shape[0], block_table.shape[1]
    _call('gemm', "gemm_qkv_rope", library().qi_gemm_bf16_qkv_rope,
          _ptr(x), _ptr(w), M, K, _ptr(q_out), _ptr(q_gain), _ptr(k_gain), C.c_float(eps), _ptr(cos), _ptr(sin),
        table_positions, _ptr(positions), _ptr(token_req), _ptr(block_table), max_blocks, page_size, num_pages,
        _ptr(k_pages), _ptr(v_pages), nq, nkv, _ptr(status), _stream())


def stage_step(host_meta: torch.Tensor, meta: torch.Tensor, device_tokens=None) -> None:
    """meta[:n] = host_meta[:n] read by a kernel straight from pinned host memory (n =
    host_meta.numel()); the first device_tokens.numel() entries come from `device_tokens`
    (int32, on the device) when given."""
    if not isinstance(host_meta, torch.Tensor) or host_meta.is_cuda or not host_meta.is_pinned() or host_meta.dtype != torch.int32:
        raise KernelError("stage_step: host_meta must be a pinned int32 host tensor")
    _req(meta, "meta", torch.int32, 1)
    n = host_meta.numel()
    if meta.numel() < n:
        raise KernelError(f"stage_step: meta has {meta.numel()} entries, {n} are needed")
    n_tok = 0
    if device_tokens is not None:
        _req(device_tokens, "device_tokens", torch.int32, 1)
        n_tok = device_tokens.numel()
    _call(None, "stage_step", library().qi_stage_step,
          C.c_void_p(host_meta.data_ptr()), _ptr(meta), n, _ptr(device_tokens), n_tok, _stream())


def publish(src: torch.Tensor, host_out: torch.Tensor, n: int) -> None:
    """host_out[:n] = src[:n], written by a kernel into pinned host memory; read it after an
    event recorded behind this call."""
    _req(src, "src", torch.int32, 1)
    if host_out.is_cuda or not host_out.is_pinned() or host_out.dtype != torch.int32:
        raise KernelError("publish: host_out must be a pinned int32 host tensor")
    if n > src.numel() or n > host_out.numel():
        raise KernelError("publish: more entries than the buffers hold")
    _call(None, "publish", library().qi_publish,
          _ptr(src), C.c_void_p(host_out.data_ptr()), n, _stream())


# --------------------------------------------------------------------------
# tensor-core matrix product (bfloat16 operands, 32-bit accumulation)

_gemm_status = {}


def gemm_bf16_supported(M: int, N: int, K: int, out_dtype) -> bool:
    """Whether `gemm_bf16` takes this problem; callers use `gemm_simt` otherwise."""
    return M > 0 and K % 8 == 0 and out_dtype in (torch.bfloat16, torch.float32)


def gemm_bf16_plan(M: int, N: int, K: int, allow_split: bool = True):
    """(orientation, tile width, K splits) the library would choose; allow_split=False for a
    product whose epilogue needs the whole sum (the fused activation). Orientation 0: the tokens
    ride the 128 rows of the tensor-core tile; 1: the weights do (few tokens); 2: tokens on the rows
    of tiles of 256 x 256 computed by pairs of CTAs (many tokens)."""
    key = (M, N, K, bool(allow_split))
    plan = _plans.get(key)
    if plan is None:
        swap, bn, splits = C.c_int(), C.c_int(), C.c_int()
        library().qi_gemm_bf16_plan(M, N, K, int(allow_split), C.byref(swap), C.byref(bn), C.byref(splits))
        plan = _plans[key] = (swap.value, bn.value, splits.value)
    return plan


_plans = {}


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, out, plan=None, status=None, epilogue: str | None = None,
              keep_partials: bool = False):
    """out[M, N] = x[M, K] @ w[N, K]^T on the tcgen05 tensor cores; x, w bfloat16; out
    bfloat16 or float32. `plan` = (orientation, tile width, splits) overrides the choice.

    epilogue="silu_mul": w's rows are (gate, up) pairs and out is [M, N / 2] =
    silu(gate) * up. keep_partials=True: when the plan splits K, the float32 partial sums
    [splits, M, N] are returned unreduced (and `out` is not written); else `out` is returned."""
    _req(x, "x", torch.bfloat16, 2)
    _req(w, "w", torch.bfloat16, 2)
    M, K = x.shape
    N = w.shape[0]
    if epilogue not in (None, "silu_mul"):
        raise KernelError(f"gemm_bf16: unknown epilogue {epilogue!r}")
    swap, bn, splits = plan if plan is not None else gemm_bf16_plan(M, N, K, allow_split=epilogue is None)
    epi = 0
    if epilogue == "silu_mul":
        epi, splits = 1, 1
    n_out = N // 2 if epi else N
    partial_only = keep_partials and splits > 1
    if not partial_only:
        _req(out, "out", ndim=2)
        if w.shape[1] != K or tuple(out.shape) != (M, n_out):
            raise KernelError(f"gemm: shapes do not agree: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    ws = torch.empty((splits, M, N), dtype=torch.float32, device=x.device) if splits > 1 else None
    if status is None:
        status = _gemm_status.get(x.device)
        if status is None:
            status = _gemm_status[x.device] = torch.zeros(1, dtype=torch.int32, device=x.device)
    _call('gemm', "gemm_bf16", library().qi_gemm_bf16,
          _ptr(x), _ptr(w), _ptr(None if partial_only else out),
                                BF16 if partial_only else _code(out), M, N, K, int(swap), bn, splits, epi,
                                _ptr(ws), _ptr(status), _stream())
    return ws if partial_only else out
