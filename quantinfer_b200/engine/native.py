"""The forward pass of a step through the library's C++ driver (csrc/forward_program.cu).

`NativeProgram.build(model)` describes a model to the driver once: its blocks'
weights, gains and constants, and the run order with each call's cache pages.
It succeeds when every part of the model is of the kinds the driver knows (the
pre-norm block of RMSNorm, paged attention with the rotary encoding or none,
RMSNorm and the gated feed-forward, the embedding and the head); any other model
keeps running through the parts' own `forward` (engine/model.py). A step then
costs the host one call instead of a few hundred: the driver picks each kernel by
the rules the parts use and takes its temporaries from one workspace.

The parts stay the description of the model: what the driver is told here is
read from them, and the tests of the parts alone run their `forward`.
"""

from __future__ import annotations

import ctypes as C

import torch

from .. import kernels
from ..errors import KernelError

MAX_GROUPS = 8


class _Linear(C.Structure):
    _fields_ = [("w", C.c_void_p), ("w_dtype", C.c_int), ("out_features", C.c_int), ("in_features", C.c_int)]


class _Block(C.Structure):
    _fields_ = [("norm1_gain", C.c_void_p), ("norm2_gain", C.c_void_p), ("norm1_eps", C.c_float), ("norm2_eps", C.c_float),
                ("qkv", _Linear), ("o", _Linear), ("gate_up", _Linear), ("down", _Linear),
                ("q_gain", C.c_void_p), ("k_gain", C.c_void_p), ("cos_t", C.c_void_p), ("sin_t", C.c_void_p),
                ("qk_eps", C.c_float), ("scale", C.c_float),
                ("nq", C.c_int), ("nkv", C.c_int), ("d", C.c_int), ("window", C.c_int), ("rotary_dim", C.c_int),
                ("table_positions", C.c_int), ("interleaved", C.c_int), ("activation", C.c_int)]


class _Call(C.Structure):
    _fields_ = [("block", C.c_int), ("group", C.c_int), ("writes", C.c_int), ("page_size", C.c_int), ("num_pages", C.c_int),
                ("k_pages", C.c_void_p), ("v_pages", C.c_void_p)]


class _ModelDesc(C.Structure):
    _fields_ = [("blocks", C.POINTER(_Block)), ("calls", C.POINTER(_Call)), ("n_blocks", C.c_int), ("n_calls", C.c_int),
                ("act_dtype", C.c_int), ("hidden", C.c_int), ("vocab", C.c_int), ("embedding", C.c_void_p),
                ("embedding_dtype", C.c_int), ("final_eps", C.c_float), ("final_gain", C.c_void_p), ("head", _Linear),
                ("status", C.c_void_p)]


class _Step(C.Structure):
    _fields_ = [("n_tokens", C.c_int), ("n_requests", C.c_int), ("n_logit_rows", C.c_int), ("all_decode", C.c_int),
                ("max_kv_len", C.c_int), ("n_tiles", C.c_int), ("n_lead_decode", C.c_int), ("reserved", C.c_int),
                ("token_ids", C.c_void_p), ("positions", C.c_void_p), ("token_req", C.c_void_p), ("q_start", C.c_void_p),
                ("start_pos", C.c_void_p), ("kv_len", C.c_void_p), ("logit_rows", C.c_void_p), ("tile_req", C.c_void_p),
                ("tile_q0", C.c_void_p), ("block_tables", C.c_void_p * MAX_GROUPS), ("max_blocks", C.c_int * MAX_GROUPS)]


def _linear(lin) -> _Linear:
    return _Linear(lin.weight.data_ptr(), kernels._code(lin.weight), lin.out_features, lin.in_features)


class NativeProgram:
    def __init__(self, model, desc, keep):
        self.vocab_size = model.spec.vocab_size      # (no reference to the model: it holds this object)
        self.desc = desc
        self._keep = keep          # the arrays the description points into
        self._sizes = {}           # step geometry -> workspace bytes

    @classmethod
    def build(cls, model, views):
        """The description of `model` with the cache views of its run order, or None when the model has a
        part of a kind the driver does not know."""
        from ..parts.attention import Attention
        from ..parts.block import PreNormBlock
        from ..parts.embedding import Embedding, LMHead
        from ..parts.ffn import GatedMLP
        from ..parts.norm import RMSNorm
        from ..parts.position import RopeHalfSplit

        if type(model.embedding) is not Embedding or type(model.head) is not LMHead or type(model.final_norm) is not RMSNorm:
            return None
        blocks = (_Block * len(model.blocks))()
        for i, b in enumerate(model.blocks):
            if (type(b) is not PreNormBlock or type(b.mixer_norm) is not RMSNorm or type(b.ffn_norm) is not RMSNorm
                    or type(b.mixer) is not Attention or type(b.ffn) is not GatedMLP):
                return None
            a, pos = b.mixer, b.mixer.position
            if pos is not None and type(pos) is not RopeHalfSplit:
                return None
            blocks[i] = _Block(
                b.mixer_norm.gain.data_ptr(), b.ffn_norm.gain.data_ptr(), b.mixer_norm.spec.eps, b.ffn_norm.spec.eps,
                _linear(a.qkv), _linear(a.o), _linear(b.ffn.gate_up), _linear(b.ffn.down),
                a.q_gain.data_ptr() if a.q_gain is not None else None, a.k_gain.data_ptr() if a.k_gain is not None else None,
                pos.cos.data_ptr() if pos is not None else None, pos.sin.data_ptr() if pos is not None else None,
                a.spec.qk_norm_eps, a.scale, a.nq, a.nkv, a.d, a.spec.window or 0, pos.rotary_dim if pos is not None else 0,
                pos.cos.shape[0] if pos is not None else 0, int(pos is not None and pos.pairing == "interleaved"),
                kernels.ACTIVATIONS[b.ffn.spec.activation])
        calls = (_Call * len(model.order))()
        for i, (call, view) in enumerate(zip(model.order, views)):
            if view.k_pages is None or view.group < 0 or view.group >= MAX_GROUPS:
                return None
            calls[i] = _Call(call.layer, view.group, int(view.writes), view.page_size, view.k_pages.shape[0],
                             view.k_pages.data_ptr(), view.v_pages.data_ptr())
        rt = model.runtime
        desc = _ModelDesc(blocks, calls, len(model.blocks), len(model.order), kernels._code(torch.empty((), dtype=rt.dtype)),
                          model.spec.hidden_size, model.spec.vocab_size, model.embedding.table.weight.data_ptr(),
                          kernels._code(model.embedding.table.weight), model.final_norm.spec.eps,
                          model.final_norm.gain.data_ptr(), _linear(model.head.proj), rt.status.data_ptr())
        return cls(model, desc, (blocks, calls, views))

    def forward(self, batch) -> torch.Tensor:
        """Runs the batch; float32 logits [len(batch.logit_rows), vocab]."""
        lib = kernels.library()
        step = _Step(batch.n_tokens, batch.n_requests, batch.n_logit_rows, int(batch.all_decode), batch.max_kv_len,
                     batch.tile_req.numel(), batch.n_lead_decode, 0, batch.token_ids.data_ptr(), batch.positions.data_ptr(), batch.token_req.data_ptr(),
                     batch.q_start.data_ptr(), batch.start_pos.data_ptr(), batch.kv_len.data_ptr(), batch.logit_rows.data_ptr(),
                     batch.tile_req.data_ptr(), batch.tile_q0.data_ptr())
        for g, table in enumerate(batch.block_tables):
            step.block_tables[g] = table.data_ptr()
            step.max_blocks[g] = table.shape[1]
        key = (batch.n_tokens, batch.n_requests, batch.n_logit_rows, batch.all_decode, batch.max_kv_len, step.n_tiles, batch.n_lead_decode,
               tuple(t.shape[1] for t in batch.block_tables))
        need = self._sizes.get(key)
        if need is None:
            lib.qi_forward_workspace_bytes.restype = C.c_longlong
            need = lib.qi_forward_workspace_bytes(C.byref(self.desc), C.byref(step))
            if need < 0:
                raise KernelError(f"forward: {lib.qi_last_error().decode()}")
            if len(self._sizes) > 4096:
                self._sizes.clear()
            self._sizes[key] = need
        device = batch.token_ids.device
        workspace = torch.empty(need, dtype=torch.uint8, device=device)
        logits = torch.empty((batch.n_logit_rows, self.vocab_size), dtype=torch.float32, device=device)
        launched = C.c_int(0)
        rc = lib.qi_forward(C.byref(self.desc), C.byref(step), C.c_void_p(workspace.data_ptr()), C.c_longlong(need),
                            C.c_void_p(logits.data_ptr() if batch.n_logit_rows else 0), C.byref(launched), kernels._stream())
        kernels.launches += launched.value
        if rc != 0:
            raise KernelError(f"forward: {lib.qi_last_error().decode()}")
        return logits
