"""Causal grouped-query attention over the paged cache.

    qkv = x . Wqkv^T                      (q, k, v projections stacked at load)
    q, k = rmsnorm_heads(q), rmsnorm_heads(k)     if qk_norm (one gain [head_dim] each)
    q, k = rotate(q, position), rotate(k, position)
    cache[position] = (k, v)
    out  = softmax(q k^T * scale, causal [, window]) v
    y    = out . Wo^T

Order and formulas: crates/quantinfer-runtime/src/qwen3/mod.rs:158-191 (three
projections :158-181, q/k norm :182-183, output projection :186-191),
batch.rs:30-65 (rotation, append, attention per request), attention.rs:39-141.
Query head h uses kv head h // (num_heads // num_kv_heads) (attention.rs:83).

Every size and constant is a field of the spec. The part asks the cache manager
for a paged entry (all keys, or a window of them); a call that reads another
layer's cache entry computes q only and writes nothing.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..cache.needs import PagedKVNeed
from ..errors import ConfigError
from ..weights.loader import TensorNeed
from .base import Part, build_part, register_part
from .linear import Linear


class Attention(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if spec.num_heads % spec.num_kv_heads:
            raise ConfigError(f"{spec.num_heads} query heads are not a multiple of {spec.num_kv_heads} kv heads")
        if spec.window is not None and spec.window <= 0:
            raise ConfigError("attention window must be positive or None")
        self.nq, self.nkv, self.d = spec.num_heads, spec.num_kv_heads, spec.head_dim
        self.scale = float(spec.scale) if spec.scale is not None else float(torch.tensor(float(self.d), dtype=torch.float32).sqrt().reciprocal())
        self.qkv = Linear(runtime, (self.nq + 2 * self.nkv) * self.d, spec.hidden_size, spec.prefix + "qkv_proj")
        self.o = Linear(runtime, spec.hidden_size, self.nq * self.d, spec.prefix + "o_proj")
        self.position = build_part("position", spec.position, runtime) if spec.position is not None else None
        self.q_gain = self.k_gain = None

    @classmethod
    def needs_of_spec(cls, s):
        p, nq, nkv, d = s.prefix, s.num_heads, s.num_kv_heads, s.head_dim
        needs = {
            p + "q_proj.weight": TensorNeed((nq * d, s.hidden_size)),
            p + "k_proj.weight": TensorNeed((nkv * d, s.hidden_size)),
            p + "v_proj.weight": TensorNeed((nkv * d, s.hidden_size)),
            p + "o_proj.weight": TensorNeed((s.hidden_size, nq * d)),
        }
        if s.qk_norm:
            needs[p + "q_norm.weight"] = TensorNeed((d,), "gain", "gain")
            needs[p + "k_norm.weight"] = TensorNeed((d,), "gain", "gain")
        return needs

    def load(self, tensors):
        p = self.spec.prefix
        qkv = [tensors[p + n + "_proj.weight"] for n in ("q", "k", "v")]
        if len({t.dtype for t in qkv}) > 1:
            qkv = [t.to(torch.float32) for t in qkv]
        self.qkv.load(torch.cat(qkv, dim=0))
        self.o.load(tensors[p + "o_proj.weight"])
        if self.spec.qk_norm:
            self.q_gain = self._gain(tensors[p + "q_norm.weight"])
            self.k_gain = self._gain(tensors[p + "k_norm.weight"])

    def cache_need(self):
        return PagedKVNeed(self.nkv, self.d, self.spec.window)

    def forward(self, x, batch, cache):
        rt = self.runtime
        n = x.shape[0]
        pos = self.position
        q = torch.empty((n, self.nq * self.d), dtype=x.dtype, device=x.device)
        table = batch.block_tables[cache.group]
        # the two fused kernels rotate whole heads in half-split pairs; any other rule takes the stand-alone kernel
        whole_head = pos is None or (pos.rotary_dim == self.d and getattr(pos, "pairing", "half_split") == "half_split")
        if whole_head and kernels.gemm_qkv_rope_supported(n, x.shape[1], self.d, pos.rotary_dim if pos else 0, x.dtype, self.qkv.weight.dtype):
            # many tokens: norm, rotation and the cache write ride in the projection's epilogue
            kernels.gemm_qkv_rope(
                x, self.qkv.weight, q, self.q_gain, self.k_gain, self.spec.qk_norm_eps,
                pos.cos if pos else None, pos.sin if pos else None, batch.positions, batch.token_req, table,
                cache.page_size, cache.k_pages if cache.writes else None, cache.v_pages if cache.writes else None,
                self.nq, self.nkv, rt.status)
            out = torch.empty_like(q)
            self.attend(q, out, batch, cache, table)
            return self.o(out, keep_partials=True)
        # K-split partial sums of the projection are added by the next kernel where it can take them
        qkv = self.qkv(x, keep_partials=self.d % 4 == 0 and whole_head)
        if (batch.all_decode and qkv.dtype in (torch.bfloat16, torch.float32) and x.dtype == torch.bfloat16
                and whole_head and (qkv.dim() == 3 or qkv.dtype == torch.bfloat16)
                and kernels.attention_tma_supported(self.nq, self.nkv, self.d, cache.page_size, table.shape[1])):
            # one token per request: the attention kernel makes its queries and the new key and value itself
            out = torch.empty_like(q)
            chunk, splits = kernels.attention_decode_plan(batch.n_requests, self.nkv, batch.max_kv_len)
            kernels.attention_decode_rope(
                qkv, out, self.q_gain, self.k_gain, self.spec.qk_norm_eps, pos.cos if pos else None,
                pos.sin if pos else None, cache.k_pages, cache.v_pages, cache.writes, table, batch.kv_len,
                batch.q_start, self.nq, self.nkv, self.d, self.scale, self.spec.window or 0, chunk, splits, rt.status)
            return self.o(out, keep_partials=True)
        kernels.qk_norm_rope_kv(
            qkv, q, self.q_gain, self.k_gain, self.spec.qk_norm_eps,
            pos.cos if pos else None, pos.sin if pos else None, pos.rotary_dim if pos else 0,
            batch.positions, batch.token_req, table, cache.page_size,
            cache.k_pages if cache.writes else None, cache.v_pages if cache.writes else None,
            self.nq, self.nkv, self.d, rt.status,
            interleaved=pos is not None and getattr(pos, "pairing", "half_split") == "interleaved")
        out = torch.empty_like(q)
        self.attend(q, out, batch, cache, table)
        return self.o(out, keep_partials=True)

    def attend(self, q, out, batch, cache, table):
        """Picks the kernel: tensor-core kernels for bfloat16 with head size 64 or 128
        (the split-key decode kernel when every entry is one token, else the flash
        kernel), the 32-bit kernel for everything else."""
        rt = self.runtime
        if q.dtype == torch.bfloat16 and kernels.attention_mma_supported(self.nq, self.nkv, self.d):
            if batch.all_decode:
                chunk, splits = kernels.attention_decode_plan(batch.n_requests, self.nkv, batch.max_kv_len)
                kernels.attention_decode(q, out, cache.k_pages, cache.v_pages, table, batch.kv_len, batch.q_start,
                                         self.nq, self.nkv, self.d, self.scale, self.spec.window or 0, chunk,
                                         splits, rt.status)
            else:
                # a mixed step: the entries of one token at its front go to the decode kernel (their rows of q
                # and out are the first rows), the others, which the tile lists hold, to the flash kernel
                lead = batch.n_lead_decode
                if lead:
                    chunk, splits = kernels.attention_decode_plan(lead, self.nkv, batch.max_kv_len)
                    kernels.attention_decode(q, out, cache.k_pages, cache.v_pages, table[:lead], batch.kv_len[:lead],
                                             batch.q_start[:lead], self.nq, self.nkv, self.d, self.scale,
                                             self.spec.window or 0, chunk, splits, rt.status)
                if batch.tile_req.numel():
                    kernels.attention_prefill(q, out, cache.k_pages, cache.v_pages, table, batch.q_start,
                                              batch.start_pos, batch.tile_req, batch.tile_q0, self.nq, self.nkv,
                                              self.d, self.scale, self.spec.window or 0, rt.status,
                                              max_kv_len=batch.max_kv_len)
            return
        kernels.attention_generic(q, out, cache.k_pages, cache.v_pages, table, batch.positions,
                                  batch.token_req, self.nq, self.nkv, self.d, self.scale,
                                  self.spec.window or 0, self.runtime.status)


register_part("mixer", "attention", Attention)
