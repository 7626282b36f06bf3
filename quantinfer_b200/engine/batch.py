"""One step's batch: for each request its next tokens, flattened, with the
per-token and per-request arrays the kernels read.

The reference concatenates the accepted items' tokens and runs the dense
operations once over all of them, with rotation tables and attention per
request by row offsets (crates/quantinfer-runtime/src/batch.rs:34-50,67-87,171-196);
an item there is a whole prompt or one decode token. Here an entry is any
portion of a prompt (from the request's current position) or one decode token,
and logits are wanted at any of its places.

Device arrays (int32), all views of one buffer that crosses in one copy:
    token_ids[n]   positions[n]   token_req[n]      per token (token_req: index of its entry)
    q_start[b+1]   start_pos[b]   kv_len[b]   slot_ids[b]      per entry
    logit_rows[r]                                    rows of the flattened batch whose logits are wanted
    tile_req[t]    tile_q0[t]                        blocks of up to 128 query rows of one entry (longest context first);
                                                     in a step that mixes decode tokens and prompt portions the entries
                                                     of one token that stand first are left out (n_lead_decode of them):
                                                     the split-key decode kernel takes those, the flash kernel the rest
    block_tables[g][b, max_blocks]                   per layer group
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import numpy as np
import torch


@dataclass
class StepEntry:
    request_id: object
    tokens: Sequence[int]
    want: Sequence[int] = ()


QUERY_TILE = 128   # query rows per entry of the tile lists (kernels.QUERY_TILE)


def _align(n: int, a: int = 4) -> int:
    return (n + a - 1) // a * a


class _OnlyOnTheDevice:
    """Stands where a batch's host-side lists would be when the step may be replayed from a
    CUDA graph: the graph keeps the kernels and their device arrays, whose contents change from
    step to step, while a host list would stay what it was at capture. Any use raises."""

    def _refuse(self, *a, **k):
        from ..errors import QuantInferError

        raise QuantInferError(
            "this step may be replayed from a CUDA graph, so its host-side lists (h_q_start, h_start_pos, h_kv_len, "
            "h_slot_ids) do not exist: read q_start, start_pos, kv_len and slot_ids on the device, or build the "
            "engine with use_graphs=False")

    __getitem__ = __iter__ = __len__ = __bool__ = _refuse


ONLY_ON_THE_DEVICE = _OnlyOnTheDevice()


@dataclass
class StepBatch:
    """What a part may read of a step. The device arrays (int32) are the interface that holds in
    every step, replayed from a graph or not: `token_ids`, `positions`, `token_req` per token;
    `q_start`, `start_pos`, `kv_len`, `slot_ids` per entry; `logit_rows`; `block_tables[group]`.
    The counts `n_tokens`, `n_requests`, `n_logit_rows` and `all_decode` are fixed for a captured
    step and may be used on the host. The `h_*` lists are a convenience for choosing a kernel or a
    grid in a step that runs once; in a step that may be replayed they raise on use. `max_kv_len`
    is an upper bound there (the context bucket), not the longest context."""

    n_tokens: int
    n_requests: int
    n_logit_rows: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    token_req: torch.Tensor
    q_start: torch.Tensor
    start_pos: torch.Tensor
    kv_len: torch.Tensor
    slot_ids: torch.Tensor
    logit_rows: torch.Tensor
    tile_req: torch.Tensor
    tile_q0: torch.Tensor
    block_tables: list
    # host copies, for parts that choose a kernel or a grid by them
    h_q_start: list = field(default_factory=list)
    h_start_pos: list = field(default_factory=list)
    h_kv_len: list = field(default_factory=list)
    h_slot_ids: list = field(default_factory=list)
    max_q_len: int = 0
    max_kv_len: int = 0
    all_decode: bool = False
    n_lead_decode: int = 0      # mixed steps: entries of one token at the front, which the tile lists leave out
    extra: dict = field(default_factory=dict)   # what fast kernels derive once per step (work lists)


def pack_batch(entries: Sequence[StepEntry], starts: Sequence[int], slots: Sequence[int],
               tables: Sequence, max_blocks: int) -> tuple:
    """Host side of a batch: one int32 array and the offsets of its parts.

    `starts[i]` is the position of entry i's first token, `slots[i]` its slot,
    `tables[g]` the block tables of group g by slot, an int32 array [slots, max_blocks]."""
    b = len(entries)
    lens = [len(e.tokens) for e in entries]
    n = sum(lens)
    r = sum(len(e.want) for e in entries)
    n_groups = len(tables)
    # Entries of one token at the front of a step that also holds longer entries (the scheduler puts the
    # decode tokens first): their attention is the decode kernel's work, where the query heads of a group
    # share each key and the keys are split over CTAs; as query tiles of their own they would each read
    # their whole context once per query head.
    n_lead = 0
    if any(ln > 1 for ln in lens):
        while n_lead < b and lens[n_lead] == 1:
            n_lead += 1
    # blocks of QUERY_TILE query rows; those that read the most keys go first
    tiles = []
    a = 0
    for i, ln in enumerate(lens):
        for t0 in range(0, ln, QUERY_TILE):
            if i >= n_lead:
                tiles.append((-(starts[i] + min(t0 + QUERY_TILE, ln)), i, a + t0))
        a += ln
    tiles.sort()
    layout, off = {}, 0
    for name, size in (("token_ids", n), ("positions", n), ("token_req", n), ("q_start", b + 1),
                       ("start_pos", b), ("kv_len", b), ("slot_ids", b), ("logit_rows", r),
                       ("tile_req", len(tiles)), ("tile_q0", len(tiles))):
        layout[name] = (off, size)
        off = _align(off + size)
    for g in range(n_groups):
        layout[f"table{g}"] = (off, b * max_blocks)
        off = _align(off + b * max_blocks)
    buf = np.full(max(off, 4), -1, dtype=np.int32)

    def part(name):
        o, s = layout[name]
        return buf[o:o + s]

    q_start = np.zeros(b + 1, dtype=np.int32)
    np.cumsum(lens, out=q_start[1:])
    part("q_start")[:] = q_start
    part("start_pos")[:] = starts
    part("kv_len")[:] = np.asarray(starts, dtype=np.int32) + np.asarray(lens, dtype=np.int32)
    part("slot_ids")[:] = slots
    part("tile_req")[:] = [t[1] for t in tiles]
    part("tile_q0")[:] = [t[2] for t in tiles]
    tok, pos, req, rows = part("token_ids"), part("positions"), part("token_req"), part("logit_rows")
    ri = 0
    for i, e in enumerate(entries):
        a, z = q_start[i], q_start[i + 1]
        tok[a:z] = e.tokens
        pos[a:z] = np.arange(starts[i], starts[i] + lens[i], dtype=np.int32)
        req[a:z] = i
        for w in e.want:
            rows[ri] = a + w
            ri += 1
    for g in range(n_groups):
        part(f"table{g}").reshape(b, max_blocks)[:] = tables[g][list(slots)]
    layout["n_lead_decode"] = n_lead
    return buf, layout, q_start, lens


def batch_from_packed(dev: torch.Tensor, layout: dict, entries, starts, slots, q_start, lens,
                      n_groups: int, max_blocks: int) -> StepBatch:
    def part(name):
        o, s = layout[name]
        return dev[o:o + s]

    b = len(entries)
    kv = [s + l for s, l in zip(starts, lens)]
    n_lead = layout.get("n_lead_decode", 0)
    return StepBatch(
        n_tokens=int(q_start[-1]), n_requests=b, n_logit_rows=layout["logit_rows"][1],
        token_ids=part("token_ids"), positions=part("positions"), token_req=part("token_req"),
        q_start=part("q_start"), start_pos=part("start_pos"), kv_len=part("kv_len"),
        slot_ids=part("slot_ids"), logit_rows=part("logit_rows"),
        tile_req=part("tile_req"), tile_q0=part("tile_q0"),
        block_tables=[part(f"table{g}").view(b, max_blocks) for g in range(n_groups)],
        h_q_start=[int(x) for x in q_start], h_start_pos=list(starts), h_kv_len=kv,
        h_slot_ids=list(slots), max_q_len=max(lens) if lens else 0, max_kv_len=max(kv) if kv else 0,
        all_decode=all(l == 1 for l in lens), n_lead_decode=n_lead,
    )
