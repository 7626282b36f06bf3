"""Reader and writer of the safetensors container, single file or index-sharded.

The format: 8 bytes little-endian header length, a JSON header mapping tensor
name -> {dtype, shape, data_offsets}, then the raw little-endian data. The
checks are the reference's (crates/quantinfer-format/src/safetensors/types.rs:15-28,48
element types and the 64 MiB header cap; json.rs:14 duplicate keys, :64-68 zero
dimensions, :94-109,132-145 ranges inside the file and not overlapping,
:118-122 byte length = product(shape) * element size; shards.rs:41-53,69-78,152-187
the index file's `weight_map` and the rule that a shard path stays inside the
index's folder).

Tensors come back as CPU torch tensors in their stored element type, backed by
a read-only memory map (no copy until they are moved to the device).
"""

from __future__ import annotations

import json
import mmap
import os
import struct
from pathlib import Path

import torch

from ..errors import WeightError

MAX_HEADER_BYTES = 64 * 1024 * 1024

_DTYPES = {
    "F32": (torch.float32, 4),
    "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
    "U32": (torch.uint32, 4),
    "U64": (torch.uint64, 8),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


def _no_duplicates(pairs):
    seen = {}
    for k, v in pairs:
        if k in seen:
            raise WeightError(f"safetensors header names {k!r} twice")
        seen[k] = v
    return seen


class SafeTensorsFile:
    """One .safetensors file: validated header, tensors read on demand."""

    def __init__(self, path):
        self.path = Path(path)
        try:
            fd = os.open(self.path, os.O_RDONLY | getattr(os, "O_NOFOLLOW", 0))
        except OSError as exc:
            raise WeightError(f"cannot open {self.path}: {exc}") from exc
        with os.fdopen(fd, "rb") as f:
            size = os.fstat(f.fileno()).st_size
            if size < 8:
                raise WeightError(f"{self.path}: too short to be a safetensors file")
            (hlen,) = struct.unpack("<Q", f.read(8))
            if hlen > MAX_HEADER_BYTES or 8 + hlen > size:
                raise WeightError(f"{self.path}: header length {hlen} is not plausible")
            raw = f.read(hlen)
            self._map = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ) if size else None
        try:
            header = json.loads(raw.decode("utf-8"), object_pairs_hook=_no_duplicates)
        except WeightError:
            raise
        except Exception as exc:
            raise WeightError(f"{self.path}: header is not valid JSON: {exc}") from exc
        if not isinstance(header, dict):
            raise WeightError(f"{self.path}: header must be a JSON object")
        self.metadata = header.pop("__metadata__", {}) or {}
        if not isinstance(self.metadata, dict) or any(
                not isinstance(k, str) or not isinstance(v, str) for k, v in self.metadata.items()):
            raise WeightError(f"{self.path}: __metadata__ must map strings to strings")
        self._data_start = 8 + hlen
        data_len = size - self._data_start
        self.entries: dict[str, tuple] = {}
        spans = []
        for name, info in header.items():
            if not isinstance(info, dict):
                raise WeightError(f"{self.path}: entry {name!r} is not an object")
            dtype, shape, offs = info.get("dtype"), info.get("shape"), info.get("data_offsets")
            if dtype not in _DTYPES:
                raise WeightError(f"{self.path}: tensor {name!r} has unsupported element type {dtype!r}")
            if not isinstance(shape, list) or any(isinstance(s, bool) or not isinstance(s, int) or s < 0 for s in shape):
                raise WeightError(f"{self.path}: tensor {name!r} has a malformed shape {shape!r}")
            if any(s == 0 for s in shape):
                raise WeightError(f"{self.path}: tensor {name!r} has a zero dimension")
            if (not isinstance(offs, list) or len(offs) != 2
                    or any(isinstance(o, bool) or not isinstance(o, int) or o < 0 for o in offs)):
                raise WeightError(f"{self.path}: tensor {name!r} has malformed data_offsets {offs!r}")
            begin, end = offs
            count = 1
            for s in shape:
                count *= s
            if end < begin or end - begin != count * _DTYPES[dtype][1]:
                raise WeightError(
                    f"{self.path}: tensor {name!r} spans {end - begin} bytes, its shape {shape} "
                    f"of {dtype} needs {count * _DTYPES[dtype][1]}")
            if end > data_len:
                raise WeightError(f"{self.path}: tensor {name!r} ends beyond the end of the file")
            self.entries[name] = (dtype, tuple(shape), begin, end)
            spans.append((begin, end, name))
        spans.sort()
        for (b0, e0, n0), (b1, e1, n1) in zip(spans, spans[1:]):
            if b1 < e0:
                raise WeightError(f"{self.path}: tensors {n0!r} and {n1!r} overlap")

    def names(self):
        return list(self.entries)

    def shape(self, name):
        return self.entries[name][1]

    def dtype(self, name):
        return _DTYPES[self.entries[name][0]][0]

    def tensor(self, name) -> torch.Tensor:
        dtype, shape, begin, end = self.entries[name]
        tdtype = _DTYPES[dtype][0]
        view = memoryview(self._map)[self._data_start + begin:self._data_start + end]
        import warnings

        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the map is read-only; the tensor is never written
            t = torch.frombuffer(view, dtype=tdtype)
        return t.reshape(shape)


class SafeTensorsFolder:
    """The weights of a model folder: `model.safetensors`, or
    `model.safetensors.index.json` with the shards its `weight_map` names."""

    def __init__(self, folder):
        self.folder = Path(folder)
        single = self.folder / "model.safetensors"
        index = self.folder / "model.safetensors.index.json"
        self._where: dict[str, SafeTensorsFile] = {}
        if single.is_file():
            f = SafeTensorsFile(single)
            for n in f.names():
                self._where[n] = f
        elif index.is_file():
            try:
                idx = json.loads(index.read_text(), object_pairs_hook=_no_duplicates)
                wm = idx["weight_map"]
                assert isinstance(wm, dict)
            except WeightError:
                raise
            except Exception as exc:
                raise WeightError(f"{index}: not a valid index file (needs an object `weight_map`): {exc}") from exc
            root = self.folder.resolve()
            files: dict[str, SafeTensorsFile] = {}
            for name, rel in wm.items():
                if not isinstance(rel, str) or os.path.isabs(rel) or ".." in Path(rel).parts:
                    raise WeightError(f"{index}: shard path {rel!r} must be relative and stay inside the folder")
                p = (self.folder / rel).resolve()
                if root not in p.parents:
                    raise WeightError(f"{index}: shard path {rel!r} leaves the model folder")
                if rel not in files:
                    files[rel] = SafeTensorsFile(self.folder / rel)
                if name not in files[rel].entries:
                    raise WeightError(f"{index}: tensor {name!r} is not in its shard {rel!r}")
                self._where[name] = files[rel]
        else:
            raise WeightError(f"{self.folder} has neither model.safetensors nor model.safetensors.index.json")

    def names(self):
        return list(self._where)

    def shape(self, name):
        return self._where[name].shape(name)

    def dtype(self, name):
        return self._where[name].dtype(name)

    def tensor(self, name) -> torch.Tensor:
        return self._where[name].tensor(name)


def write_safetensors(path, tensors: dict, metadata: dict | None = None) -> None:
    """Writes CPU tensors to one file, in the order given."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = []
    for name, t in tensors.items():
        if t.dtype not in _NAMES:
            raise WeightError(f"cannot store tensor {name!r} of type {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
        order.append(name)
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * ((8 - len(raw) % 8) % 8)
    tmp = Path(str(path) + ".tmp")
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            if t.dtype == torch.bfloat16:
                t = t.view(torch.int16)
            f.write(t.numpy().tobytes())
    os.replace(tmp, path)
