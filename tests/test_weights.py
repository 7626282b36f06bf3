"""Weights: the container reader, the loader's one clear error, random folders (no GPU)."""

import json
import struct

import pytest
import torch

from helpers import TINY_CONFIGS, make_folder
from quantinfer_b200.config import config_from_dict
from quantinfer_b200.engine.model import tensor_needs_of_spec
from quantinfer_b200.errors import WeightError
from quantinfer_b200.weights import (SafeTensorsFile, SafeTensorsFolder, load_folder, write_model_folder,
                                     write_safetensors)


def _needs(name):
    return tensor_needs_of_spec(config_from_dict(TINY_CONFIGS[name]).to_model_spec())


def test_random_folder_loads_and_keeps_stored_types(tmp_path):
    folder = make_folder(tmp_path / "A", "A")
    t = load_folder(folder, _needs("A"))
    assert t["model.embed_tokens.weight"].dtype == torch.bfloat16          # bfloat16 stays bfloat16
    assert t["model.layers.0.input_layernorm.weight"].dtype == torch.float32   # a 32-bit tensor stays so
    assert t["model.layers.1.self_attn.q_norm.weight"].shape == (16,)
    assert "lm_head.weight" not in t    # tied
    g = t["model.norm.weight"]
    assert float(g.min()) >= 0.9 and float(g.max()) <= 1.1
    w = t["model.layers.0.mlp.down_proj.weight"].float()
    assert abs(float(w.std()) - 0.02) < 0.002


def test_random_weights_are_reproducible_and_seeded(tmp_path):
    a = load_folder(make_folder(tmp_path / "a", "B"), _needs("B"))
    b = load_folder(make_folder(tmp_path / "b", "B"), _needs("B"))
    assert all(torch.equal(a[k], b[k]) for k in a)
    cfg = config_from_dict(TINY_CONFIGS["B"])
    c = load_folder(write_model_folder(tmp_path / "c", cfg, seed=99), _needs("B"))
    assert not torch.equal(a["lm_head.weight"], c["lm_head.weight"])


def test_same_bytes_as_the_safetensors_package(tmp_path):
    from safetensors.torch import load_file

    folder = make_folder(tmp_path / "C", "C")
    theirs = load_file(str(folder / "model.safetensors"))
    ours = load_folder(folder, _needs("C"))
    assert set(theirs) == set(ours)
    assert all(torch.equal(theirs[k], ours[k]) for k in ours)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = make_folder(tmp_path / "B", "B")
    from safetensors.torch import load_file, save_file

    t = load_file(str(folder / "model.safetensors"))
    del t["model.layers.1.mlp.up_proj.weight"]
    del t["lm_head.weight"]
    t["model.layers.7.extra.weight"] = torch.zeros(3)
    t["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 96, dtype=torch.bfloat16)
    t["model.norm.weight"] = torch.zeros(96, dtype=torch.int32)
    save_file(t, str(folder / "model.safetensors"))
    with pytest.raises(WeightError) as e:
        load_folder(folder, _needs("B"))
    msg = str(e.value)
    assert "missing tensors (2)" in msg and "model.layers.1.mlp.up_proj.weight" in msg and "lm_head.weight" in msg
    assert "unexpected tensors (1)" in msg and "model.layers.7.extra.weight" in msg
    assert "wrong shapes (1)" in msg and "has [16, 96], expected [32, 96]" in msg
    assert "wrong element types (1)" in msg and "model.norm.weight" in msg


def test_tensors_the_model_does_not_use_are_skipped_with_one_line(tmp_path):
    from safetensors.torch import load_file, save_file

    folder = make_folder(tmp_path / "B", "B")
    path = str(folder / "model.safetensors")
    t = load_file(path)
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(16)
    t["something.else"] = torch.zeros(2, 2, dtype=torch.bfloat16)
    save_file(t, path)
    lines = []
    got = load_folder(folder, _needs("B"), warn=lines.append)
    assert set(got) == set(_needs("B"))
    assert len(lines) == 1 and "2 tensors" in lines[0] and "something.else" in lines[0] and "inv_freq" in lines[0]
    # asked to be strict, the same folder is refused, and the error names them
    with pytest.raises(WeightError, match=r"unexpected tensors \(2\)"):
        load_folder(folder, _needs("B"), strict=True)


def test_a_tied_configuration_with_a_stored_head_uses_the_table(tmp_path):
    from safetensors.torch import load_file, save_file

    folder = make_folder(tmp_path / "A", "A")            # A ties its head to the embedding table
    path = str(folder / "model.safetensors")
    t = load_file(path)
    t["lm_head.weight"] = torch.full_like(t["model.embed_tokens.weight"], 7.0)   # differs from the table
    save_file(t, path)
    lines = []
    got = load_folder(folder, _needs("A"), warn=lines.append)
    assert "lm_head.weight" not in got
    assert len(lines) == 1 and "lm_head.weight" in lines[0] and "tied" in lines[0]


def test_values_that_are_not_finite_are_refused_by_name_when_asked(tmp_path):
    from safetensors.torch import load_file, save_file

    folder = make_folder(tmp_path / "C", "C")
    load_folder(folder, _needs("C"), check_finite=True)      # a clean folder passes the check
    path = str(folder / "model.safetensors")
    t = load_file(path)
    t["model.layers.1.mlp.gate_proj.weight"][3, 5] = float("nan")
    t["model.layers.0.post_attention_layernorm.weight"][2] = float("-inf")
    t["model.layers.0.post_attention_layernorm.weight"][9] = float("inf")
    save_file(t, path)
    load_folder(folder, _needs("C"))                          # off by default
    with pytest.raises(WeightError) as e:
        load_folder(folder, _needs("C"), check_finite=True)
    msg = str(e.value)
    assert "model.layers.1.mlp.gate_proj.weight (1 of" in msg
    assert "model.layers.0.post_attention_layernorm.weight (2 of 168" in msg


def test_sharded_folder(tmp_path):
    folder = make_folder(tmp_path / "A", "A")
    from safetensors.torch import load_file

    t = load_file(str(folder / "model.safetensors"))
    names = list(t)
    (folder / "model.safetensors").unlink()
    half = len(names) // 2
    write_safetensors(folder / "model-00001-of-00002.safetensors", {k: t[k] for k in names[:half]})
    write_safetensors(folder / "model-00002-of-00002.safetensors", {k: t[k] for k in names[half:]})
    wm = {k: "model-00001-of-00002.safetensors" for k in names[:half]}
    wm.update({k: "model-00002-of-00002.safetensors" for k in names[half:]})
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    got = load_folder(folder, _needs("A"))
    assert all(torch.equal(got[k], t[k]) for k in names)
    # a shard path may not leave the folder
    wm[names[0]] = "../elsewhere.safetensors"
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    with pytest.raises(WeightError, match="relative and stay inside"):
        SafeTensorsFolder(folder)
    # a tensor must be in the shard the index names
    wm[names[0]] = "model-00002-of-00002.safetensors"
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    with pytest.raises(WeightError, match="is not in its shard"):
        SafeTensorsFolder(folder)


def _raw(path, header: dict, data: bytes):
    raw = json.dumps(header).encode()
    path.write_bytes(struct.pack("<Q", len(raw)) + raw + data)
    return path


@pytest.mark.parametrize("header, data, message", [
    ({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}, b"\0" * 8, "needs 8"),
    ({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 4, "beyond the end"),
    ({"a": {"dtype": "F8", "shape": [2], "data_offsets": [0, 2]}}, b"\0" * 2, "unsupported element type"),
    ({"a": {"dtype": "F32", "shape": [0], "data_offsets": [0, 0]}}, b"", "zero dimension"),
    ({"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]},
      "b": {"dtype": "F32", "shape": [1], "data_offsets": [2, 6]}}, b"\0" * 8, "overlap"),
    ({"__metadata__": {"k": 1}}, b"", "__metadata__"),
])
def test_container_checks(tmp_path, header, data, message):
    with pytest.raises(WeightError, match=message):
        SafeTensorsFile(_raw(tmp_path / "x.safetensors", header, data))


def test_duplicate_names_and_bad_lengths(tmp_path):
    raw = b'{"a":{"dtype":"F32","shape":[1],"data_offsets":[0,4]},"a":{"dtype":"F32","shape":[1],"data_offsets":[4,8]}}'
    p = tmp_path / "dup.safetensors"
    p.write_bytes(struct.pack("<Q", len(raw)) + raw + b"\0" * 8)
    with pytest.raises(WeightError, match="twice"):
        SafeTensorsFile(p)
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(WeightError, match="header length"):
        SafeTensorsFile(p)
    p.write_bytes(b"\0\0")
    with pytest.raises(WeightError, match="too short"):
        SafeTensorsFile(p)


def test_folder_without_weights(tmp_path):
    with pytest.raises(WeightError, match="neither model.safetensors nor"):
        SafeTensorsFolder(tmp_path)
