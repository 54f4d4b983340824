"""Safetensors container, binding by name, errors, random weights (CPU)."""
import json
import os
import struct

import pytest
import torch
from safetensors import safe_open
from safetensors.torch import save_file

from synaptix_b200.config import Qwen3Config
from synaptix_b200.models import model_skeleton
from synaptix_b200.weights import (DictSource, RandomSource, SafetensorsError, SafetensorsFile,
                                   SafetensorsSource, TensorSpec, WeightError, bind_tensors,
                                   write_model_folder, write_safetensors)
from tiny import TINY_A, TINY_B, make_folder


def test_writer_is_read_by_the_safetensors_package(tmp_path):
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.randn(7), "c": torch.arange(6, dtype=torch.int64).view(2, 3)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t, metadata={"k": "v"})
    with safe_open(p, "pt") as f:
        assert sorted(f.keys()) == ["a", "b", "c"]
        for k in t:
            assert torch.equal(f.get_tensor(k), t[k])
        assert f.metadata() == {"k": "v"}


def test_reader_reads_the_safetensors_package(tmp_path):
    t = {"w": torch.randn(4, 6).to(torch.bfloat16), "g": torch.randn(6), "h": torch.randn(2, 2).to(torch.float16)}
    p = str(tmp_path / "model.safetensors")
    save_file(t, p)
    f = SafetensorsFile(p)
    assert f.tensors["w"].dtype == "BF16" and f.tensors["w"].shape == (4, 6)
    assert torch.equal(f.get("w"), t["w"]) and torch.equal(f.get("g"), t["g"])
    src = SafetensorsSource(str(tmp_path))
    assert src.get("w").dtype == torch.bfloat16          # stored bfloat16 stays bfloat16
    assert src.get("g").dtype == torch.float32           # stored 32-bit stays 32-bit
    assert src.get("h").dtype == torch.float32           # float16 is widened, losing nothing
    assert torch.equal(src.get("h"), t["h"].float())


def test_integer_tables_come_back_as_int32():
    src = DictSource({"t": torch.arange(5, dtype=torch.int64)})
    assert src.get("t").dtype == torch.int32


def test_container_errors(tmp_path):
    p = str(tmp_path / "bad.safetensors")
    open(p, "wb").write(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(p)
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    open(p, "wb").write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)       # data cut short
    with pytest.raises(SafetensorsError, match="'w'"):
        SafetensorsFile(p)
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 12]}}).encode()
    open(p, "wb").write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 16)      # byte count != shape
    with pytest.raises(SafetensorsError, match="needs 16 bytes"):
        SafetensorsFile(p)
    hdr = b'{"w":{"dtype":"F32","shape":[1],"data_offsets":[0,4]},"w":{"dtype":"F32","shape":[1],"data_offsets":[0,4]}}'
    open(p, "wb").write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 4)
    with pytest.raises(SafetensorsError, match="twice"):
        SafetensorsFile(p)
    hdr = json.dumps({"w": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}).encode()
    open(p, "wb").write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 4)
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        SafetensorsFile(p)
    with pytest.raises(SafetensorsError, match="neither"):
        SafetensorsSource(str(tmp_path / "empty"))


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    specs = {"a": TensorSpec((2, 3)), "b": TensorSpec((4,), "gain"), "c": TensorSpec((5,)), "opt": TensorSpec((1,), optional=True)}
    src = DictSource({"a": torch.zeros(3, 2), "c": torch.zeros(5), "x": torch.zeros(1), "y": torch.zeros(1)})
    with pytest.raises(WeightError) as ei:
        bind_tensors(specs, src)
    e = ei.value
    assert e.missing == ["b"] and e.unexpected == ["x", "y"]
    assert e.wrong_shape == [("a", (3, 2), (2, 3))]
    msg = str(e)
    assert "missing (1): b" in msg and "unexpected (2): x, y" in msg and "a is [3, 2], expected [2, 3]" in msg


def test_model_names_and_counts():
    # 11 tensors a layer + embedding + final norm (+ output head when untied)
    a = model_skeleton(Qwen3Config.from_dict(TINY_A)).all_tensor_specs()
    b = model_skeleton(Qwen3Config.from_dict(TINY_B)).all_tensor_specs()
    assert len([n for n, s in a.items() if not s.optional]) == 2 * 11 + 2
    assert len([n for n, s in b.items() if not s.optional]) == 3 * 11 + 3
    assert a["model.layers.1.self_attn.k_proj.weight"].shape == (32, 64)
    assert b["model.layers.2.self_attn.q_norm.weight"].shape == (32,)
    assert b["model.layers.0.mlp.down_proj.weight"].shape == (96, 160)
    assert b["lm_head.weight"].shape == (389, 96) and not b["lm_head.weight"].optional
    assert a["lm_head.weight"].optional


def test_model_folder_errors_name_the_tensors(tmp_path):
    d = make_folder("B", str(tmp_path / "m"))
    cfg = Qwen3Config.from_dict(TINY_B)
    model = model_skeleton(cfg)
    with safe_open(os.path.join(d, "model.safetensors"), "pt") as f:
        t = {k: f.get_tensor(k) for k in f.keys()}
    del t["model.layers.1.mlp.up_proj.weight"]
    del t["lm_head.weight"]
    t["model.layers.0.self_attn.q_norm.weight"] = torch.zeros(16)
    t["model.layers.7.extra"] = torch.zeros(1)
    with pytest.raises(WeightError) as ei:
        bind_tensors(model.all_tensor_specs(), DictSource(t))
    assert ei.value.missing == ["lm_head.weight", "model.layers.1.mlp.up_proj.weight"]
    assert ei.value.unexpected == ["model.layers.7.extra"]
    assert [w[0] for w in ei.value.wrong_shape] == ["model.layers.0.self_attn.q_norm.weight"]


def test_random_weights_are_seeded_per_tensor_name():
    specs = {"m": TensorSpec((64, 32)), "e": TensorSpec((100, 32), "embedding"), "g": TensorSpec((512,), "gain")}
    a = RandomSource(specs, 3, std_matrix=0.02, std_embedding=0.05, std_gain=0.1)
    b = RandomSource({"g": specs["g"], "m": specs["m"]}, 3, std_matrix=0.02, std_gain=0.1)
    assert torch.equal(a.get("m"), b.get("m")) and torch.equal(a.get("g"), b.get("g"))   # order and company do not matter
    assert not torch.equal(a.get("m"), RandomSource(specs, 4).get("m"))
    assert a.get("m").dtype == torch.bfloat16
    assert abs(a.get("m").float().std().item() - 0.02) < 0.002
    assert abs(a.get("e").float().std().item() - 0.05) < 0.005
    g = a.get("g").float()
    assert abs(g.mean().item() - 1.0) < 0.02 and abs(g.std().item() - 0.1) < 0.02
    g32 = RandomSource(specs, 3, gain_dtype=torch.float32).get("g")
    assert g32.dtype == torch.float32


def test_written_folder_loads_back(tmp_path):
    cfg = Qwen3Config.from_dict(TINY_A)
    d = write_model_folder(cfg, str(tmp_path / "a"), 0, std_gain=0.1)
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    src = SafetensorsSource(d)
    t = bind_tensors(model_skeleton(cfg).all_tensor_specs(), src)
    assert "lm_head.weight" not in t and len(t) == 24
    d2 = write_model_folder(cfg, str(tmp_path / "b"), 0, std_gain=0.1)
    assert open(os.path.join(d, "model.safetensors"), "rb").read() == open(os.path.join(d2, "model.safetensors"), "rb").read()
