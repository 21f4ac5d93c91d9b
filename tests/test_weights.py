"""Safetensors container, tensors by name, and the one error that lists what does not fit."""
import json
import os
import struct

import pytest
import torch

from ferrox_b200 import SafetensorsError, WeightsError, resolve, write_random_model
from ferrox_b200.parts.build import build_model
from ferrox_b200.weights import loader as wl
from ferrox_b200.weights.safetensors_io import ModelFiles, SafetensorsFile, write_safetensors
from tiny_configs import TINY_A, TINY_B

import plain_qwen2moe as plain


def test_write_and_read_back(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).reshape(2, 3)}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, t, metadata={"k": "v"})
    f = SafetensorsFile(path)
    assert f.metadata == {"k": "v"}
    for n, v in t.items():
        got = f.tensor(n)
        assert got.dtype == v.dtype and torch.equal(got, v)


def test_plain_reader_agrees_with_engine_reader(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), TINY_A, seed=3)
    a = plain.read_safetensors(os.path.join(folder, "model.safetensors"))
    f = ModelFiles(folder)
    assert set(a) == set(f.names())
    for n in a:
        assert torch.equal(a[n], f.tensor(n).to(torch.float32))


def _raw(path, header: dict, data: bytes, pad=b""):
    h = json.dumps(header).encode() + pad
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + data)


def test_container_errors(tmp_path):
    p = str(tmp_path / "bad.safetensors")
    open(p, "wb").write(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="exceeds"):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 100) + b"{}")
    with pytest.raises(SafetensorsError, match="does not fit"):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 4) + b"{{{{")
    with pytest.raises(SafetensorsError, match="not JSON"):
        SafetensorsFile(p)
    _raw(p, {"w": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 12]}}, b"\0" * 12)
    with pytest.raises(SafetensorsError, match="needs 16"):
        SafetensorsFile(p)
    _raw(p, {"w": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}, b"\0" * 12)
    with pytest.raises(SafetensorsError, match="gap"):
        SafetensorsFile(p)
    _raw(p, {"w": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
             "v": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}, b"\0" * 12)
    with pytest.raises(SafetensorsError, match="overlaps"):
        SafetensorsFile(p)
    _raw(p, {"w": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 12)
    with pytest.raises(SafetensorsError, match="cover 8 bytes"):
        SafetensorsFile(p)
    _raw(p, {"w": {"dtype": "Q4", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 8)
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        SafetensorsFile(p)
    with pytest.raises(SafetensorsError, match="neither"):
        ModelFiles(str(tmp_path))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), TINY_A, seed=0)
    tensors = plain.read_safetensors(os.path.join(folder, "model.safetensors"))
    del tensors["model.layers.1.self_attn.k_proj.bias"]
    del tensors["model.layers.0.mlp.experts.3.up_proj.weight"]
    tensors["model.layers.0.mlp.experts.4.up_proj.weight"] = torch.zeros(32, 64)  # an expert too many
    tensors["model.norm.weight"] = torch.zeros(65)
    tensors["lm_head.weight"] = tensors["lm_head.weight"].T.contiguous()
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    _, spec = resolve(TINY_A)
    model = build_model(spec)
    with pytest.raises(WeightsError) as e:
        wl.open_folder(folder, model.tensor_decls(), "cpu", torch.float32)
    msg = str(e.value)
    assert "missing (2)" in msg and "model.layers.1.self_attn.k_proj.bias" in msg
    assert "model.layers.0.mlp.experts.3.up_proj.weight" in msg
    assert "unexpected (1)" in msg and "experts.4.up_proj" in msg
    assert "wrong shape (2)" in msg and "model.norm.weight: expected [64], found [65]" in msg
    assert "lm_head.weight: expected [256, 64], found [64, 256]" in msg


def test_tied_model_rejects_a_head_tensor(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), TINY_B, seed=1)
    tensors = plain.read_safetensors(os.path.join(folder, "model.safetensors"))
    assert "lm_head.weight" not in tensors
    tensors["lm_head.weight"] = torch.zeros(384, 128)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    _, spec = resolve(TINY_B)
    with pytest.raises(WeightsError, match="unexpected"):
        wl.open_folder(folder, build_model(spec).tensor_decls(), "cpu", torch.float32)


def test_optional_gate_vector_may_be_absent(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), TINY_A, seed=0, optional_tensors=False)
    names = set(ModelFiles(folder).names())
    assert not any("shared_expert_gate" in n for n in names)
    _, spec = resolve(TINY_A)
    wl.open_folder(folder, build_model(spec).tensor_decls(), "cpu", torch.float32)  # no error


def test_resident_dtypes():
    bf, f32 = torch.bfloat16, torch.float32
    assert wl.resident_dtype(bf, bf) == bf
    assert wl.resident_dtype(f32, bf) == f32  # stored in 32 bits: stays so
    assert wl.resident_dtype(torch.float16, bf) == bf
    assert wl.resident_dtype(bf, f32) == f32
    assert wl.resident_dtype(torch.int64, bf) == torch.int32


def test_random_mode_is_seeded_and_order_free(tmp_path):
    a = write_random_model(str(tmp_path / "a"), TINY_A, seed=7)
    b = write_random_model(str(tmp_path / "b"), TINY_A, seed=7)
    c = write_random_model(str(tmp_path / "c"), TINY_A, seed=8)
    ta, tb, tc = (plain.read_safetensors(os.path.join(f, "model.safetensors")) for f in (a, b, c))
    assert all(torch.equal(ta[n], tb[n]) for n in ta)
    assert not torch.equal(ta["lm_head.weight"], tc["lm_head.weight"])
    assert torch.equal(ta["model.norm.weight"], torch.ones(64))
    w = ta["model.layers.0.self_attn.q_proj.weight"]
    assert abs(float(w.std()) - 0.02) < 0.003 and abs(float(w.mean())) < 0.002
    with open(os.path.join(a, "config.json")) as f:
        assert json.load(f)["architectures"] == ["Qwen2MoeForCausalLM"]
    # sharded folders read the same
    half = sorted(ta)[: len(ta) // 2]
    os.makedirs(tmp_path / "s")
    write_safetensors(str(tmp_path / "s" / "p1.safetensors"), {n: ta[n] for n in half})
    write_safetensors(str(tmp_path / "s" / "p2.safetensors"), {n: ta[n] for n in ta if n not in half})
    with open(tmp_path / "s" / "model.safetensors.index.json", "w") as f:
        json.dump({"weight_map": {n: ("p1.safetensors" if n in half else "p2.safetensors") for n in ta}}, f)
    mf = ModelFiles(str(tmp_path / "s"))
    assert all(torch.equal(mf.tensor(n), ta[n]) for n in ta)


def test_the_random_rule_is_a_function_of_key_and_index_only():
    """A tensor's values depend on (seed, name, element index) alone: a longer draw starts with the shorter one, an
    odd length ends inside a pair, and the stream looks like N(mean, std)."""
    from ferrox_b200.weights import random_init as ri

    key = ri.tensor_key(3, "model.layers.0.mlp.gate.weight")
    assert key == ri.tensor_key(3, "model.layers.0.mlp.gate.weight") != ri.tensor_key(4, "model.layers.0.mlp.gate.weight")
    long = ri.normal_cpu(key, 200_001, 0.0, 1.0)
    assert torch.equal(ri.normal_cpu(key, 777, 0.0, 1.0), long[:777])
    assert abs(float(long.mean())) < 0.01 and abs(float(long.std()) - 1.0) < 0.01
    assert 3.5 < float(long.abs().max()) < 6.5
    # a normal's fourth moment, and no correlation inside the pairs that share a radius
    assert abs(float((long ** 4).mean()) - 3.0) < 0.15
    assert abs(float((long[0:-1:2] * long[1::2]).mean())) < 0.01
    shifted = ri.normal_cpu(key, 1000, 1.0, 0.02)
    assert abs(float(shifted.mean()) - 1.0) < 0.003 and abs(float(shifted.std()) - 0.02) < 0.003
