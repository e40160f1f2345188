"""The safetensors container and the loader's errors, after the reference's
`safetensors/safetensors_test.go:62-257` (single file, shards, duplicate across shards,
missing shard, malformed or empty index, missing model) plus the one error that lists
missing, unexpected and misshapen tensors, the dtype policy and the random-weights mode."""
from __future__ import annotations

import json
import os
import struct

import pytest
import torch

import janis_b200
from janis_b200.weights.loader import (TensorSpec, WeightsError, check_tensors, load_tensors, random_tensor,
                                       random_tensors, stored_to_kept)
from janis_b200.weights.safetensors import SafetensorsError, SafetensorsFile, open_model, write_safetensors
from tests.conftest import TINY_A, TINY_B, write_tiny


def test_write_then_read_every_dtype(tmp_path):
    t = {"a.f32": torch.randn(3, 5), "b.bf16": torch.randn(4, 2).bfloat16(), "c.f16": torch.randn(7).half(),
         "d.i32": torch.arange(6, dtype=torch.int32).view(2, 3), "e.i64": torch.tensor([2 ** 40, -1]),
         "f.u8": torch.tensor([0, 255], dtype=torch.uint8), "g.bool": torch.tensor([True, False, True]),
         "h.scalar": torch.tensor(3.5)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t, {"k": "v"})
    f = SafetensorsFile(p)
    assert f.names() == sorted(t) and f.metadata == {"k": "v"}
    for n, want in t.items():
        got = f.read(n)
        assert got.dtype == want.dtype and got.shape == want.shape and torch.equal(got, want), n
    f.close()


def test_the_library_package_reads_what_we_write(tmp_path):
    """An independent reader (the installed safetensors package) agrees with the writer."""
    st = pytest.importorskip("safetensors.torch")
    t = {"w": torch.randn(5, 3).bfloat16(), "n": torch.randn(4)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t)
    back = st.load_file(p)
    assert set(back) == set(t) and all(torch.equal(back[k], t[k]) for k in t)
    st.save_file(t, str(tmp_path / "y.safetensors"))
    f = SafetensorsFile(str(tmp_path / "y.safetensors"))
    assert all(torch.equal(f.read(k), t[k]) for k in t)


def _raw_file(path, header: dict, data: bytes = b""):
    blob = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)) + blob + data)


@pytest.mark.parametrize("make,match", [
    (lambda p: open(p, "wb").write(b"\x01\x02"), "too short"),
    (lambda p: open(p, "wb").write(struct.pack("<Q", 10 ** 9) + b"{}"), "does not fit"),
    (lambda p: open(p, "wb").write(struct.pack("<Q", 5) + b"{not}"), "not valid JSON"),
    (lambda p: _raw_file(p, {"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}, b"\0" * 8), "outside"),
    (lambda p: _raw_file(p, {"t": {"dtype": "F32", "shape": [3], "data_offsets": [0, 16]}}, b"\0" * 16), "need 12"),
    (lambda p: _raw_file(p, {"t": {"dtype": "F8_E4M3", "shape": [1], "data_offsets": [0, 1]}}, b"\0"), "unsupported dtype"),
    (lambda p: _raw_file(p, {"t": {"dtype": "F32"}}), "malformed header entry"),
])
def test_broken_files_are_errors(tmp_path, make, match):
    p = str(tmp_path / "bad.safetensors")
    make(p)
    with pytest.raises(SafetensorsError, match=match):
        SafetensorsFile(p)


def test_shards(tmp_path):
    d = str(tmp_path)
    write_safetensors(os.path.join(d, "s1.safetensors"), {"a": torch.ones(2), "b": torch.zeros(3)})
    write_safetensors(os.path.join(d, "s2.safetensors"), {"c": torch.full((2, 2), 7.0)})
    write_safetensors(os.path.join(d, "s3.safetensors"), {"d": torch.arange(3.0)})
    idx = {"weight_map": {"a": "s1.safetensors", "b": "s1.safetensors", "c": "s2.safetensors", "d": "s3.safetensors"}}
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as f:
        json.dump(idx, f)
    m = open_model(d)
    assert m.names() == ["a", "b", "c", "d"] and torch.equal(m.read("c"), torch.full((2, 2), 7.0))
    with pytest.raises(SafetensorsError, match="'z' not found"):
        m.read("z")
    m.close()
    # the same tensor in two shards
    write_safetensors(os.path.join(d, "s3.safetensors"), {"a": torch.ones(2)})
    with pytest.raises(SafetensorsError, match="duplicate tensor 'a' across shards"):
        open_model(d)
    # a shard that is not there
    os.unlink(os.path.join(d, "s3.safetensors"))
    with pytest.raises(SafetensorsError, match="s3.safetensors"):
        open_model(d)


@pytest.mark.parametrize("index,match", [("{broken", "cannot read the shard index"), ("{}", "weight_map is missing or empty"),
                                         ('{"weight_map": {}}', "weight_map is missing or empty")])
def test_bad_index(tmp_path, index, match):
    (tmp_path / "model.safetensors.index.json").write_text(index)
    with pytest.raises(SafetensorsError, match=match):
        open_model(str(tmp_path))


def test_no_model_at_all(tmp_path):
    with pytest.raises(SafetensorsError, match="no model.safetensors"):
        open_model(str(tmp_path))


def test_one_error_lists_missing_unexpected_and_misshapen(tmp_path):
    d = str(tmp_path)
    write_tiny(d, TINY_A, seed=1)
    _, _, model = janis_b200.build_model(TINY_A)
    specs = model.tensor_specs()
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    tensors = {n: f.read(n) for n in f.names()}
    f.close()
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 32, dtype=torch.bfloat16)
    tensors["model.layers.0.input_layernorm.weight"] = torch.zeros(64, dtype=torch.int32)
    tensors["model.layers.9.extra.weight"] = torch.zeros(2)
    tensors["lm_head.weight"] = torch.zeros(4)                # ignorable for a tied model
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    with pytest.raises(WeightsError) as e:
        load_tensors(d, specs, "cpu", model.ignorable_tensors)
    msg = str(e.value)
    assert "missing tensors (2)" in msg and "model.layers.1.mlp.up_proj.weight  [128, 64]" in msg
    assert "model.norm.weight" in msg
    assert "unexpected tensors (1)" in msg and "model.layers.9.extra.weight" in msg and "lm_head" not in msg
    assert "wrong shape or dtype (2)" in msg
    assert "q_proj.weight: expected shape [64, 64], found [64, 32]" in msg
    assert "input_layernorm.weight: expected floating point, found dtype I32" in msg


def test_a_config_of_another_size_does_not_load(tmp_path):
    d = str(tmp_path)
    write_tiny(d, TINY_A, seed=1)
    _, _, model = janis_b200.build_model(TINY_B)
    with pytest.raises(WeightsError, match="missing tensors"):
        load_tensors(d, model.tensor_specs(), "cpu")


def test_dtype_policy(tmp_path):
    assert stored_to_kept(torch.zeros(2, dtype=torch.bfloat16), False).dtype == torch.bfloat16
    assert stored_to_kept(torch.zeros(2, dtype=torch.float16), False).dtype == torch.bfloat16
    assert stored_to_kept(torch.zeros(2, dtype=torch.float32), False).dtype == torch.float32
    assert stored_to_kept(torch.zeros(2, dtype=torch.float64), False).dtype == torch.float32
    assert stored_to_kept(torch.zeros(2, dtype=torch.int64), True).dtype == torch.int32
    d = str(tmp_path)
    write_tiny(d, TINY_B, seed=2, norms_f32=True)
    _, _, model = janis_b200.build_model(TINY_B)
    t = load_tensors(d, model.tensor_specs(), "cpu")
    assert t["model.norm.weight"].dtype == torch.float32                       # stored in 32-bit, stays so
    assert t["model.layers.0.mlp.down_proj.weight"].dtype == torch.bfloat16


def test_random_weights_are_a_function_of_seed_and_name(tmp_path):
    a = random_tensor("x.weight", TensorSpec((8, 4)), 5)
    assert torch.equal(a, random_tensor("x.weight", TensorSpec((8, 4)), 5))
    assert not torch.equal(a, random_tensor("y.weight", TensorSpec((8, 4)), 5))
    assert not torch.equal(a, random_tensor("x.weight", TensorSpec((8, 4)), 6))
    both = random_tensors({"x.weight": TensorSpec((8, 4)), "z": TensorSpec((3,), init_std=0.1)}, 5)
    assert torch.equal(both["x.weight"], a)                                    # order and company do not matter
    d1, d2 = str(tmp_path / "a"), str(tmp_path / "b")
    janis_b200.write_random_model(d1, TINY_B, seed=9)
    janis_b200.write_random_model(d2, TINY_B, seed=9)
    with open(os.path.join(d1, "model.safetensors"), "rb") as f1, open(os.path.join(d2, "model.safetensors"), "rb") as f2:
        assert f1.read() == f2.read()
    cfg = janis_b200.Gemma2Config.from_dict(json.load(open(os.path.join(d1, "config.json"))))
    assert cfg == janis_b200.Gemma2Config.from_dict(TINY_B)
    f = SafetensorsFile(os.path.join(d1, "model.safetensors"))
    w = f.read("model.layers.0.mlp.gate_proj.weight").float()
    n = f.read("model.layers.0.input_layernorm.weight").float()
    assert abs(w.std().item() - 0.02) < 0.002 and abs(n.std().item() - 0.1) < 0.03
    f.close()


def test_random_weights_have_the_asked_spread_and_do_not_repeat():
    """Mean 0, the standard deviation asked for, a bell (kurtosis near 3, nothing beyond 6 deviations), no
    correlation between neighbours, between rows or between tensors, and a prefix of a longer tensor of the same
    name equals the shorter one (a value is a function of seed, name and index alone: chunks cannot matter)."""
    n = (1 << 24) + 12345                              # more than one chunk of the generator
    a = random_tensor("m.weight", TensorSpec((n,), init_std=0.02), 7, dtype=torch.float32)
    x = (a / 0.02).double()
    assert abs(x.mean().item()) < 3e-3 and abs(x.std().item() - 1.0) < 3e-3
    assert 2.8 < (x ** 4).mean().item() < 3.1 and x.abs().max().item() <= 6.0
    assert abs((x[:-1] * x[1:]).mean().item()) < 3e-3 and abs((x[:-4096] * x[4096:]).mean().item()) < 3e-3
    b = random_tensor("n.weight", TensorSpec((n,), init_std=0.02), 7, dtype=torch.float32)
    assert abs(((b / 0.02).double() * x).mean().item()) < 3e-3
    short = random_tensor("m.weight", TensorSpec((1000,), init_std=0.02), 7, dtype=torch.float32)
    assert torch.equal(short, a[:1000])
    ints = random_tensor("t.table", TensorSpec((5000,), integer=True), 7)
    assert ints.dtype == torch.int32 and 0 <= int(ints.min()) and int(ints.max()) < 2 ** 15 and len(ints.unique()) > 4000


@pytest.mark.gpu
def test_random_weights_are_the_same_bits_on_every_device():
    for spec, dt in ((TensorSpec((300, 77), init_std=0.02), torch.bfloat16), (TensorSpec((5000,), init_std=0.1), torch.float32),
                     (TensorSpec((64, 3), integer=True), torch.bfloat16)):
        cpu = random_tensor("model.layers.3.x.weight", spec, 11, "cpu", dt)
        gpu = random_tensor("model.layers.3.x.weight", spec, 11, "cuda:0", dt)
        assert gpu.is_cuda and torch.equal(cpu, gpu.cpu())
