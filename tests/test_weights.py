import json
import struct

import numpy as np
import pytest
import torch

from gguf2bin_b200.config import model_spec_from_dict
from gguf2bin_b200.engine.model import expected_tensors
from gguf2bin_b200.weights import (Expected, SafetensorsFile, WeightsError, load_weights,
                                   runtime_dtype, write_random_model, write_safetensors)
from helpers import TINY
from plain import qwen3_plain as P


def folder_with(tmp_path, tensors, name="a"):
    (tmp_path / "config.json").write_text(json.dumps(TINY[name]))
    write_safetensors(tmp_path / "model.safetensors",
                      [(n, tuple(t.shape), t.dtype, (lambda t=t: t)) for n, t in tensors.items()])
    return tmp_path


def good_tensors(name="a", dtype=torch.float32):
    exp = expected_tensors(model_spec_from_dict(TINY[name]))
    return {n: torch.zeros(e.shape, dtype=dtype) for n, e in exp.items() if not e.optional}, exp


def test_random_model_roundtrip_and_own_reader(tmp_path):
    folder = write_random_model(tmp_path / "m", TINY["b"], seed=5, dtype="bfloat16")
    exp = expected_tensors(model_spec_from_dict(TINY["b"]))
    got = load_weights(folder, exp, torch.bfloat16, "cpu")
    cfg, W = P.read_model_folder(folder)                      # the tests' own reader agrees
    assert set(W) == set(got)
    for n, t in got.items():
        assert t.dtype == torch.bfloat16 and tuple(t.shape) == tuple(exp[n].shape)
        assert np.array_equal(t.float().numpy(), W[n])
    m = got["model.layers.1.mlp.up_proj.weight"].float()
    assert abs(m.std().item() - 0.02) < 0.002 and abs(m.mean().item()) < 0.002
    nrm = got["model.layers.2.input_layernorm.weight"].float()
    assert abs(nrm.mean().item() - 1.0) < 0.05 and 0.05 < nrm.std().item() < 0.15
    again = write_random_model(tmp_path / "m2", TINY["b"], seed=5, dtype="bfloat16")
    assert (folder / "model.safetensors").read_bytes() == (again / "model.safetensors").read_bytes()
    other = write_random_model(tmp_path / "m3", TINY["b"], seed=6, dtype="bfloat16")
    assert (folder / "model.safetensors").read_bytes() != (other / "model.safetensors").read_bytes()


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    tensors, exp = good_tensors()
    del tensors["model.layers.0.self_attn.q_norm.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64)
    tensors["model.layers.1.mlp.down_proj.weight"] = torch.zeros(128, 64)
    with pytest.raises(WeightsError) as e:
        load_weights(folder_with(tmp_path, tensors), exp, torch.float32, "cpu")
    msg = str(e.value)
    assert "missing (2)" in msg and "model.layers.0.self_attn.q_norm.weight" in msg
    assert "model.norm.weight" in msg
    assert "unexpected (1)" in msg and "q_proj.bias" in msg
    assert "wrong shape (1)" in msg and "found [128, 64], expected [64, 128]" in msg


def test_tied_head_may_be_absent_or_present(tmp_path):
    tensors, exp = good_tensors("a")
    assert "lm_head.weight" not in tensors and exp["lm_head.weight"].optional
    load_weights(folder_with(tmp_path, tensors), exp, torch.float32, "cpu")
    tensors["lm_head.weight"] = torch.zeros(256, 64)
    load_weights(folder_with(tmp_path, tensors), exp, torch.float32, "cpu")
    t2, exp_b = good_tensors("b")
    del t2["lm_head.weight"]                                  # untied: required
    with pytest.raises(WeightsError, match="lm_head.weight"):
        load_weights(folder_with(tmp_path, t2, "b"), exp_b, torch.float32, "cpu")


def test_precision_policy():
    assert runtime_dtype(torch.bfloat16, torch.bfloat16) == torch.bfloat16
    assert runtime_dtype(torch.float16, torch.bfloat16) == torch.bfloat16
    assert runtime_dtype(torch.float32, torch.bfloat16) == torch.float32   # 32-bit stays
    assert runtime_dtype(torch.bfloat16, torch.float32) == torch.float32
    assert runtime_dtype(torch.int64, torch.bfloat16) == torch.int32
    assert runtime_dtype(torch.int64, torch.float32) == torch.int32


def test_mixed_storage_is_kept(tmp_path):
    tensors, exp = good_tensors("a", torch.bfloat16)
    tensors["model.norm.weight"] = torch.ones(64, dtype=torch.float32)
    got = load_weights(folder_with(tmp_path, tensors), exp, torch.bfloat16, "cpu")
    assert got["model.norm.weight"].dtype == torch.float32
    assert got["model.embed_tokens.weight"].dtype == torch.bfloat16


def test_broken_files(tmp_path):
    p = tmp_path / "model.safetensors"
    (tmp_path / "config.json").write_text(json.dumps(TINY["a"]))
    exp = {"x": Expected((4,))}
    with pytest.raises(WeightsError, match="neither"):
        load_weights(tmp_path / "nowhere", exp, torch.float32, "cpu")
    p.write_bytes(b"\x01\x02")
    with pytest.raises(WeightsError, match="too short"):
        load_weights(tmp_path, exp, torch.float32, "cpu")
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(WeightsError, match="header length"):
        load_weights(tmp_path, exp, torch.float32, "cpu")
    hdr = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)          # truncated data
    with pytest.raises(WeightsError, match="truncated"):
        load_weights(tmp_path, exp, torch.float32, "cpu")
    p.write_bytes(struct.pack("<Q", 5) + b"{nope")
    with pytest.raises(WeightsError, match="JSON"):
        load_weights(tmp_path, exp, torch.float32, "cpu")
    hdr = json.dumps({"x": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 4)
    with pytest.raises(WeightsError, match="unsupported dtype"):
        load_weights(tmp_path, exp, torch.float32, "cpu")


def test_shards_and_duplicates(tmp_path):
    a, b = torch.arange(4.0), torch.arange(6.0).reshape(2, 3)
    write_safetensors(tmp_path / "s1.safetensors", [("a", (4,), torch.float32, lambda: a)])
    write_safetensors(tmp_path / "s2.safetensors", [("b", (2, 3), torch.float32, lambda: b)])
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}))
    got = load_weights(tmp_path, {"a": Expected((4,)), "b": Expected((2, 3))}, torch.float32, "cpu")
    assert torch.equal(got["a"], a) and torch.equal(got["b"], b)
    write_safetensors(tmp_path / "s2.safetensors", [("b", (2, 3), torch.float32, lambda: b),
                                                    ("a", (4,), torch.float32, lambda: a)])
    with pytest.raises(WeightsError, match="more than one shard"):
        load_weights(tmp_path, {"a": Expected((4,)), "b": Expected((2, 3))}, torch.float32, "cpu")


def test_random_values_follow_the_plain_definition(monkeypatch):
    """The package's numpy generator against the element-at-a-time copy of its definition,
    bit for bit; a tensor made in several chunks equals the one made at once; the stream of
    a tensor does not depend on the other tensors."""
    import torch
    from plain import philox_normal_plain as Q
    from gguf2bin_b200.weights import normal_values, random_tensor, random_init
    for seed, tensor, n in ((0, 0, 9), (77, 5, 1003), (2 ** 40 + 3, 290, 64)):
        z = normal_values(n, seed, tensor)
        ref = np.array([Q.standard_normal(seed, tensor, i) for i in range(n)], np.float32)
        assert np.array_equal(z.view(np.uint32), ref.view(np.uint32))
    assert np.array_equal(normal_values(40, 3, 1, first=8), normal_values(48, 3, 1)[8:])
    e_m, e_s = Expected((7, 13)), Expected((19,), init="scale")
    m = random_tensor(e_m, 5, 2, torch.bfloat16, 0.02, 0.1)
    s = random_tensor(e_s, 5, 3, torch.float32, 0.02, 0.1)
    bits = m.view(torch.int16).numpy().astype(np.uint16).reshape(-1)
    assert [int(b) for b in bits] == [Q.to_bfloat16_bits(Q.value(5, 2, i, "matrix", 0.02)) for i in range(91)]
    assert [float(v) for v in s] == [float(Q.value(5, 3, i, "scale", 0.1)) for i in range(19)]
    monkeypatch.setattr(random_init, "_CHUNK", 16)
    assert torch.equal(random_tensor(e_m, 5, 2, torch.bfloat16, 0.02, 0.1), m)
    big = normal_values(400_000, 1, 0)
    assert abs(big.mean()) < 0.01 and abs(big.std() - 1) < 0.01
    assert abs((big ** 4).mean() / big.var() ** 2 - 3) < 0.05 and np.abs(big).max() > 4
