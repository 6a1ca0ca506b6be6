"""Weights by name: round trip, the one error that lists everything, dtype rules, random mode."""
import json
import os
import struct
import tempfile

import pytest
import torch

from builderforce_inference_b200.registry import describe_model
from builderforce_inference_b200.weights import (SafetensorsError, SafetensorsFile, WeightsError, expected_tensors,
                                                 load_folder, random_tensors, write_model_folder,
                                                 write_safetensors)
from helpers import TINY_A, TINY_B, model_folder
from plain import qwen3_plain as P

CPU = torch.device("cpu")


def _load(folder, cfg, dtype=torch.float32):
    spec = describe_model(cfg)
    return load_folder(folder, expected_tensors(spec), spec.ignored_names, dtype, CPU)


def test_folder_round_trip_and_names():
    folder = model_folder("B", torch.bfloat16)
    t = _load(folder, TINY_B, torch.bfloat16)
    assert t["model.layers.2.self_attn.q_proj.weight"].shape == (192, 96)
    assert t["model.layers.0.self_attn.k_norm.weight"].shape == (32,)
    assert t["lm_head.weight"].shape == (384, 96)
    assert all(v.dtype == torch.bfloat16 for v in t.values())
    # the independent reader of the plain implementation sees the same bytes
    raw = P.read_safetensors(os.path.join(folder, "model.safetensors"))
    assert set(raw) == set(t)
    for k in t:
        assert torch.equal(raw[k], t[k])


def test_float32_run_widens_exactly_and_bfloat16_run_keeps_32bit_tensors():
    folder = model_folder("A", torch.bfloat16)
    wide = _load(folder, TINY_A, torch.float32)
    kept = _load(folder, TINY_A, torch.bfloat16)
    for k in wide:
        assert wide[k].dtype == torch.float32 and torch.equal(wide[k], kept[k].float())
    f32 = model_folder("A", torch.float32)
    t = _load(f32, TINY_A, torch.bfloat16)
    assert all(v.dtype == torch.float32 for v in t.values())     # stored in 32-bit, stays so


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    spec = describe_model(TINY_A)
    tensors = dict(random_tensors(expected_tensors(spec), 1, torch.float32, CPU))
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 32)
    tensors["model.layers.9.extra.weight"] = torch.zeros(3)
    d = tempfile.mkdtemp()
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(TINY_A, f)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors.items())
    with pytest.raises(WeightsError) as e:
        _load(d, TINY_A)
    err = e.value
    assert sorted(err.missing) == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.9.extra.weight"]
    assert err.wrong_shape == [("model.layers.0.self_attn.q_proj.weight", (64, 32), (64, 64))]
    msg = str(err)
    for word in ("model.norm.weight", "model.layers.9.extra.weight", "[64, 32]", "[64, 64]"):
        assert word in msg


def test_tied_model_ignores_a_stored_head_and_untied_model_needs_it():
    spec = describe_model(TINY_A)
    tensors = dict(random_tensors(expected_tensors(spec), 1, torch.float32, CPU))
    tensors["lm_head.weight"] = torch.zeros(256, 64)
    d = tempfile.mkdtemp()
    write_safetensors(os.path.join(d, "model.safetensors"), tensors.items())
    assert "lm_head.weight" not in _load(d, TINY_A)
    specb = describe_model(TINY_B)
    tb = dict(random_tensors(expected_tensors(specb), 1, torch.float32, CPU))
    del tb["lm_head.weight"]
    d2 = tempfile.mkdtemp()
    write_safetensors(os.path.join(d2, "model.safetensors"), tb.items())
    with pytest.raises(WeightsError, match="lm_head.weight"):
        _load(d2, TINY_B)


def test_integer_tables_become_int32_and_bad_dtypes_are_named():
    d = tempfile.mkdtemp()
    write_safetensors(os.path.join(d, "model.safetensors"),
                      [("table", torch.arange(6, dtype=torch.int64).reshape(2, 3)),
                       ("flag", torch.ones(2, dtype=torch.bool))])
    from builderforce_inference_b200.parts.base import ParamSpec
    out = load_folder(d, {"table": ParamSpec((2, 3), "table")}, ["flag"], torch.bfloat16, CPU)
    assert out["table"].dtype == torch.int32 and out["table"].tolist() == [[0, 1, 2], [3, 4, 5]]
    with pytest.raises(WeightsError, match="unusable dtype"):
        load_folder(d, {"flag": ParamSpec((2,), "norm")}, ["table"], torch.bfloat16, CPU)


def test_truncated_and_malformed_files():
    folder = model_folder("A", torch.float32)
    src = os.path.join(folder, "model.safetensors")
    raw = open(src, "rb").read()
    d = tempfile.mkdtemp()
    bad = os.path.join(d, "model.safetensors")
    open(bad, "wb").write(raw[:len(raw) - 100])
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(bad)
    open(bad, "wb").write(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(bad)
    hdr = b'{"a":{"dtype":"F32","shape":[1],"data_offsets":[0,4]},"a":{"dtype":"F32","shape":[1],"data_offsets":[0,4]}}'
    open(bad, "wb").write(struct.pack("<Q", len(hdr)) + hdr + b"\0\0\0\0")
    with pytest.raises(SafetensorsError, match="duplicate"):
        SafetensorsFile(bad)
    with pytest.raises(FileNotFoundError):
        _load(tempfile.mkdtemp(), TINY_A)


def test_sharded_folder():
    spec = describe_model(TINY_A)
    tensors = dict(random_tensors(expected_tensors(spec), 2, torch.float32, CPU))
    names = sorted(tensors)
    d = tempfile.mkdtemp()
    half = len(names) // 2
    parts = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
    for fname, ns in parts.items():
        write_safetensors(os.path.join(d, fname), [(n, tensors[n]) for n in ns])
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as f:
        json.dump({"weight_map": {n: fn for fn, ns in parts.items() for n in ns}}, f)
    got = _load(d, TINY_A)
    assert all(torch.equal(got[n], tensors[n]) for n in names)


def test_random_weights_depend_on_seed_and_name_only():
    spec = describe_model(TINY_A)
    exp = expected_tensors(spec)
    a = dict(random_tensors(exp, 5, torch.float32, CPU))
    b = dict(random_tensors(dict(reversed(list(exp.items()))), 5, torch.float32, CPU))
    c = dict(random_tensors(exp, 6, torch.float32, CPU))
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.norm.weight"], c["model.norm.weight"])
    w = a["model.layers.0.mlp.gate_proj.weight"]
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
    n = a["model.layers.0.input_layernorm.weight"]
    assert abs(float(n.mean()) - 1.0) < 0.05 and 0.05 < float(n.std()) < 0.2
    d = tempfile.mkdtemp()
    write_model_folder(TINY_A, 5, d, torch.float32)
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    assert json.load(open(os.path.join(d, "config.json")))["vocab_size"] == 256


def test_random_fill_is_the_closed_formula_bit_for_bit():
    """The product's numpy fill against the plain restatement in Python integers, float32 and
    bfloat16, for matrices and norm weights, at scattered indices of a large tensor too."""
    from plain import random_fill_plain as R
    from builderforce_inference_b200.parts.base import ParamSpec
    from builderforce_inference_b200.weights.random_init import random_tensor
    for role, shape in (("matrix", (37, 53)), ("norm", (301,)), ("table", (70001, 3))):
        t = random_tensor("some.tensor", ParamSpec(shape, role), 9, torch.float32, CPU).reshape(-1)
        tb = random_tensor("some.tensor", ParamSpec(shape, role), 9, torch.bfloat16, CPU).reshape(-1)
        n = t.numel()
        for i in sorted({0, 1, 2, 63, 64, n // 3, 65535 % n, 65536 % n, n - 2, n - 1}):
            want = R.value(9, "some.tensor", i, role)
            assert float(t[i]) == want, (role, i)
            assert int(tb[i].view(torch.int16)) & 0xFFFF == R.bf16_bits(want), (role, i)
    big = random_tensor("w", ParamSpec((1000, 1000)), 3, torch.float32, CPU)
    assert abs(float(big.std()) - 0.02) < 2e-4 and abs(float(big.mean())) < 1e-4
    assert float(big.abs().max()) <= 0.02 * 4.9
