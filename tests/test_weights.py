"""Safetensors by name, one clear error for every mismatch, and the random-weights mode."""
import json
import os
import struct

import pytest
import torch

from pih_b200.config import config_from_dict
from pih_b200.models import expected_tensors
from pih_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, load_weights, random_tensors,
                              write_random_model, write_safetensors)


def _expected(raw):
    spec = config_from_dict(raw).model_spec()
    return spec, {n: i.shape for n, i in expected_tensors(spec).items()}


def test_expected_names_are_the_checkpoint_names(tiny_configs):
    _, exp_a = _expected(tiny_configs["A"])
    assert "lm_head.weight" not in exp_a                       # tied
    assert len(exp_a) == 2 + 11 * 2
    assert exp_a["model.layers.1.self_attn.q_proj.weight"] == (64, 64)
    assert exp_a["model.layers.0.self_attn.k_norm.weight"] == (16,)
    _, exp_b = _expected(tiny_configs["B"])
    assert exp_b["lm_head.weight"] == (384, 96) and len(exp_b) == 3 + 11 * 3
    assert exp_b["model.layers.2.self_attn.q_proj.weight"] == (192, 96)   # heads * head_dim != hidden
    assert exp_b["model.layers.2.self_attn.o_proj.weight"] == (96, 192)
    assert exp_b["model.layers.0.mlp.down_proj.weight"] == (96, 224)


def test_random_model_folder_loads_and_is_reproducible(tmp_path, tiny_configs):
    cfg = config_from_dict(tiny_configs["B"])
    d1 = write_random_model(str(tmp_path / "m1"), cfg, seed=1, sigma=0.05)
    d2 = write_random_model(str(tmp_path / "m2"), cfg, seed=1, sigma=0.05)
    d3 = write_random_model(str(tmp_path / "m3"), cfg, seed=2, sigma=0.05)
    assert sorted(os.listdir(d1)) == ["config.json", "model.safetensors"]
    _, exp = _expected(tiny_configs["B"])
    w1, w2, w3 = (load_weights(d, exp) for d in (d1, d2, d3))
    assert set(w1) == set(exp)
    for n in exp:
        assert w1[n].dtype == torch.bfloat16 and tuple(w1[n].shape) == exp[n]
        assert torch.equal(w1[n], w2[n])
    assert not torch.equal(w1["lm_head.weight"], w3["lm_head.weight"])
    norm = w1["model.layers.0.input_layernorm.weight"].float()
    assert abs(float(norm.mean()) - 1.0) < 0.05 and abs(float(w1["lm_head.weight"].float().std()) - 0.05) < 0.005
    with open(os.path.join(d1, "config.json")) as f:
        assert config_from_dict(json.load(f)) == cfg


def test_values_depend_on_the_name_only(tiny_configs):
    spec, _ = _expected(tiny_configs["A"])
    full = random_tensors(expected_tensors(spec), seed=3)
    one = {"model.norm.weight": expected_tensors(spec)["model.norm.weight"]}
    assert torch.equal(random_tensors(one, seed=3)["model.norm.weight"], full["model.norm.weight"])


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path, tiny_configs):
    spec, exp = _expected(tiny_configs["A"])
    tensors = random_tensors(expected_tensors(spec), seed=0)
    del tensors["model.layers.0.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.9.extra.weight"] = torch.zeros(3, dtype=torch.bfloat16)
    tensors["model.layers.1.self_attn.q_norm.weight"] = torch.zeros(17, dtype=torch.bfloat16)
    tensors["model.embed_tokens.weight"] = torch.zeros(64, 256, dtype=torch.bfloat16)
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    with pytest.raises(WeightError) as info:
        load_weights(str(tmp_path), exp)
    e = info.value
    assert e.missing == ["model.layers.0.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.9.extra.weight"]
    assert [w[0] for w in e.wrong_shape] == ["model.embed_tokens.weight", "model.layers.1.self_attn.q_norm.weight"]
    text = str(e)
    for needle in ("missing (2)", "unexpected (1)", "wrong shape (2)", "model.norm.weight",
                   "model.layers.9.extra.weight", "is [17], expected [16]"):
        assert needle in text


def test_stored_dtypes_are_kept_and_integers_become_int32(tmp_path):
    tensors = {"a": torch.randn(4, 3).to(torch.bfloat16), "b": torch.randn(5), "c": torch.arange(6, dtype=torch.int64)}
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    got = load_weights(str(tmp_path), {"a": (4, 3), "b": (5,), "c": (6,)})
    assert got["a"].dtype == torch.bfloat16 and got["b"].dtype == torch.float32 and got["c"].dtype == torch.int32
    assert torch.equal(got["b"], tensors["b"]) and got["c"].tolist() == list(range(6))


def test_tied_head_may_be_stored_anyway(tmp_path, tiny_configs):
    spec, exp = _expected(tiny_configs["A"])
    tensors = random_tensors(expected_tensors(spec), seed=0)
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    got = load_weights(str(tmp_path), exp, optional={"lm_head.weight": (256, 64)})
    assert "lm_head.weight" in got


def test_sharded_folder(tmp_path, tiny_configs):
    spec, exp = _expected(tiny_configs["A"])
    tensors = random_tensors(expected_tensors(spec), seed=0)
    names = sorted(tensors)
    half = len(names) // 2
    write_safetensors(str(tmp_path / "s1.safetensors"), {n: tensors[n] for n in names[:half]})
    write_safetensors(str(tmp_path / "s2.safetensors"), {n: tensors[n] for n in names[half:]})
    index = {"weight_map": {n: ("s1.safetensors" if i < half else "s2.safetensors") for i, n in enumerate(names)}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    got = load_weights(str(tmp_path), exp)
    assert all(torch.equal(got[n], tensors[n]) for n in names)


def test_container_faults_are_refused(tmp_path):
    p = str(tmp_path / "x.safetensors")
    header = json.dumps({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}).encode()
    with open(p, "wb") as f:                       # payload shorter than the record says
        f.write(struct.pack("<Q", len(header)) + header + b"\0" * 4)
    with pytest.raises(SafetensorsError):
        SafetensorsFile(p)
    header = json.dumps({"a": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}).encode()
    with open(p, "wb") as f:                       # a gap before the first tensor
        f.write(struct.pack("<Q", len(header)) + header + b"\0" * 12)
    with pytest.raises(SafetensorsError, match="gap"):
        SafetensorsFile(p)
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", 1 << 40))
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(p)


def test_matches_the_safetensors_package_when_it_is_there(tmp_path):
    st = pytest.importorskip("safetensors.torch")
    tensors = {"w": torch.randn(7, 5).to(torch.bfloat16), "v": torch.randn(3)}
    ours, theirs = str(tmp_path / "ours.safetensors"), str(tmp_path / "theirs.safetensors")
    write_safetensors(ours, tensors)
    st.save_file(tensors, theirs)
    back = st.load_file(ours)
    with SafetensorsFile(theirs) as f:
        for n in tensors:
            assert torch.equal(back[n], tensors[n]) and torch.equal(f.read_tensor(n), tensors[n])
