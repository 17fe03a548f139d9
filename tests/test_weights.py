"""Safetensors container, loading by name, the one error, random-weights mode (no GPU)."""
import json
import os
import struct

import pytest
import torch

from helpers import TINY_A, TINY_B, make_weights
from yalm_b200.config import config_from_dict
from yalm_b200.engine.lm import tensor_needs_of
from yalm_b200.weights import (SafetensorsError, WeightsError, check_tensors,
                               load_checkpoint, read_file, write_file, write_model_dir)


def test_container_round_trip_and_type_rules(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(4, 2).to(torch.bfloat16),
         "c": torch.randn(6).to(torch.float16), "i": torch.arange(7, dtype=torch.int64)}
    write_file(str(tmp_path / "model.safetensors"), t, {"k": "v"})
    raw = read_file(str(tmp_path / "model.safetensors"))
    for k in t:
        assert raw[k].dtype == t[k].dtype and torch.equal(raw[k], t[k])
    got = load_checkpoint(str(tmp_path))
    assert got["a"].dtype == torch.float32                       # stored in 32 bits: stays
    assert got["b"].dtype == torch.bfloat16
    assert got["c"].dtype == torch.float16 and torch.equal(got["c"], t["c"])   # as stored until bound
    assert got["i"].dtype == torch.int32                         # integer tables as int32
    assert torch.equal(got["i"], t["i"].to(torch.int32))


def test_readable_by_the_safetensors_package(tmp_path):
    st = pytest.importorskip("safetensors.torch")
    t = {"x": torch.randn(2, 3).to(torch.bfloat16), "y": torch.randn(5)}
    write_file(str(tmp_path / "m.safetensors"), t)
    back = st.load_file(str(tmp_path / "m.safetensors"))
    assert torch.equal(back["x"], t["x"]) and torch.equal(back["y"], t["y"])


def test_truncated_and_malformed_files(tmp_path):
    p = str(tmp_path / "model.safetensors")
    write_file(p, {"a": torch.randn(64, 64)})
    data = open(p, "rb").read()
    open(p, "wb").write(data[:len(data) - 100])
    with pytest.raises(SafetensorsError, match="truncated|outside the file"):
        read_file(p)
    open(p, "wb").write(data[:4])
    with pytest.raises(SafetensorsError, match="truncated"):
        read_file(p)
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 12]}}).encode()
    open(p, "wb").write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 12)
    with pytest.raises(SafetensorsError, match="needs 16 bytes but has 12"):
        read_file(p)
    hdr = json.dumps({"a": {"dtype": "F8_E5M2", "shape": [2], "data_offsets": [0, 2]}}).encode()
    open(p, "wb").write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 2)
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        read_file(p)


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    cfg = config_from_dict(TINY_A)
    needs = tensor_needs_of(cfg)
    w = make_weights(TINY_A, 0)
    check_tensors(needs, w)
    del w["model.layers.1.mlp.up_proj.weight"], w["model.norm.weight"]
    w["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64)
    w["extra.bias"] = torch.zeros(3)
    with pytest.raises(WeightsError) as e:
        check_tensors(needs, w)
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["extra.bias"]
    assert err.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (32, 64), (16, 64))]
    msg = str(err)
    for word in ("model.norm.weight", "extra.bias", "expected [32, 64], found [16, 64]"):
        assert word in msg


def test_tied_model_needs_no_lm_head():
    needs = tensor_needs_of(config_from_dict(TINY_B))
    assert "lm_head.weight" not in needs and "model.embed_tokens.weight" in needs
    assert needs["model.layers.0.self_attn.q_proj.weight"].shape == (3 * 32, 96)
    assert needs["model.layers.0.self_attn.k_proj.weight"].shape == (1 * 32, 96)
    assert needs["model.layers.2.mlp.down_proj.weight"].shape == (96, 256)


def test_random_weights_mode_writes_a_model_folder(tmp_path):
    cfg = config_from_dict(TINY_B)
    needs = tensor_needs_of(cfg)
    write_model_dir(str(tmp_path / "m1"), cfg, needs, seed=5)
    write_model_dir(str(tmp_path / "m2"), cfg, needs, seed=5)
    write_model_dir(str(tmp_path / "m3"), cfg, needs, seed=6)
    a, b, c = (load_checkpoint(str(tmp_path / n)) for n in ("m1", "m2", "m3"))
    assert set(a) == set(needs)
    check_tensors(needs, a)
    for k in a:
        assert torch.equal(a[k], b[k])
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    assert a["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert a["model.norm.weight"].dtype == torch.float32
    assert abs(a["model.norm.weight"].mean().item() - 1.0) < 0.05
    assert 0.015 < a["model.layers.0.mlp.gate_proj.weight"].float().std().item() < 0.025
    back = json.load(open(tmp_path / "m1" / "config.json"))
    assert config_from_dict(back) == cfg.__class__.from_dict(dict(cfg.to_dict(), torch_dtype="bfloat16"))


def test_sharded_folder_and_duplicate_names(tmp_path):
    w = make_weights(TINY_A, 0)
    names = sorted(w)
    os.makedirs(tmp_path / "m")
    write_file(str(tmp_path / "m" / "model-00001-of-00002.safetensors"), {n: w[n] for n in names[:9]})
    write_file(str(tmp_path / "m" / "model-00002-of-00002.safetensors"), {n: w[n] for n in names[9:]})
    got = load_checkpoint(str(tmp_path / "m"))
    assert set(got) == set(w)
    write_file(str(tmp_path / "m" / "model-00003.safetensors"), {names[0]: w[names[0]]})
    with pytest.raises(WeightsError, match="more than one file"):
        load_checkpoint(str(tmp_path / "m"))
    with pytest.raises(WeightsError, match="no .safetensors"):
        os.makedirs(tmp_path / "empty")
        load_checkpoint(str(tmp_path / "empty"))


def test_tensors_an_exporter_may_add_are_no_error():
    """Rotary frequency buffers, and a copy of the head beside tied embeddings, are not
    read and not reported; any other extra tensor still is."""
    cfg = config_from_dict(dict(TINY_B))
    assert cfg.tie_word_embeddings
    assert cfg.ignorable_tensor("model.layers.0.self_attn.rotary_emb.inv_freq")
    assert cfg.ignorable_tensor("lm_head.weight")
    assert not cfg.ignorable_tensor("model.layers.0.self_attn.q_proj.bias")
    assert not config_from_dict(dict(TINY_A)).ignorable_tensor("lm_head.weight")


def test_packed_single_file_round_trip(tmp_path):
    """A model folder packed into one file: same tensors in their stored types, the
    configuration in the metadata; a plain safetensors file without it is refused."""
    from yalm_b200.weights import load_packed, pack_model_dir, read_metadata
    from yalm_b200.weights.pack import CONFIG_KEY, main
    cfg = config_from_dict(dict(TINY_B))
    write_model_dir(str(tmp_path / "m"), cfg, tensor_needs_of(cfg), seed=4, dtype=torch.bfloat16)
    assert main([str(tmp_path / "m"), str(tmp_path / "one.safetensors")]) == 0
    d, t = load_packed(str(tmp_path / "one.safetensors"))
    assert config_from_dict(d) == config_from_dict(dict(cfg.to_dict(), torch_dtype="bfloat16"))
    ref = load_checkpoint(str(tmp_path / "m"))
    assert set(t) == set(ref) and all(t[k].dtype == ref[k].dtype and torch.equal(t[k], ref[k]) for k in ref)
    assert CONFIG_KEY in read_metadata(str(tmp_path / "one.safetensors"))
    with pytest.raises(WeightsError, match="no configuration"):
        load_packed(str(tmp_path / "m" / "model.safetensors"))
    pack_model_dir(str(tmp_path / "m"), str(tmp_path / "two.safetensors"))
