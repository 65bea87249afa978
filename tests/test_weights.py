"""Weights: the safetensors container, loading by name, the one error that lists everything, dtypes,
and the random-weights mode."""
import json
import os
import struct

import pytest
import torch

from burn_lm_b200 import WeightsError, write_random_model
from burn_lm_b200.model import tensor_specs_of
from burn_lm_b200.weights import SafetensorsError, SafetensorsFile, TensorSpec, load_tensors, write_safetensors
from tiny import TINY_A, TINY_B


def test_container_round_trip_and_independent_reader(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int64).view(2, 3)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t)
    f = SafetensorsFile(p)
    assert sorted(f.names()) == ["a", "b", "c"]
    for k, v in t.items():
        assert torch.equal(f.get(k), v) and f.dtype(k) == v.dtype and tuple(f.shape(k)) == tuple(v.shape)
    f.close()
    from safetensors.torch import load_file      # another implementation reads what this one wrote
    other = load_file(p)
    for k, v in t.items():
        assert torch.equal(other[k], v)


def test_container_errors(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 5) + b"{oops")
    with pytest.raises(SafetensorsError, match="not valid JSON"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="do not fit"):
        SafetensorsFile(str(p))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = str(tmp_path / "m")
    write_random_model(folder, TINY_A, seed=1, dtype="float32")
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    tensors = {n: f.get(n).clone() for n in f.names()}
    f.close()
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 63)
    tensors["lm_head.weight"] = torch.zeros(256, 64)          # tied model: the head is not a stored tensor
    tensors["model.layers.9.extra"] = torch.zeros(1)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    with pytest.raises(WeightsError) as e:
        load_tensors(folder, tensor_specs_of(TINY_A), torch.float32, "cpu")
    err = e.value
    assert sorted(err.missing) == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert sorted(err.unexpected) == ["lm_head.weight", "model.layers.9.extra"]
    assert [w[0] for w in err.wrong_shape] == ["model.layers.0.self_attn.q_proj.weight"]
    msg = str(err)
    for needle in ("missing (2)", "unexpected (2)", "wrong shape (1)", "expected (64, 64) found (64, 63)"):
        assert needle in msg


def test_missing_file(tmp_path):
    with pytest.raises(WeightsError, match="model.safetensors"):
        load_tensors(str(tmp_path), [], torch.float32, "cpu")


def test_dtypes_are_kept(tmp_path):
    folder = str(tmp_path)
    write_safetensors(os.path.join(folder, "model.safetensors"), {
        "w16": torch.randn(4, 4).to(torch.bfloat16), "w32": torch.randn(4, 4), "h": torch.randn(4, 4).to(torch.float16),
        "table": torch.arange(5, dtype=torch.int64)})
    specs = [TensorSpec("w16", (4, 4)), TensorSpec("w32", (4, 4)), TensorSpec("h", (4, 4)), TensorSpec("table", (5,), kind="int")]
    bf = load_tensors(folder, specs, torch.bfloat16, "cpu")
    assert bf["w16"].dtype == torch.bfloat16 and bf["w32"].dtype == torch.float32      # 32-bit stays 32-bit
    assert bf["h"].dtype == torch.bfloat16 and bf["table"].dtype == torch.int32
    fp = load_tensors(folder, specs, torch.float32, "cpu")
    assert all(fp[k].dtype == torch.float32 for k in ("w16", "w32", "h")) and fp["table"].dtype == torch.int32
    assert torch.equal(fp["w16"], bf["w16"].float())                                  # widened exactly
    with pytest.raises(WeightsError, match="wrong shape"):
        load_tensors(folder, [TensorSpec("table", (5,)), *specs[:3]], torch.float32, "cpu")   # int stored, float wanted


def test_ignorable_names(tmp_path):
    folder = str(tmp_path)
    write_safetensors(os.path.join(folder, "model.safetensors"), {"w": torch.zeros(2), "model.layers.0.self_attn.rotary_emb.inv_freq": torch.zeros(3)})
    got = load_tensors(folder, [TensorSpec("w", (2,))], torch.float32, "cpu",
                       ignorable=(r"model\.layers\.\d+\.self_attn\.rotary_emb\.inv_freq",))
    assert list(got) == ["w"]


def test_random_mode_is_seeded_and_order_free(tmp_path):
    a = write_random_model(str(tmp_path / "a"), TINY_B, seed=4, dtype="bfloat16")
    b = write_random_model(str(tmp_path / "b"), TINY_B, seed=4, dtype="bfloat16")
    c = write_random_model(str(tmp_path / "c"), TINY_B, seed=5, dtype="bfloat16")
    fa, fb, fc = (SafetensorsFile(os.path.join(x, "model.safetensors")) for x in (a, b, c))
    assert sorted(fa.names()) == sorted(s.name for s in tensor_specs_of(TINY_B))
    assert "lm_head.weight" in fa.names()
    for n in fa.names():
        assert torch.equal(fa.get(n), fb.get(n))
        assert fa.dtype(n) == torch.bfloat16
    assert not torch.equal(fa.get("lm_head.weight"), fc.get("lm_head.weight"))
    w = fa.get("model.layers.0.mlp.gate_proj.weight").float()
    g = fa.get("model.norm.weight").float()
    assert abs(w.std().item() - 0.02) < 0.002 and abs(w.mean().item()) < 0.001
    assert abs(g.mean().item() - 1.0) < 0.05 and 0.05 < g.std().item() < 0.15
    cfg = json.load(open(os.path.join(a, "config.json")))
    assert cfg["hidden_size"] == 192 and cfg["torch_dtype"] == "bfloat16"
    tied = write_random_model(str(tmp_path / "t"), TINY_A, seed=4, dtype="float32")
    ft = SafetensorsFile(os.path.join(tied, "model.safetensors"))
    assert "lm_head.weight" not in ft.names() and ft.dtype("model.norm.weight") == torch.float32
    for f in (fa, fb, fc, ft):
        f.close()


def _stored(folder):
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    tensors = {n: f.get(n).clone() for n in f.names()}
    f.close()
    return tensors


def test_a_tied_model_may_store_its_head_when_it_equals_the_table(tmp_path):
    from burn_lm_b200.model import plan_of
    folder = write_random_model(str(tmp_path / "m"), TINY_A, seed=2, dtype="float32")
    _, _, plan = plan_of(TINY_A)
    assert plan.duplicate_tensors == (("lm_head.weight", "model.embed_tokens.weight"),)
    tensors = _stored(folder)
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    got = load_tensors(folder, tensor_specs_of(TINY_A), torch.float32, "cpu", plan.ignorable_tensors, plan.duplicate_tensors)
    assert "lm_head.weight" not in got and "model.embed_tokens.weight" in got
    tensors["lm_head.weight"][3, 5] += 1.0
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    with pytest.raises(WeightsError, match="differing") as e:
        load_tensors(folder, tensor_specs_of(TINY_A), torch.float32, "cpu", plan.ignorable_tensors, plan.duplicate_tensors)
    assert e.value.differing == [("lm_head.weight", "model.embed_tokens.weight")] and not e.value.unexpected
    # an untied model names no such pair: there the head is simply a wanted tensor
    assert plan_of(TINY_B)[2].duplicate_tensors == ()


def test_a_folder_of_shards_with_an_index(tmp_path):
    """model.safetensors.index.json with two files loads as the single file does; a tensor the index's files
    do not hold is reported as missing."""
    folder = write_random_model(str(tmp_path / "m"), TINY_B, seed=3, dtype="bfloat16")
    specs = tensor_specs_of(TINY_B)
    whole = load_tensors(folder, specs, torch.bfloat16, "cpu")
    tensors = _stored(folder)
    names = sorted(tensors)
    parts = {"model-00001-of-00002.safetensors": names[: len(names) // 2], "model-00002-of-00002.safetensors": names[len(names) // 2:]}
    sharded = str(tmp_path / "s")
    os.makedirs(sharded)
    for fname, ns in parts.items():
        write_safetensors(os.path.join(sharded, fname), {n: tensors[n] for n in ns})
    index = {"metadata": {}, "weight_map": {n: fname for fname, ns in parts.items() for n in ns}}
    json.dump(index, open(os.path.join(sharded, "model.safetensors.index.json"), "w"))
    json.dump(TINY_B, open(os.path.join(sharded, "config.json"), "w"))
    got = load_tensors(sharded, specs, torch.bfloat16, "cpu")
    assert sorted(got) == sorted(whole) and all(torch.equal(got[n], whole[n]) for n in whole)
    first = parts["model-00001-of-00002.safetensors"]
    write_safetensors(os.path.join(sharded, "model-00001-of-00002.safetensors"), {n: tensors[n] for n in first[1:]})
    with pytest.raises(WeightsError) as e:
        load_tensors(sharded, specs, torch.bfloat16, "cpu")
    assert e.value.missing == [first[0]]
