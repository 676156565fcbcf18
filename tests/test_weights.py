"""safetensors reading and the loader's one error that lists missing, unexpected and misshapen tensors."""
import json
import struct

import pytest
import torch

from roost_b200.config import Qwen3Config
from roost_b200.engine.model import parameter_declarations
from roost_b200.weights import loader
from roost_b200.weights.random_init import random_tensors, write_random_model
from roost_b200.weights.safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors
from tests.conftest import TINY_A, TINY_B
from tests.plain import qwen3_plain as plain


def _spec(cfg):
    spec = Qwen3Config.from_dict(cfg).to_spec()
    return spec, parameter_declarations(spec)


def test_round_trip_keeps_dtypes_and_values(tmp_path):
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.randn(7), "c": torch.arange(6, dtype=torch.int64).reshape(2, 3),
         "d": torch.randn(2, 2).to(torch.float16), "e": torch.empty(0, 4)}
    write_safetensors(tmp_path / "x.safetensors", t)
    with SafetensorsFile(tmp_path / "x.safetensors") as f:
        for k, v in t.items():
            got = f.tensor(k)
            assert got.dtype == v.dtype and got.shape == v.shape and torch.equal(got, v)
    # the plain reader (written separately) reads the same bytes
    got = plain.read_safetensors(tmp_path / "x.safetensors")
    assert torch.equal(got["a"], t["a"]) and torch.equal(got["b"], t["b"])
    # the loader's storage rule: bfloat16 and float32 stay, float16 widens, integers become int32
    assert loader._stored(t["a"]).dtype == torch.bfloat16 and loader._stored(t["b"]).dtype == torch.float32
    assert loader._stored(t["d"]).dtype == torch.float32 and loader._stored(t["c"]).dtype == torch.int32


def _raw(path, header: dict, data: bytes):
    blob = json.dumps(header).encode()
    path.write_bytes(struct.pack("<Q", len(blob)) + blob + data)


def test_header_checks(tmp_path):
    p = tmp_path / "h.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(p)
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(p)
    _raw(p, {"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}, b"\0" * 4)
    with pytest.raises(SafetensorsError, match="needs 8"):
        SafetensorsFile(p)
    _raw(p, {"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}, "b": {"dtype": "F32", "shape": [1], "data_offsets": [8, 12]}}, b"\0" * 12)
    with pytest.raises(SafetensorsError, match="tile"):
        SafetensorsFile(p)
    _raw(p, {"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}}, b"\0" * 8)
    with pytest.raises(SafetensorsError, match="trailing"):
        SafetensorsFile(p)
    _raw(p, {"a": {"dtype": "Q4", "shape": [1], "data_offsets": [0, 4]}}, b"\0" * 4)
    with pytest.raises(SafetensorsError, match="dtype"):
        SafetensorsFile(p)
    _raw(p, {"__metadata__": {"x": "y"}, "a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}}, b"\0" * 4)
    assert list(SafetensorsFile(p).names()) == ["a"]


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    spec, decls = _spec(TINY_B)
    tensors = random_tensors(TINY_B, 3)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(192)
    tensors["model.layers.2.self_attn.k_proj.weight"] = torch.zeros(64, 96)
    tensors["lm_head.weight"] = torch.zeros(387, 95)
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    write_safetensors(tmp_path / "model.safetensors", tensors)
    with pytest.raises(loader.WeightError) as e:
        loader.load_checkpoint(tmp_path, decls, spec.weight_names)
    err = e.value
    assert sorted(err.missing) == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert sorted(n for n, _, _ in err.wrong_shape) == ["lm_head.weight", "model.layers.2.self_attn.k_proj.weight"]
    for name in err.missing + err.unexpected + [n for n, _, _ in err.wrong_shape]:
        assert name in str(err)
    assert "[64, 96]" in str(err) and "[32, 96]" in str(err)


def test_concatenation_and_tied_head(tmp_path):
    write_random_model(tmp_path, TINY_A, seed=4, std=0.05)
    spec, decls = _spec(TINY_A)
    assert "lm_head" not in decls and spec.tie_embeddings
    params = loader.load_checkpoint(tmp_path, decls, spec.weight_names)
    raw = plain.read_safetensors(tmp_path / "model.safetensors")
    p = "model.layers.1."
    assert torch.equal(params["blocks.1.mixer"]["qkv"], torch.cat([raw[p + "self_attn.q_proj.weight"], raw[p + "self_attn.k_proj.weight"],
                                                                   raw[p + "self_attn.v_proj.weight"]]))
    assert torch.equal(params["blocks.1.feed_forward"]["gate_up"], torch.cat([raw[p + "mlp.gate_proj.weight"], raw[p + "mlp.up_proj.weight"]]))
    assert params["embed"]["table"].dtype == torch.float32       # stored in 32-bit, kept in 32-bit
    assert not loader.checkpoint_has(tmp_path, "lm_head.weight")
    with pytest.raises(loader.WeightError, match="neither"):
        loader.checkpoint_files(tmp_path / "nowhere")


def test_a_checkpoint_in_two_shards_is_read_through_its_index(tmp_path):
    """model.safetensors.index.json names a shard for every tensor; the loader reads each tensor from the shard the index
    names and gives the same parameters as the one-file form. A tensor a shard holds without the index naming it, and a
    tensor the index names for a shard that lacks it, are told in the same one error as the tensors the model misses."""
    spec, decls = _spec(TINY_B)
    tensors = random_tensors(TINY_B, 5)
    one = tmp_path / "one"
    one.mkdir()
    write_safetensors(one / "model.safetensors", tensors)
    want = loader.load_checkpoint(one, decls, spec.weight_names)
    names = list(tensors)
    first, second = names[::2], names[1::2]          # neighbours of a concatenated parameter land in different shards
    two = tmp_path / "two"
    two.mkdir()
    shards = {"model-00001-of-00002.safetensors": first, "model-00002-of-00002.safetensors": second}
    weight_map = {}
    for shard, held in shards.items():
        write_safetensors(two / shard, {n: tensors[n] for n in held})
        weight_map.update({n: shard for n in held})
    (two / "model.safetensors.index.json").write_text(json.dumps({"metadata": {"total_size": 0}, "weight_map": weight_map}))
    assert [f.name for f in loader.checkpoint_files(two)] == sorted(shards)
    assert loader.checkpoint_has(two, "lm_head.weight") and not loader.checkpoint_has(two, "model.layers.0.self_attn.q_proj.bias")
    got = loader.load_checkpoint(two, decls, spec.weight_names)
    assert got.keys() == want.keys()
    for scope in want:
        for local in want[scope]:
            assert torch.equal(got[scope][local], want[scope][local]), (scope, local)
    # the index forgets one tensor (it is still in its shard) and names another for the wrong shard
    forgotten, misplaced = "model.layers.1.mlp.down_proj.weight", "model.norm.weight"
    bad = dict(weight_map)
    del bad[forgotten]
    bad[misplaced] = [s for s in shards if s != weight_map[misplaced]][0]
    (two / "model.safetensors.index.json").write_text(json.dumps({"weight_map": bad}))
    with pytest.raises(loader.WeightError) as e:
        loader.load_checkpoint(two, decls, spec.weight_names)
    err = e.value
    assert sorted(err.missing) == sorted([forgotten, misplaced])
    assert len(err.index_faults) == 3 and "shard index" in str(err)
    assert any(forgotten in f and "does not name it" in f for f in err.index_faults)
    assert any(misplaced in f and "does not hold it" in f for f in err.index_faults)
    (two / "model.safetensors.index.json").write_text(json.dumps({"weights": {}}))
    with pytest.raises(loader.WeightError, match="weight_map"):
        loader.load_checkpoint(two, decls, spec.weight_names)


def test_random_weights_mode_is_seeded_and_order_independent(tmp_path):
    a = random_tensors(TINY_B, seed=1, std=0.02, norm_std=0.1)
    b = random_tensors(TINY_B, seed=1, std=0.02, norm_std=0.1)
    c = random_tensors(TINY_B, seed=2, std=0.02, norm_std=0.1)
    assert all(torch.equal(a[k], b[k]) for k in a) and not torch.equal(a["lm_head.weight"], c["lm_head.weight"])
    assert all(v.dtype == torch.bfloat16 for v in a.values())
    w = a["model.layers.0.mlp.down_proj.weight"].float()
    assert abs(float(w.std()) - 0.02) < 0.002
    n = a["model.layers.0.input_layernorm.weight"].float()
    assert 0.05 < float(n.std()) < 0.15 and abs(float(n.mean()) - 1) < 0.05
    # a tensor's values do not depend on the other tensors: another depth gives the same layer 0
    d = random_tensors(dict(TINY_B, num_hidden_layers=1, layer_types=["full_attention"]), seed=1, std=0.02, norm_std=0.1)
    assert torch.equal(d["model.layers.0.self_attn.q_proj.weight"], a["model.layers.0.self_attn.q_proj.weight"])
    out = write_random_model(tmp_path / "m", TINY_B, seed=1, std=0.02, norm_std=0.1)
    assert json.loads((out / "config.json").read_text()) == TINY_B
    assert torch.equal(plain.read_safetensors(out / "model.safetensors")["model.norm.weight"], a["model.norm.weight"])
