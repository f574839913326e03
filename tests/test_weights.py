"""Weights: safetensors by name, the one error that lists everything, random folders (CPU)."""
import json
import os
import struct

import pytest
import torch

import tiny_configs
from supersonic_b200.config import config_from_dict
from supersonic_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, WeightStore,
                                     random_store, write_model_folder, write_safetensors)


def _folder(tmp_path, cfg=tiny_configs.A, seed=3):
    c = config_from_dict(cfg)
    return c, write_model_folder(c, seed, str(tmp_path / "m"))


def test_random_folder_round_trip(tmp_path):
    c, d = _folder(tmp_path)
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    s = WeightStore.from_dir(d)
    s.check(c.tensor_shapes())
    q = s.get("model.layers.1.self_attn.q_proj.weight")
    assert q.dtype == torch.bfloat16 and tuple(q.shape) == (64, 64)
    assert abs(q.float().std().item() - 0.02) < 0.002
    n = s.get("model.norm.weight").float()
    assert abs(n.mean().item() - 1.0) < 0.05 and 0.05 < n.std().item() < 0.15
    assert json.load(open(os.path.join(d, "config.json")))["architectures"] == ["LlamaForCausalLM"]


def test_seed_decides_values_and_order_does_not(tmp_path):
    c = config_from_dict(tiny_configs.B)
    a, b, other = random_store(c, 5), random_store(c, 5), random_store(c, 6)
    name = "model.layers.2.mlp.down_proj.weight"
    assert torch.equal(a.get(name), b.get(name)) and not torch.equal(a.get(name), other.get(name))
    d = write_model_folder(c, 5, str(tmp_path / "m"))
    assert torch.equal(WeightStore.from_dir(d).get(name), a.get(name))


def test_one_error_lists_missing_unexpected_and_shapes(tmp_path):
    c = config_from_dict(tiny_configs.A)
    tensors = dict(random_store(c, 0)._tensors)
    del tensors["model.layers.0.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    tensors["model.layers.1.self_attn.k_proj.weight"] = torch.zeros(16, 64, dtype=torch.bfloat16)
    with pytest.raises(WeightError) as e:
        WeightStore.from_tensors(tensors, "here").check(c.tensor_shapes())
    msg = str(e.value)
    assert "model.layers.0.mlp.up_proj.weight" in msg and "model.norm.weight" in msg
    assert "unexpected (1): model.layers.0.self_attn.rotary_emb.inv_freq" in msg
    assert "model.layers.1.self_attn.k_proj.weight expected [32, 64], found [16, 64]" in msg
    assert e.value.missing == ["model.norm.weight", "model.layers.0.mlp.up_proj.weight"] or \
        set(e.value.missing) == {"model.norm.weight", "model.layers.0.mlp.up_proj.weight"}
    assert len(e.value.wrong_shape) == 1 and len(e.value.unexpected) == 1


def test_untied_config_needs_lm_head(tmp_path):
    c, d = _folder(tmp_path, tiny_configs.A)                   # tied: no lm_head in the folder
    untied = config_from_dict(dict(tiny_configs.A, tie_word_embeddings=False))
    with pytest.raises(WeightError, match="lm_head.weight"):
        WeightStore.from_dir(d).check(untied.tensor_shapes())


def test_storage_dtypes(tmp_path):
    path = str(tmp_path / "x.safetensors")
    t32, t16, ti = torch.randn(3, 4), torch.randn(2, 2).half(), torch.arange(6).reshape(2, 3)
    write_safetensors(path, [("a", torch.float32, [3, 4]), ("b", torch.float16, [2, 2]),
                             ("c", torch.int64, [2, 3])], [("a", t32), ("b", t16), ("c", ti)])
    os.rename(path, str(tmp_path / "model.safetensors"))
    s = WeightStore.from_dir(str(tmp_path))
    assert s.get("a").dtype == torch.float32 and torch.equal(s.get("a"), t32)     # 32-bit stays
    assert s.get("b").dtype == torch.bfloat16                                      # 16-bit -> bfloat16
    assert s.get("c").dtype == torch.int32 and s.get("c").tolist() == ti.tolist()  # tables -> int32


def test_sharded_folder(tmp_path):
    c = config_from_dict(tiny_configs.A)
    names = list(c.tensor_shapes())
    rs = random_store(c, 1)
    half = len(names) // 2
    weight_map = {}
    for i, part in enumerate((names[:half], names[half:])):
        fn = f"model-{i + 1:05d}-of-00002.safetensors"
        write_safetensors(str(tmp_path / fn), [(n, torch.bfloat16, c.tensor_shapes()[n]) for n in part],
                          [(n, rs.get(n)) for n in part])
        weight_map.update({n: fn for n in part})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    s = WeightStore.from_dir(str(tmp_path))
    s.check(c.tensor_shapes())
    assert torch.equal(s.get(names[-1]), rs.get(names[-1]))


def test_corrupt_files(tmp_path):
    with pytest.raises(SafetensorsError, match="no model.safetensors"):
        WeightStore.from_dir(str(tmp_path))
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 10 ** 9) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 4) + b"nope")
    with pytest.raises(SafetensorsError, match="not JSON"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"w": {"dtype": "BF16", "shape": [4, 4], "data_offsets": [0, 32]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 16)          # truncated data
    with pytest.raises(SafetensorsError, match="does not match"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"w": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 4)
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        SafetensorsFile(str(p))


def test_buffers_are_passed_over_and_unexpected_tensors_can_be_a_warning():
    import warnings
    import torch
    from supersonic_b200.weights import WeightError, WeightStore
    store = WeightStore.from_tensors({"a": torch.zeros(2, 3), "x.rotary_emb.inv_freq": torch.zeros(4),
                                      "stray": torch.zeros(1)})
    ignorable = lambda n: n.endswith("rotary_emb.inv_freq")
    with pytest.raises(WeightError) as e:
        store.check({"a": [2, 3]}, ignorable=ignorable)
    assert e.value.unexpected == ["stray"]
    with warnings.catch_warnings(record=True) as seen:
        warnings.simplefilter("always")
        store.check({"a": [2, 3]}, ignorable=ignorable, allow_unexpected=True)
    assert len(seen) == 1 and "stray" in str(seen[0].message)
    with pytest.raises(WeightError) as e, warnings.catch_warnings():       # missing tensors stay an error
        warnings.simplefilter("ignore")
        store.check({"a": [2, 3], "b": [1]}, ignorable=ignorable, allow_unexpected=True)
    assert e.value.missing == ["b"] and e.value.unexpected == []
