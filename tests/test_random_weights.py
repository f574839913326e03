"""The weight generator: the package's host version against the tests' own scalar statement,
and its statistics.  (The device version is compared in tests/test_kernels_gpu.py.)"""
import numpy as np
import torch

import plain_random as pr
import tiny_configs
from supersonic_b200.config import config_from_dict
from supersonic_b200.weights import random_fill, random_store
from supersonic_b200.weights.store import random_tensor


def bits(t):
    return t.view(torch.int16).numpy().astype(np.int64) & 0xFFFF


def test_host_fill_equals_the_scalar_recipe():
    for seed, name, mean, std in ((0, "model.embed_tokens.weight", 0.0, 0.02), (7, "model.norm.weight", 1.0, 0.1),
                                  (2 ** 40 + 5, "model.layers.3.mlp.up_proj.weight", 0.0, 0.08)):
        got = bits(random_fill.fill_host(seed, name, (37, 11), mean, std)).reshape(-1)
        want = [pr.value_bits(seed, name, i, mean, std) for i in range(37 * 11)]
        assert got.tolist() == want


def test_a_piece_equals_the_whole():
    key = random_fill.tensor_key(3, "w")
    whole = random_fill._normals(key, 0, 5000)
    assert np.array_equal(whole[1234:1300], random_fill._normals(key, 1234, 66))


def test_name_and_seed_matter_order_does_not():
    cfg = config_from_dict(tiny_configs.A)
    a = random_tensor(cfg, 0, "model.layers.0.self_attn.q_proj.weight")
    b = random_tensor(cfg, 0, "model.layers.1.self_attn.q_proj.weight")
    c = random_tensor(cfg, 1, "model.layers.0.self_attn.q_proj.weight")
    assert not torch.equal(a, b) and not torch.equal(a, c)
    store = random_store(cfg, 0)
    assert torch.equal(store.get("model.layers.0.self_attn.q_proj.weight"), a)


def test_moments():
    n = random_fill._normals(random_fill.tensor_key(5, "x"), 0, 400000)
    assert abs(n.mean()) < 0.01 and abs(n.var() - 1.0) < 0.01
    assert abs((n ** 3).mean()) < 0.03 and abs((n ** 4).mean() - 3.0) < 0.15     # near-normal: kurtosis 2.9
    assert np.abs(n).max() <= 6.0
    # neighbouring elements and neighbouring tensors are uncorrelated
    assert abs(np.corrcoef(n[:-1], n[1:])[0, 1]) < 0.01
    m = random_fill._normals(random_fill.tensor_key(5, "y"), 0, 400000)
    assert abs(np.corrcoef(n, m)[0, 1]) < 0.01
