"""Shared fixtures.  Tests marked ``gpu`` need a CUDA device and run the compiled kernels;
everything else runs on the CPU."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """Model folders (config.json + model.safetensors) of the tiny configurations, written
    once per session into a temporary folder; values are (folder, config dict, float64 weights)."""
    import plain_llama as pl
    import tiny_configs
    from supersonic_b200.config import config_from_dict
    from supersonic_b200.weights import write_model_folder
    out = {}
    for name, (cfg, seed, std) in tiny_configs.CONFIGS.items():
        d = str(tmp_path_factory.mktemp(name))
        write_model_folder(config_from_dict(cfg), seed, d, std=std, norm_jitter=0.1)
        pc, pw = pl.read_model_folder(d)
        out[name] = (d, pc, pw)
    return out
