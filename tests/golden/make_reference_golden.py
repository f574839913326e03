"""Writes tests/golden/reference_kernels_logits.npz: logits of a tiny random model computed by
DeanoC/SuperSonic's own CUDA kernels (compiled unmodified by ``baseline/reference_kernels.py``,
chained in the order of the reference's prompt engine by ``tests/reference_model.py``).  Needs a
CUDA device; the file it writes lets a machine without one check the plain implementation
against the reference's arithmetic (``tests/test_plain_impl.py``).

    python -m baseline.reference_kernels && python tests/golden/make_reference_golden.py [OUT.npz]
"""
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import plain_llama as pl  # noqa: E402
import tiny_configs  # noqa: E402
from supersonic_b200.config import config_from_dict  # noqa: E402
from supersonic_b200.weights import write_model_folder  # noqa: E402

TOKENS = {"A": [17, 3, 250, 99, 0, 42, 42, 7, 128, 64, 5, 200, 31, 8],
          "B": [17, 3, 250, 99, 0, 42, 42, 7, 128, 64, 5, 200, 383, 1, 1, 77, 300, 12, 19, 240]}


def model(name):
    cfg, seed, std = tiny_configs.CONFIGS[name]
    with tempfile.TemporaryDirectory() as d:
        write_model_folder(config_from_dict(cfg), seed, d, std=std)
        return pl.read_model_folder(d)


if __name__ == "__main__":
    import reference_model      # needs a CUDA device and the compiled reference kernels
    out = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "reference_kernels_logits.npz")
    arrays = {}
    for name, tokens in TOKENS.items():
        pc, pw = model(name)
        arrays[f"tokens_{name}"] = np.array(tokens)
        arrays[f"logits_{name}"] = reference_model.forward(pc, pw, tokens)[:, :64].astype(np.float32)
    np.savez_compressed(out, **arrays)
    print("wrote", out)
