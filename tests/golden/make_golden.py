"""Writes tests/golden/plain_logits.npz: logits of the plain implementation on one tiny
random model, kept as a guard against accidental changes of the plain implementation
itself (what ties the plain implementation to the reference's own output is
``reference_kernels_logits.npz`` beside it, written by ``make_reference_golden.py``).

    python tests/golden/make_golden.py
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

TOKENS = [17, 3, 250, 99, 0, 42, 42, 7, 128, 64, 5, 200]


def compute():
    cfg, seed, std = tiny_configs.CONFIGS["B"]
    with tempfile.TemporaryDirectory() as d:
        write_model_folder(config_from_dict(cfg), seed, d, std=std)
        pc, pw = pl.read_model_folder(d)
        return pl.forward(pc, pw, TOKENS)


if __name__ == "__main__":
    logits = compute()
    np.savez_compressed(os.path.join(HERE, "plain_logits.npz"), tokens=np.array(TOKENS),
                        logits=logits[:, :48].astype(np.float32))
    print("wrote", logits.shape)
