"""Loader for the fixtures under ``tests/golden`` (see ``make_golden.py`` there)."""

import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name: str) -> dict:
    """Return the fixture as a dict of CPU torch tensors (fp32 / bool / int)."""
    out = {}
    with np.load(os.path.join(GOLDEN_DIR, name + ".npz")) as z:
        for key in z.files:
            a = z[key]
            if key.startswith("bf16:"):
                a = (a.astype(np.uint32) << 16).view(np.float32)
                key = key[5:]
            if a.dtype == np.uint32:
                a = a.astype(np.int64)
            out[key] = torch.from_numpy(np.ascontiguousarray(a))
    return out
