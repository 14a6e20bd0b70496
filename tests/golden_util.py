"""Load the committed golden fixtures (bf16 arrays are stored as uint16 views)."""
import os

import numpy as np
from ml_dtypes import bfloat16

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    out = {}
    for k in z.files:
        if k.startswith("__bf16__"):
            continue
        v = z[k]
        out[k] = v.view(bfloat16) if ("__bf16__" + k) in z.files else v
    return out


def bits(a):
    a = np.ascontiguousarray(a)
    return a.view(np.uint16) if a.dtype == bfloat16 else a
