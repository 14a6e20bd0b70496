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


# ---------------------------------------------------------------------------
# Seeded decode-FFN stack at the Llama-3-70B dimensions (hidden 8192, intermediate 28672).
# The fixture ffn_stack_70b.npz stores only the seeds and the [8, 8192] hidden state after every
# layer; the weights (366 MB per layer) are regenerated from the seeds by whoever needs them.
# ---------------------------------------------------------------------------
STACK70B = dict(hidden=8192, intermediate=28672, layers=2, batch=8, group_size=128, seed=7000)


def stack70b_weight(K, N, seed, group_size=128, scale_lo=0.001, scale_hi=0.02):
    """Layout-A (qweight, qzeros, scales) with uniform nibbles: the packed words are drawn
    directly as uniform 32-bit patterns, which is the same distribution as packing uniform
    nibbles, and eight times cheaper to generate."""
    rng = np.random.default_rng(seed)
    qw = rng.integers(-2 ** 31, 2 ** 31, size=(K, N // 8), dtype=np.int64).astype(np.int32)
    qz = rng.integers(-2 ** 31, 2 ** 31, size=(K // group_size, N // 8), dtype=np.int64).astype(np.int32)
    s = rng.uniform(scale_lo, scale_hi, size=(K // group_size, N)).astype(bfloat16)
    return qw, qz, s


def stack70b_layer(l, cfg=STACK70B):
    """(gate, up, down, gamma) of layer l; scales of down chosen so the residual stream stays O(1)."""
    H, I, gs, seed = cfg["hidden"], cfg["intermediate"], cfg["group_size"], cfg["seed"] + 10 * l
    gate = stack70b_weight(H, I, seed, gs)
    up = stack70b_weight(H, I, seed + 1, gs)
    down = stack70b_weight(I, H, seed + 2, gs, 0.0002, 0.001)
    gamma = (np.random.default_rng(seed + 3).standard_normal(H) * 0.1 + 1.0).astype(bfloat16)
    return gate, up, down, gamma


def stack70b_input(cfg=STACK70B):
    return np.random.default_rng(cfg["seed"] - 1).standard_normal((cfg["batch"], cfg["hidden"])).astype(bfloat16)
