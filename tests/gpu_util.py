"""Helpers shared by the GPU parity tests: numpy <-> torch bf16, seeded AWQ tensors."""
import numpy as np
import torch
from ml_dtypes import bfloat16

from oracle import awq_oracle as O


def to_dev(a, device="cuda"):
    a = np.ascontiguousarray(a)
    if a.dtype == bfloat16:
        return torch.from_numpy(a.view(np.int16)).to(device).view(torch.bfloat16)
    return torch.from_numpy(a).to(device)


def to_host(t):
    t = t.detach()
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).cpu().numpy().view(bfloat16)
    return t.cpu().numpy()


def synth_awq(K, N, gs=128, seed=0, scale_lo=0.001, scale_hi=0.02):
    """Seeded layout-A tensors with the benchmark's distributions: nibbles and zero nibbles
    uniform 0..15, scales ~U(lo, hi) rounded to bf16."""
    rng = np.random.default_rng(seed)
    nibs = rng.integers(0, 16, size=(K, N), dtype=np.uint8)
    z = rng.integers(0, 16, size=(K // gs, N), dtype=np.uint8)
    s = rng.uniform(scale_lo, scale_hi, size=(K // gs, N)).astype(bfloat16)
    return O.pack_awq_int32(nibs), O.pack_awq_int32(z), s


def dev_weight(qw, qz, s, gs=128):
    from mlir_air_b200.ops import AwqWeight
    return AwqWeight.from_numpy(qw, qz, s, gs)


def randn_bf16(shape, seed):
    return np.random.default_rng(seed).standard_normal(shape).astype(bfloat16)
