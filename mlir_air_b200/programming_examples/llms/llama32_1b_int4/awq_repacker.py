"""HF AutoAWQ tensors <-> mlir-air's layouts, with a self-test that also exercises the GPU.

Callables of mlir-air's llms/llama32_1b_int4/awq_repacker.py: `unpack_awq_int32` (:41),
`dequant_to_bf16` (:57), `repack_hf_awq_linear` (:85), `repack_for_gemv` (:112),
`_gen_synthetic_awq` (:143), `self_test` (:166) and the command line (:242-245).  The host functions
are numpy; self-test steps [d] and [e] run the CUDA library against them.
"""
import argparse

import numpy as np
from ml_dtypes import bfloat16

from mlir_air_b200 import layouts

AWQ_PACK_ORDER = np.array(layouts.AWQ_PACK_ORDER, dtype=np.int64)
AWQ_UNPACK_PERM = np.argsort(AWQ_PACK_ORDER)

unpack_awq_int32 = layouts.unpack_awq_int32


def dequant_f32(qweight, qzeros, scales, group_size):
    """(q - z) * bf16(s) in f32, [K, N]."""
    q = unpack_awq_int32(qweight).astype(np.int32)
    z = np.repeat(unpack_awq_int32(qzeros).astype(np.int32), group_size, axis=0)
    s = np.repeat(np.asarray(scales).astype(bfloat16).astype(np.float32), group_size, axis=0)
    if z.shape != q.shape or s.shape != q.shape:
        raise ValueError("qzeros / scales do not match qweight and group_size")
    return ((q - z) * s).astype(np.float32)


def dequant_to_bf16(qweight, qzeros, scales, group_size):
    """Dense bf16 [in_features, out_features]; scales are rounded to bf16 first."""
    return dequant_f32(qweight, qzeros, scales, group_size).astype(bfloat16)


def repack_hf_awq_linear(qweight, qzeros, scales, group_size):
    return layouts.A_to_B(qweight, qzeros, scales, group_size)


def repack_for_gemv(qweight, qzeros, scales, group_size, M_TILE=8, K_CHUNK=2048, N_CORES=8):
    A_q, A_s, A_z = repack_hf_awq_linear(qweight, qzeros, scales, group_size)
    M, K = A_q.shape[0], A_q.shape[1] * 2
    return layouts.pack_gemv_tiles(A_q, A_s, A_z, M, K, group_size, M_TILE, K_CHUNK, N_CORES, M)


def _gen_synthetic_awq(K, N, group_size, seed=42):
    """Same rng call order as the reference generator, so the same tensors for a seed."""
    rng = np.random.default_rng(seed)
    G = K // group_size
    nibs = rng.integers(0, 16, size=(K, N), dtype=np.uint8)
    z_nibs = rng.integers(0, 16, size=(G, N), dtype=np.uint8)
    scales = rng.uniform(0.005, 0.02, size=(G, N)).astype(np.float16)
    return layouts.pack_awq_int32(nibs), layouts.pack_awq_int32(z_nibs), scales, nibs, z_nibs


def self_test(K=512, N=128, group_size=128, seed=42, verbose=True, gpu=None):
    say = print if verbose else (lambda *a, **k: None)
    qweight, qzeros, scales, nibs, z_nibs = _gen_synthetic_awq(K, N, group_size, seed)
    if not (np.array_equal(unpack_awq_int32(qweight), nibs) and np.array_equal(unpack_awq_int32(qzeros), z_nibs)):
        raise AssertionError("unpack_awq_int32 does not invert the AWQ packing")
    say(f"  [a] AWQ_PACK_ORDER unpack: PASS ({K}x{N} nibbles)")

    w_dense = dequant_to_bf16(qweight, qzeros, scales, group_size)
    A_q, A_s, A_z = repack_hf_awq_linear(qweight, qzeros, scales, group_size)
    from mlir_air_b200.programming_examples import _common as C
    w_repacked = C.dequant_B(A_q, A_s, A_z).astype(bfloat16)
    if not np.array_equal(w_dense.view(np.uint16), w_repacked.T.view(np.uint16)):
        raise AssertionError("dense vs repacked dequant mismatch")
    say("  [b] dense vs repacked dequant: PASS")

    x = np.random.default_rng(seed + 1).standard_normal(K).astype(bfloat16)
    y_b = (C.dequant_B(A_q, A_s, A_z) @ x.astype(np.float32)).astype(bfloat16)
    y_d = (w_dense.astype(np.float32).T @ x.astype(np.float32)).astype(bfloat16)
    corr = np.corrcoef(y_b.astype(np.float32), y_d.astype(np.float32))[0, 1]
    if not corr >= 0.9999:
        raise AssertionError(f"end-to-end correlation {corr:.6f} below 0.9999 threshold")
    say(f"  [c] end-to-end (layout B golden vs dense): PASS (corr={corr:.6f})")

    if gpu is None:
        import torch
        gpu = torch.cuda.is_available()
    if not gpu:
        say("  [d], [e] skipped: no CUDA device")
        return
    import torch
    from mlir_air_b200 import ops
    w = ops.AwqWeight.from_numpy(qweight, qzeros, scales, group_size)
    got = ops.dequant(w).view(torch.int16).cpu().numpy().view(np.uint16)
    if not np.array_equal(got, w_dense.view(np.uint16)):
        raise AssertionError("GPU dequant is not bit-exact with dequant_to_bf16")
    say("  [d] GPU dequant == dequant_to_bf16 (bit-exact): PASS")
    ws = ops.Workspace(K, N)
    xd = torch.from_numpy(x.view(np.int16)).cuda().view(torch.bfloat16).view(1, -1)
    y = ops.gemv(xd, w, ws).view(torch.int16).cpu().numpy().view(bfloat16)[0]
    ws.check()
    ref = (x.astype(np.float32) @ dequant_f32(qweight, qzeros, scales, group_size)).astype(bfloat16)
    err = float(np.linalg.norm(y.astype(np.float64) - ref.astype(np.float64)) / np.linalg.norm(ref.astype(np.float64)))
    if not err <= 1e-2:
        raise AssertionError(f"GPU GEMV rel-L2 {err:.3e} exceeds 1e-2")
    say(f"  [e] GPU GEMV vs golden: PASS (rel-L2={err:.2e})")


def main(argv=None):
    ap = argparse.ArgumentParser(prog="awq_repacker.py", description="HF AutoAWQ -> mlir-air packed-BO repacker + self-test.")
    ap.add_argument("--k", type=int, default=512)
    ap.add_argument("--n", type=int, default=128)
    ap.add_argument("--gs", type=int, default=128)
    ap.add_argument("--seed", type=int, default=42)
    args = ap.parse_args(argv)
    print(f"AWQ repacker self-test: K={args.k}, N={args.n}, GS={args.gs}, seed={args.seed}")
    self_test(K=args.k, N=args.n, group_size=args.gs, seed=args.seed)
    print("All self-tests PASSED.")


if __name__ == "__main__":
    main()
