"""int4-AWQ prefill GEMM  C[M, N] = A[M, K] @ dequant(W)  on a B200.

Entry points of mlir-air's matrix_multiplication/int4_awq/matmul_int4_packed.py: `packed_tile_bytes`
(:49), `pack_inputs` (:57), `cpu_reference` (:89), `build_module` (:109), command line (:399-418).
Argument order of the runner: activations first, packed weights second.
"""
import numpy as np
from ml_dtypes import bfloat16

from mlir_air_b200 import layouts
from mlir_air_b200.backend import KernelSpec
from mlir_air_b200.programming_examples import _common as C


def packed_tile_bytes(n_tile, k_chunk, gs):
    return layouts.gemv_tile_bytes(n_tile, k_chunk, gs)


def pack_inputs(W_q, W_s, W_z, M, K, N, GS, N_TILE, K_CHUNK):
    """[N / N_TILE, K / K_CHUNK, tile_bytes]; W_q [N, K/2] u8, W_s [K/GS, N] bf16, W_z [K/GS, N] u8."""
    return layouts.pack_gemm_tiles(W_q, W_s, W_z, K, N, GS, N_TILE, K_CHUNK)


def cpu_reference(W_q, W_s, W_z, A):
    return (A.astype(np.float32) @ C.dequant_B(W_q, W_s, W_z).T).astype(bfloat16)


def build_module(m, k, n, gs, tile_m, tile_k_l2, tile_k_l1, tile_n, herd_m, herd_n, m_per_segment=1):
    if n % tile_n or k % tile_k_l1 or tile_k_l1 % gs:
        raise ValueError("N over tile_n, K over tile_k_l1 over gs must tile")
    return KernelSpec("matmul_int4_packed", dict(M=m, K=k, N=n, GS=gs, N_TILE=tile_n, K_CHUNK=tile_k_l1))


def main(argv=None):
    ap = C.base_parser("matmul_int4_packed.py", "int4-AWQ GEMM: C = A @ dequant(W)")
    for flag, default in (("--m", 64), ("--k", 128), ("--n", 128), ("--gs", 128), ("--tile-m", 16),
                          ("--tile-k-l2", 128), ("--tile-k-l1", 128), ("--tile-n", 16), ("--herd-m", 2), ("--herd-n", 4)):
        ap.add_argument(flag, type=int, default=default, dest=flag[2:].replace("-", "_"))
    ap.add_argument("--compile-mode", choices=["compile-and-run", "compile-only"], default="compile-and-run",
                    dest="compile_mode")
    args = ap.parse_args(argv)
    spec = build_module(args.m, args.k, args.n, args.gs, args.tile_m, args.tile_k_l2, args.tile_k_l1, args.tile_n,
                        args.herd_m, args.herd_n)
    W_q, W_s, W_z = C.seeded_layout_B(args.n, args.k, args.gs)
    A = np.random.randn(args.m, args.k).astype(bfloat16)
    packed = pack_inputs(W_q, W_s, W_z, args.m, args.k, args.n, args.gs, args.tile_n, args.tile_k_l1)
    C.finish(args, spec, dict(instance_name="matmul_int4_packed"), [A, packed], [cpu_reference(W_q, W_s, W_z, A)],
             rtol=0.1, atol=0.05, max_mismatch_percentage=0.05, min_correlation=0.999)


if __name__ == "__main__":
    main()
