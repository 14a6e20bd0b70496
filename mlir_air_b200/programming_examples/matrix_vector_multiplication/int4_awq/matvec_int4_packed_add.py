"""int4-AWQ GEMV with fused residual add  D = dequant(A) @ B + R  on a B200.

Entry points of mlir-air's matvec_int4_packed_add.py: `build_module` (:100), `cpu_reference` (:302),
command line (:327-349); packing is `matvec_int4_packed.pack_inputs`.
"""
import numpy as np
from ml_dtypes import bfloat16

from mlir_air_b200.backend import KernelSpec
from mlir_air_b200.programming_examples import _common as C
from mlir_air_b200.programming_examples.matrix_vector_multiplication.int4_awq.matvec_int4_packed import pack_inputs


def build_module(M, K, GS=128, M_TILE=8, K_CHUNK=2048, N_CORES=8, M_PER_LAUNCH=None):
    M_PER_LAUNCH = M if M_PER_LAUNCH is None else M_PER_LAUNCH
    if M % M_PER_LAUNCH or M_PER_LAUNCH % (N_CORES * M_TILE) or K % K_CHUNK or K_CHUNK % GS:
        raise ValueError("M / M_PER_LAUNCH / N_CORES / M_TILE or K / K_CHUNK / GS do not tile")
    return KernelSpec("matvec_int4_packed_add", dict(M=M, K=K, GS=GS, M_TILE=M_TILE, K_CHUNK=K_CHUNK,
                                                     N_CORES=N_CORES, M_PER_LAUNCH=M_PER_LAUNCH))


def cpu_reference(A_q, A_s, A_z, B, R):
    """The residual joins the f32 sum before the single bf16 rounding."""
    acc = np.asarray(B).astype(np.float32) @ C.dequant_B(A_q, A_s, A_z).T
    return (acc + np.asarray(R).astype(np.float32)).astype(bfloat16)


def main(argv=None):
    ap = C.base_parser("matvec_int4_packed_add.py", "int4-AWQ GEMV with fused residual add: D = dequant(A) @ B + R")
    C.add_gemv_tiling(ap, 2048, 2048)
    ap.add_argument("--m-per-launch", type=int, default=None, dest="m_per_launch")
    C.add_compile_mode(ap)
    args = ap.parse_args(argv)
    kc = C.resolve_k_chunk(args)
    spec = build_module(args.m, args.k, args.gs, args.m_tile, kc, args.n_cores, args.m_per_launch)
    A_q, A_s, A_z = C.seeded_layout_B(args.m, args.k, args.gs)
    B = np.random.randn(args.k).astype(bfloat16)
    R = np.random.randn(args.m).astype(bfloat16)
    packed = pack_inputs(A_q, A_s, A_z, args.m, args.k, args.gs, args.m_tile, kc, args.n_cores,
                         args.m_per_launch or args.m)
    C.finish(args, spec, dict(instance_name="matvec_int4_packed_add"), [packed, B, R],
             [cpu_reference(A_q, A_s, A_z, B, R)], rtol=0.1, atol=0.05, min_correlation=0.999)


if __name__ == "__main__":
    main()
