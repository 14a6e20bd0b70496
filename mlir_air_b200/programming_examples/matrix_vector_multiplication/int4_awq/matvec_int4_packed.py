"""int4-AWQ GEMV  D[M] = dequant(A_q, A_s, A_z)[M, K] @ B[K]  on a B200.

Same entry points as mlir-air's matrix_vector_multiplication/int4_awq/matvec_int4_packed.py:
`pack_inputs` (:57), `build_module` (:106), `cpu_reference` (:272) and the command line (:291-317),
plus `--batch`.  The runner receives [PACKED, B] and returns D.
"""
import numpy as np
from ml_dtypes import bfloat16

from mlir_air_b200 import layouts
from mlir_air_b200.backend import KernelSpec
from mlir_air_b200.programming_examples import _common as C


def pack_inputs(A_q, A_s, A_z, M, K, GS, M_TILE, K_CHUNK, N_CORES, M_PER_LAUNCH):
    """[total_tiles, tile_bytes] uint8, one [Q | S | Z] slab per (launch, core, outer, k-chunk)."""
    return layouts.pack_gemv_tiles(A_q, A_s, A_z, M, K, GS, M_TILE, K_CHUNK, N_CORES, M_PER_LAUNCH)


def build_module(M, K, GS=128, M_TILE=8, K_CHUNK=2048, N_CORES=8, M_PER_LAUNCH=None):
    M_PER_LAUNCH = M if M_PER_LAUNCH is None else M_PER_LAUNCH
    if M % M_PER_LAUNCH or M_PER_LAUNCH % (N_CORES * M_TILE) or K % K_CHUNK or K_CHUNK % GS:
        raise ValueError("M / M_PER_LAUNCH / N_CORES / M_TILE or K / K_CHUNK / GS do not tile")
    return KernelSpec("matvec_int4_packed", dict(M=M, K=K, GS=GS, M_TILE=M_TILE, K_CHUNK=K_CHUNK, N_CORES=N_CORES,
                                                 M_PER_LAUNCH=M_PER_LAUNCH))


def cpu_reference(A_q, A_s, A_z, B):
    """f32 accumulate, one bf16 rounding; B may be [K] or [batch, K]."""
    return (np.asarray(B).astype(np.float32) @ C.dequant_B(A_q, A_s, A_z).T).astype(bfloat16)


def main(argv=None):
    ap = C.base_parser("matvec_int4_packed.py", "int4-AWQ GEMV: D = dequant(A) @ B")
    C.add_gemv_tiling(ap, 2048, 2048)
    ap.add_argument("--m-per-launch", type=int, default=None, dest="m_per_launch")
    ap.add_argument("--batch", type=int, default=1)
    C.add_compile_mode(ap)
    args = ap.parse_args(argv)
    kc = C.resolve_k_chunk(args)
    spec = build_module(args.m, args.k, args.gs, args.m_tile, kc, args.n_cores, args.m_per_launch)
    A_q, A_s, A_z = C.seeded_layout_B(args.m, args.k, args.gs)
    B = np.random.randn(*((args.k,) if args.batch == 1 else (args.batch, args.k))).astype(bfloat16)
    packed = pack_inputs(A_q, A_s, A_z, args.m, args.k, args.gs, args.m_tile, kc, args.n_cores,
                         args.m_per_launch or args.m)
    C.finish(args, spec, dict(instance_name="matvec_int4_packed"), [packed, B], [cpu_reference(A_q, A_s, A_z, B)],
             rtol=0.1, atol=0.05, min_correlation=0.999)


if __name__ == "__main__":
    main()
