"""RMSNorm -> gate/up int4-AWQ GEMV -> SwiGLU (the decode FFN front half) on a B200.

Entry points of mlir-air's decode_ffn_swiglu/matvec_int4_swiglu_rms.py: `build_module` (:93),
`cpu_reference` (:490), command line (:524-541).  The M rows of the weight are gate/up interleaved
(row 2i = gate_i, 2i+1 = up_i); inputs are [PACKED, RMS_in bf16 [2, K]] (row 0 = x, row 1 = gamma),
output bf16 [M/2].  K does not have to equal K_CHUNK here.
"""
import numpy as np
from ml_dtypes import bfloat16

from mlir_air_b200.backend import KernelSpec
from mlir_air_b200.programming_examples import _common as C
from mlir_air_b200.programming_examples.matrix_vector_multiplication.int4_awq.matvec_int4_packed import pack_inputs


def build_module(M, K, GS=128, M_TILE=8, K_CHUNK=2048, N_CORES=8):
    if M % 2 or M % (N_CORES * M_TILE) or K % K_CHUNK or K_CHUNK % GS:
        raise ValueError("M must be even and tile over N_CORES * M_TILE; K over K_CHUNK over GS")
    return KernelSpec("matvec_int4_swiglu_rms", dict(M=M, K=K, GS=GS, M_TILE=M_TILE, K_CHUNK=K_CHUNK,
                                                     N_CORES=N_CORES, M_PER_LAUNCH=M, eps=1e-5))


def cpu_reference(A_q, A_s, A_z, RMS_in, eps=1e-5):
    x, w = RMS_in[0].astype(np.float32), RMS_in[1].astype(np.float32)
    rstd = 1.0 / np.sqrt(float((x * x).sum()) / x.shape[0] + eps)
    normed = ((x * rstd) * w).astype(bfloat16).astype(np.float32)
    raw = (C.dequant_B(A_q, A_s, A_z) @ normed).astype(bfloat16).astype(np.float32)
    gate, up = raw[0::2], raw[1::2]
    return (gate * 0.5 * (np.tanh(gate / 2.0) + 1.0) * up).astype(bfloat16)


def main(argv=None):
    ap = C.base_parser("matvec_int4_swiglu_rms.py", "int4-AWQ FFN GEMV with fused RMSNorm input and SwiGLU output.")
    C.add_gemv_tiling(ap, 16384, 2048)
    C.add_compile_mode(ap)
    args = ap.parse_args(argv)
    kc = C.resolve_k_chunk(args)
    spec = build_module(args.m, args.k, args.gs, args.m_tile, kc, args.n_cores)
    A_q, A_s, A_z = C.seeded_layout_B(args.m, args.k, args.gs)
    x = np.random.randn(args.k).astype(bfloat16)
    gamma = (np.random.randn(args.k) * 0.1 + 1.0).astype(bfloat16)
    RMS_in = np.stack([x, gamma], axis=0).astype(bfloat16)
    packed = pack_inputs(A_q, A_s, A_z, args.m, args.k, args.gs, args.m_tile, kc, args.n_cores, args.m)
    C.finish(args, spec, dict(instance_name="matvec_int4_swiglu_rms"), [packed, RMS_in],
             [cpu_reference(A_q, A_s, A_z, RMS_in)], rtol=0.15, atol=0.5, min_correlation=0.99)


if __name__ == "__main__":
    main()
