"""The post-attention half of a decode layer on int4-AWQ weights with the FFN in ONE launch, on a B200.

Entry points of mlir-air's llms/llama32_1b_int4/multi_launch_builder/o_gemv_ffn_int4_fused.py:
`build_o_gemv_ffn_int4_fused_module` (:154), `build_module` (:172), the stage goldens
`lgu_cpu_reference` (:127) and `ld_cpu_reference` (:1078) chained behind the O-projection golden of
matvec_int4_packed_add.py (:1189-1191), and the command line with its 8-argument ABI and seeded
inputs (:1097-1248).  The reference wires three herds with cascades inside one launch; here the O
projection is the decode GEMV with residual and RMSNorm, gate/up + SwiGLU and down + residual run as
one launch of the stack kernel (awq_b200_ffn_stack_decode_bf16 on a one-layer plan).
"""
import numpy as np
from ml_dtypes import bfloat16

from mlir_air_b200.backend import KernelSpec
from mlir_air_b200.programming_examples import _common as C
from mlir_air_b200.programming_examples.matrix_vector_multiplication.int4_awq.matvec_int4_packed import pack_inputs
from mlir_air_b200.programming_examples.matrix_vector_multiplication.int4_awq.matvec_int4_packed_add import (
    cpu_reference as la_cpu_reference)


def lgu_cpu_reference(A_q, A_s, A_z, res1, gamma, eps=1e-5):
    """RMSNorm(res1, gamma) -> interleaved gate/up GEMV -> SwiGLU, bf16 at the reference's rounding points."""
    x, w = res1.astype(np.float32), gamma.astype(np.float32)
    rstd = 1.0 / np.sqrt(float((x * x).sum()) / res1.shape[0] + eps)
    normed = ((x * rstd) * w).astype(bfloat16).astype(np.float32)
    raw = (C.dequant_B(A_q, A_s, A_z) @ normed).astype(bfloat16).astype(np.float32)
    gate, up = raw[0::2], raw[1::2]
    return (gate * 0.5 * (np.tanh(gate / 2.0) + 1.0) * up).astype(bfloat16)


def ld_cpu_reference(A_q, A_s, A_z, swiglu, R):
    """D = bf16(bf16(dequant @ swiglu) + R): the product is rounded before the residual joins."""
    raw = (C.dequant_B(A_q, A_s, A_z) @ swiglu.astype(np.float32)).astype(bfloat16).astype(np.float32)
    return (raw + R.astype(np.float32)).astype(bfloat16)


def build_module(K, M_LA, M_LGU, K_LD, GS=128, M_TILE=8, K_CHUNK=2048, N_LA=8, N_LGU=8, N_LD=8):
    if K != M_LA:
        raise ValueError("the builder requires K == M_LA so that res1 doubles as the residual of the down projection")
    if M_LGU % 2:
        raise ValueError("M_LGU must be even (gate/up rows interleaved)")
    for m, k, n in ((M_LA, K, N_LA), (M_LGU, K, N_LGU), (M_LA, K_LD, N_LD)):
        if m % (n * M_TILE) or k % K_CHUNK or K_CHUNK % GS:
            raise ValueError(f"[{m} x {k}] does not tile with {n} cores x M_TILE {M_TILE}, K_CHUNK {K_CHUNK}, GS {GS}")
    return KernelSpec("o_gemv_ffn_int4_fused", dict(emb_dim=K, hidden_dim=M_LGU // 2, GS=GS, M_TILE=M_TILE, K_CHUNK=K_CHUNK,
                                                    N_CORES=N_LA, eps=1e-5))


def build_o_gemv_ffn_int4_fused_module(emb_dim=2048, hidden_dim=8192, gs=128, m_tile=8, k_chunk=2048, n_cores=8):
    """Same signature as o_gemv_ffn_int4_multi.build_o_gemv_ffn_int4_module."""
    return build_module(K=emb_dim, M_LA=emb_dim, M_LGU=2 * hidden_dim, K_LD=hidden_dim, GS=gs, M_TILE=m_tile,
                        K_CHUNK=k_chunk, N_LA=n_cores, N_LGU=n_cores, N_LD=n_cores)


def main(argv=None):
    ap = C.base_parser("o_gemv_ffn_int4_fused.py", "Full int4-AWQ post-attention block, FFN in one launch")
    ap.add_argument("--emb-dim", type=int, default=2048)
    ap.add_argument("--hidden-dim", type=int, default=8192)
    ap.add_argument("--gs", type=int, default=128)
    ap.add_argument("--m-tile", type=int, default=8, dest="m_tile")
    ap.add_argument("--k-chunk", type=int, default=2048, dest="k_chunk")
    ap.add_argument("--n-cores", type=int, default=8, dest="n_cores")
    C.add_compile_mode(ap)
    args = ap.parse_args(argv)
    emb, hid, gs = args.emb_dim, args.hidden_dim, args.gs
    print(f"O GEMV + FFN full-int4 1-launch fused: emb_dim={emb}, hidden_dim={hid}, k_chunk={args.k_chunk}")
    spec = build_o_gemv_ffn_int4_fused_module(emb, hid, gs, args.m_tile, args.k_chunk, args.n_cores)
    if args.print_module_only or args.compile_mode == "compile-only":
        C.finish(args, spec, dict(instance_name="o_gemv_ffn_int4_fused"), [], [])
    # one np.random.seed(42) stream, drawn in the reference's order (:1154-1185)
    la = C.seeded_layout_B(emb, emb, gs)
    B_la = np.random.randn(emb).astype(bfloat16)
    R_la = np.random.randn(emb).astype(bfloat16)

    def more(M, K):
        unp = np.random.randint(0, 16, size=(M, K), dtype=np.uint8)
        return ((unp[:, 0::2] | (unp[:, 1::2] << 4)).astype(np.uint8),
                np.random.uniform(0.005, 0.02, size=(K // gs, M)).astype(bfloat16),
                np.random.randint(7, 9, size=(K // gs, M), dtype=np.uint8))

    lgu = more(2 * hid, emb)
    gamma = (np.random.randn(emb) * 0.1 + 1.0).astype(bfloat16)
    ld = more(emb, hid)
    res1_ref = la_cpu_reference(*la, B_la, R_la)
    swiglu_ref = lgu_cpu_reference(*lgu, res1_ref, gamma)
    D_ref = ld_cpu_reference(*ld, swiglu_ref, res1_ref)
    pk = lambda w, m, k: pack_inputs(*w, m, k, gs, args.m_tile, args.k_chunk, args.n_cores, m)  # noqa: E731
    inputs = [pk(la, emb, emb), B_la, R_la, pk(lgu, 2 * hid, emb), gamma, pk(ld, emb, hid)]
    C.finish(args, spec, dict(instance_name="o_gemv_ffn_int4_fused"), inputs, [D_ref, res1_ref], rtol=0.2, atol=2.0,
             min_correlation=0.99, max_rel_l2=1e-2)


if __name__ == "__main__":
    main()
