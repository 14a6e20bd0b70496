"""O projection + residual, RMSNorm, gate/up + SwiGLU, down + residual: the post-attention half of a
decode layer on int4-AWQ weights, on a B200.

Entry points of mlir-air's llms/llama32_1b_int4/multi_launch_builder/o_gemv_ffn_int4_multi.py:
`build_o_gemv_ffn_int4_module` (:110), the golden `o_gemv_ffn_int4_reference` (:273), the weight
generator `_gen_int4_weights` (:291), and the command line with its 15-argument ABI and seeded
inputs (:313-476).  The reference stitches three launches; here the three stages are the decode GEMV
with residual, the RMSNorm + gate/up GEMV with SwiGLU in its epilogue, and the GEMV with residual again.
"""
import sys

import numpy as np
from ml_dtypes import bfloat16

from mlir_air_b200.backend import KernelSpec
from mlir_air_b200.programming_examples import _common as C
from mlir_air_b200.programming_examples.matrix_vector_multiplication.int4_awq.matvec_int4_packed import pack_inputs


def _packed_dims(M, K, GS, M_TILE, K_CHUNK, N_CORES, M_PER_LAUNCH):
    """(number of tiles, bytes per tile) of a packed GEMV weight (:99-107)."""
    n_gpc = K_CHUNK // GS
    tile_bytes = M_TILE * K_CHUNK // 2 + 3 * n_gpc * M_TILE
    return (M // M_TILE) * (K // K_CHUNK), tile_bytes


def build_o_gemv_ffn_int4_module(emb_dim=2048, hidden_dim=8192, gs=128, m_tile=8, k_chunk=2048, n_cores=8):
    for m, k in ((emb_dim, emb_dim), (2 * hidden_dim, emb_dim), (emb_dim, hidden_dim)):
        if m % (n_cores * m_tile) or k % k_chunk or k_chunk % gs:
            raise ValueError(f"[{m} x {k}] does not tile with n_cores * m_tile = {n_cores * m_tile}, k_chunk {k_chunk}, gs {gs}")
    return KernelSpec("o_gemv_ffn_int4", dict(emb_dim=emb_dim, hidden_dim=hidden_dim, GS=gs, M_TILE=m_tile, K_CHUNK=k_chunk,
                                              N_CORES=n_cores, eps=1e-5))


def o_gemv_ffn_int4_reference(wo, attn_out, x_residual, ffn_norm_w, wgate, wup, wdown, eps=1e-5):
    """CPU reference on dequantised bf16 weights [out, in] (:273-288): res1 stays f32."""
    f = np.float32
    res1 = wo.astype(f) @ attn_out.astype(f) + x_residual.astype(f)
    rstd = 1.0 / np.sqrt((res1 * res1).mean() + eps)
    normed = ((res1 * rstd) * ffn_norm_w.astype(f)).astype(bfloat16).astype(f)
    gate, up = wgate.astype(f) @ normed, wup.astype(f) @ normed
    swiglu = ((gate * 0.5 * (np.tanh(gate / 2.0) + 1.0)) * up).astype(bfloat16).astype(f)
    return (wdown.astype(f) @ swiglu + res1).astype(bfloat16)


def _gen_int4_weights(M, K, gs, seed):
    """(A_q, A_s, A_z, dequantised bf16 [M, K]) from default_rng(seed): nibbles, scales ~U(0.005, 0.02),
    zeros in {7, 8} (:291-310)."""
    rng = np.random.default_rng(seed)
    unp = rng.integers(0, 16, size=(M, K), dtype=np.uint8)
    A_q = (unp[:, 0::2] | (unp[:, 1::2] << 4)).astype(np.uint8)
    A_s = rng.uniform(0.005, 0.02, size=(K // gs, M)).astype(bfloat16)
    A_z = rng.integers(7, 9, size=(K // gs, M), dtype=np.uint8)
    return A_q, A_s, A_z, C.dequant_B(A_q, A_s, A_z).astype(bfloat16)


def main(argv=None):
    ap = C.base_parser("o_gemv_ffn_int4_multi.py", "Full int4-AWQ post-attention block (O proj, FFN), three stages")
    ap.add_argument("--emb-dim", type=int, default=2048)
    ap.add_argument("--hidden-dim", type=int, default=8192)
    ap.add_argument("--gs", type=int, default=128)
    ap.add_argument("--m-tile", type=int, default=8, dest="m_tile")
    ap.add_argument("--k-chunk", type=int, default=2048, dest="k_chunk")
    ap.add_argument("--n-cores", type=int, default=8, dest="n_cores")
    C.add_compile_mode(ap)
    args = ap.parse_args(argv)
    emb, hid = args.emb_dim, args.hidden_dim
    print(f"O GEMV + FFN full-int4 3-launch: emb_dim={emb}, hidden_dim={hid}, k_chunk={args.k_chunk}")
    spec = build_o_gemv_ffn_int4_module(emb, hid, args.gs, args.m_tile, args.k_chunk, args.n_cores)
    if args.print_module_only or args.compile_mode == "compile-only":
        C.finish(args, spec, dict(instance_name="o_gemv_ffn_int4"), [], [])
    np.random.seed(42)
    wo_q, wo_s, wo_z, wo_bf16 = _gen_int4_weights(emb, emb, args.gs, 100)
    gu_q, gu_s, gu_z, gu_bf16 = _gen_int4_weights(2 * hid, emb, args.gs, 150)  # rows 2i = gate_i, 2i + 1 = up_i
    wd_q, wd_s, wd_z, wd_bf16 = _gen_int4_weights(emb, hid, args.gs, 200)
    attn_out = np.random.randn(emb).astype(bfloat16)
    x_residual = np.random.randn(emb).astype(bfloat16)
    ffn_norm_w = (np.random.randn(emb) * 0.1 + 1.0).astype(bfloat16)
    packed_rms = np.zeros((2, emb), dtype=bfloat16)
    packed_rms[1] = ffn_norm_w
    pk = lambda q, s, z, m, k: pack_inputs(q, s, z, m, k, args.gs, args.m_tile, args.k_chunk, args.n_cores, m)  # noqa: E731
    expected = o_gemv_ffn_int4_reference(wo_bf16, attn_out, x_residual, ffn_norm_w, gu_bf16[0::2], gu_bf16[1::2], wd_bf16)
    z_emb, z_hid = np.zeros(emb, dtype=bfloat16), np.zeros(hid, dtype=bfloat16)
    inputs = [pk(wo_q, wo_s, wo_z, emb, emb), attn_out, z_emb, x_residual, z_emb, z_emb, packed_rms,
              pk(gu_q, gu_s, gu_z, 2 * hid, emb), z_hid, np.zeros((1, 1), dtype=bfloat16), z_hid, z_hid.copy(),
              pk(wd_q, wd_s, wd_z, emb, hid), z_emb]
    C.finish(args, spec, dict(instance_name="o_gemv_ffn_int4"), inputs, [expected], rtol=0.2, atol=2.0, min_correlation=0.99,
             max_rel_l2=1e-2)


if __name__ == "__main__":
    main()
