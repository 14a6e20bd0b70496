"""RMSNorm + int4-AWQ Q/K/V GEMVs + half-split RoPE on Q and K: the attention-input half of a
decode layer on a B200.

Entry points of mlir-air's llms/llama32_1b_int4/multi_launch_builder/rms_qkv_int4_rope_multi.py:
`build_rms_qkv_int4_rope_module` (:361), the goldens `_rms_norm_ref` (:527) and `_rope_ref` (:533),
and the command line with its 13-argument ABI and seeded inputs (:557-728).  The reference stitches
six launches (RMSNorm, three GEMVs, two RoPE); here Q, K and V are one GEMV launch over the
concatenated weight and RoPE rotates the Q and K parts of its output.
"""
import sys

import numpy as np
from ml_dtypes import bfloat16

from mlir_air_b200.backend import KernelSpec
from mlir_air_b200.programming_examples import _common as C
from mlir_air_b200.programming_examples.matrix_vector_multiplication.int4_awq.matvec_int4_packed import (
    cpu_reference as int4_gemv_ref, pack_inputs)


def build_rms_qkv_int4_rope_module(emb_dim=2048, kv_dim=512, n_heads=32, n_kv_heads=8, head_dim=64, gs=128, m_tile=8,
                                   k_chunk=2048, n_cores=8, rope_herd_x=1, print_kernels=False):
    if n_heads * head_dim != emb_dim or n_kv_heads * head_dim != kv_dim:
        raise ValueError("n_heads * head_dim must be emb_dim and n_kv_heads * head_dim must be kv_dim")
    if emb_dim % k_chunk or k_chunk % gs or emb_dim % (n_cores * m_tile) or kv_dim % (n_cores * m_tile):
        raise ValueError("emb_dim / kv_dim do not tile with k_chunk / gs / n_cores / m_tile")
    return KernelSpec("rms_qkv_int4_rope", dict(emb_dim=emb_dim, kv_dim=kv_dim, n_heads=n_heads, n_kv_heads=n_kv_heads,
                                                head_dim=head_dim, GS=gs, M_TILE=m_tile, K_CHUNK=k_chunk, N_CORES=n_cores))


def _rms_norm_ref(x_1d, weight, eps=1e-5):
    x_f32 = np.asarray(x_1d).astype(np.float32)
    rms = np.sqrt(np.mean(x_f32 ** 2) + eps)
    return (x_f32 / rms * np.asarray(weight).astype(np.float32)).astype(bfloat16)


def _rope_ref(x_flat, lut_flat, head_dim):
    """LUT row: [cos_0 .. cos_{half-1} | sin_0 .. sin_{half-1}];
    out[i] = x[i] cos[i] - x[i + half] sin[i], out[i + half] = x[i] sin[i] + x[i + half] cos[i]."""
    half = head_dim // 2
    x = np.asarray(x_flat).astype(np.float32).reshape(-1, head_dim)
    lut = np.asarray(lut_flat).astype(np.float32).reshape(-1, head_dim)
    out = np.empty_like(x)
    out[:, :half] = x[:, :half] * lut[:, :half] - x[:, half:] * lut[:, half:]
    out[:, half:] = x[:, :half] * lut[:, half:] + x[:, half:] * lut[:, :half]
    return out.astype(bfloat16).flatten()


def generate_rope_lut(head_dim=64, rope_base=500000.0, seq_len=2048, dtype=bfloat16):
    """[seq_len, head_dim] rows [cos | sin] (llama32_1b/llama32_1b_weights.py:395-440)."""
    inv_freq = 1.0 / (rope_base ** (np.arange(0, head_dim, 2, dtype=np.float64) / head_dim))
    ang = np.outer(np.arange(seq_len, dtype=np.float64), inv_freq)
    return np.concatenate([np.cos(ang), np.sin(ang)], axis=1).astype(dtype)


def main(argv=None):
    EMB_DIM, KV_DIM, N_HEADS, N_KV_HEADS, HEAD_DIM, GS, M_TILE, K_CHUNK, N_CORES = 2048, 512, 32, 8, 64, 128, 8, 2048, 8
    ap = C.base_parser("rms_qkv_int4_rope_multi.py", "RMSNorm + int4 QKV GEMV + RoPE QK multi-launch decode test")
    ap.add_argument("--print-kernels", action="store_true")
    C.add_compile_mode(ap)
    args = ap.parse_args(argv)
    print(f"RMS+int4 QKV+RoPE Multi-Launch (decode): emb={EMB_DIM}, kv={KV_DIM}, heads={N_HEADS}/{N_KV_HEADS}, "
          f"dk={HEAD_DIM}, gs={GS}")
    spec = build_rms_qkv_int4_rope_module(EMB_DIM, KV_DIM, N_HEADS, N_KV_HEADS, HEAD_DIM, GS, M_TILE, K_CHUNK, N_CORES,
                                          print_kernels=args.print_kernels)
    np.random.seed(42)
    x_in = np.random.uniform(-1.0, 1.0, (EMB_DIM,)).astype(bfloat16)
    norm_w = np.random.uniform(0.5, 1.5, (EMB_DIM,)).astype(bfloat16)

    def gen_awq_weights(m, k, gs):
        unp = np.random.randint(0, 16, size=(m, k), dtype=np.uint8)
        a_q = (unp[:, 0::2] | (unp[:, 1::2] << 4)).astype(np.uint8)
        a_s = np.random.uniform(0.005, 0.02, size=(k // gs, m)).astype(bfloat16)
        a_z = np.random.randint(7, 9, size=(k // gs, m), dtype=np.uint8)
        return a_q, a_s, a_z

    wq, wk, wv = (gen_awq_weights(m, EMB_DIM, GS) for m in (EMB_DIM, KV_DIM, KV_DIM))
    packed = [pack_inputs(*w, m, EMB_DIM, GS, M_TILE, K_CHUNK, N_CORES, m) for w, m in ((wq, EMB_DIM), (wk, KV_DIM), (wv, KV_DIM))]
    base_lut_row = generate_rope_lut(HEAD_DIM, seq_len=1)[0]
    lut_q = np.tile(base_lut_row, (N_HEADS, 1)).flatten().astype(bfloat16)
    lut_k = np.tile(base_lut_row, (N_KV_HEADS, 1)).flatten().astype(bfloat16)
    print("Computing CPU reference...")
    normed_ref = _rms_norm_ref(x_in, norm_w)
    q_ref, k_ref = int4_gemv_ref(*wq, normed_ref), int4_gemv_ref(*wk, normed_ref)
    z = lambda n: np.zeros(n, dtype=bfloat16)
    inputs = [x_in, norm_w, z(EMB_DIM), packed[0], z(EMB_DIM), packed[1], z(KV_DIM), packed[2], z(KV_DIM), lut_q, lut_k]
    C.finish(args, spec, dict(instance_name="rms_qkv_int4_rope"), inputs,
             [_rope_ref(q_ref, lut_q, HEAD_DIM), _rope_ref(k_ref, lut_k, HEAD_DIM)], rtol=0.2, atol=0.5, min_correlation=0.99)


if __name__ == "__main__":
    main()
