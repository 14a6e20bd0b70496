"""Generate tests/golden/*.npz by running mlir-air's OWN Python golden functions.

Run once where the mlir-air tree is available:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py --reference /path/to/mlir-air

The reference example files import the `air` MLIR bindings at module top; those
are not needed by the numpy golden functions, so `air.*` is replaced by inert
stand-ins (a meta-path finder returning MagicMock modules whose `module_builder`
is the identity decorator).  Everything stored comes out of the reference's own
`unpack_awq_int32`, `dequant_to_bf16`, `repack_hf_awq_linear`, `_gen_synthetic_awq`,
`pack_inputs` (x3) and `cpu_reference` (x4); the inline goldens that live under
`__main__` in dequant_awq.py / ffn_decode.py / ffn_prefill.py are replayed here
line for line from their seeds.  The tests never need the reference tree.
"""

import argparse
import importlib
import importlib.abc
import importlib.machinery
import os
import sys
from unittest import mock

import numpy as np
from ml_dtypes import bfloat16

_STAR = ["module_builder", "launch", "segment", "herd", "dma_memcpy_nd", "MemorySpace", "T",
         "IntegerType", "MemRefType", "IntegerAttr", "StringAttr", "UnitAttr", "AffineMap",
         "AffineExpr", "AffineConstantExpr", "AffineSymbolExpr", "VectorType", "IndexType",
         "Channel", "ChannelGet", "ChannelPut", "BF16Type", "F32Type"]


class _AirStub(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, name, path, target=None):
        if name == "air" or name.startswith("air."):
            return importlib.machinery.ModuleSpec(name, self, is_package=True)
        return None

    def create_module(self, spec):
        m = mock.MagicMock(name=spec.name)
        m.__name__ = spec.name
        m.__path__ = []
        m.__spec__ = spec
        m.__all__ = list(_STAR)
        m.module_builder = lambda f: f
        return m

    def exec_module(self, module):
        pass


def _import_from(path, modname):
    sys.path.insert(0, path)
    try:
        return importlib.import_module(modname)
    finally:
        sys.path.pop(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("MLIR_AIR_SRC"), required="MLIR_AIR_SRC" not in os.environ,
                    help="checkout of mlir-air (or set MLIR_AIR_SRC)")
    ap.add_argument("--out", default=os.path.dirname(os.path.abspath(__file__)))
    ap.add_argument("--big", action="store_true",
                    help="also replay the reference's 2048x2048 GEMV test shape (about 15 s)")
    ap.add_argument("--only", default="", help="comma-separated fixture names to (re)write; default: all")
    args = ap.parse_args()
    only = set(filter(None, args.only.split(",")))
    sys.dont_write_bytecode = True
    sys.meta_path.insert(0, _AirStub())
    pe = os.path.join(args.reference, "programming_examples")

    rp = _import_from(os.path.join(pe, "llms", "llama32_1b_int4"), "awq_repacker")
    mv = _import_from(os.path.join(pe, "matrix_vector_multiplication", "int4_awq"), "matvec_int4_packed")
    mva = _import_from(os.path.join(pe, "matrix_vector_multiplication", "int4_awq"), "matvec_int4_packed_add")
    sw = _import_from(os.path.join(pe, "decode_ffn_swiglu"), "matvec_int4_swiglu_rms")
    mm = _import_from(os.path.join(pe, "matrix_multiplication", "int4_awq"), "matmul_int4_packed")
    dq = _import_from(os.path.join(pe, "dequant_awq"), "dequant_awq")
    fd = _import_from(os.path.join(pe, "ffn_swiglu", "decode"), "ffn_decode")
    for extra in ("llms", os.path.join("llms", "llama32_1b"), os.path.join("llms", "llama32_1b_int4")):
        sys.path.insert(0, os.path.join(pe, extra))
    qkv = _import_from(os.path.join(pe, "llms", "llama32_1b_int4", "multi_launch_builder"), "rms_qkv_int4_rope_multi")
    lw = _import_from(os.path.join(pe, "llms", "llama32_1b"), "llama32_1b_weights")
    ap_ = _import_from(os.path.join(pe, "llms", "llama32_1b_int4"), "awq_pack")
    ofm = _import_from(os.path.join(pe, "llms", "llama32_1b_int4", "multi_launch_builder"), "o_gemv_ffn_int4_multi")
    off = _import_from(os.path.join(pe, "llms", "llama32_1b_int4", "multi_launch_builder"), "o_gemv_ffn_int4_fused")

    def save(name, **arrs):
        if only and name not in only:
            return
        out = {}
        for k, v in arrs.items():
            v = np.asarray(v)
            out[k] = v.view(np.uint16) if v.dtype == bfloat16 else v
            if v.dtype == bfloat16:
                out["__bf16__" + k] = np.array(1)
        np.savez_compressed(os.path.join(args.out, name + ".npz"), **out)
        print("wrote", name, {k: tuple(np.asarray(v).shape) for k, v in arrs.items()})

    # --- awq_repacker.self_test vectors (K=512, N=128, gs=128, seed 42) ----------
    rp.self_test(K=512, N=128, group_size=128, seed=42, verbose=True)
    K, N, GS = 512, 128, 128
    qweight, qzeros, scales, nibs, z_nibs = rp._gen_synthetic_awq(K, N, GS, seed=42)
    w_dense = rp.dequant_to_bf16(qweight, qzeros, scales, GS)
    A_q, A_s, A_z = rp.repack_hf_awq_linear(qweight, qzeros, scales, GS)
    x = np.random.default_rng(43).standard_normal(K).astype(bfloat16)
    y = mv.cpu_reference(A_q, A_s, A_z, x)
    packed = rp.repack_for_gemv(qweight, qzeros, scales, GS, M_TILE=8, K_CHUNK=512, N_CORES=8)
    save("awq_repacker_selftest", qweight=qweight, qzeros=qzeros, scales=scales, nibs=nibs,
         z_nibs=z_nibs, w_dense=w_dense, A_q=A_q, A_s=A_s, A_z=A_z, x=x, y=y, packed=packed)

    # second shape with two int32 blocks per 16 columns and 3 groups, gs=64
    qweight, qzeros, scales, nibs, z_nibs = rp._gen_synthetic_awq(192, 48, 64, seed=7)
    save("awq_repacker_gs64", qweight=qweight, qzeros=qzeros, scales=scales, nibs=nibs,
         z_nibs=z_nibs, w_dense=rp.dequant_to_bf16(qweight, qzeros, scales, 64))

    # --- awq_pack.py: the dequant, the NPU packer and the min/max quantiser on seeded inputs ---
    qweight, qzeros, scales, _, _ = rp._gen_synthetic_awq(256, 64, 128, seed=11)
    Wb = (np.random.default_rng(12).standard_normal((256, 48)) * 0.05).astype(bfloat16)  # [K, N] prefill orientation
    Wq, Ws, Wz = ap_.fake_quantize_awq_int4(np.ascontiguousarray(Wb.T), gs=64)
    save("awq_pack_256x64", qweight=qweight, qzeros=qzeros, scales=scales.astype(bfloat16),
         dense=ap_.awq_dequant_layer(qweight, qzeros, scales.astype(bfloat16), gs=128),
         packed=ap_.awq_pack_for_npu(qweight, qzeros, scales.astype(bfloat16), gs=128, n_tile=16, k_chunk=128, M_seq=64),
         W=Wb, W_q=Wq, W_s=Ws, W_z=Wz,
         W_packed=ap_.pack_weight_for_int4_gemm(Wb, 64, gs=64, n_tile=16, k_chunk=128))

    # --- o_gemv_ffn_int4_{multi,fused}.py: the post-attention block goldens at a small shape ---
    emb, hid, gs_ = 256, 512, 128
    np.random.seed(42)
    wo = ofm._gen_int4_weights(emb, emb, gs_, 100)
    gu = ofm._gen_int4_weights(2 * hid, emb, gs_, 150)
    wd = ofm._gen_int4_weights(emb, hid, gs_, 200)
    attn = np.random.randn(emb).astype(bfloat16)
    xres = np.random.randn(emb).astype(bfloat16)
    fnw = (np.random.randn(emb) * 0.1 + 1.0).astype(bfloat16)
    res1 = mva.cpu_reference(wo[0], wo[1], wo[2], attn, xres)
    swi = off.lgu_cpu_reference(gu[0], gu[1], gu[2], res1, fnw)
    save("o_gemv_ffn_int4_256x512", wo_q=wo[0], wo_s=wo[1], wo_z=wo[2], gu_q=gu[0], gu_s=gu[1], gu_z=gu[2], wd_q=wd[0],
         wd_s=wd[1], wd_z=wd[2], attn_out=attn, x_residual=xres, ffn_norm_w=fnw,
         multi_out=ofm.o_gemv_ffn_int4_reference(wo[3], attn, xres, fnw, gu[3][0::2], gu[3][1::2], wd[3]),
         res1=res1, swiglu=swi, fused_out=off.ld_cpu_reference(wd[0], wd[1], wd[2], swi, res1))

    # --- rms_qkv_int4_rope_multi.py: RMSNorm -> Q/K/V int4 GEMVs -> half-split RoPE on Q and K, its
    #     __main__ data recipe (:640-687) at a small shape, positions 0..3 of the reference's LUT ---
    EMB, KVD, NH, NKV, HD = 256, 64, 4, 1, 64
    np.random.seed(42)
    x_in = np.random.uniform(-1.0, 1.0, (EMB,)).astype(bfloat16)
    norm_w = np.random.uniform(0.5, 1.5, (EMB,)).astype(bfloat16)

    def gen_awq_weights(m, k, gs):
        unp = np.random.randint(0, 16, size=(m, k), dtype=np.uint8)
        a_q = (unp[:, 0::2] | (unp[:, 1::2] << 4)).astype(np.uint8)
        a_s = np.random.uniform(0.005, 0.02, size=(k // gs, m)).astype(bfloat16)
        a_z = np.random.randint(7, 9, size=(k // gs, m), dtype=np.uint8)
        return a_q, a_s, a_z

    wq, wk, wv = gen_awq_weights(EMB, EMB, 128), gen_awq_weights(KVD, EMB, 128), gen_awq_weights(KVD, EMB, 128)
    cfg = lw.LlamaConfig()
    cfg.head_dim = HD
    lut = lw.generate_rope_lut(cfg, seq_len=4, dtype=bfloat16)
    normed = qkv._rms_norm_ref(x_in, norm_w)
    q_ref, k_ref, v_ref = (mv.cpu_reference(*w, normed) for w in (wq, wk, wv))
    pos = 3
    lut_q = np.tile(lut[pos], (NH, 1)).flatten().astype(bfloat16)
    lut_k = np.tile(lut[pos], (NKV, 1)).flatten().astype(bfloat16)
    save("rms_qkv_int4_rope_256", x_in=x_in, norm_w=norm_w, wq_q=wq[0], wq_s=wq[1], wq_z=wq[2], wk_q=wk[0], wk_s=wk[1],
         wk_z=wk[2], wv_q=wv[0], wv_s=wv[1], wv_z=wv[2], lut=lut, pos=np.array(pos), normed=normed, q=q_ref, k=k_ref,
         v=v_ref, q_roped=qkv._rope_ref(q_ref, lut_q, HD), k_roped=qkv._rope_ref(k_ref, lut_k, HD),
         rope_base=np.array(cfg.rope_base))

    # --- the example scripts' seeded inputs (np.random.seed(42)), small shapes ---
    def gemv_inputs(M, K, GS, residual=False, rms=False):
        np.random.seed(42)
        unp = np.random.randint(0, 16, size=(M, K), dtype=np.uint8)
        A_q = (unp[:, 0::2] | (unp[:, 1::2] << 4)).astype(np.uint8)
        A_s = np.random.uniform(0.005, 0.02, size=(K // GS, M)).astype(bfloat16)
        A_z = np.random.randint(7, 9, size=(K // GS, M), dtype=np.uint8)
        B = np.random.randn(K).astype(bfloat16)
        extra = None
        if residual:
            extra = np.random.randn(M).astype(bfloat16)
        if rms:
            extra = (np.random.randn(K) * 0.1 + 1.0).astype(bfloat16)
        return A_q, A_s, A_z, B, extra

    M, K, GS = 64, 512, 128
    A_q, A_s, A_z, B, _ = gemv_inputs(M, K, GS)
    save("matvec_int4_packed_64x512", A_q=A_q, A_s=A_s, A_z=A_z, B=B,
         D=mv.cpu_reference(A_q, A_s, A_z, B),
         packed=mv.pack_inputs(A_q, A_s, A_z, M, K, GS, 8, 256, 4, 32))
    A_q, A_s, A_z, B, R = gemv_inputs(M, K, GS, residual=True)
    save("matvec_int4_packed_add_64x512", A_q=A_q, A_s=A_s, A_z=A_z, B=B, R=R,
         D=mva.cpu_reference(A_q, A_s, A_z, B, R))
    M, K = 256, 512
    A_q, A_s, A_z, xin, gamma = gemv_inputs(M, K, GS, rms=True)
    RMS_in = np.stack([xin, gamma], axis=0).astype(bfloat16)
    save("matvec_int4_swiglu_rms_256x512", A_q=A_q, A_s=A_s, A_z=A_z, RMS_in=RMS_in,
         D=sw.cpu_reference(A_q, A_s, A_z, RMS_in))

    if args.big:
        M = K = 2048
        A_q, A_s, A_z, B, _ = gemv_inputs(M, K, 128)
        save("matvec_int4_packed_2048x2048_D", D=mv.cpu_reference(A_q, A_s, A_z, B))

    # matmul_int4_packed defaults (m 64, k 128, n 128) and a 2-group shape
    for (Mm, Kk, Nn) in [(64, 128, 128), (32, 256, 64)]:
        np.random.seed(42)
        unp = np.random.randint(0, 16, size=(Nn, Kk), dtype=np.uint8)
        W_q = (unp[:, 0::2] | (unp[:, 1::2] << 4)).astype(np.uint8)
        W_s = np.random.uniform(0.005, 0.02, size=(Kk // 128, Nn)).astype(bfloat16)
        W_z = np.random.randint(7, 9, size=(Kk // 128, Nn), dtype=np.uint8)
        A = np.random.randn(Mm, Kk).astype(bfloat16)
        save(f"matmul_int4_packed_{Mm}x{Kk}x{Nn}", W_q=W_q, W_s=W_s, W_z=W_z, A=A,
             C=mm.cpu_reference(W_q, W_s, W_z, A),
             packed=mm.pack_inputs(W_q, W_s, W_z, Mm, Kk, Nn, 128, 16, 128))

    # dequant_awq.py: seed 0, N=1024, gs=128, herd 4; golden loop of :391-396
    n, gs, herd = 1024, 128, 4
    np.random.seed(0)
    int4_vals = np.random.randint(0, 16, n).astype(np.uint8)
    sc = np.random.uniform(0.01, 0.1, n // gs).astype(bfloat16)
    zr = np.random.randint(7, 10, n // gs).astype(np.uint8)
    ref = np.zeros(n, dtype=bfloat16)
    for i in range(n):
        g = i // gs
        ref[i] = bfloat16((float(int4_vals[i]) - float(zr[g])) * float(sc[g]))
    save("dequant_awq_1024", int4_vals=int4_vals, scales=sc, zeros=zr, ref=ref,
         packed=dq.pack_inputs(int4_vals, sc, zr, n, gs, herd),
         tile_bytes=np.array(dq.packed_tile_bytes(n // herd, gs)))

    # ffn_swiglu/decode (dim 128, 4 cols, seed 0) and prefill (seq 16) goldens
    dim, cols = 128, 4
    np.random.seed(0)
    xv = (np.random.randn(dim) * 0.1).astype(bfloat16)
    Wg = (np.random.randn(dim, dim) * 0.1).astype(bfloat16)
    Wu = (np.random.randn(dim, dim) * 0.1).astype(bfloat16)
    Wd = (np.random.randn(dim, dim) * 0.1).astype(bfloat16)
    xf = xv.astype(np.float32)
    gate = Wg.astype(np.float32) @ xf
    up = Wu.astype(np.float32) @ xf
    inter = gate * (1.0 / (1.0 + np.exp(-gate))) * up
    out = (Wd.astype(np.float32) @ inter).astype(bfloat16)
    dim_m = dim // cols
    pk = np.concatenate([
        np.concatenate([fd.transpose_32bit_words(W[c * dim_m:(c + 1) * dim_m, :], dim_m, dim)
                        for c in range(cols)]) for W in (Wg, Wu, Wd)]).astype(bfloat16)
    save("ffn_decode_128", x=xv, W_gate=Wg, W_up=Wu, W_down=Wd, out=out, packed_weights=pk)

    seq = 16
    np.random.seed(0)
    xm = (np.random.randn(seq, dim) * 0.1).astype(bfloat16)
    Wg = (np.random.randn(dim, dim) * 0.1).astype(bfloat16)
    Wu = (np.random.randn(dim, dim) * 0.1).astype(bfloat16)
    Wd = (np.random.randn(dim, dim) * 0.1).astype(bfloat16)
    xf = xm.astype(np.float32)
    gate = xf @ Wg.astype(np.float32).T
    up = xf @ Wu.astype(np.float32).T
    inter = gate * (1.0 / (1.0 + np.exp(-gate))) * up
    out = (inter @ Wd.astype(np.float32).T).astype(bfloat16)
    dim_n = dim // cols
    pk = np.concatenate([
        np.concatenate([W[:, c * dim_n:(c + 1) * dim_n].reshape(-1) for c in range(cols)])
        for W in (Wg, Wu, Wd)]).astype(bfloat16)
    save("ffn_prefill_16x128", x=xm, W_gate=Wg, W_up=Wu, W_down=Wd, out=out, packed_weights=pk)


if __name__ == "__main__":
    main()
