"""GPU parity: every CUDA entry point, called through the C ABI, against the numpy oracle
and the committed golden fixtures.  Bit-exact for the dequantised weights and all byte /
integer repacks; rel-L2 <= 1e-2 (f32 accumulate) for GEMV / FFN / GEMM outputs."""
import numpy as np
import pytest
import torch
from ml_dtypes import bfloat16

from oracle import awq_oracle as O
from golden_util import load, bits
from gpu_util import to_dev, to_host, synth_awq, dev_weight, randn_bf16

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-2  # the benchmark definition's tolerance for GEMV / GEMM / FFN outputs


@pytest.fixture(scope="module")
def ops():
    from mlir_air_b200 import ops as _ops
    return _ops


@pytest.fixture(autouse=True)
def _auto_kernels(ops):
    ops.set_decode_kernel("auto")
    ops.set_gemm_kernel("auto")
    yield
    ops.set_decode_kernel("auto")
    ops.set_gemm_kernel("auto")


# ------------------------------------------------------------------ dequant (rows a1/a2)
@pytest.mark.parametrize("name,gs", [("awq_repacker_selftest", 128), ("awq_repacker_gs64", 64)])
def test_dequant_golden_bit_exact(ops, name, gs):
    g = load(name)
    w = dev_weight(g["qweight"], g["qzeros"], g["scales"], gs)
    out = to_host(ops.dequant(w))
    assert np.array_equal(bits(out), bits(g["w_dense"]))


def test_dequant_cfg1_bit_exact(ops):
    qw, qz, s = synth_awq(2048, 2048, 128, seed=0)
    out = to_host(ops.dequant(dev_weight(qw, qz, s)))
    assert np.array_equal(bits(out), bits(O.dequant_to_bf16(qw, qz, s, 128)))


@pytest.mark.parametrize("K,N,gs", [(128, 8, 128), (256, 40, 64), (96, 1032, 32), (4096, 11008, 128)])
def test_dequant_shapes_bit_exact(ops, K, N, gs):
    qw, qz, s = synth_awq(K, N, gs, seed=K + N)
    out = to_host(ops.dequant(dev_weight(qw, qz, s, gs)))
    assert np.array_equal(bits(out), bits(O.dequant_to_bf16(qw, qz, s, gs)))


def test_dequant_extreme_values(ops):
    """All 256 (q, z) pairs against scales at the ends of the bf16 range used by AWQ."""
    K, N = 128, 16 * 16
    nibs = np.tile(np.repeat(np.arange(16, dtype=np.uint8), 16)[None, :], (K, 1))
    z = np.tile(np.arange(16, dtype=np.uint8), 16)[None, :]
    s = np.array([1e-6, 0.001, 0.0123, 0.02, 1.0, 3.3895e38 / 16] * 43, dtype=np.float32)[:N][None, :].astype(bfloat16)
    qw, qz = O.pack_awq_int32(nibs), O.pack_awq_int32(z)
    out = to_host(ops.dequant(dev_weight(qw, qz, s)))
    assert np.array_equal(bits(out), bits(O.dequant_to_bf16(qw, qz, s, 128)))


def test_dequant_empty(ops):
    w = dev_weight(np.zeros((0, 4), np.int32), np.zeros((0, 4), np.int32), np.zeros((0, 32), bfloat16))
    assert ops.dequant(w).shape == (0, 32)


def test_dequant_1d_example_golden(ops):
    g = load("dequant_awq_1024")
    pq = (g["int4_vals"][0::2] | (g["int4_vals"][1::2] << 4)).astype(np.uint8)
    out = ops.dequant_1d(to_dev(pq), to_dev(g["scales"]), to_dev(g["zeros"]), 1024, 128)
    assert np.array_equal(bits(to_host(out)), bits(g["ref"]))


def test_bad_arguments_raise(ops):
    from mlir_air_b200._lib import AwqBackendError
    qw, qz, s = synth_awq(256, 64, 128, seed=1)
    w = dev_weight(qw, qz, s)
    w.group_size = 100  # K % gs != 0
    with pytest.raises(AwqBackendError):
        ops.dequant(w)


# ------------------------------------------------------------------ layout converters (row a3)
def test_repack_B_A_roundtrip_exact(ops):
    g = load("awq_repacker_selftest")
    w = ops.repack_B_to_A(to_dev(g["A_q"]), to_dev(g["A_s"]), to_dev(g["A_z"]), 128)
    assert np.array_equal(to_host(w.qweight), g["qweight"])
    assert np.array_equal(to_host(w.qzeros), g["qzeros"])
    assert np.array_equal(bits(to_host(w.scales)), bits(g["scales"].astype(bfloat16)))
    A_q, A_s, A_z = ops.repack_A_to_B(w)
    assert np.array_equal(to_host(A_q), g["A_q"]) and np.array_equal(to_host(A_z), g["A_z"])
    assert np.array_equal(bits(to_host(A_s)), bits(g["A_s"]))


def test_interleave_gate_up_exact(ops):
    K, I = 256, 72
    gq, gz, gs_ = synth_awq(K, I, 128, seed=3)
    uq, uz, us = synth_awq(K, I, 128, seed=4)
    w = ops.interleave_gate_up(dev_weight(gq, gz, gs_), dev_weight(uq, uz, us))
    nib = np.empty((K, 2 * I), np.uint8)
    nib[:, 0::2], nib[:, 1::2] = O.unpack_awq_int32(gq), O.unpack_awq_int32(uq)
    zn = np.empty((K // 128, 2 * I), np.uint8)
    zn[:, 0::2], zn[:, 1::2] = O.unpack_awq_int32(gz), O.unpack_awq_int32(uz)
    sc = np.empty((K // 128, 2 * I), bfloat16)
    sc[:, 0::2], sc[:, 1::2] = gs_, us
    assert np.array_equal(to_host(w.qweight), O.pack_awq_int32(nib))
    assert np.array_equal(to_host(w.qzeros), O.pack_awq_int32(zn))
    assert np.array_equal(bits(to_host(w.scales)), bits(sc))


# ------------------------------------------------------------------ decode GEMV (rows a4/a5)
GEMV_SHAPES = [(1, 512, 256), (3, 1024, 1056), (8, 2048, 4096), (2, 256, 32), (5, 11008, 4096)]


@pytest.mark.parametrize("kernel", ["generic", "streamk", "streamk_bf16"])
@pytest.mark.parametrize("B,K,N", GEMV_SHAPES)
def test_gemv_vs_oracle(ops, kernel, B, K, N):
    ops.set_decode_kernel(kernel)
    qw, qz, s = synth_awq(K, N, 128, seed=B * 7 + K)
    x = randn_bf16((B, K), seed=11)
    r = randn_bf16((B, N), seed=12)
    w = dev_weight(qw, qz, s)
    ws = ops.Workspace(K, N)
    y = to_host(ops.gemv(to_dev(x), w, ws))
    yr = to_host(ops.gemv(to_dev(x), w, ws, residual=to_dev(r)))
    yf = to_host(ops.gemv(to_dev(x), w, ws, f32_out=True))
    ws.check()
    assert O.rel_l2(y, O.gemv_A_ref(x, qw, qz, s, 128)) <= REL_L2_TOL
    assert O.rel_l2(yr, O.gemv_A_ref(x, qw, qz, s, 128, residual=r)) <= REL_L2_TOL
    ref32 = x.astype(np.float32) @ O.dequant_f32(qw, qz, s, 128)
    assert O.rel_l2(yf, ref32) <= 1e-4
    # second golden of the north star: bf16-rounded weights
    ref_b = (x.astype(np.float32) @ O.dequant_to_bf16(qw, qz, s, 128).astype(np.float32)).astype(bfloat16)
    assert O.rel_l2(y, ref_b) <= REL_L2_TOL


def test_gemv_cfg2_full_size(ops):
    """Benchmark configuration 2: [B, 4096] x [4096, 11008], B = 1 and 8."""
    qw, qz, s = synth_awq(4096, 11008, 128, seed=0)
    wf = O.dequant_f32(qw, qz, s, 128)
    w = dev_weight(qw, qz, s)
    ws = ops.Workspace(4096, 11008)
    for B in (1, 8):
        x = randn_bf16((B, 4096), seed=B)
        ref = (x.astype(np.float32) @ wf).astype(bfloat16)
        for kernel in ("streamk", "streamk_bf16", "generic"):
            ops.set_decode_kernel(kernel)
            y = to_host(ops.gemv(to_dev(x), w, ws))
            assert O.rel_l2(y, ref) <= REL_L2_TOL, (kernel, B)
    ws.check()


def test_gemv_streamk_is_deterministic(ops):
    """With the fixed-order reduction selected, repeated runs give identical bits, and the default
    (atomic) reduction agrees with it to f32 summation error."""
    ops.set_decode_kernel("streamk")
    ops.set_deterministic(True)
    qw, qz, s = synth_awq(4096, 4096, 128, seed=5)
    w = dev_weight(qw, qz, s)
    ws = ops.Workspace(4096, 4096)
    x = to_dev(randn_bf16((8, 4096), seed=6))
    y0 = to_host(ops.gemv(x, w, ws))
    try:
        for _ in range(3):
            assert np.array_equal(bits(to_host(ops.gemv(x, w, ws))), bits(y0))
        f_det = to_host(ops.gemv(x, w, ws, f32_out=True))
        ops.set_deterministic(False)
        f_fast = to_host(ops.gemv(x, w, ws, f32_out=True))
        assert O.rel_l2(f_fast, f_det) <= 1e-6
    finally:
        ops.set_deterministic(False)
    ws.check()


def test_gemv_batch_over_8(ops):
    qw, qz, s = synth_awq(1024, 512, 128, seed=8)
    x = randn_bf16((19, 1024), seed=9)
    w = dev_weight(qw, qz, s)
    ws = ops.Workspace(1024, 512)
    ref = O.gemv_A_ref(x, qw, qz, s, 128)
    for kernel in ("streamk", "streamk_bf16", "generic"):
        ops.set_decode_kernel(kernel)
        assert O.rel_l2(to_host(ops.gemv(to_dev(x), w, ws)), ref) <= REL_L2_TOL
    ws.check()


def test_gemv_linearity_full_size(ops):
    """Size-independent property at the 70B down-projection shape: y(x1) + y(x2) == y(x1 + x2)
    in f32 partials (up to f32 summation error), and a zero input gives exactly zero."""
    K, N = 28672, 8192
    qw, qz, s = synth_awq(K, N, 128, seed=2)
    w = dev_weight(qw, qz, s)
    ws = ops.Workspace(K, N)
    x1 = np.zeros((1, K), bfloat16); x1[0, ::2] = randn_bf16(K // 2, 1)
    x2 = np.zeros((1, K), bfloat16); x2[0, 1::2] = randn_bf16(K // 2, 2)
    y1 = to_host(ops.gemv(to_dev(x1), w, ws, f32_out=True))
    y2 = to_host(ops.gemv(to_dev(x2), w, ws, f32_out=True))
    y12 = to_host(ops.gemv(to_dev((x1.astype(np.float32) + x2.astype(np.float32)).astype(bfloat16)), w, ws, f32_out=True))
    assert O.rel_l2(y1 + y2, y12) <= 1e-4
    y0 = to_host(ops.gemv(to_dev(np.zeros((1, K), bfloat16)), w, ws, f32_out=True))
    assert np.all(y0 == 0)
    ws.check()


def test_gemv_reference_example_fixture(ops):
    """matvec_int4_packed.py inputs (layout B, seed 42) -> repack on the GPU -> GEMV, judged with
    the reference's own tolerances (rtol .1, atol .05, corr >= .999) and with rel-L2."""
    for name, has_r in (("matvec_int4_packed_64x512", False), ("matvec_int4_packed_add_64x512", True)):
        g = load(name)
        w = ops.repack_B_to_A(to_dev(g["A_q"]), to_dev(g["A_s"]), to_dev(g["A_z"]), 128)
        ws = ops.Workspace(w.K, w.N)
        res = to_dev(g["R"].reshape(1, -1)) if has_r else None
        y = to_host(ops.gemv(to_dev(g["B"].reshape(1, -1)), w, ws, residual=res))[0]
        a, e = y.astype(np.float64), g["D"].astype(np.float64)
        assert np.isclose(a, e, rtol=0.1, atol=0.05).all()
        assert np.corrcoef(a, e)[0, 1] >= 0.999
        assert O.rel_l2(y, g["D"]) <= REL_L2_TOL


# ------------------------------------------------------------------ RMSNorm + SwiGLU (row a6)
def test_rmsnorm_vs_oracle(ops):
    x = randn_bf16((5, 4096), seed=1)
    gamma = (np.random.default_rng(2).standard_normal(4096) * 0.1 + 1.0).astype(bfloat16)
    out = to_host(ops.rmsnorm(to_dev(x), to_dev(gamma), 1e-5))
    ref = np.stack([O.rmsnorm_ref(r, gamma, 1e-5) for r in x])
    # one bf16 ulp at most (f32 summation order), and almost all elements identical
    d = np.abs(bits(out).astype(np.int32) - bits(ref).astype(np.int32))
    assert d.max() <= 1 and (d != 0).mean() < 0.01


def test_swiglu_rms_reference_example_fixture(ops):
    g = load("matvec_int4_swiglu_rms_256x512")
    w = ops.repack_B_to_A(to_dev(g["A_q"]), to_dev(g["A_s"]), to_dev(g["A_z"]), 128)  # [K, 2I] interleaved
    ws = ops.Workspace(w.K, w.N)
    for kernel in ("generic", "streamk", "streamk_bf16"):
        ops.set_decode_kernel(kernel)
        normed = ops.rmsnorm(to_dev(g["RMS_in"][0:1]), to_dev(g["RMS_in"][1]), 1e-5)
        y = to_host(ops.gateup_swiglu(normed, w, ws))[0]
        a, e = y.astype(np.float64), g["D"].astype(np.float64)
        assert np.isclose(a, e, rtol=0.15, atol=0.5).all()
        assert np.corrcoef(a, e)[0, 1] >= 0.99
        assert O.rel_l2(y, g["D"]) <= REL_L2_TOL
    ws.check()


def _ffn_weights(H, I, seed):
    gate = synth_awq(H, I, 128, seed=seed)
    up = synth_awq(H, I, 128, seed=seed + 1)
    down = synth_awq(I, H, 128, seed=seed + 2)
    return gate, up, down


@pytest.mark.parametrize("kernel", ["generic", "streamk", "streamk_bf16"])
@pytest.mark.parametrize("B,H,I", [(1, 512, 1408), (4, 1024, 2816), (16, 512, 1024)])
def test_ffn_decode_vs_oracle(ops, kernel, B, H, I):
    ops.set_decode_kernel(kernel)
    gate, up, down = _ffn_weights(H, I, seed=H + I)
    x = randn_bf16((B, H), seed=3)
    gamma = (np.random.default_rng(4).standard_normal(H) * 0.1 + 1.0).astype(bfloat16)
    wgu = ops.interleave_gate_up(dev_weight(*gate), dev_weight(*up))
    wd = dev_weight(*down)
    ws = ops.Workspace(max(H, I), max(2 * I, H))
    # plain FFN (config 3 form) and the stack layer form (norm + residual)
    y = to_host(ops.ffn_decode(to_dev(x), wgu, wd, ws))
    assert O.rel_l2(y, O.ffn_A_ref(x, gate, up, down, 128)) <= REL_L2_TOL
    y2 = to_host(ops.ffn_decode(to_dev(x), wgu, wd, ws, gamma=to_dev(gamma), residual=to_dev(x)))
    assert O.rel_l2(y2, O.ffn_layer_A_ref(x, gamma, gate, up, down, 128)) <= REL_L2_TOL
    t = to_host(ops.gateup_swiglu(to_dev(x), wgu, ws))
    assert O.rel_l2(t, O.gateup_swiglu_A_ref(x, gate, up, 128)) <= REL_L2_TOL
    ws.check()


def test_ffn_cfg3_full_size(ops):
    """Benchmark configuration 3: hidden 4096, intermediate 11008, batch 1 / 4 / 16."""
    H, I = 4096, 11008
    gate, up, down = _ffn_weights(H, I, seed=0)
    wgu = ops.interleave_gate_up(dev_weight(*gate), dev_weight(*up))
    wd = dev_weight(*down)
    ws = ops.Workspace(I, 2 * I)
    fg, fu, fd = (O.dequant_f32(*m, 128) for m in (gate, up, down))
    for B in (1, 4, 16):
        x = randn_bf16((B, H), seed=B)
        xf = x.astype(np.float32)
        g = (xf @ fg).astype(bfloat16).astype(np.float32)
        u = (xf @ fu).astype(bfloat16).astype(np.float32)
        t = (g * 0.5 * (np.tanh(g / 2.0) + 1.0) * u).astype(bfloat16)
        ref = (t.astype(np.float32) @ fd).astype(bfloat16)
        y = to_host(ops.ffn_decode(to_dev(x), wgu, wd, ws))
        assert O.rel_l2(y, ref) <= REL_L2_TOL, B
    ws.check()


def test_fp16_activation_formats_agree_with_bf16(ops):
    """The internal fp16 activation format is exact for bf16 values with 2^-14 <= |x| <= 65504: feeding the same
    values as fp16 gives the same bits as feeding bf16, for both kernels.  (standard-normal values: the few below
    2^-14 are themselves multiples of 2^-24 only by luck, which is why the tiny-activation test below exists.)"""
    import torch
    K, N = 1024, 1536
    qw, qz, s = synth_awq(K, N, 128, seed=31)
    w = dev_weight(qw, qz, s)
    ws = ops.Workspace(K, N)
    x = to_dev(randn_bf16((5, K), seed=32))
    for kernel in ("streamk", "generic"):
        ops.set_decode_kernel(kernel)
        y_b = to_host(ops.gemv(x, w, ws))
        y_h = to_host(ops.gemv(x.to(torch.float16), w, ws, x_f16=True))
        assert np.array_equal(bits(y_b), bits(y_h)), kernel
        t_b = ops.gateup_swiglu(x, w, ws)
        t_h = ops.gateup_swiglu(x, w, ws, out_f16=True)
        assert torch.equal(t_b.float(), t_h.float()), kernel
    n_b = ops.rmsnorm(x, to_dev(randn_bf16(K, seed=33)), 1e-5)
    n_h = ops.rmsnorm(x, to_dev(randn_bf16(K, seed=33)), 1e-5, out_f16=True)
    assert torch.equal(n_b.float(), n_h.float())
    ws.check()


def test_tiny_activations_lose_bits_in_fp16_but_stay_inside_the_bar(ops):
    """Activations far below 2^-14 land in fp16 subnormals (2^-24 absolute resolution) on the default path: the
    result is no longer bit-identical to the bf16 path, but still within the tolerance of the oracle; the bf16
    activation path is exact for them.  (Scales of 0.5 to 1 keep the sums near 3e-3: split-K partial sums are handed over
    with an absolute resolution of 2^-20, which sums of 4e-5, what the usual scales would give, would feel.)"""
    K, N = 1024, 1536
    qw, qz, s = synth_awq(K, N, 128, seed=51, scale_lo=0.5, scale_hi=1.0)
    w = dev_weight(qw, qz, s)
    x = (np.random.default_rng(52).standard_normal((4, K)) * 3e-5).astype(bfloat16)  # most |x| < 2^-14 = 6.1e-5
    assert (np.abs(x.astype(np.float32)) < 2.0 ** -14).mean() > 0.9
    ref = O.gemv_A_ref(x, qw, qz, s, 128)
    ws = ops.Workspace(K, N)
    try:
        ops.set_decode_kernel("streamk")
        y_h = to_host(ops.gemv(to_dev(x), w, ws))
        ops.set_decode_kernel("streamk_bf16")
        y_b = to_host(ops.gemv(to_dev(x), w, ws))
        ws.check()
    finally:
        ops.set_decode_kernel("auto")
    assert O.rel_l2(y_b, ref) <= 2e-3
    assert O.rel_l2(y_h, ref) <= REL_L2_TOL
    assert not np.array_equal(bits(y_h), bits(y_b)), "fp16 subnormals cannot hold these values exactly"


def test_fp16_overflow_is_reported_and_bf16_path_handles_it(ops):
    from mlir_air_b200._lib import AwqBackendError
    K, N = 256, 512
    qw, qz, s = synth_awq(K, N, 128, seed=41)
    w = dev_weight(qw, qz, s)
    x = randn_bf16((2, K), seed=42)
    x[0, 3] = bfloat16(1.0e6)  # beyond fp16
    ref = O.gemv_A_ref(x, qw, qz, s, 128)
    ops.set_decode_kernel("streamk")
    ws = ops.Workspace(K, N)
    ops.gemv(to_dev(x), w, ws)
    with pytest.raises(AwqBackendError):
        ws.check()
    ops.set_decode_kernel("streamk_bf16")
    ws = ops.Workspace(K, N)
    y = to_host(ops.gemv(to_dev(x), w, ws))
    ws.check()
    assert O.rel_l2(y, ref) <= REL_L2_TOL


# ------------------------------------------------------------------ prefill GEMM (row a9)
@pytest.mark.parametrize("name", ["matmul_int4_packed_64x128x128", "matmul_int4_packed_32x256x64"])
def test_gemm_reference_example_fixture(ops, name):
    g = load(name)
    w = ops.repack_B_to_A(to_dev(g["W_q"]), to_dev(g["W_s"]), to_dev(g["W_z"]), 128)
    for kernel in ("generic", "auto"):
        ops.set_gemm_kernel(kernel)
        c = to_host(ops.gemm(to_dev(g["A"]), w))
        a, e = c.astype(np.float64), g["C"].astype(np.float64)
        assert (~np.isclose(a, e, rtol=0.1, atol=0.05)).mean() <= 0.0005
        assert np.corrcoef(a.ravel(), e.ravel())[0, 1] >= 0.999
        assert O.rel_l2(c, g["C"]) <= REL_L2_TOL


@pytest.mark.parametrize("M,K,N", [(64, 256, 128), (100, 512, 200), (256, 1024, 512), (2048, 512, 256)])
def test_gemm_vs_oracle(ops, M, K, N):
    qw, qz, s = synth_awq(K, N, 128, seed=M + N)
    A = randn_bf16((M, K), seed=5)
    ref = (A.astype(np.float32) @ O.dequant_f32(qw, qz, s, 128)).astype(bfloat16)
    for kernel in ("generic", "auto"):
        ops.set_gemm_kernel(kernel)
        c = to_host(ops.gemm(to_dev(A), dev_weight(qw, qz, s)))
        ops.gemm_check()
        assert O.rel_l2(c, ref) <= REL_L2_TOL, kernel


@pytest.mark.parametrize("M,K,N", [(128, 128, 256), (1, 128, 32), (130, 384, 288), (300, 1024, 1056), (512, 2048, 768)])
def test_gemm_tensor_core_kernel(ops, M, K, N):
    """The tcgen05 kernel alone: ragged M and N tiles, several tiles per CTA, against both goldens
    (f32 weights, and the bf16-rounded weights the kernel actually multiplies)."""
    ops.set_gemm_kernel("tc")
    qw, qz, s = synth_awq(K, N, 128, seed=3 * M + N)
    A = randn_bf16((M, K), seed=7)
    c = to_host(ops.gemm(to_dev(A), dev_weight(qw, qz, s)))
    ops.gemm_check()
    ref_f32w = (A.astype(np.float32) @ O.dequant_f32(qw, qz, s, 128)).astype(bfloat16)
    ref_bf16w = (A.astype(np.float32) @ O.dequant_to_bf16(qw, qz, s, 128).astype(np.float32)).astype(bfloat16)
    assert O.rel_l2(c, ref_bf16w) <= 3e-3   # same products, f32 summation order only
    assert O.rel_l2(c, ref_f32w) <= REL_L2_TOL


@pytest.mark.parametrize("M,K,N", [(192, 128, 256), (1, 128, 32), (130, 384, 288), (300, 1024, 1056), (512, 2048, 768), (2048, 512, 256),
                                   (65, 256, 4096)])
def test_gemm_tensor_memory_kernel(ops, M, K, N):
    """The tcgen05 kernel that keeps the dequantised weights in tensor memory (operands swapped, 192-row tiles): ragged
    row and column tiles, several tiles per CTA, all three epilogues, against both goldens."""
    ops.set_gemm_kernel("tm")
    try:
        qw, qz, s = synth_awq(K, N, 128, seed=3 * M + N)
        A = randn_bf16((M, K), seed=7)
        w = dev_weight(qw, qz, s)
        c = to_host(ops.gemm(to_dev(A), w))
        ops.gemm_check()
        ref_f32w = (A.astype(np.float32) @ O.dequant_f32(qw, qz, s, 128)).astype(bfloat16)
        ref_bf16w = (A.astype(np.float32) @ O.dequant_to_bf16(qw, qz, s, 128).astype(np.float32)).astype(bfloat16)
        assert O.rel_l2(c, ref_bf16w) <= 3e-3   # same products, f32 summation order only
        assert O.rel_l2(c, ref_f32w) <= REL_L2_TOL
        R = randn_bf16((M, N), seed=9)
        cr = to_host(ops.gemm(to_dev(A), w, residual=to_dev(R)))
        assert O.rel_l2(cr, O.gemv_A_ref(A, qw, qz, s, 128, residual=R)) <= REL_L2_TOL
        if N % 64 == 0:
            gate, up = synth_awq(K, N // 2, 128, seed=4), synth_awq(K, N // 2, 128, seed=5)
            wgu = ops.interleave_gate_up(dev_weight(*gate), dev_weight(*up))
            t = to_host(ops.gemm(to_dev(A), wgu, swiglu=True))
            assert O.rel_l2(t, O.gateup_swiglu_A_ref(A, gate, up, 128)) <= REL_L2_TOL
        ops.gemm_check()
    finally:
        ops.set_gemm_kernel("auto")


def test_gemm_cfg4_full_size(ops):
    """Benchmark configuration 4: [2048, 4096] x [4096, 14336]."""
    M, K, N = 2048, 4096, 14336
    qw, qz, s = synth_awq(K, N, 128, seed=0)
    A = randn_bf16((M, K), seed=1)
    ops.set_gemm_kernel("tc")
    c = to_host(ops.gemm(to_dev(A), dev_weight(qw, qz, s)))
    ops.gemm_check()
    ref = (A.astype(np.float32) @ O.dequant_f32(qw, qz, s, 128)).astype(bfloat16)
    assert O.rel_l2(c, ref) <= REL_L2_TOL
    # identical A rows give identical C rows; a zero A gives exactly zero (size-independent checks)
    A2 = np.tile(A[:1], (256, 1))
    c2 = to_host(ops.gemm(to_dev(A2), dev_weight(qw, qz, s)))
    assert (bits(c2) == bits(c2[:1])).all() and np.array_equal(bits(c2[0]), bits(c[0]))
    c0 = to_host(ops.gemm(to_dev(np.zeros((128, K), bfloat16)), dev_weight(qw, qz, s)))
    assert not c0.astype(np.float32).any()
    ops.gemm_check()


@pytest.mark.parametrize("B", [9, 12, 16, 17, 27, 32, 45])
def test_gemv_multi_row_pass(ops, B):
    """9-16 rows share one pass over the weights with two 8-row tiles per decoded fragment, 17-32 rows
    with four; 45 rows are 32 + 13.  All three epilogues, a partial last strip (N = 1312), against the oracle and against
    the same rows taken 8 at a time."""
    K, N = 1024, 1312
    qw, qz, s = synth_awq(K, N, 128, seed=31)
    x = randn_bf16((B, K), seed=32)
    r = randn_bf16((B, N), seed=33)
    w = dev_weight(qw, qz, s)
    ws = ops.Workspace(K, N)
    ops.set_decode_kernel("streamk")
    try:
        y = to_host(ops.gemv(to_dev(x), w, ws, residual=to_dev(r)))
        assert O.rel_l2(y, O.gemv_A_ref(x, qw, qz, s, 128, residual=r)) <= REL_L2_TOL
        y8 = np.concatenate([to_host(ops.gemv(to_dev(x[i:i + 8]), w, ws, residual=to_dev(r[i:i + 8]))) for i in range(0, B, 8)])
        assert O.rel_l2(y, y8) <= 2e-3
        yf = to_host(ops.gemv(to_dev(x), w, ws, f32_out=True))
        assert yf.dtype == np.float32 and O.rel_l2(yf, x.astype(np.float32) @ O.dequant_f32(qw, qz, s, 128)) <= 2e-3
        gate, up = synth_awq(K, 640, 128, seed=34), synth_awq(K, 640, 128, seed=35)
        wgu = ops.interleave_gate_up(dev_weight(*gate), dev_weight(*up))
        t = to_host(ops.gateup_swiglu(to_dev(x), wgu, ws))
        assert O.rel_l2(t, O.gateup_swiglu_A_ref(x, gate, up, 128)) <= REL_L2_TOL
    finally:
        ops.set_decode_kernel("auto")
    ws.check()
