"""RMSNorm -> int4 Q/K/V GEMVs -> half-split RoPE (rms_qkv_int4_rope_multi.py): the oracle against the
fixture made from the reference's own functions (CPU), and the CUDA path against both (GPU)."""
import numpy as np
import pytest
from ml_dtypes import bfloat16

from golden_util import bits, load
from oracle import awq_oracle as O

HD, NH, NKV = 64, 4, 1


@pytest.fixture(scope="module")
def g():
    return load("rms_qkv_int4_rope_256")


def _lut_rows(g, n):
    return np.tile(g["lut"][int(g["pos"])], (n, 1))


def test_oracle_matches_reference_fixture(g):
    # LUT and RMSNorm of this block and RoPE: bit-exact restatements
    assert np.array_equal(bits(O.rope_lut_ref(HD, float(g["rope_base"]), 4)), bits(g["lut"]))
    assert np.array_equal(bits(O.rms_norm_1d_ref(g["x_in"], g["norm_w"])), bits(g["normed"]))
    assert np.array_equal(bits(O.rope_halfsplit_ref(g["q"], _lut_rows(g, NH), HD)), bits(g["q_roped"]))
    assert np.array_equal(bits(O.rope_halfsplit_ref(g["k"], _lut_rows(g, NKV), HD)), bits(g["k_roped"]))
    # the GEMVs: vectorised golden against the reference's scalar-loop cpu_reference
    for n in ("q", "k", "v"):
        w = O.layout_B_to_A(g[f"w{n}_q"], g[f"w{n}_s"], g[f"w{n}_z"])
        assert O.rel_l2(O.gemv_A_ref(g["normed"], *w, 128)[0], g[n]) <= 1e-3
    # the whole block in one call
    ws = [O.layout_B_to_A(g[f"w{n}_q"], g[f"w{n}_s"], g[f"w{n}_z"]) for n in ("q", "k", "v")]
    q_r, k_r, v = O.rms_qkv_rope_A_ref(g["x_in"][None], g["norm_w"], *ws, g["lut"][int(g["pos"])][None], NH, NKV, HD, 128)
    assert O.rel_l2(q_r[0], g["q_roped"]) <= 1e-3 and O.rel_l2(k_r[0], g["k_roped"]) <= 1e-3 and O.rel_l2(v[0], g["v"]) <= 1e-3


def test_rope_is_a_rotation():
    """Size-independent property: position 0 is the identity, and a rotation keeps each pair's norm."""
    rng = np.random.default_rng(0)
    x = rng.standard_normal((6, 128)).astype(bfloat16)
    lut = O.rope_lut_ref(128, 500000.0, 9, dtype=np.float32)
    assert np.array_equal(bits(O.rope_halfsplit_ref(x, np.tile(lut[0], (6, 1)), 128)), bits(x))
    y = O.rope_halfsplit_ref(x.astype(np.float32), np.tile(lut[8], (6, 1)), 128).astype(np.float32)
    xf = x.astype(np.float32)
    n_in = xf[:, :64] ** 2 + xf[:, 64:] ** 2
    n_out = y[:, :64] ** 2 + y[:, 64:] ** 2
    assert np.allclose(n_in, n_out, rtol=2e-2, atol=1e-3)


@pytest.mark.gpu
def test_rope_kernel_bit_exact_and_block_parity(g):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from gpu_util import dev_weight, to_dev, to_host
    from mlir_air_b200 import ops
    # RoPE alone, on the reference's own q / k: same bits
    lut_row = to_dev(g["lut"][int(g["pos"])][None])
    q_r = to_host(ops.rope_halfsplit(to_dev(g["q"][None]), lut_row, NH, HD, out=torch.empty((1, 256), dtype=torch.bfloat16, device="cuda")))
    assert np.array_equal(bits(q_r[0]), bits(g["q_roped"]))
    k = to_dev(g["k"][None])
    ops.rope_halfsplit(k, lut_row, NKV, HD)  # in place
    assert np.array_equal(bits(to_host(k)[0]), bits(g["k_roped"]))
    # a batch with one position per token, rotating a strided view of a wider buffer
    rng = np.random.default_rng(1)
    B, heads, hd = 5, 3, 128
    xw = rng.standard_normal((B, heads * hd + 64)).astype(bfloat16)
    lut = O.rope_lut_ref(hd, 10000.0, 32)[[0, 3, 7, 31, 12]]
    buf = to_dev(xw)
    out = to_host(ops.rope_halfsplit(buf[:, :heads * hd], to_dev(lut), heads, hd, out=torch.empty((B, heads * hd), dtype=torch.bfloat16, device="cuda")))
    ref = O.rope_halfsplit_ref(xw[:, :heads * hd], np.repeat(lut, heads, axis=0), hd)
    assert np.array_equal(bits(out), bits(ref))
    # the block: rmsnorm -> one GEMV over Wq | Wk | Wv -> RoPE
    ws = [dev_weight(*O.layout_B_to_A(g[f"w{n}_q"], g[f"w{n}_s"], g[f"w{n}_z"])) for n in ("q", "k", "v")]
    w = ops.AwqWeight(torch.cat([t.qweight for t in ws], 1).contiguous(), torch.cat([t.qzeros for t in ws], 1).contiguous(),
                      torch.cat([t.scales for t in ws], 1).contiguous(), 128)
    wsp = ops.Workspace(w.K, w.N)
    normed = ops.rmsnorm(to_dev(g["x_in"][None]), to_dev(g["norm_w"]), 1e-5)
    qkv = ops.gemv(normed, w, wsp)
    wsp.check()
    assert O.rel_l2(to_host(normed)[0], g["normed"]) <= 1e-2
    ops.rope_halfsplit(qkv[:, :256], lut_row, NH, HD)
    ops.rope_halfsplit(qkv[:, 256:320], lut_row, NKV, HD)
    y = to_host(qkv)[0]
    assert O.rel_l2(y[:256], g["q_roped"]) <= 1e-2
    assert O.rel_l2(y[256:320], g["k_roped"]) <= 1e-2
    assert O.rel_l2(y[320:], g["v"]) <= 1e-2
