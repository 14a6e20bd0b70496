"""Pin the numpy oracle against vectors produced by mlir-air's own golden functions
(tests/golden/make_golden.py).  CPU only."""
import numpy as np
import pytest
from ml_dtypes import bfloat16

from oracle import awq_oracle as O
from golden_util import load, bits


def test_selftest_unpack_exact():
    g = load("awq_repacker_selftest")
    assert np.array_equal(O.unpack_awq_int32(g["qweight"]), g["nibs"])
    assert np.array_equal(O.unpack_awq_int32(g["qzeros"]), g["z_nibs"])
    assert np.array_equal(O.pack_awq_int32(g["nibs"]), g["qweight"])
    assert np.array_equal(O.pack_awq_int32(g["z_nibs"]), g["qzeros"])


def test_selftest_generator_matches_reference_rng():
    g = load("awq_repacker_selftest")
    qw, qz, sc, nibs, zn = O.gen_synthetic_awq(512, 128, 128, seed=42)
    assert np.array_equal(qw, g["qweight"]) and np.array_equal(qz, g["qzeros"])
    assert np.array_equal(sc, g["scales"]) and np.array_equal(nibs, g["nibs"])


@pytest.mark.parametrize("name,gs", [("awq_repacker_selftest", 128), ("awq_repacker_gs64", 64)])
def test_dequant_bit_exact(name, gs):
    g = load(name)
    w = O.dequant_to_bf16(g["qweight"], g["qzeros"], g["scales"], gs)
    assert np.array_equal(bits(w), bits(g["w_dense"]))
    # the f32 (unrounded) weight rounds to the same bf16
    wf = O.dequant_f32(g["qweight"], g["qzeros"], g["scales"], gs)
    assert np.array_equal(bits(wf.astype(bfloat16)), bits(g["w_dense"]))


def test_repack_A_to_B_and_back():
    g = load("awq_repacker_selftest")
    A_q, A_s, A_z = O.repack_hf_awq_linear(g["qweight"], g["qzeros"], g["scales"], 128)
    assert np.array_equal(A_q, g["A_q"]) and np.array_equal(A_z, g["A_z"])
    assert np.array_equal(bits(A_s), bits(g["A_s"]))
    qw, qz, sc = O.layout_B_to_A(A_q, A_s, A_z)
    assert np.array_equal(qw, g["qweight"]) and np.array_equal(qz, g["qzeros"])
    assert np.array_equal(bits(sc), bits(g["scales"].astype(bfloat16)))


def test_repack_for_gemv_tiles():
    g = load("awq_repacker_selftest")
    packed = O.pack_inputs_gemv(g["A_q"], g["A_s"], g["A_z"], 128, 512, 128, 8, 512, 8, 128)
    assert np.array_equal(packed, g["packed"])
    A_q, A_s, A_z = O.unpack_inputs_gemv(packed, 128, 512, 128, 8, 512, 8, 128)
    assert np.array_equal(A_q, g["A_q"]) and np.array_equal(A_z, g["A_z"])
    assert np.array_equal(bits(A_s), bits(g["A_s"]))


def test_selftest_gemv_scalar_loop_golden():
    g = load("awq_repacker_selftest")
    y = O.gemv_ref(g["A_q"], g["A_s"], g["A_z"], g["x"])
    # vectorised f32 matmul vs the reference's scalar f32 loop: summation order only
    assert O.rel_l2(y, g["y"]) < 4e-3
    ya = O.gemv_A_ref(g["x"], g["qweight"], g["qzeros"], g["scales"], 128)[0]
    assert np.array_equal(bits(ya), bits(y))


def test_matvec_int4_packed_small():
    g = load("matvec_int4_packed_64x512")
    assert O.rel_l2(O.gemv_ref(g["A_q"], g["A_s"], g["A_z"], g["B"]), g["D"]) < 4e-3
    packed = O.pack_inputs_gemv(g["A_q"], g["A_s"], g["A_z"], 64, 512, 128, 8, 256, 4, 32)
    assert np.array_equal(packed, g["packed"])
    A_q, A_s, A_z = O.unpack_inputs_gemv(packed, 64, 512, 128, 8, 256, 4, 32)
    assert np.array_equal(A_q, g["A_q"]) and np.array_equal(A_z, g["A_z"])
    assert np.array_equal(bits(A_s), bits(g["A_s"]))


def test_matvec_int4_packed_reference_shape_2048():
    """The reference's own lit shape (M=K=2048, seed 42): inputs regenerated from the
    seed exactly as matvec_int4_packed.py:345-351 does, output of the scalar loop stored."""
    g = load("matvec_int4_packed_2048x2048_D")
    np.random.seed(42)
    unp = np.random.randint(0, 16, size=(2048, 2048), dtype=np.uint8)
    A_q = (unp[:, 0::2] | (unp[:, 1::2] << 4)).astype(np.uint8)
    A_s = np.random.uniform(0.005, 0.02, size=(16, 2048)).astype(bfloat16)
    A_z = np.random.randint(7, 9, size=(16, 2048), dtype=np.uint8)
    B = np.random.randn(2048).astype(bfloat16)
    assert O.rel_l2(O.gemv_ref(A_q, A_s, A_z, B), g["D"]) < 4e-3


def test_matvec_int4_packed_add_small():
    g = load("matvec_int4_packed_add_64x512")
    d = O.gemv_add_ref(g["A_q"], g["A_s"], g["A_z"], g["B"], g["R"])
    assert O.rel_l2(d, g["D"]) < 4e-3


def test_swiglu_rms_small_bit_exact():
    g = load("matvec_int4_swiglu_rms_256x512")
    d = O.swiglu_rms_ref(g["A_q"], g["A_s"], g["A_z"], g["RMS_in"])
    assert np.array_equal(bits(d), bits(g["D"]))  # same vectorised formula -> same bits


@pytest.mark.parametrize("name,dims", [("matmul_int4_packed_64x128x128", (64, 128, 128)),
                                       ("matmul_int4_packed_32x256x64", (32, 256, 64))])
def test_matmul_int4_packed(name, dims):
    M, K, N = dims
    g = load(name)
    assert np.array_equal(bits(O.gemm_ref(g["W_q"], g["W_s"], g["W_z"], g["A"])), bits(g["C"]))
    packed = O.pack_inputs_gemm(g["W_q"], g["W_s"], g["W_z"], M, K, N, 128, 16, 128)
    assert np.array_equal(packed, g["packed"])
    W_q, W_s, W_z = O.unpack_inputs_gemm(packed, K, N, 128, 16, 128)
    assert np.array_equal(W_q, g["W_q"]) and np.array_equal(W_z, g["W_z"])
    assert np.array_equal(bits(W_s), bits(g["W_s"]))


def test_dequant_awq_example():
    g = load("dequant_awq_1024")
    assert tuple(g["tile_bytes"]) == O.dequant_tile_bytes(256, 128)
    assert np.array_equal(O.pack_inputs_dequant(g["int4_vals"], g["scales"], g["zeros"], 1024, 128, 4),
                          g["packed"])
    assert np.array_equal(bits(O.dequant_1d(g["int4_vals"], g["scales"], g["zeros"], 128)), bits(g["ref"]))


def test_ffn_bf16_goldens():
    g = load("ffn_decode_128")
    assert np.array_equal(bits(O.ffn_bf16_ref(g["x"], g["W_gate"], g["W_up"], g["W_down"])), bits(g["out"]))
    pk = np.concatenate([O.pack_ffn_weights_decode(g[k], 128, 32, 4) for k in ("W_gate", "W_up", "W_down")])
    assert np.array_equal(bits(pk.astype(bfloat16)), bits(g["packed_weights"]))
    g = load("ffn_prefill_16x128")
    assert np.array_equal(bits(O.ffn_bf16_ref(g["x"], g["W_gate"], g["W_up"], g["W_down"])), bits(g["out"]))
    pk = np.concatenate([O.pack_ffn_weights_prefill(g[k], 128, 32, 4) for k in ("W_gate", "W_up", "W_down")])
    assert np.array_equal(bits(pk.astype(bfloat16)), bits(g["packed_weights"]))


def test_layout_A_goldens_agree_with_layout_B_goldens():
    g = load("matvec_int4_swiglu_rms_256x512")
    A_q, A_s, A_z = g["A_q"], g["A_s"], g["A_z"]
    # rows are gate/up interleaved: split into two layout-A matrices
    gate = O.layout_B_to_A(A_q[0::2], A_s[:, 0::2], A_z[:, 0::2])
    up = O.layout_B_to_A(A_q[1::2], A_s[:, 1::2], A_z[:, 1::2])
    d = O.gateup_swiglu_A_ref(g["RMS_in"][0], gate, up, 128, gamma=g["RMS_in"][1])[0]
    assert O.rel_l2(d, g["D"]) < 4e-3
