"""Host layout converters (mlir_air_b200.layouts) against the reference-generated fixtures
and the oracle.  CPU only; exact."""
import numpy as np
from ml_dtypes import bfloat16

from mlir_air_b200 import layouts as L
from oracle import awq_oracle as O
from golden_util import load, bits


def test_unpack_pack_match_reference_vectors():
    g = load("awq_repacker_selftest")
    assert np.array_equal(L.unpack_awq_int32(g["qweight"]), g["nibs"])
    assert np.array_equal(L.pack_awq_int32(g["nibs"]), g["qweight"])
    assert np.array_equal(L.pack_awq_int32(g["z_nibs"]), g["qzeros"])


def test_A_to_B_and_back():
    g = load("awq_repacker_selftest")
    A_q, A_s, A_z = L.A_to_B(g["qweight"], g["qzeros"], g["scales"], 128)
    assert np.array_equal(A_q, g["A_q"]) and np.array_equal(A_z, g["A_z"]) and np.array_equal(bits(A_s), bits(g["A_s"]))
    qw, qz, sc = L.B_to_A(A_q, A_s, A_z)
    assert np.array_equal(qw, g["qweight"]) and np.array_equal(qz, g["qzeros"])


def test_gemv_tiles_match_reference_pack_inputs():
    g = load("matvec_int4_packed_64x512")
    args = (64, 512, 128, 8, 256, 4, 32)
    packed = L.pack_gemv_tiles(g["A_q"], g["A_s"], g["A_z"], *args)
    assert np.array_equal(packed, g["packed"])
    A_q, A_s, A_z = L.unpack_gemv_tiles(packed, *args)
    assert np.array_equal(A_q, g["A_q"]) and np.array_equal(A_z, g["A_z"]) and np.array_equal(bits(A_s), bits(g["A_s"]))
    g = load("awq_repacker_selftest")  # repack_for_gemv output
    assert np.array_equal(L.pack_gemv_tiles(g["A_q"], g["A_s"], g["A_z"], 128, 512, 128, 8, 512, 8, 128), g["packed"])


def test_gemm_tiles_match_reference_pack_inputs():
    for name, (K, N) in (("matmul_int4_packed_64x128x128", (128, 128)), ("matmul_int4_packed_32x256x64", (256, 64))):
        g = load(name)
        packed = L.pack_gemm_tiles(g["W_q"], g["W_s"], g["W_z"], K, N, 128, 16, 128)
        assert np.array_equal(packed, g["packed"])
        W_q, W_s, W_z = L.unpack_gemm_tiles(packed, K, N, 128, 16, 128)
        assert np.array_equal(W_q, g["W_q"]) and np.array_equal(W_z, g["W_z"]) and np.array_equal(bits(W_s), bits(g["W_s"]))


def test_dequant_tiles_match_reference_pack_inputs():
    g = load("dequant_awq_1024")
    assert tuple(g["tile_bytes"]) == L.dequant_tile_bytes(256, 128)
    packed = L.pack_dequant_tiles(g["int4_vals"], g["scales"], g["zeros"], 1024, 128, 4)
    assert np.array_equal(packed, g["packed"])
    pq, s, z = L.unpack_dequant_tiles(packed, 1024, 128, 4)
    assert np.array_equal(pq, (g["int4_vals"][0::2] | (g["int4_vals"][1::2] << 4)))
    assert np.array_equal(bits(s), bits(g["scales"])) and np.array_equal(z, g["zeros"])


def test_random_tilings_roundtrip_and_agree_with_oracle():
    rng = np.random.default_rng(0)
    for (M, K, GS, MT, KC, NC, MPL) in [(64, 512, 128, 8, 256, 4, 32), (128, 256, 64, 16, 128, 2, 64), (32, 128, 32, 4, 128, 8, 32)]:
        A_q = rng.integers(0, 256, (M, K // 2), dtype=np.uint8)
        A_s = rng.uniform(0.001, 0.02, (K // GS, M)).astype(bfloat16)
        A_z = rng.integers(0, 16, (K // GS, M), dtype=np.uint8)
        p = L.pack_gemv_tiles(A_q, A_s, A_z, M, K, GS, MT, KC, NC, MPL)
        assert np.array_equal(p, O.pack_inputs_gemv(A_q, A_s, A_z, M, K, GS, MT, KC, NC, MPL))
        q2, s2, z2 = L.unpack_gemv_tiles(p, M, K, GS, MT, KC, NC, MPL)
        assert np.array_equal(q2, A_q) and np.array_equal(z2, A_z) and np.array_equal(bits(s2), bits(A_s))


def test_interleave_rows():
    rng = np.random.default_rng(1)
    mk = lambda: (rng.integers(0, 256, (8, 64), dtype=np.uint8), rng.uniform(0, 1, (1, 8)).astype(bfloat16),
                  rng.integers(0, 16, (1, 8), dtype=np.uint8))
    g, u = mk(), mk()
    q, s, z = L.interleave_rows_gate_up(g, u)
    assert np.array_equal(q[0::2], g[0]) and np.array_equal(q[1::2], u[0])
    assert np.array_equal(bits(s[:, 1::2]), bits(u[1])) and np.array_equal(z[:, 0::2], g[2])
