"""The awq_pack.py callables (awq_dequant_layer, awq_pack_for_npu, fake_quantize_awq_int4,
pack_weight_for_int4_gemm) against outputs of mlir-air's own functions on the same seeded inputs
(tests/golden/awq_pack_256x64.npz, written by tests/golden/make_golden.py): integer and byte work, so
everything is compared bit for bit."""
import numpy as np
import pytest
from ml_dtypes import bfloat16

from golden_util import bits, load
from mlir_air_b200.programming_examples.llms.llama32_1b_int4 import awq_pack as P


@pytest.fixture(scope="module")
def g():
    return load("awq_pack_256x64")


def test_dequant_layer_bit_exact(g):
    w = P.awq_dequant_layer(g["qweight"], g["qzeros"], g["scales"], gs=128)
    assert w.dtype == bfloat16 and np.array_equal(bits(w), bits(g["dense"]))


def test_pack_for_npu_bit_exact_and_round_trips(g):
    packed = P.awq_pack_for_npu(g["qweight"], g["qzeros"], g["scales"], gs=128, n_tile=16, k_chunk=128, M_seq=64)
    assert packed.dtype == np.uint8 and packed.shape == g["packed"].shape
    assert np.array_equal(packed, g["packed"])
    # and back: per-tile buffer -> layout B -> layout A gives the checkpoint tensors again
    from mlir_air_b200 import layouts
    K, N = g["qweight"].shape[0], g["qweight"].shape[1] * 8
    qw, qz, sc = layouts.B_to_A(*layouts.unpack_gemm_tiles(packed, K, N, 128, 16, 128))
    assert np.array_equal(qw, g["qweight"]) and np.array_equal(qz, g["qzeros"]) and np.array_equal(bits(sc), bits(g["scales"]))


def test_fake_quantize_bit_exact(g):
    W_q, W_s, W_z = P.fake_quantize_awq_int4(np.ascontiguousarray(g["W"].T), gs=64)
    assert np.array_equal(W_q, g["W_q"]) and np.array_equal(W_z, g["W_z"]) and np.array_equal(bits(W_s), bits(g["W_s"]))
    # the quantiser is asymmetric min/max: every group's extremes map to 0 and 15 (unless the group is constant)
    nib = np.stack([W_q & 15, W_q >> 4], -1).reshape(W_q.shape[0], -1).reshape(W_q.shape[0], -1, 64)
    assert nib.min() == 0 and nib.max() == 15 and (nib.max(axis=2) - nib.min(axis=2) == 15).all()


def test_pack_weight_for_int4_gemm_bit_exact(g):
    packed = P.pack_weight_for_int4_gemm(g["W"], 64, gs=64, n_tile=16, k_chunk=128)
    assert np.array_equal(packed, g["W_packed"])


def test_shape_checks(g):
    with pytest.raises(AssertionError):
        P.awq_dequant_layer(g["qweight"], g["qzeros"], g["scales"], gs=96)          # K not divisible
    with pytest.raises(AssertionError):
        P.awq_dequant_layer(g["qweight"], g["qzeros"][:1], g["scales"], gs=128)     # zeros of another shape
    with pytest.raises(AssertionError):
        P.fake_quantize_awq_int4(np.zeros((8, 100), bfloat16), gs=64)


@pytest.mark.gpu
def test_gpu_forms_agree(g):
    """The device forms: awq_b200_dequant_bf16 gives awq_dequant_layer's bits, awq_b200_repack_C_to_B + _B_to_A
    take the per-tile buffer back to the checkpoint tensors, and a weight quantised by fake_quantize_awq_int4
    multiplies as its dequantised form does."""
    import torch
    from gpu_util import to_dev, to_host
    from mlir_air_b200 import ops
    from oracle import awq_oracle as O
    assert np.array_equal(bits(P.dequant_layer_gpu(g["qweight"], g["qzeros"], g["scales"], 128)), bits(g["dense"]))
    K, N = g["qweight"].shape[0], g["qweight"].shape[1] * 8
    w = P.packed_to_device(g["packed"], K, N, gs=128, n_tile=16, k_chunk=128)
    assert torch.equal(w.qweight.cpu(), torch.from_numpy(g["qweight"])) and torch.equal(w.qzeros.cpu(), torch.from_numpy(g["qzeros"]))
    assert np.array_equal(bits(to_host(w.scales)), bits(g["scales"]))
    wq = P.quantize_to_device(g["W"], gs=64)
    x = np.random.default_rng(1).standard_normal((3, g["W"].shape[0])).astype(bfloat16)
    ws = ops.Workspace(wq.K, wq.N)
    y = to_host(ops.gemv(to_dev(x), wq, ws))
    ws.check()
    deq = O.dequant_f32(*(t.cpu().numpy() if t.dtype != torch.bfloat16 else to_host(t) for t in (wq.qweight, wq.qzeros, wq.scales)), 64)
    assert O.rel_l2(y, (x.astype(np.float32) @ deq).astype(bfloat16)) <= 1e-2
    # 4-bit min/max quantisation of N(0, 0.05) weights: the quantised weight is close to the original
    assert O.rel_l2(deq, g["W"].astype(np.float32)) < 0.12
