"""AWQ packers and the min/max int4 quantiser: the callables of mlir-air's
programming_examples/llms/llama32_1b_int4/awq_pack.py, same names, arguments and results.

    awq_dequant_layer(qweight_i32, qzeros_i32, scales_bf16, gs=128)          awq_pack.py:84-104
    awq_pack_for_npu(..., gs=128, n_tile=16, k_chunk=128, M_seq=2048)        awq_pack.py:112-146
    fake_quantize_awq_int4(W_bf16, gs=128)                                   awq_pack.py:287-316
    pack_weight_for_int4_gemm(W_bf16, M_seq, gs=128, n_tile=16, k_chunk=128) awq_pack.py:319-332

All four are integer / byte work done once per weight on the host.  The per-tile packed buffers
(`awq_pack_for_npu`, `pack_weight_for_int4_gemm`) are the format the reference's NPU kernel wants;
this library's kernels take the AutoAWQ tensors as they are, so `awq_to_device` is what a caller
here uses instead, and `packed_to_device` takes a per-tile buffer back to a resident weight
(unpacked on the GPU by awq_b200_repack_C_to_B / awq_b200_repack_B_to_A).  `dequant_layer_gpu`
is the device form of `awq_dequant_layer` (bit-identical).
"""
from __future__ import annotations

import numpy as np
from ml_dtypes import bfloat16

from mlir_air_b200 import layouts


def _awq_unpack_int32_to_nibbles(packed_i32, n_outer):
    """(n_outer, n_packed) int32 -> (n_outer, 8 n_packed) uint8 in natural column order
    (awq_pack.py:66-76)."""
    return layouts.unpack_awq_int32(np.asarray(packed_i32)).reshape(n_outer, -1)


def _check_awq(qweight_i32, qzeros_i32, scales_bf16, gs):
    K, n_packed = qweight_i32.shape
    N, n_groups = n_packed * 8, K // gs
    assert K % gs == 0, f"K={K} not divisible by gs={gs}"
    assert qzeros_i32.shape == (n_groups, n_packed)
    assert scales_bf16.shape == (n_groups, N)
    return K, N, n_groups


def awq_dequant_layer(qweight_i32, qzeros_i32, scales_bf16, gs=128):
    """AWQ qweight / qzeros / scales -> dense (K, N) bf16 weight, W[k, n] = (q - z) * s in f32 with
    one rounding (awq_pack.py:84-104).  Group by group, so no K x N temporaries of the repeated
    zeros and scales are built; the arithmetic per element is the reference's."""
    K, N, n_groups = _check_awq(qweight_i32, qzeros_i32, scales_bf16, gs)
    q = _awq_unpack_int32_to_nibbles(qweight_i32, K).reshape(n_groups, gs, N)
    z = _awq_unpack_int32_to_nibbles(qzeros_i32, n_groups).astype(np.float32)
    s = np.asarray(scales_bf16).astype(np.float32)
    w = (q.astype(np.float32) - z[:, None, :]) * s[:, None, :]
    return w.reshape(K, N).astype(bfloat16)


def awq_pack_for_npu(qweight_i32, qzeros_i32, scales_bf16, gs=128, n_tile=16, k_chunk=128, M_seq=2048):
    """AWQ tensors -> per-tile packed buffer (N / n_tile, K / k_chunk, tile_bytes) uint8: nibble values
    kept, re-shuffled to output-major rows with two k per byte (awq_pack.py:112-146, through
    matmul_int4_packed.pack_inputs :57-86).  M_seq does not enter the layout."""
    K, N, _ = _check_awq(qweight_i32, qzeros_i32, scales_bf16, gs)
    A_q, A_s, A_z = layouts.A_to_B(np.asarray(qweight_i32), np.asarray(qzeros_i32), np.asarray(scales_bf16), gs)
    return layouts.pack_gemm_tiles(A_q, A_s, A_z, K, N, gs, n_tile, k_chunk)


def fake_quantize_awq_int4(W_bf16, gs=128):
    """Asymmetric uint4 quantisation per group of `gs` along K of a [M, K] bf16 weight
    (awq_pack.py:287-316): scale = (max - min) / 15 (1e-7 where a group is constant),
    zero = round(-min / scale) clipped to 0..15, q = round(w / scale + zero) clipped.
    Returns (W_q uint8 [M, K/2], low nibble = even k; W_s bf16 [K/gs, M]; W_z uint8 [K/gs, M])."""
    M, K = W_bf16.shape
    assert K % gs == 0, f"K={K} not divisible by gs={gs}"
    n_groups = K // gs
    w = np.asarray(W_bf16).astype(np.float32).reshape(M, n_groups, gs)
    w_min, w_max = w.min(axis=2), w.max(axis=2)
    scale = (w_max - w_min) / 15.0
    scale = np.where(scale == 0, 1e-7, scale)
    zero = np.round(-w_min / scale).clip(0, 15).astype(np.uint8)
    q = np.round(w / scale[:, :, None] + zero.astype(np.float32)[:, :, None]).clip(0, 15).astype(np.uint8).reshape(M, K)
    W_q = (q[:, 0::2] | (q[:, 1::2] << 4)).astype(np.uint8)
    return W_q, scale.T.astype(bfloat16), np.ascontiguousarray(zero.T)


def pack_weight_for_int4_gemm(W_bf16, M_seq, gs=128, n_tile=16, k_chunk=128):
    """Quantise a prefill-orientation [K, N] bf16 weight and pack it per tile
    (awq_pack.py:319-332): [N / n_tile, K / k_chunk, tile_bytes] uint8."""
    W_NK = np.ascontiguousarray(np.asarray(W_bf16).T)
    N, K = W_NK.shape
    W_q, W_s, W_z = fake_quantize_awq_int4(W_NK, gs=gs)
    return layouts.pack_gemm_tiles(W_q, W_s, W_z, K, N, gs, n_tile, k_chunk)


# ---------------------------------------------------------------------------------------------
# What a caller of this library does with the same tensors
# ---------------------------------------------------------------------------------------------
def awq_to_device(qweight_i32, qzeros_i32, scales_bf16, gs=128, device="cuda"):
    """The AutoAWQ tensors as a resident weight: no repacking, the kernels read this layout."""
    from mlir_air_b200.ops import AwqWeight
    _check_awq(qweight_i32, qzeros_i32, scales_bf16, gs)
    return AwqWeight.from_numpy(qweight_i32, qzeros_i32, scales_bf16, gs, device=device)


def quantize_to_device(W_bf16_KN, gs=128, device="cuda"):
    """[K, N] bf16 weight -> min/max int4 quantisation (fake_quantize_awq_int4) -> resident weight."""
    from mlir_air_b200 import ops
    import torch
    W_q, W_s, W_z = fake_quantize_awq_int4(np.ascontiguousarray(np.asarray(W_bf16_KN).T), gs=gs)
    return ops.repack_B_to_A(torch.from_numpy(W_q).to(device),
                             torch.from_numpy(np.ascontiguousarray(W_s).view(np.int16)).to(device).view(torch.bfloat16),
                             torch.from_numpy(W_z).to(device), gs)


def packed_to_device(packed, K, N, gs=128, n_tile=16, k_chunk=128, device="cuda"):
    """A per-tile packed GEMM buffer (what awq_pack_for_npu returns) -> resident weight, unpacked on
    the GPU."""
    from mlir_air_b200 import ops
    import torch
    return ops.repack_C_to_A(torch.from_numpy(np.ascontiguousarray(packed, dtype=np.uint8)).to(device), N, K, gs,
                             n_tile, k_chunk)


def dequant_layer_gpu(qweight_i32, qzeros_i32, scales_bf16, gs=128):
    """awq_dequant_layer on the GPU (awq_b200_dequant_bf16): same bits."""
    from mlir_air_b200 import ops
    w = ops.dequant(awq_to_device(qweight_i32, qzeros_i32, scales_bf16, gs))
    return w.view(__import__("torch").int16).cpu().numpy().view(bfloat16)
