"""Host logic of the tensor-parallel FFN, on CPU: shard bounds, shard slicing, and the
per-rank partial + allreduce composition run as two gloo ranks against the unsharded oracle."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from ml_dtypes import bfloat16

from mlir_air_b200 import ffn
from mlir_air_b200 import layouts as L
from oracle import awq_oracle as O


def test_shard_bounds_even_and_uneven():
    assert ffn.tp_shard_bounds(28672, 8) == [(i * 3584, (i + 1) * 3584) for i in range(8)]
    b = ffn.tp_shard_bounds(11008, 8)  # 86 groups: 11, 11, 11, 11, 11, 11, 10, 10
    assert [(hi - lo) // 128 for lo, hi in b] == [11] * 6 + [10] * 2
    assert b[0][0] == 0 and b[-1][1] == 11008 and all(b[i][1] == b[i + 1][0] for i in range(7))
    assert all(lo % 128 == 0 and hi % 128 == 0 for lo, hi in b)
    assert ffn.tp_shard_bounds(11008, 1) == [(0, 11008)]
    with pytest.raises(Exception):
        ffn.tp_shard_bounds(1000, 2)
    with pytest.raises(Exception):
        ffn.tp_shard_bounds(256, 3)


def _interleaved(gate, up, gs):
    K, I = O.unpack_awq_int32(gate[0]).shape
    nib = np.empty((K, 2 * I), np.uint8)
    nib[:, 0::2], nib[:, 1::2] = O.unpack_awq_int32(gate[0]), O.unpack_awq_int32(up[0])
    zn = np.empty((K // gs, 2 * I), np.uint8)
    zn[:, 0::2], zn[:, 1::2] = O.unpack_awq_int32(gate[1]), O.unpack_awq_int32(up[1])
    sc = np.empty((K // gs, 2 * I), bfloat16)
    sc[:, 0::2], sc[:, 1::2] = gate[2], up[2]
    return L.pack_awq_int32(nib), L.pack_awq_int32(zn), sc


def _weights(H, I, gs=128):
    def synth(K, N, seed):
        r = np.random.default_rng(seed)
        return (O.pack_awq_int32(r.integers(0, 16, (K, N), dtype=np.uint8)),
                O.pack_awq_int32(r.integers(0, 16, (K // gs, N), dtype=np.uint8)),
                r.uniform(0.001, 0.02, (K // gs, N)).astype(bfloat16))
    return synth(H, I, 1), synth(H, I, 2), synth(I, H, 3)


def _rank_partial(x, gu, down, bounds, gs=128):
    """What one rank computes: swiglu on its gate/up columns, then its K-slice of down, in f32."""
    i0, i1 = bounds
    gq, gz, gsx = ffn.slice_gateup(*gu, i0, i1)
    nib = O.unpack_awq_int32(np.ascontiguousarray(gq))
    zn = O.unpack_awq_int32(np.ascontiguousarray(gz))
    gate = (O.pack_awq_int32(nib[:, 0::2]), O.pack_awq_int32(zn[:, 0::2]), np.ascontiguousarray(gsx[:, 0::2]))
    up = (O.pack_awq_int32(nib[:, 1::2]), O.pack_awq_int32(zn[:, 1::2]), np.ascontiguousarray(gsx[:, 1::2]))
    t = O.gateup_swiglu_A_ref(x, gate, up, gs)
    dq, dz, ds = (np.ascontiguousarray(a) for a in ffn.slice_down(*down, i0, i1, gs))
    return t.astype(np.float32) @ O.dequant_f32(dq, dz, ds, gs)


def _worker(rank, world, port, H, I, out_dict):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        gate, up, down = _weights(H, I)
        x = np.random.default_rng(0).standard_normal((3, H)).astype(bfloat16)
        bounds = ffn.tp_shard_bounds(I, world)[rank]
        part = torch.from_numpy(_rank_partial(x, _interleaved(gate, up, 128), down, bounds))
        dist.all_reduce(part)  # the one exchange step of the layer
        y = (part.numpy() + x.astype(np.float32)).astype(bfloat16)
        ref = O.ffn_A_ref(x, gate, up, down, 128, residual=x)
        out_dict[rank] = O.rel_l2(y, ref)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("I", [512, 640])  # 4 groups (even) and 5 groups (uneven over 2 ranks)
def test_two_gloo_ranks_match_unsharded_oracle(I):
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        out = mgr.dict()
        port = 29500 + (os.getpid() + I) % 500
        procs = [ctx.Process(target=_worker, args=(r, 2, port, 256, I, out)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        assert len(out) == 2 and all(v <= 1e-2 for v in out.values()), dict(out)


def test_stack_launch_accounting():
    class _L:  # just enough of a layer for the accounting helper
        pass
    s = ffn.DecodeFFNStack.__new__(ffn.DecodeFFNStack)
    s.layers, s.tp, s.plan, s.gemm_ws = [None] * 80, 1, None, None  # no split-K workspace: batches above 8 take GEMV passes
    assert s.launches_per_step(8) == 240 and s.launches_per_step(16) == 80 * 5
    s.uses_gemm = lambda batch: False
    s.plan = object()  # with a fused plan: one launch for up to 8 rows, per-layer kernels beyond
    assert s.launches_per_step(8) == 1 and s.launches_per_step(16) == 80 * 5
    s.plan = None
    s.tp = 8
    assert s.launches_per_step(8) == 1 + 80 * 3


def test_which_batched_decode_gemm_a_stack_takes():
    """Up to 32 rows the kernel with fp8 operands, but only where a layer (on this rank) is large enough for its three
    launches per product to pay: the full 70B layer and its halves, not an eighth of it, a 7B layer up to 16 rows only."""
    class _W:
        def __init__(self, K, N):
            self.K, self.N, self.group_size = K, N, 128

    class _L:
        def __init__(self, H, I):
            self.gateup, self.down, self.gamma = _W(H, 2 * I), _W(I, H), object()

    class _Ws:
        def fits_f8(self, M, K, N):
            return M <= 32

    def stack(H, I):
        s = ffn.DecodeFFNStack.__new__(ffn.DecodeFFNStack)
        s.layers, s.tp, s.plan, s.gemm_ws = [_L(H, I)] * 2, 1, None, _Ws()
        return s
    full, half, eighth, small = stack(8192, 28672), stack(8192, 14336), stack(8192, 3584), stack(4096, 11008)
    assert full.uses_gemm_f8(9) and full.uses_gemm_f8(32) and not full.uses_gemm_f8(33) and not full.uses_gemm_f8(8)
    assert half.uses_gemm_f8(16) and half.uses_gemm_f8(32)
    assert not eighth.uses_gemm_f8(16) and not eighth.uses_gemm_f8(32) and eighth.uses_gemm(32)
    assert small.uses_gemm_f8(16) and not small.uses_gemm_f8(32)
    assert stack(8192, 7168).uses_gemm_f8(16) and not stack(8192, 7168).uses_gemm_f8(17)
    assert full.launches_per_step(32) == 2 * 7 and eighth.launches_per_step(32) == 2 * 5 and full.launches_per_step(64) == 2 * 5
