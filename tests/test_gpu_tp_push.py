"""Tensor-parallel decode stack on 2 (and, where the box has them, 4) GPUs: the peer-memory hand-over
(awq_b200_gemv_f32_push + awq_b200_tp_reduce_add_rmsnorm_act) and the one-launch tensor-parallel stack
(awq_b200_ffn_stack_decode_tp_bf16) against the NCCL allreduce path and the unsharded numpy oracle.
Skipped on boxes with fewer GPUs than ranks."""
import os

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp
from ml_dtypes import bfloat16

from oracle import awq_oracle as O

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, H, I, L, B, out):
    import torch.distributed as dist
    from gpu_util import synth_awq, to_dev, to_host
    from mlir_air_b200 import ffn, ops
    from mlir_air_b200.ops import AwqWeight
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        group = dist.group.WORLD
        i0, i1 = ffn.tp_shard_bounds(I, world)[rank]
        layers, full = [], []
        for l in range(L):
            gate = synth_awq(H, I, 128, seed=10 * l)
            up = synth_awq(H, I, 128, seed=10 * l + 1)
            down = synth_awq(I, H, 128, seed=10 * l + 2, scale_lo=0.0005, scale_hi=0.004)
            gamma = (np.random.default_rng(10 * l + 3).standard_normal(H) * 0.1 + 1.0).astype(bfloat16)
            full.append((gate, up, down, gamma))
            gu = ops.interleave_gate_up(AwqWeight.from_numpy(*gate, 128), AwqWeight.from_numpy(*up, 128))
            layers.append(ffn.FFNLayer(ffn.shard_gateup(gu, i0, i1), ffn.shard_down(AwqWeight.from_numpy(*down, 128), i0, i1),
                                       to_dev(gamma)))
        x = np.random.default_rng(7).standard_normal((B, H)).astype(bfloat16)
        push = ffn.DecodeFFNStack(layers, H, max_batch=8, group=group, peer_push=True, fused=False)
        nccl = ffn.DecodeFFNStack(layers, H, max_batch=8, group=group, fused=False)
        one = ffn.DecodeFFNStack(layers, H, max_batch=8, group=group)  # the whole stack in one launch per rank
        assert push.peers is not None and nccl.peers is None and one.uses_fused(B) and one.plan_peers is not None
        y_push = to_host(push.step(to_dev(x)))
        y_push2 = to_host(push.step(to_dev(x)))  # the slots and flags are reusable
        push.check()
        y_nccl = to_host(nccl.step(to_dev(x)))
        nccl.check()
        # replayed as a CUDA graph, twice
        push.load_input(to_dev(x))
        g1 = to_host(push.replay(B).clone())
        push.load_input(to_dev(x))
        g2 = to_host(push.replay(B).clone())
        push.check()
        y_one = to_host(one.step(to_dev(x)))
        y_one2 = to_host(one.step(to_dev(x)))  # the flag counters run on from launch to launch
        one.load_input(to_dev(x))
        y_one3 = to_host(one.replay(B).clone())
        one.load_input(to_dev(x))
        y_one4 = to_host(one.replay(B).clone())
        one.check()
        one.resync()  # what all ranks do after a failed launch on any of them: slots, flags and launch count back to zero
        y_one5 = to_host(one.step(to_dev(x)))
        one.check()
        h = x
        for gate, up, down, gamma in full:
            h = O.ffn_layer_A_ref(h, gamma, gate, up, down, 128)
        out[rank] = dict(how=push.peers.how, oracle=O.rel_l2(y_push, h), again=O.rel_l2(y_push2, h),
                         vs_nccl=O.rel_l2(y_push, y_nccl), graph1=O.rel_l2(g1, h), graph2=O.rel_l2(g2, h),
                         nccl_oracle=O.rel_l2(y_nccl, h), one=O.rel_l2(y_one, h), one2=O.rel_l2(y_one2, h),
                         one3=O.rel_l2(y_one3, h), one4=O.rel_l2(y_one4, h), one5=O.rel_l2(y_one5, h),
                         one_vs_nccl=O.rel_l2(y_one, y_nccl))
        torch.cuda.synchronize()
        dist.barrier()
    except Exception:  # noqa: BLE001 -- show it before the hard exit below
        import traceback
        traceback.print_exc()
    finally:
        # captured graphs hold the communicator's collectives: leave without tearing it down
        os._exit(0 if rank in out else 1)


@pytest.mark.parametrize("world,B,H,I,L", [(2, 8, 1024, 2816, 3), (2, 1, 2048, 5632, 2), (4, 8, 1024, 2816, 3)])
def test_tp_push_matches_nccl_and_oracle(world, B, H, I, L):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        out = mgr.dict()
        port = 29600 + (os.getpid() + H) % 300
        procs = [ctx.Process(target=_worker, args=(r, world, port, H, I, L, B, out)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(300)
        for p in procs:
            if p.is_alive():
                p.kill()
        assert all(p.exitcode == 0 for p in procs), dict(out)
        res = dict(out)
    assert len(res) == world, res
    for r, d in res.items():
        assert d["oracle"] <= 1e-2 and d["again"] <= 1e-2 and d["graph1"] <= 1e-2 and d["graph2"] <= 1e-2, res
        assert d["vs_nccl"] <= 5e-3, res
        assert max(d["one"], d["one2"], d["one3"], d["one4"], d["one5"]) <= 1e-2 and d["one_vs_nccl"] <= 5e-3, res


def _worker_gemm(rank, world, port, H, I, L, B, out):
    import torch.distributed as dist
    from gpu_util import synth_awq, to_dev, to_host
    from mlir_air_b200 import ffn, ops
    from mlir_air_b200.ops import AwqWeight
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        group = dist.group.WORLD
        i0, i1 = ffn.tp_shard_bounds(I, world)[rank]
        layers, full = [], []
        for l in range(L):
            gate = synth_awq(H, I, 128, seed=10 * l)
            up = synth_awq(H, I, 128, seed=10 * l + 1)
            down = synth_awq(I, H, 128, seed=10 * l + 2, scale_lo=0.0005, scale_hi=0.004)
            gamma = (np.random.default_rng(10 * l + 3).standard_normal(H) * 0.1 + 1.0).astype(bfloat16)
            full.append((gate, up, down, gamma))
            gu = ops.interleave_gate_up(AwqWeight.from_numpy(*gate, 128), AwqWeight.from_numpy(*up, 128))
            layers.append(ffn.FFNLayer(ffn.shard_gateup(gu, i0, i1), ffn.shard_down(AwqWeight.from_numpy(*down, 128), i0, i1),
                                       to_dev(gamma)))
        x = np.random.default_rng(7).standard_normal((B, H)).astype(bfloat16)
        st = ffn.DecodeFFNStack(layers, H, max_batch=64, group=group)
        # with the size bar out of the way: up to 32 rows the fp8-operand GEMM (a third launch per product splits the token
        # rows), the 16-bit one beyond
        st.GEMM_F8_MIN_WEIGHTS = {16: 0, 32: 0}
        assert st.uses_gemm(B) and st.uses_gemm_f8(B) == (B <= 32)
        assert st.launches_per_step(B) == (7 if B <= 32 else 5) * L + 1
        y = to_host(st.step(to_dev(x)))
        y2 = to_host(st.step(to_dev(x)))
        st.load_input(to_dev(x))
        g1 = to_host(st.replay(B).clone())
        st.check()
        old = ffn.DecodeFFNStack(layers, H, max_batch=64, group=group)
        old.gemm_ws = None  # the per-layer GEMV passes with the allreduce in between
        assert not old.uses_gemm(B)
        y_old = to_host(old.step(to_dev(x)))
        old.check()
        h = x
        for gate, up, down, gamma in full:
            h = O.ffn_layer_A_ref(h, gamma, gate, up, down, 128)
        out[rank] = dict(oracle=O.rel_l2(y, h), again=bool(np.array_equal(y.view(np.uint16), y2.view(np.uint16))),
                         graph=O.rel_l2(g1, h), vs_gemv=O.rel_l2(y, y_old))
        torch.cuda.synchronize()
        dist.barrier()
    except Exception:  # noqa: BLE001 -- show it before the hard exit below
        import traceback
        traceback.print_exc()
    finally:
        os._exit(0 if rank in out else 1)


# (the third case: 11 groups of the intermediate dimension on 2 ranks, shards of 6 and 5 groups; the fourth: 4 ranks)
@pytest.mark.parametrize("world,B,H,I,L", [(2, 32, 1024, 2816, 3), (2, 17, 2048, 5632, 2), (2, 64, 1024, 1408, 2), (4, 40, 1024, 2816, 2)])
def test_tp_batched_decode_gemm_matches_oracle(world, B, H, I, L):
    """Batches of 9 to 64 rows on tensor-parallel ranks: gate/up shard and down shard through the batched-decode GEMM, the
    down partial as f32 (awq_b200_gemm_decode_f32), one allreduce per layer, residual add fused with the next norm."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        out = mgr.dict()
        port = 29600 + (os.getpid() + H + B) % 300
        procs = [ctx.Process(target=_worker_gemm, args=(r, world, port, H, I, L, B, out)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(300)
        for p in procs:
            if p.is_alive():
                p.kill()
        assert all(p.exitcode == 0 for p in procs), dict(out)
        res = dict(out)
    assert len(res) == world, res
    for r, d in res.items():
        assert d["oracle"] <= 1e-2 and d["graph"] <= 1e-2 and d["vs_gemv"] <= 1e-2 and d["again"], res
