"""Device-side waits that run out, on one GPU and without faulting anything: a kernel that waits for data nobody
sends gives up after the run-time limit (awq_b200_set_wait_limit), leaves an error word in its workspace, drains
and returns; the next *_check call reports AWQ_ERR_DEVICE_TIMEOUT; after awq_b200_workspace_init the same
workspace serves a normal call.  The counterpart of the reference raising when a run does not reach
ERT_CMD_STATE_COMPLETED (python/air/backend/xrt.py:204-218)."""
import ctypes

import numpy as np
import pytest
from ml_dtypes import bfloat16

from oracle import awq_oracle as O

pytestmark = pytest.mark.gpu

WAIT_CYCLES = 2_000_000  # about a millisecond


@pytest.fixture()
def short_waits():
    from mlir_air_b200 import _lib
    lib = _lib.load()
    assert lib.awq_b200_set_wait_limit(WAIT_CYCLES) == 0
    yield lib
    assert lib.awq_b200_set_wait_limit(0) == 0  # back to the default


def _small_stack(ops, H, I, L, seed):
    from gpu_util import dev_weight, synth_awq, to_dev
    layers_np, gus, downs, gammas = [], [], [], []
    for l in range(L):
        gate, up = synth_awq(H, I, 128, seed=seed + 10 * l), synth_awq(H, I, 128, seed=seed + 10 * l + 1)
        down = synth_awq(I, H, 128, seed=seed + 10 * l + 2, scale_lo=0.0005, scale_hi=0.004)
        gamma = (np.random.default_rng(seed + 10 * l + 3).standard_normal(H) * 0.1 + 1.0).astype(bfloat16)
        layers_np.append((gate, up, down, gamma))
        gus.append(ops.interleave_gate_up(dev_weight(*gate), dev_weight(*up)))
        downs.append(dev_weight(*down))
        gammas.append(to_dev(gamma))
    return layers_np, ops.FFNStackPlan(gus, downs, gammas)


def test_stack_kernel_gives_up_when_a_rank_never_sends(short_waits):
    """The tensor-parallel stack launch as rank 0 of 2, where the "other rank" is a zeroed local buffer that
    nothing ever writes: the warps that collect the ranks' partial sums poll it, run into the limit and leave."""
    import torch
    from gpu_util import randn_bf16, to_dev, to_host
    from mlir_air_b200 import _lib, ops
    lib = short_waits
    H, I, L, B = 512, 1024, 2, 4
    layers_np, plan = _small_stack(ops, H, I, L, seed=300)
    ws = ops.Workspace(max(H, I), max(2 * I, H))
    slot = int(lib.awq_b200_ffn_stack_tp_slot_bytes(H, 2))
    stride = slot + 256
    mine = torch.zeros(2 * stride, dtype=torch.uint8, device="cuda")
    silent = torch.zeros(2 * stride, dtype=torch.uint8, device="cuda")  # the rank that never joins
    bases = (ctypes.c_void_p * 2)(mine.data_ptr(), silent.data_ptr())
    x = to_dev(randn_bf16((B, H), seed=1))
    out = torch.empty_like(x)
    inter = torch.empty((B, I), dtype=torch.float16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    rc = lib.awq_b200_ffn_stack_decode_tp_bf16(plan.ptr, L, x.data_ptr(), out.data_ptr(), inter.data_ptr(), 1e-5, B, H, I, 128,
                                               bases, stride, slot, 2, 0, ws.buf.data_ptr(), ws.nbytes, stream)
    assert rc == 0, _lib.last_error()  # the launch itself is fine; the failure is on the device
    t1.record()
    rc = lib.awq_b200_workspace_check(ws.buf.data_ptr(), stream)
    assert rc == _lib.AWQ_ERR_DEVICE_TIMEOUT, (rc, _lib.last_error())
    assert "wait gave up" in _lib.last_error()
    assert t0.elapsed_time(t1) < 500.0, "the kernel must drain within a few waits, not hang"
    # the context is alive and the workspace is usable again after re-initialisation
    _lib.check(lib.awq_b200_workspace_init(ws.buf.data_ptr(), ws.nbytes, stream), "workspace_init")
    xh = randn_bf16((B, H), seed=2)
    y = to_host(ops.ffn_stack_decode(plan, to_dev(xh), ws))
    ws.check()
    ref = xh
    for gate, up, down, gamma in layers_np:
        ref = O.ffn_layer_A_ref(ref, gamma, gate, up, down, 128)
    assert O.rel_l2(y, ref) <= 1e-2


def test_peer_reduce_gives_up_when_no_flag_is_raised(short_waits):
    """awq_b200_tp_reduce_add_rmsnorm_act waits for the arrival flags of every rank; here nobody raises them."""
    import torch
    from gpu_util import randn_bf16, to_dev
    from mlir_air_b200 import _lib, ops
    lib = short_waits
    B, K = 4, 1024
    ws = ops.Workspace(K, K)
    h = to_dev(randn_bf16((B, K), seed=3))
    partial = torch.zeros((B, K), dtype=torch.float32, device="cuda")
    flags = torch.zeros(16, dtype=torch.int32, device="cuda")
    h_out = torch.full_like(h, 7.0)
    parts = (ctypes.c_void_p * 2)(partial.data_ptr(), partial.data_ptr())
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.awq_b200_tp_reduce_add_rmsnorm_act(h.data_ptr(), parts, flags.data_ptr(), 2, None, 1e-5, h_out.data_ptr(), None, 0, B, K,
                                                ws.buf.data_ptr(), stream)
    assert rc == 0, _lib.last_error()
    rc = lib.awq_b200_workspace_check(ws.buf.data_ptr(), stream)
    assert rc == _lib.AWQ_ERR_DEVICE_TIMEOUT, (rc, _lib.last_error())
    assert torch.all(h_out.float() == 7.0), "nothing may be written after the wait gave up"
    # with the flags raised the same call goes through
    _lib.check(lib.awq_b200_workspace_init(ws.buf.data_ptr(), ws.nbytes, stream), "workspace_init")
    flags[:2] = 1
    rc = lib.awq_b200_tp_reduce_add_rmsnorm_act(h.data_ptr(), parts, flags.data_ptr(), 2, None, 1e-5, h_out.data_ptr(), None, 0, B, K,
                                                ws.buf.data_ptr(), stream)
    assert rc == 0, _lib.last_error()
    ws.check()
    assert torch.equal(h_out, h)  # h + 0 + 0


def test_overflow_inside_the_ffn_is_reported_not_hidden():
    """An intermediate beyond the fp16 range: the fp16 path must say so (the SwiGLU output becomes an infinity, the
    down projection's sums are then not finite and trip the hand-over's range check or show in the output), and
    the bf16 activation path computes the layer."""
    import torch
    from gpu_util import dev_weight, randn_bf16, synth_awq, to_dev, to_host
    from mlir_air_b200 import ops
    from mlir_air_b200._lib import AwqBackendError
    H, I, B = 512, 1024, 2
    gate = synth_awq(H, I, 128, seed=1, scale_lo=1.0, scale_hi=2.0)  # gate, up ~ 2e2: silu(g) * u beyond 65504 for some columns
    up = synth_awq(H, I, 128, seed=2, scale_lo=1.0, scale_hi=2.0)
    down = synth_awq(I, H, 128, seed=3, scale_lo=1e-5, scale_hi=2e-5)
    x = randn_bf16((B, H), seed=4)
    ref = O.ffn_A_ref(x, gate, up, down, 128)
    assert np.abs(O.gateup_swiglu_A_ref(x, gate, up, 128).astype(np.float32)).max() > 65504.0
    wgu, wd = ops.interleave_gate_up(dev_weight(*gate), dev_weight(*up)), dev_weight(*down)
    ops.set_decode_kernel("streamk")
    try:
        ws = ops.Workspace(max(H, I), max(2 * I, H))
        y = to_host(ops.ffn_decode(to_dev(x), wgu, wd, ws))
        reported = False
        try:
            ws.check()
        except AwqBackendError:
            reported = True
        assert reported or not np.isfinite(y.astype(np.float32)).all(), "an overflow was turned into finite numbers silently"
        ops.set_decode_kernel("streamk_bf16")
        ws = ops.Workspace(max(H, I), max(2 * I, H))
        y = to_host(ops.ffn_decode(to_dev(x), wgu, wd, ws))
        ws.check()
        assert O.rel_l2(y, ref) <= 1e-2
    finally:
        ops.set_decode_kernel("auto")
