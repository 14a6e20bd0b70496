"""The allocation-free GEMV entry point (awq_b200_gemv_bf16_static).

It exists for hosts that cannot give the library a scratch buffer -- a plugin slot whose
signature only has the reference's inputs and outputs, or a server that forbids cudaMalloc
after start-up -- so its scratch is a fixed array inside the library.  These tests call it
through the C ABI and compare it with the regular entry point, twice in a row on different
inputs, because the array keeps the previous call's contents.

Collected last on purpose (file name), so a run that stops at the first failure has already
run every other test.
"""
import ctypes

import numpy as np
import pytest

REL_L2_TOL = 1e-2  # same bound as the other GEMV parity tests


def test_static_rejects_oversize_without_touching_the_gpu():
    from mlir_air_b200 import _lib
    lib = _lib.load()
    dummy = ctypes.c_void_p(16)
    rc = lib.awq_b200_gemv_bf16_static(dummy, dummy, dummy, dummy, None, dummy, 1, 128, 32768 + 32, 128, None)
    assert rc == _lib.AWQ_ERR_INVALID_ARGUMENT
    assert "exceeds the built-in scratch" in _lib.last_error()
    rc = lib.awq_b200_gemv_bf16_static(dummy, dummy, dummy, dummy, None, dummy, 65, 128, 256, 128, None)
    assert rc == _lib.AWQ_ERR_INVALID_ARGUMENT


@pytest.mark.gpu
def test_static_matches_workspace_entry_point_two_calls_in_a_row():
    import torch
    from mlir_air_b200 import _lib, ops
    from oracle import awq_oracle as O
    from gpu_util import to_dev, to_host, synth_awq, dev_weight, randn_bf16

    lib = _lib.load()
    K, N = 4096, 4096  # 16 strips x 32 groups over 148 CTAs: every strip is shared between CTAs
    qw, qz, s = synth_awq(K, N, 128, seed=21)
    w = dev_weight(qw, qz, s)
    ws = ops.Workspace(K, N)
    ops.set_decode_kernel("streamk_bf16")  # the allocation-free entry multiplies bf16 activations as they are
    stream = torch.cuda.current_stream().cuda_stream
    try:
        # 8 and 3 rows: one pass; 20 rows: three passes of 8 rows over the one shared set of accumulators
        for call, (B, seed) in enumerate([(8, 1), (3, 2), (20, 3)]):
            x = randn_bf16((B, K), seed=seed)
            r = randn_bf16((B, N), seed=seed + 10)
            xd, rd = to_dev(x), to_dev(r)
            y_ref = torch.empty((B, N), dtype=torch.bfloat16, device="cuda")
            y_new = torch.full((B, N), float("nan"), dtype=torch.bfloat16, device="cuda")
            _lib.check(lib.awq_b200_gemv_bf16(xd.data_ptr(), w.qweight.data_ptr(), w.qzeros.data_ptr(),
                                              w.scales.data_ptr(), rd.data_ptr(), y_ref.data_ptr(), B, K, N, 128,
                                              ws.buf.data_ptr(), ws.nbytes, stream), "gemv_bf16")
            _lib.check(lib.awq_b200_gemv_bf16_static(xd.data_ptr(), w.qweight.data_ptr(), w.qzeros.data_ptr(),
                                                     w.scales.data_ptr(), rd.data_ptr(), y_new.data_ptr(), B, K, N,
                                                     128, stream), "gemv_bf16_static")
            # a wait that gave up would be reported here (and only here: the next static call clears the word)
            _lib.check(lib.awq_b200_static_check(stream), "static_check")
            a, e = to_host(y_new), to_host(y_ref)
            assert np.isfinite(a.astype(np.float32)).all(), f"call {call}: output not fully written"
            assert O.rel_l2(a, e) <= REL_L2_TOL, f"call {call}"
            assert O.rel_l2(a, O.gemv_A_ref(x, qw, qz, s, 128, residual=r)) <= REL_L2_TOL, f"call {call}"
        ws.check()
    finally:
        ops.set_decode_kernel("auto")


@pytest.mark.gpu
def test_static_reports_unsupported_shapes():
    import torch
    from mlir_air_b200 import _lib
    from gpu_util import synth_awq, dev_weight, to_dev, randn_bf16
    lib = _lib.load()
    K, N = 128, 40  # N % 32 != 0: the stream-K kernel cannot run, and there is no fallback here
    w = dev_weight(*synth_awq(K, N, 128, seed=3))
    x = to_dev(randn_bf16((1, K), seed=1))
    y = torch.empty((1, N), dtype=torch.bfloat16, device="cuda")
    rc = lib.awq_b200_gemv_bf16_static(x.data_ptr(), w.qweight.data_ptr(), w.qzeros.data_ptr(), w.scales.data_ptr(),
                                       None, y.data_ptr(), 1, K, N, 128, torch.cuda.current_stream().cuda_stream)
    assert rc == _lib.AWQ_ERR_UNSUPPORTED
