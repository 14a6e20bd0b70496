"""GPU parity of the one-launch decode FFN stack (awq_b200_ffn_stack_decode_bf16) against the
numpy oracle (the layer chain of o_gemv_ffn_int4_multi.py:9-12 repeated over the layers) and
against the per-layer kernels."""
import numpy as np
import pytest
from ml_dtypes import bfloat16

from oracle import awq_oracle as O

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-2  # the benchmark definition's tolerance for GEMV / FFN outputs


@pytest.fixture(scope="module")
def ops():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from mlir_air_b200 import ops as _ops
    _ops.set_decode_kernel("auto")
    _ops.set_deterministic(False)
    return _ops


def _layers_np(H, I, L, seed):
    from gpu_util import synth_awq
    out = []
    for l in range(L):
        gate = synth_awq(H, I, 128, seed=seed + 10 * l)
        up = synth_awq(H, I, 128, seed=seed + 10 * l + 1)
        down = synth_awq(I, H, 128, seed=seed + 10 * l + 2, scale_lo=0.0005, scale_hi=0.004)
        gamma = (np.random.default_rng(seed + 10 * l + 3).standard_normal(H) * 0.1 + 1.0).astype(bfloat16)
        out.append((gate, up, down, gamma))
    return out


def _plan(ops, layers_np):
    from gpu_util import dev_weight, to_dev
    gus, downs, gammas = [], [], []
    for gate, up, down, gamma in layers_np:
        gus.append(ops.interleave_gate_up(dev_weight(*gate), dev_weight(*up)))
        downs.append(dev_weight(*down))
        gammas.append(to_dev(gamma))
    return ops.FFNStackPlan(gus, downs, gammas), gus, downs, gammas


def _oracle_stack(x, layers_np):
    h = x
    for gate, up, down, gamma in layers_np:
        h = O.ffn_layer_A_ref(h, gamma, gate, up, down, 128)
    return h


@pytest.mark.parametrize("B,H,I,L", [(1, 512, 1408, 2), (4, 1024, 2816, 3), (8, 512, 1024, 4), (3, 2048, 5632, 2)])
def test_stack_vs_oracle(ops, B, H, I, L):
    from gpu_util import randn_bf16, to_dev, to_host
    layers_np = _layers_np(H, I, L, seed=H + I)
    plan, gus, downs, gammas = _plan(ops, layers_np)
    ws = ops.Workspace(max(H, I), max(2 * I, H))
    assert plan.workspace_bytes() <= ws.nbytes
    x = randn_bf16((B, H), seed=5)
    ref = _oracle_stack(x, layers_np)
    y = to_host(ops.ffn_stack_decode(plan, to_dev(x), ws))
    ws.check()
    assert y.shape == (B, H)
    assert O.rel_l2(y, ref) <= REL_L2_TOL
    # the same through the per-layer entry point
    h = to_dev(x)
    for l in range(L):
        h = ops.ffn_decode(h, gus[l], downs[l], ws, gamma=gammas[l], residual=h)
    # two correct f32 summation orders differ by bf16 rounding flips that later layers amplify
    assert O.rel_l2(y, to_host(h)) <= 5e-3
    # a second call on the same workspace (state reset by the launcher), output aliasing the input
    hx = to_dev(x)
    ops.ffn_stack_decode(plan, hx, ws, out=hx)
    ws.check()
    assert O.rel_l2(to_host(hx), ref) <= REL_L2_TOL


def test_stack_llama70b_dims_matches_per_layer_kernels(ops):
    """Benchmark configuration 5 dims (hidden 8192, intermediate 28672), 3 layers, batch 8 and 1: the
    fused launch against the same stack run layer by layer, eager and as a replayed CUDA graph."""
    import torch
    from mlir_air_b200 import ffn
    H, I, L = 8192, 28672, 3
    layers = [ffn.random_layer(H, I, seed=l) for l in range(L)]
    fused = ffn.DecodeFFNStack(layers, H, max_batch=16)
    plain = ffn.DecodeFFNStack(layers, H, max_batch=16, fused=False)
    assert fused.uses_fused(8) and not fused.uses_fused(16) and not plain.uses_fused(8)
    assert fused.launches_per_step(8) == 1
    gen = torch.Generator(device="cuda").manual_seed(1234)
    for B in (8, 1):
        x = (torch.randn((B, H), device="cuda", generator=gen) * 0.5).to(torch.bfloat16)
        a = fused.step(x).float()
        b = plain.step(x).float()
        fused.check()
        plain.check()
        assert torch.isfinite(a).all()
        # two valid paths (fp16 against bf16 intermediates, different summation orders), each inside the bar against
        # the oracle: between them the same bar
        rel = float((a - b).norm() / b.norm())
        assert rel <= REL_L2_TOL, (B, rel)
        fused.load_input(x)
        g1 = fused.replay(B).float().clone()
        fused.load_input(x)
        g2 = fused.replay(B).float().clone()
        fused.check()
        assert float((g1 - b).norm() / b.norm()) <= REL_L2_TOL
        assert float((g2 - b).norm() / b.norm()) <= REL_L2_TOL
    # a batch the fused kernel does not take goes through the per-layer kernels
    x = (torch.randn((16, H), device="cuda") * 0.5).to(torch.bfloat16)
    rel = float((fused.step(x).float() - plain.step(x).float()).norm() / plain.step(x).float().norm())
    assert rel <= 5e-3


def test_stack_llama70b_dims_vs_oracle_golden(ops):
    """Benchmark configuration 5 dims against the numpy oracle: tests/golden/ffn_stack_70b.npz holds the
    hidden state after each of two seeded layers (hidden 8192, intermediate 28672, batch 8), computed on
    the CPU by tests/golden/make_golden_stack70b.py.  The weights are regenerated here from the seeds.
    Checked per layer from the golden input of that layer and end to end, for the one-launch stack
    kernel and for the per-layer kernels."""
    import golden_util
    from gpu_util import dev_weight, to_dev, to_host
    g = golden_util.load("ffn_stack_70b")
    cfg = {k: int(g[k]) for k in golden_util.STACK70B}
    assert cfg == golden_util.STACK70B, "fixture was generated for another configuration"
    H, I, L = cfg["hidden"], cfg["intermediate"], cfg["layers"]
    gold = g["h"]  # [L, 8, H] bf16
    x = golden_util.stack70b_input(cfg)
    gus, downs, gammas = [], [], []
    for l in range(L):
        gate, up, down, gamma = golden_util.stack70b_layer(l, cfg)
        gus.append(ops.interleave_gate_up(dev_weight(*gate), dev_weight(*up)))
        downs.append(dev_weight(*down))
        gammas.append(to_dev(gamma))
        del gate, up, down
    ws = ops.Workspace(max(H, I), max(2 * I, H))
    errs = {}
    # per layer, from the golden input of that layer: one-launch kernel on a one-layer plan, and the per-layer entry point
    for l in range(L):
        h_in = to_dev(x if l == 0 else gold[l - 1])
        plan1 = ops.FFNStackPlan([gus[l]], [downs[l]], [gammas[l]])
        errs[f"fused layer {l}"] = O.rel_l2(to_host(ops.ffn_stack_decode(plan1, h_in, ws)), gold[l])
        ws.check()
        errs[f"per-layer layer {l}"] = O.rel_l2(
            to_host(ops.ffn_decode(h_in, gus[l], downs[l], ws, gamma=gammas[l], residual=h_in)), gold[l])
        ws.check()
    # end to end: both layers in one launch, batch 8 and batch 1 (row 0 alone)
    plan = ops.FFNStackPlan(gus, downs, gammas)
    errs["fused end to end"] = O.rel_l2(to_host(ops.ffn_stack_decode(plan, to_dev(x), ws)), gold[L - 1])
    errs["fused end to end, batch 1"] = O.rel_l2(to_host(ops.ffn_stack_decode(plan, to_dev(x[:1]), ws)), gold[L - 1][:1])
    ws.check()
    bad = {k: v for k, v in errs.items() if not v <= REL_L2_TOL}
    assert not bad, errs


def test_stack_rejects_what_it_cannot_run(ops):
    import torch
    from gpu_util import dev_weight, synth_awq, to_dev
    from mlir_air_b200._lib import AwqBackendError
    H, I = 512, 1024
    layers_np = _layers_np(H, I, 1, seed=1)
    plan, *_ = _plan(ops, layers_np)
    ws = ops.Workspace(I, 2 * I)
    x = torch.zeros((9, H), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(AwqBackendError):
        ops.ffn_stack_decode(plan, x, ws)  # more than 8 rows
    with pytest.raises(AwqBackendError):  # group size 64
        g64 = dev_weight(*synth_awq(H, 2 * I, 64, seed=2), gs=64)
        d64 = dev_weight(*synth_awq(I, H, 64, seed=3), gs=64)
        ops.FFNStackPlan([g64], [d64], [to_dev(layers_np[0][3])])
    # an empty batch is a no-op
    out = ops.ffn_stack_decode(plan, torch.zeros((0, H), dtype=torch.bfloat16, device="cuda"), ws)
    assert out.shape == (0, H)


@pytest.mark.parametrize("M,K,N", [(64, 1024, 2816), (32, 512, 1024), (200, 1024, 512)])
def test_gemm_epilogues_vs_oracle(ops, M, K, N):
    """Tensor-core GEMM with the decode block's epilogues (batched-decode golden, M = batch):
    residual joined before the one rounding; SwiGLU over interleaved gate/up pairs."""
    from gpu_util import dev_weight, randn_bf16, synth_awq, to_dev, to_host
    ops.set_gemm_kernel("tc")
    try:
        A = randn_bf16((M, K), seed=1)
        w = synth_awq(K, N, 128, seed=2)
        R = randn_bf16((M, N), seed=3)
        y = to_host(ops.gemm(to_dev(A), dev_weight(*w), residual=to_dev(R)))
        ops.gemm_check()
        assert O.rel_l2(y, O.gemv_A_ref(A, *w, 128, residual=R)) <= REL_L2_TOL
        gate, up = synth_awq(K, N // 2, 128, seed=4), synth_awq(K, N // 2, 128, seed=5)
        wgu = ops.interleave_gate_up(dev_weight(*gate), dev_weight(*up))
        t = to_host(ops.gemm(to_dev(A), wgu, swiglu=True))
        ops.gemm_check()
        assert t.shape == (M, N // 2)
        assert O.rel_l2(t, O.gateup_swiglu_A_ref(A, gate, up, 128)) <= REL_L2_TOL
    finally:
        ops.set_gemm_kernel("auto")


def test_stack_large_batch_takes_the_gemm_path(ops):
    """Batches 9 to 64 on one GPU: two batched-decode tensor-core GEMMs per layer; same results as one pass of the
    stack kernel per 8 rows and as the oracle; run twice to show that a step leaves the split-K workspace clean."""
    import torch
    from gpu_util import randn_bf16, to_dev, to_host
    from mlir_air_b200 import ffn
    H, I, L = 1024, 2816, 2
    layers_np = _layers_np(H, I, L, seed=77)
    plan, gus, downs, gammas = _plan(ops, layers_np)
    stack = ffn.DecodeFFNStack([ffn.FFNLayer(g, d, gm) for g, d, gm in zip(gus, downs, gammas)], H, max_batch=64)
    assert stack.uses_gemm(9) and stack.uses_gemm(64) and not stack.uses_gemm(8)
    # layers of this size take the 16-bit kernel at every batch; with the size bar out of the way, the kernel with fp8
    # operands up to 32 rows (a third launch per product splits the token rows)
    assert not stack.uses_gemm_f8(16) and stack.launches_per_step(32) == 5 * L
    stack.GEMM_F8_MIN_WEIGHTS = {16: 0, 32: 0}
    assert stack.uses_gemm_f8(9) and stack.uses_gemm_f8(32) and not stack.uses_gemm_f8(33)
    assert stack.launches_per_step(64) == 5 * L and stack.launches_per_step(32) == 7 * L
    for B in (9, 17, 32, 40, 64):
        x = randn_bf16((B, H), seed=B)
        y = to_host(stack.step(to_dev(x)))
        ops.gemm_check()
        assert O.rel_l2(y, _oracle_stack(x, layers_np)) <= REL_L2_TOL
        assert np.array_equal(y.view(np.uint16), to_host(stack.step(to_dev(x))).view(np.uint16))
        # the stack kernel on the same rows, 8 at a time
        parts = [to_host(stack.step(to_dev(x[i:i + 8]))) for i in range(0, B, 8)]
        # (the 16-bit GEMM rounds the weights to fp16, the fp8-operand GEMM and the GEMV keep (q - z) s in f32)
        assert O.rel_l2(y, np.concatenate(parts, 0)) <= REL_L2_TOL
        stack.load_input(to_dev(x))
        g1 = to_host(stack.replay(B).clone())
        assert O.rel_l2(g1, _oracle_stack(x, layers_np)) <= REL_L2_TOL
    stack.check()


@pytest.mark.parametrize("B", [32, 64])
def test_stack_batched_decode_gemm_vs_oracle_hidden_2048(ops, B):
    """The GEMM path of the stack at hidden 2048 / intermediate 5632, 32 and 64 token rows, two layers, against the oracle:
    eager and as a replayed CUDA graph."""
    from gpu_util import randn_bf16, to_dev, to_host
    from mlir_air_b200 import ffn
    H, I, L = 2048, 5632, 2
    layers_np = _layers_np(H, I, L, seed=91)
    plan, gus, downs, gammas = _plan(ops, layers_np)
    stack = ffn.DecodeFFNStack([ffn.FFNLayer(g, d, gm) for g, d, gm in zip(gus, downs, gammas)], H, max_batch=64)
    assert stack.uses_gemm(B)
    x = randn_bf16((B, H), seed=B + 1)
    ref = _oracle_stack(x, layers_np)
    assert O.rel_l2(to_host(stack.step(to_dev(x))), ref) <= REL_L2_TOL
    stack.load_input(to_dev(x))
    assert O.rel_l2(to_host(stack.replay(B).clone()), ref) <= REL_L2_TOL
    stack.check()


# (M, K, N): one k-block pair and one tile; a ragged last tile; more units than SMs with tiles shared by several SMs and
# SMs covering several tiles; K deeper than the input ring many times over
@pytest.mark.parametrize("M,K,N", [(9, 128, 256), (16, 256, 32), (33, 1024, 1312), (64, 2048, 5632), (64, 8192, 512),
                                   (17, 512, 800), (48, 1024, 2048), (12, 5632, 2048)])
def test_gemm_decode_vs_oracle(ops, M, K, N):
    """Batched-decode GEMM (stream-K over column tiles and k-blocks, split-K sums as integers) against the oracle, all
    three epilogues; a second call on the same workspace gives the same bits."""
    from gpu_util import dev_weight, randn_bf16, synth_awq, to_dev, to_host
    bits = lambda a: a.view(np.uint16)  # noqa: E731
    A = randn_bf16((M, K), seed=M + 1)
    w = synth_awq(K, N, 128, seed=N + 2)
    R = randn_bf16((M, N), seed=3)
    ws = ops.GemmDecodeWorkspace(N, batch=M)
    dw = dev_weight(*w)
    y = to_host(ops.gemm_decode(to_dev(A), dw, ws))
    ops.gemm_check()
    ref_bf16w = (A.astype(np.float32) @ O.dequant_to_bf16(*w, 128).astype(np.float32)).astype(bfloat16)
    assert O.rel_l2(y, ref_bf16w) <= 3e-3  # same products, summation order only
    assert O.rel_l2(y, O.gemv_A_ref(A, *w, 128)) <= REL_L2_TOL
    # the f32 sums themselves (what a tensor-parallel rank hands to the allreduce): rounded, they are the bf16 output
    import torch
    yf = ops.gemm_decode(to_dev(A), dw, ws, f32_out=True)
    assert yf.dtype == torch.float32 and np.array_equal(bits(to_host(yf.to(torch.bfloat16))), bits(y))
    yr = to_host(ops.gemm_decode(to_dev(A), dw, ws, residual=to_dev(R)))
    ops.gemm_check()
    assert O.rel_l2(yr, O.gemv_A_ref(A, *w, 128, residual=R)) <= REL_L2_TOL
    assert np.array_equal(bits(yr), bits(to_host(ops.gemm_decode(to_dev(A), dw, ws, residual=to_dev(R)))))
    if N % 64 == 0:
        gate, up = synth_awq(K, N // 2, 128, seed=4), synth_awq(K, N // 2, 128, seed=5)
        wgu = ops.interleave_gate_up(dev_weight(*gate), dev_weight(*up))
        t = to_host(ops.gemm_decode(to_dev(A), wgu, ws, swiglu=True))
        ops.gemm_check()
        assert t.shape == (M, N // 2)
        assert O.rel_l2(t, O.gateup_swiglu_A_ref(A, gate, up, 128)) <= REL_L2_TOL


@pytest.mark.parametrize("M,K,N", [(9, 128, 256), (33, 1024, 1312), (64, 2048, 5632), (17, 8192, 512)])
def test_gemm_decode_fp16_operands_vs_oracle(ops, M, K, N):
    """The same product on fp16 token rows and weights dequantised to fp16 (what the decode stack runs between its
    kernels): every epilogue against the oracle, nearer to it than the bf16 form, fp16 and bf16 outputs of one
    value agreeing, and repeatable bits."""
    import torch
    from gpu_util import dev_weight, randn_bf16, synth_awq, to_dev, to_host
    bits = lambda a: a.view(np.uint16)  # noqa: E731
    A = randn_bf16((M, K), seed=M + 7)
    w = synth_awq(K, N, 128, seed=N + 8)
    R = randn_bf16((M, N), seed=9)
    ws = ops.GemmDecodeWorkspace(N, batch=M)
    dw = dev_weight(*w)
    Ah = to_dev(A).to(torch.float16)  # exact: |values| of a unit normal sit well inside fp16's normal range
    yf = ops.gemm_decode(Ah, dw, ws, f32_out=True)
    ops.gemm_check()
    exact = A.astype(np.float32) @ O.dequant_f32(*w, 128)
    err_h = O.rel_l2(yf.cpu().numpy(), exact)
    err_b = O.rel_l2(ops.gemm_decode(to_dev(A), dw, ws, f32_out=True).cpu().numpy(), exact)
    assert err_h <= 5e-4 and err_h < 0.5 * err_b, (err_h, err_b)  # 11 against 8 significant bits of every weight
    y = to_host(ops.gemm_decode(Ah, dw, ws))
    assert np.array_equal(bits(y), bits(to_host(yf.to(torch.bfloat16))))
    assert O.rel_l2(y, O.gemv_A_ref(A, *w, 128)) <= 3e-3
    y16 = ops.gemm_decode(Ah, dw, ws, out_f16=True)
    assert y16.dtype == torch.float16 and torch.equal(y16, yf.to(torch.float16))
    yr = to_host(ops.gemm_decode(Ah, dw, ws, residual=to_dev(R)))
    ops.gemm_check()
    assert O.rel_l2(yr, O.gemv_A_ref(A, *w, 128, residual=R)) <= 3e-3
    assert np.array_equal(bits(yr), bits(to_host(ops.gemm_decode(Ah, dw, ws, residual=to_dev(R)))))
    if N % 64 == 0:
        gate, up = synth_awq(K, N // 2, 128, seed=4), synth_awq(K, N // 2, 128, seed=5)
        wgu = ops.interleave_gate_up(dev_weight(*gate), dev_weight(*up))
        t = ops.gemm_decode(Ah, wgu, ws, swiglu=True)
        t16 = ops.gemm_decode(Ah, wgu, ws, swiglu=True, out_f16=True)
        ops.gemm_check()
        assert t16.dtype == torch.float16 and torch.equal(t16, t.to(torch.float16))  # the bf16 value, stored as fp16
        assert O.rel_l2(to_host(t), O.gateup_swiglu_A_ref(A, gate, up, 128)) <= 3e-3


# (M, K, N) as above, up to 32 rows; the last: a row whose elements span 20 binades and a row of zeros
@pytest.mark.parametrize("M,K,N", [(9, 128, 256), (16, 256, 32), (32, 1024, 1312), (17, 512, 800), (32, 8192, 512),
                                   (12, 5632, 2048), (24, 2048, 5632)])
def test_gemm_decode_fp8_operands_vs_oracle(ops, M, K, N):
    """The product with the packed nibbles and the split token rows as the tensor core's fp8 operands, zero point and scale
    applied in f32: every epilogue against the oracle (no weight is rounded, so it sits nearer to the exact product than
    the 16-bit kernels), bf16 and fp16 inputs, outputs of one value agreeing, repeatable bits."""
    import torch
    from gpu_util import dev_weight, randn_bf16, synth_awq, to_dev, to_host
    bits = lambda a: a.view(np.uint16)  # noqa: E731
    A = randn_bf16((M, K), seed=M + 11)
    A[0] = (A[0].astype(np.float32) * np.exp2(np.random.default_rng(5).integers(-18, 3, K))).astype(bfloat16)  # a wide row
    A[M - 1] = 0  # and an empty one
    w = synth_awq(K, N, 128, seed=N + 12)
    R = randn_bf16((M, N), seed=13)
    ws = ops.GemmDecodeWorkspace(N, batch=M, K=K)
    assert ws.fits_f8(M, K, N) and not ws.fits_f8(33, K, N)
    dw = dev_weight(*w)
    yf = ops.gemm_decode(to_dev(A), dw, ws, f32_out=True, f8=True)
    ops.gemm_check()
    exact = A.astype(np.float32) @ O.dequant_f32(*w, 128)
    assert O.rel_l2(yf.cpu().numpy(), exact) <= 1e-4
    assert float(np.abs(yf.cpu().numpy()[M - 1]).max()) == 0.0
    for m in (0, 1):  # the wide row on its own, and an ordinary one
        assert O.rel_l2(yf.cpu().numpy()[m], exact[m]) <= 1e-4
    y = to_host(ops.gemm_decode(to_dev(A), dw, ws, f8=True))
    assert np.array_equal(bits(y), bits(to_host(yf.to(torch.bfloat16))))
    assert O.rel_l2(y, O.gemv_A_ref(A, *w, 128)) <= 3e-3
    Ah = to_dev(A).to(torch.float16)  # fp16 token rows: the bf16 values that fp16 holds exactly, others rounded by the cast
    yh = ops.gemm_decode(Ah, dw, ws, f32_out=True, f8=True)
    assert O.rel_l2(yh.cpu().numpy(), Ah.float().cpu().numpy() @ O.dequant_f32(*w, 128)) <= 1e-4
    # genuine fp16 values (11 significant bits) are rounded to the 8 that the two pieces hold, like a bf16 conversion
    Ag = (to_dev(A).float() * 1.0009765625).to(torch.float16)
    yg = ops.gemm_decode(Ag, dw, ws, f32_out=True, f8=True)
    assert O.rel_l2(yg.cpu().numpy(), Ag.float().cpu().numpy() @ O.dequant_f32(*w, 128)) <= 3e-3
    y16 = ops.gemm_decode(to_dev(A), dw, ws, out_f16=True, f8=True)
    assert y16.dtype == torch.float16 and torch.equal(y16, yf.to(torch.float16))
    yr = to_host(ops.gemm_decode(to_dev(A), dw, ws, residual=to_dev(R), f8=True))
    ops.gemm_check()
    assert O.rel_l2(yr, O.gemv_A_ref(A, *w, 128, residual=R)) <= 3e-3
    assert np.array_equal(bits(yr), bits(to_host(ops.gemm_decode(to_dev(A), dw, ws, residual=to_dev(R), f8=True))))
    if N % 64 == 0:
        gate, up = synth_awq(K, N // 2, 128, seed=4), synth_awq(K, N // 2, 128, seed=5)
        wgu = ops.interleave_gate_up(dev_weight(*gate), dev_weight(*up))
        t = ops.gemm_decode(to_dev(A), wgu, ws, swiglu=True, f8=True)
        t16 = ops.gemm_decode(to_dev(A), wgu, ws, swiglu=True, out_f16=True, f8=True)
        ops.gemm_check()
        assert t16.dtype == torch.float16 and torch.equal(t16, t.to(torch.float16))
        assert O.rel_l2(to_host(t), O.gateup_swiglu_A_ref(A, gate, up, 128)) <= 3e-3


def test_gemm_decode_rejects_what_it_cannot_run(ops):
    import torch
    from gpu_util import dev_weight, randn_bf16, synth_awq, to_dev
    from mlir_air_b200._lib import AwqBackendError
    w = dev_weight(*synth_awq(256, 256, 128, seed=1))
    ws = ops.GemmDecodeWorkspace(256, batch=16)
    with pytest.raises(AwqBackendError):  # more rows than the kernel takes
        ops.gemm_decode(to_dev(randn_bf16((65, 256), seed=1)), w, ws)
    with pytest.raises(AwqBackendError):  # workspace too small for these rows (sized for 16, called with 17)
        ops.gemm_decode(to_dev(randn_bf16((17, 256), seed=1)), w, ws)
    assert ops.gemm_decode(torch.zeros((0, 256), dtype=torch.bfloat16, device="cuda"), w, ws).shape == (0, 256)
    x = to_dev(randn_bf16((16, 256), seed=1))
    with pytest.raises(AwqBackendError):  # the residual joins a bf16 output only
        ops.gemm_decode(x, w, ws, residual=x, out_f16=True)
    with pytest.raises(AwqBackendError):  # f32 sums carry no epilogue
        ops.gemm_decode(x, w, ws, f32_out=True, swiglu=True)
    with pytest.raises(AwqBackendError):
        ops.gemm_decode(x.float(), w, ws)
    with pytest.raises(AwqBackendError):  # the fp8-operand kernel needs room for the split token rows
        ops.gemm_decode(x, w, ws, f8=True)
    ws8 = ops.GemmDecodeWorkspace(256, batch=64, K=256)
    with pytest.raises(AwqBackendError):  # and takes 32 rows at most
        ops.gemm_decode(to_dev(randn_bf16((33, 256), seed=1)), w, ws8, f8=True)
