"""Runner and backend with the reference's interface, executing on a B200.

Mirrors `XRTRunner` (python/air/backend/xrt_runner.py:60-373) and `XRTBackend`
(python/air/backend/xrt.py:221-929): the same constructor keywords (NPU-only ones are
accepted and ignored), `run_test(module, inputs, expected_outputs, rtol, atol,
max_mismatch_percentage, min_correlation) -> 0 | -1` printing `PASS!` / `failed.`,
`compile(module) -> artifact`, `load(artifact) -> invoker(*arrays) -> tuple(arrays)`, `unload()`,
`last_latency_us`.  A "module" here is a `KernelSpec` (what the example's `build_module`
returns): there is no IR to compile, so `compile` validates the spec and loads the library.

The invoker behaves like the XRT one (xrt.py:742-791): it allocates device buffers per call,
copies every argument in, runs, copies every buffer back and returns them all as fresh host
arrays (inputs first, outputs after).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np
from ml_dtypes import bfloat16

from . import _lib, layouts
from ._lib import AwqBackendError

AirBackendError = AwqBackendError  # the reference's exception name


@dataclass
class KernelSpec:
    """What `build_module` returns: the kernel instance and its compile-time shape parameters
    (the `-DDIM_*` macros of the AIE kernels become run-time arguments here)."""
    instance_name: str
    params: Dict[str, int] = field(default_factory=dict)

    def __str__(self):  # `-p/--print-module-only` prints the resolved plan instead of MLIR
        items = ", ".join(f"{k}={v}" for k, v in self.params.items())
        return f"b200.kernel @{self.instance_name}({items})"


def _to_dev(a: np.ndarray):
    import torch
    a = np.ascontiguousarray(a)
    if a.dtype == bfloat16:
        return torch.from_numpy(a.view(np.int16)).cuda().view(torch.bfloat16)
    return torch.from_numpy(a).cuda()


def _to_host(t, like: np.ndarray):
    import torch
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).cpu().numpy().view(bfloat16).reshape(like.shape)
    return t.cpu().numpy().reshape(like.shape)


# ---- one host-level implementation per kernel instance: args are the example's buffers ----------
def _run_dequant(p, args):
    from . import ops
    packed, out = args
    pq, s, z = layouts.unpack_dequant_tiles(packed, p["n"], p["group_size"], p["herd_n"])
    y = ops.dequant_1d(_to_dev(pq), _to_dev(s), _to_dev(z), p["n"], p["group_size"])
    return [y], [1]


def _resident(p, slot, build):
    """`build()`, or what an earlier call built for argument `slot` when the caller declared that
    argument static (KernelCache.load_and_run: written on first use, resident afterwards)."""
    if slot is None or slot not in p.get("__static__", ()):
        return build()
    store = p["__resident__"]
    if slot not in store:
        store[slot] = build()
    return store[slot]


def _weight_from_gemv_tiles(p, packed, M, slot=None):
    """Per-tile packed buffer -> resident layout-A weight, unpacked on the GPU
    (awq_b200_repack_C_to_B, then awq_b200_repack_B_to_A)."""
    from . import ops

    def build():
        layouts._check_gemv_tiling(M, p["K"], p["GS"], p["M_TILE"], p["K_CHUNK"], p["N_CORES"], p.get("M_PER_LAUNCH") or M)
        return ops.repack_C_to_A(_to_dev(np.ascontiguousarray(packed, dtype=np.uint8).reshape(-1)), M, p["K"], p["GS"],
                                 p["M_TILE"], p["K_CHUNK"])

    return _resident(p, slot, build)


def _workspace(p, K, N):
    from . import ops
    if "__resident__" in p:
        return _resident(dict(p, __static__=("ws",)), "ws", lambda: ops.Workspace(K, N))
    return ops.Workspace(K, N)


def _run_matvec(p, args):
    from . import ops
    packed, x, out = args
    w = _weight_from_gemv_tiles(p, packed, p["M"], slot=0)
    ws = _workspace(p, w.K, w.N)
    y = ops.gemv(_to_dev(np.asarray(x).reshape(-1, p["K"])), w, ws)
    ws.check()
    return [y], [2]


def _run_matvec_add(p, args):
    from . import ops
    packed, x, r, out = args
    w = _weight_from_gemv_tiles(p, packed, p["M"], slot=0)
    ws = _workspace(p, w.K, w.N)
    y = ops.gemv(_to_dev(np.asarray(x).reshape(-1, p["K"])), w, ws, residual=_to_dev(np.asarray(r).reshape(-1, p["M"])))
    ws.check()
    return [y], [3]


def _run_swiglu_rms(p, args):
    from . import ops
    packed, rms_in, out = args
    w = _weight_from_gemv_tiles(p, packed, p["M"], slot=0)  # rows gate/up interleaved -> [K, 2I] interleaved columns
    ws = _workspace(p, w.K, w.N)
    rms_in = np.asarray(rms_in).reshape(2, p["K"])
    normed = ops.rmsnorm(_to_dev(rms_in[0:1]), _to_dev(rms_in[1]), p.get("eps", 1e-5))
    y = ops.gateup_swiglu(normed, w, ws)
    ws.check()
    return [y], [2]


def _run_rms_qkv_rope(p, args):
    """The 13-argument ABI of rms_qkv_int4_rope_multi.py:17-31: x_in, norm_w, normed, wq_packed, q,
    wk_packed, k, wv_packed, v, lut_q, lut_k, q_roped, k_roped.  Q, K and V are one GEMV over the
    concatenated weight; RoPE rotates the Q and K parts of its output."""
    import torch
    from . import ops
    x_in, norm_w, _, wq_p, _, wk_p, _, wv_p, _, lut_q, lut_k, _, _ = args
    emb, kv, hd = p["emb_dim"], p["kv_dim"], p["head_dim"]
    tile = dict(K=emb, GS=p["GS"], M_TILE=p["M_TILE"], K_CHUNK=p["K_CHUNK"], N_CORES=p["N_CORES"])

    def build_qkv():
        ws_ = [_weight_from_gemv_tiles(tile, wq_p, emb), _weight_from_gemv_tiles(tile, wk_p, kv),
               _weight_from_gemv_tiles(tile, wv_p, kv)]
        return ops.AwqWeight(torch.cat([t.qweight for t in ws_], 1).contiguous(),
                             torch.cat([t.qzeros for t in ws_], 1).contiguous(),
                             torch.cat([t.scales for t in ws_], 1).contiguous(), p["GS"])

    # resident when all three weight arguments (3, 5, 7) are declared static
    w = _resident(p, 3 if {3, 5, 7} <= set(p.get("__static__", ())) else None, build_qkv)
    ws = _workspace(p, w.K, w.N)
    normed = ops.rmsnorm(_to_dev(np.asarray(x_in).reshape(1, emb)), _to_dev(np.asarray(norm_w)), p.get("eps", 1e-5))
    qkv = ops.gemv(normed, w, ws)
    ws.check()
    q, k, v = qkv[:, :emb].clone(), qkv[:, emb:emb + kv].clone(), qkv[:, emb + kv:].clone()
    # the reference tiles one LUT row over the heads (:676-677); a token's row is its first head's
    lut_row_q = _to_dev(np.asarray(lut_q).reshape(-1, hd)[0:1])
    lut_row_k = _to_dev(np.asarray(lut_k).reshape(-1, hd)[0:1])
    q_r = ops.rope_halfsplit(qkv[:, :emb], lut_row_q, p["n_heads"], hd, out=torch.empty_like(q))
    k_r = ops.rope_halfsplit(qkv[:, emb:emb + kv], lut_row_k, p["n_kv_heads"], hd, out=torch.empty_like(k))
    return [normed, q, k, v, q_r, k_r], [2, 4, 6, 8, 11, 12]


def _run_matmul(p, args):
    from . import ops
    A, packed, out = args
    if p["N"] % p["N_TILE"] or p["K"] % p["K_CHUNK"] or p["K_CHUNK"] % p["GS"]:
        raise ValueError("N, K, N_TILE, K_CHUNK and GS do not tile")
    w = _resident(p, 1, lambda: ops.repack_C_to_A(_to_dev(np.ascontiguousarray(packed, dtype=np.uint8).reshape(-1)), p["N"],
                                                  p["K"], p["GS"], p["N_TILE"], p["K_CHUNK"]))
    y = ops.gemm(_to_dev(np.asarray(A).reshape(p["M"], p["K"])), w)
    ops.gemm_check()
    return [y], [2]


def _run_ffn_int4(p, args):
    """x, then (qweight, qzeros, scales) of gate/up-interleaved and of down, then `inter` and `out`."""
    from . import ops
    x, gq, gz, gs_, dq, dz, ds, inter, out = args
    H, I, gsz = p["hidden"], p["intermediate"], p["GS"]
    wgu = ops.AwqWeight.from_numpy(gq, gz, gs_, gsz)
    wd = ops.AwqWeight.from_numpy(dq, dz, ds, gsz)
    ws = ops.Workspace(max(H, I), max(2 * I, H))
    xd = _to_dev(np.asarray(x).reshape(-1, H))
    it = ops.gateup_swiglu(xd, wgu, ws)  # bf16 intermediate, returned to the caller for checking
    y = ops.gemv(it, wd, ws)
    ws.check()
    return [it, y], [7, 8]


def _run_ffn_int4_prefill(p, args):
    """x [seq, hidden], then (qweight, qzeros, scales) of gate/up-interleaved and of down, then `inter` and `out`:
    the prefill FFN on AWQ weights as two tensor-core GEMMs, SwiGLU in the first one's epilogue."""
    from . import ops
    x, gq, gz, gs_, dq, dz, ds, inter, out = args
    H, gsz = p["hidden"], p["GS"]
    wgu = _resident(p, 1, lambda: ops.AwqWeight.from_numpy(gq, gz, gs_, gsz))
    wd = _resident(p, 4, lambda: ops.AwqWeight.from_numpy(dq, dz, ds, gsz))
    xd = _to_dev(np.asarray(x).reshape(-1, H))
    it = ops.gemm(xd, wgu, swiglu=True)
    y = ops.gemm(it, wd)
    ops.gemm_check()
    return [it, y], [7, 8]


def _o_gemv_ffn(p, wo_p, attn_out, x_residual, gu_p, gamma, wd_p, slots, one_launch):
    """The post-attention half of a decode layer: res1 = W_o attn + x; out = W_d swiglu(W_gu rms(res1, gamma)) + res1
    (o_gemv_ffn_int4_multi.py:9-12).  Returns (res1, swiglu or None, out) as device tensors [1, emb] / [1, hidden]."""
    import torch
    from . import ops
    emb, hid = p["emb_dim"], p["hidden_dim"]
    tile = dict(GS=p["GS"], M_TILE=p["M_TILE"], K_CHUNK=p["K_CHUNK"], N_CORES=p["N_CORES"], __static__=p.get("__static__", ()),
                __resident__=p.get("__resident__", {}))
    wo = _weight_from_gemv_tiles(dict(tile, K=emb), wo_p, emb, slot=slots[0])
    wgu = _weight_from_gemv_tiles(dict(tile, K=emb), gu_p, 2 * hid, slot=slots[1])  # rows gate/up interleaved
    wd = _weight_from_gemv_tiles(dict(tile, K=hid), wd_p, emb, slot=slots[2])
    ws = _workspace(p, max(emb, hid), max(2 * hid, emb))
    g = _to_dev(np.asarray(gamma).reshape(emb))
    res1 = ops.gemv(_to_dev(np.asarray(attn_out).reshape(1, emb)), wo, ws, residual=_to_dev(np.asarray(x_residual).reshape(1, emb)))
    swiglu = None
    if one_launch:
        # RMSNorm, gate/up + SwiGLU, down + residual in ONE launch, intermediates staying inside the kernel's scratch
        plan = _resident(dict(p, __static__=("plan",) if slots[1] in p.get("__static__", ()) else ()), "plan",
                         lambda: ops.FFNStackPlan([wgu], [wd], [g]))
        out = ops.ffn_stack_decode(plan, res1, ws, eps=p.get("eps", 1e-5))
    else:
        normed = ops.rmsnorm(res1, g, p.get("eps", 1e-5))
        swiglu = ops.gateup_swiglu(normed, wgu, ws)
        out = ops.gemv(swiglu, wd, ws, residual=res1)
    ws.check()
    return res1, swiglu, out


def _run_o_gemv_ffn_int4(p, args):
    """The 15-argument ABI of o_gemv_ffn_int4_multi.py:13-31 (arguments 2, 4, 5, 8, 9, 10, 13 are dead there and
    ignored here): res1 lands in row 0 of argument 6, the SwiGLU output in argument 11, the result in argument 14."""
    import torch
    wo_p, attn_out, _, x_res, _, _, packed_rms, gu_p, _, _, _, _, wd_p, _, out = args
    emb = p["emb_dim"]
    packed_rms = np.asarray(packed_rms).reshape(2, emb)
    res1, swiglu, y = _o_gemv_ffn(p, wo_p, attn_out, x_res, gu_p, packed_rms[1], wd_p, (0, 7, 12), one_launch=False)
    rms_out = torch.cat([res1.reshape(1, emb), _to_dev(packed_rms[1:2])], 0)
    return [rms_out, swiglu, y], [6, 11, 14]


def _run_o_gemv_ffn_int4_fused(p, args):
    """The 8-argument ABI of o_gemv_ffn_int4_fused.py:33-42: wo_packed, attn_out, x_residual, gate/up_packed,
    ffn_norm_w, wdown_packed, output, res1 copy."""
    wo_p, attn_out, x_res, gu_p, gamma, wd_p, out, res1_out = args
    res1, _, y = _o_gemv_ffn(p, wo_p, attn_out, x_res, gu_p, gamma, wd_p, (0, 3, 5), one_launch=True)
    return [y, res1], [6, 7]


def _run_ffn_bf16(p, args):
    """bf16 FFN examples: x, packed [gate | up | down] weights, then the gate / up / inter buffers
    (function arguments in the reference, ffn_decode.py:300-303) and the output."""
    from . import ops
    x, packed, gate_buf, up_buf, inter_buf, out = args
    dim, cols = p["dim"], p["num_cols"]
    unpack = layouts.unpack_ffn_weights_prefill if p["mode"] == "prefill" else layouts.unpack_ffn_weights_decode
    flat = np.asarray(packed).reshape(3, dim * dim)
    Wg, Wu, Wd = (unpack(flat[i], dim, cols) for i in range(3))
    if p["mode"] == "prefill":
        # that example packs B = W^T column blocks of `W[:, cols]`, and its golden multiplies by W^T
        Wg, Wu, Wd = (np.ascontiguousarray(w) for w in (Wg, Wu, Wd))
    xd = _to_dev(np.asarray(x).reshape(-1, dim))
    g = ops.linear_bf16(xd, _to_dev(Wg))
    u = ops.linear_bf16(xd, _to_dev(Wu))
    t = ops.silu_mul(g, u)
    y = ops.linear_bf16(t, _to_dev(Wd))
    return [g, u, t, y], [2, 3, 4, 5]


def _run_matvec_bf16(p, args):
    """A bf16 [M, K], B bf16 [K], C bf16 [M] (matrix_vector_multiplication/bf16/matvec.py)."""
    from . import ops
    A, B, out = args
    y = ops.linear_bf16(_to_dev(np.asarray(B).reshape(1, p["K"])),
                        _resident(p, 0, lambda: _to_dev(np.asarray(A).reshape(p["M"], p["K"]))))
    return [y], [2]


def _run_swiglu_rms_bf16(p, args):
    """A bf16 [M, K] (gate/up rows interleaved), RMS_in bf16 [2, K], D bf16 [M/2]
    (decode_ffn_swiglu/matvec_swiglu_rms.py)."""
    from . import ops
    A, rms_in, out = args
    rms_in = np.asarray(rms_in).reshape(2, p["K"])
    normed = ops.rmsnorm(_to_dev(rms_in[0:1]), _to_dev(rms_in[1]), p.get("eps", 1e-5))
    gu = ops.linear_bf16(normed, _resident(p, 0, lambda: _to_dev(np.asarray(A).reshape(p["M"], p["K"]))))
    return [ops.silu_mul(gu[0, 0::2].contiguous(), gu[0, 1::2].contiguous())], [2]


def _run_silu_and_mul(p, args):
    from . import ops
    gate, up, out = args
    return [ops.silu_mul(_to_dev(np.asarray(gate).reshape(-1)), _to_dev(np.asarray(up).reshape(-1)))], [2]


_INSTANCES: Dict[str, Callable] = {
    "matvec_bf16": _run_matvec_bf16,
    "silu_and_mul": _run_silu_and_mul,
    "matvec_swiglu_rms": _run_swiglu_rms_bf16,
    "ffn_swiglu": _run_ffn_bf16,
    "dequant": _run_dequant,
    "matvec_int4_packed": _run_matvec,
    "matvec_int4_packed_add": _run_matvec_add,
    "matvec_int4_swiglu_rms": _run_swiglu_rms,
    "matmul_int4_packed": _run_matmul,
    "rms_qkv_int4_rope": _run_rms_qkv_rope,
    "ffn_swiglu_int4": _run_ffn_int4,
    "ffn_swiglu_int4_prefill": _run_ffn_int4_prefill,
    "o_gemv_ffn_int4": _run_o_gemv_ffn_int4,
    "o_gemv_ffn_int4_fused": _run_o_gemv_ffn_int4_fused,
}


class B200Backend:
    """Counterpart of XRTBackend.  Keyword arguments that only steer the AIE compiler are ignored."""

    def __init__(self, verbose: bool = False, n_perf_iters: int = 0, n_warmup_iters: int = 10,
                 instance_name: str = "", **npu_only_kwargs):
        self.verbose = verbose
        self.n_perf_iters = n_perf_iters
        self.n_warmup_iters = n_warmup_iters
        self.instance_name = instance_name
        self.ignored_kwargs = dict(npu_only_kwargs)
        self.currently_loaded = False
        self.last_latency_us: Optional[float] = None

    def __del__(self):
        self.unload()

    def compile(self, module: KernelSpec):
        if self.currently_loaded:
            raise AwqBackendError("Cannot compile while an artifact is loaded. Call unload() first.")
        if not isinstance(module, KernelSpec):
            raise AwqBackendError(f"expected a KernelSpec from build_module, got {type(module).__name__}")
        name = module.instance_name or self.instance_name
        if name not in _INSTANCES:
            raise AwqBackendError(f"no B200 kernel for instance '{name}' (have: {sorted(_INSTANCES)})")
        _lib.load()  # the "link" step: fails loudly if libawq_b200.so has not been built
        return KernelSpec(name, dict(module.params))

    def load(self, artifact: KernelSpec):
        import torch
        if self.currently_loaded:
            raise AwqBackendError("Cannot load while an artifact is loaded. Call unload() first.")
        if not torch.cuda.is_available():
            raise AwqBackendError("load() needs a CUDA device; there is no CPU path")
        fn, params = _INSTANCES[artifact.instance_name], artifact.params

        def invoker(*args):
            args = [np.asarray(a) for a in args]
            outs, idx = fn(params, args)
            if self.n_perf_iters > 0:  # time whole invocations, as xrt.py:768-779 times run.start()+wait2()
                for _ in range(self.n_warmup_iters):
                    fn(params, args)
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(self.n_perf_iters):
                    fn(params, args)
                e1.record()
                torch.cuda.synchronize()
                self.last_latency_us = e0.elapsed_time(e1) * 1e3 / self.n_perf_iters
            torch.cuda.synchronize()
            result = [a.copy() for a in args]
            for t, i in zip(outs, idx):
                result[i] = _to_host(t, args[i])
            return tuple(result)

        self.currently_loaded = True
        return invoker

    def compile_and_load(self, module):
        return self.load(self.compile(module))

    def unload(self):
        self.currently_loaded = False


class B200Runner:
    """Counterpart of XRTRunner: compile, run once, compare against the expected outputs."""

    def __init__(self, verbose: bool = False, n_perf_iters: int = 0, n_warmup_iters: int = 10,
                 perf_flops: Optional[float] = None, report_precision: bool = False, instance_name: str = "",
                 **npu_only_kwargs):
        self.verbose = verbose
        self.n_perf_iters = n_perf_iters
        self.n_warmup_iters = n_warmup_iters
        self.perf_flops = perf_flops
        self.report_precision = report_precision
        self.instance_name = instance_name
        self.ignored_kwargs = dict(npu_only_kwargs)
        self.last_latency_us: Optional[float] = None
        self.last_outputs: List[np.ndarray] = []

    def run_test(self, mlir_module, inputs: Sequence[np.ndarray], expected_outputs: Sequence[np.ndarray] = (),
                 stochastic_expected_outputs: Sequence = (), rtol: float = 1e-3, atol: float = 1e-8,
                 max_mismatch_percentage: float = 0, min_correlation: Optional[float] = None,
                 max_rel_l2: Optional[float] = None) -> int:
        """The reference's acceptance rule (rtol / atol / mismatch budget / correlation floor) and, with
        `max_rel_l2`, this library's own bound on |actual - expected| / |expected| per float output."""
        if stochastic_expected_outputs:
            raise AwqBackendError("stochastic_expected_outputs is not used by the int4-AWQ examples")
        if not expected_outputs:
            raise AwqBackendError("expected_outputs must not be empty")
        backend = B200Backend(verbose=self.verbose, n_perf_iters=self.n_perf_iters,
                              n_warmup_iters=self.n_warmup_iters, instance_name=self.instance_name)
        placeholders = [np.zeros(o.shape, o.dtype) for o in expected_outputs]
        invoker = backend.load(backend.compile(mlir_module))
        actual = invoker(*list(inputs), *placeholders)
        self.last_latency_us = backend.last_latency_us
        if self.n_perf_iters > 0 and self.last_latency_us is not None:
            line = f"Latency (us): {self.last_latency_us:.1f}"
            if self.perf_flops is not None:
                line += f" | Throughput: {self.perf_flops / (self.last_latency_us * 1e-6) / 1e9:.6e} GFLOP/s"
            print(line)
        backend.unload()
        self.last_outputs = list(actual[len(inputs):])
        ok = self._check_outputs(self.last_outputs, list(expected_outputs), rtol, atol, max_mismatch_percentage,
                                 min_correlation, max_rel_l2)
        print("PASS!" if ok else "failed.")
        return 0 if ok else -1

    def _check_outputs(self, actual_outputs, expected_outputs, rtol, atol, max_mismatch_percentage, min_correlation,
                       max_rel_l2=None):
        """Same acceptance rule as xrt_runner.py:423-521: float outputs by np.isclose on f64 with a
        mismatch budget and an optional Pearson-correlation floor; integer outputs exactly.  Also
        prints the rel-L2 error, which is what this library's own tests bound."""
        if len(actual_outputs) != len(expected_outputs):
            raise AwqBackendError("number of outputs differs from number of expected outputs")
        ok = True
        for i, (act, exp) in enumerate(zip(actual_outputs, expected_outputs)):
            act = np.reshape(act, exp.shape)
            if exp.dtype in (np.float16, np.float32, np.float64, bfloat16):
                a, e = act.astype(np.float64), exp.astype(np.float64)
                bad = ~np.isclose(a, e, rtol=rtol, atol=atol)
                allowed = int(e.size * max_mismatch_percentage / 100)
                rel_l2 = float(np.linalg.norm(a - e) / max(np.linalg.norm(e), 1e-30))
                print(f"Output {i}: rel-L2 {rel_l2:.3e}, {int(bad.sum())} / {e.size} outside rtol={rtol} atol={atol}")
                if max_rel_l2 is not None and not rel_l2 <= max_rel_l2:
                    ok = False
                    print(f"ERROR: Output {i} rel-L2 {rel_l2:.3e} exceeds {max_rel_l2:g}")
                if self.report_precision:
                    err = np.abs(a - e)
                    print(f"[precision] Output {i} ({err.size} elements): mean_rel_L1={err.mean() / (np.abs(e).mean() + 1e-30):.3e}"
                          f" | rel_err max={(err / (np.abs(e) + 1e-30)).max():.3e} | abs_err max={err.max():.3e}")
                if bad.sum() > allowed:
                    ok = False
                    print(f"ERROR: Output {i} does not meet expected output.")
                    for idx in list(zip(*np.where(bad)))[:20]:
                        print(f"  Index {idx}: expected={e[idx]}, actual={a[idx]}, diff={abs(a[idx] - e[idx])}")
                if min_correlation is not None and e.size > 0:
                    corr = float(np.corrcoef(a.ravel(), e.ravel())[0, 1])
                    print(f"Output {i} correlation: {corr:.6f} (threshold: {min_correlation})")
                    if not np.isfinite(corr) or corr < min_correlation:
                        ok = False
                        print(f"ERROR: Output {i} correlation {corr:.6f} below threshold {min_correlation}")
            elif not np.array_equal(act, exp):
                ok = False
                print(f"ERROR: Output {i} does not meet expected output ({int((act != exp).sum())} mismatches).")
        return ok


# drop-in names for scripts written against the reference
XRTRunner = B200Runner
XRTBackend = B200Backend
