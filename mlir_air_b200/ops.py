"""Device-level operators: torch CUDA tensors in, torch CUDA tensors out, every one a
single call into the C ABI on torch's current stream.  torch is used for device
memory and streams only; no operator here has a PyTorch implementation."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from . import _lib


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _want(t: torch.Tensor, dtype, name: str):
    if not t.is_cuda:
        raise _lib.AwqBackendError(f"{name} must be a CUDA tensor")
    if t.dtype != dtype:
        raise _lib.AwqBackendError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise _lib.AwqBackendError(f"{name} must be contiguous")
    return t


@dataclass
class AwqWeight:
    """One AWQ-quantised linear layer in HF AutoAWQ layout (layout A), resident on a GPU.

    qweight int32 [K, N/8], qzeros int32 [K/gs, N/8], scales bf16 [K/gs, N].
    """
    qweight: torch.Tensor
    qzeros: torch.Tensor
    scales: torch.Tensor
    group_size: int = 128

    def __post_init__(self):
        _want(self.qweight, torch.int32, "qweight")
        _want(self.qzeros, torch.int32, "qzeros")
        _want(self.scales, torch.bfloat16, "scales")
        K, nb = self.qweight.shape
        if self.qzeros.shape != (K // self.group_size, nb) or self.scales.shape != (K // self.group_size, nb * 8):
            raise _lib.AwqBackendError(
                f"qzeros {tuple(self.qzeros.shape)} / scales {tuple(self.scales.shape)} do not match "
                f"qweight {tuple(self.qweight.shape)} with group size {self.group_size}")

    @property
    def K(self):
        return self.qweight.shape[0]

    @property
    def N(self):
        return self.qweight.shape[1] * 8

    @property
    def nbytes(self):
        return sum(t.numel() * t.element_size() for t in (self.qweight, self.qzeros, self.scales))

    @classmethod
    def from_numpy(cls, qweight, qzeros, scales, group_size=128, device="cuda"):
        """Host arrays (scales bf16 as ml_dtypes.bfloat16, or fp16/fp32 rounded to bf16 as
        awq_repacker.py:74-78 does) -> device-resident weight."""
        import numpy as np
        from ml_dtypes import bfloat16
        s = np.ascontiguousarray(np.asarray(scales).astype(bfloat16)).view(np.int16)
        return cls(torch.from_numpy(np.ascontiguousarray(qweight, dtype=np.int32)).to(device),
                   torch.from_numpy(np.ascontiguousarray(qzeros, dtype=np.int32)).to(device),
                   torch.from_numpy(s).to(device).view(torch.bfloat16), group_size)


class Workspace:
    """Caller-owned scratch for the decode kernels (strip counters + split-K partials).
    One per stream: calls that share a workspace must not overlap on the GPU."""

    def __init__(self, K: int, N: int, device="cuda", batch: int = 64):
        self.nbytes = int(_lib.load().awq_b200_workspace_bytes(int(batch), int(K), int(N)))
        self.buf = torch.empty(self.nbytes, dtype=torch.uint8, device=device)
        with torch.cuda.device(self.buf.device):
            _lib.call("awq_b200_workspace_init", self.buf.data_ptr(), self.nbytes, _stream())

    def fits(self, K, N, batch=64):
        return int(_lib.load().awq_b200_workspace_bytes(int(batch), int(K), int(N))) <= self.nbytes

    def check(self):
        """Synchronise and raise if a device-side wait timed out."""
        with torch.cuda.device(self.buf.device):
            _lib.call("awq_b200_workspace_check", self.buf.data_ptr(), _stream())


ACT_BF16, ACT_F16, OUT_F32 = 0, 1, 2


def _act_dtype(f16: bool):
    return torch.float16 if f16 else torch.bfloat16


def set_decode_kernel(mode: str):
    """"auto", "generic", "streamk" (fp16 activation path) or "streamk_bf16" (bf16 activations as they are)."""
    _lib.call("awq_b200_set_decode_kernel", {"auto": 0, "generic": 1, "streamk": 2, "streamk_bf16": 3}[mode])


def set_deterministic(on: bool):
    """Kept for callers of earlier versions; a no-op: split-K partials are summed as integers, so every result is
    bit-reproducible already."""
    _lib.call("awq_b200_set_deterministic", 1 if on else 0)


def set_gemm_kernel(mode: str):
    _lib.call("awq_b200_set_gemm_kernel", {"auto": 0, "generic": 1, "tc": 2, "tm": 3}[mode])


def dequant(w: AwqWeight, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """bf16 [K, N] = (q - z) * s, bit-exact with awq_repacker.dequant_to_bf16."""
    if out is None:
        out = torch.empty((w.K, w.N), dtype=torch.bfloat16, device=w.qweight.device)
    _want(out, torch.bfloat16, "out")
    _lib.call("awq_b200_dequant_bf16", _ptr(w.qweight), _ptr(w.qzeros), _ptr(w.scales), _ptr(out), w.K, w.N,
              w.group_size, _stream())
    return out


def dequant_1d(packed_q, scales, zeros, n, group_size, out=None):
    if out is None:
        out = torch.empty(n, dtype=torch.bfloat16, device=packed_q.device)
    _lib.call("awq_b200_dequant_1d_bf16", _ptr(_want(packed_q, torch.uint8, "packed_q")),
              _ptr(_want(scales, torch.bfloat16, "scales")), _ptr(_want(zeros, torch.uint8, "zeros")), _ptr(out),
              int(n), int(group_size), _stream())
    return out


def _x2d(x, K, f16=False):
    _want(x, _act_dtype(f16), "x")
    if x.dim() == 1:
        x = x.view(1, -1)
    if x.dim() != 2 or x.shape[1] != K:
        raise _lib.AwqBackendError(f"x must be [B, {K}], got {tuple(x.shape)}")
    return x


def gemv(x, w: AwqWeight, ws: Workspace, residual=None, out=None, f32_out=False, x_f16=False):
    """y [B, N] = x [B, K] @ W (+ residual); bf16 with one rounding, or the f32 partial.
    x is bf16, or fp16 (the library's internal activation format) with x_f16."""
    x = _x2d(x, w.K, x_f16)
    B = x.shape[0]
    if out is None:
        out = torch.empty((B, w.N), dtype=torch.float32 if f32_out else torch.bfloat16, device=x.device)
    if f32_out and residual is not None:
        raise _lib.AwqBackendError("f32 partial output takes no residual")
    if residual is not None:
        _want(residual, torch.bfloat16, "residual")
    _want(out, torch.float32 if f32_out else torch.bfloat16, "out")
    _lib.call("awq_b200_gemv_act", _ptr(x), ACT_F16 if x_f16 else ACT_BF16, _ptr(w.qweight), _ptr(w.qzeros),
              _ptr(w.scales), _ptr(residual), _ptr(out), 1 if f32_out else 0, B, w.K, w.N, w.group_size, _ptr(ws.buf),
              ws.nbytes, _stream())
    return out


def gateup_swiglu(x, w_gateup: AwqWeight, ws: Workspace, out=None, x_f16=False, out_f16=False):
    """out [B, I] = silu(gate) * up for a gate/up-interleaved [K, 2I] weight."""
    x = _x2d(x, w_gateup.K, x_f16)
    B, I = x.shape[0], w_gateup.N // 2
    if out is None:
        out = torch.empty((B, I), dtype=_act_dtype(out_f16), device=x.device)
    _lib.call("awq_b200_gateup_swiglu_act", _ptr(x), ACT_F16 if x_f16 else ACT_BF16, _ptr(w_gateup.qweight),
              _ptr(w_gateup.qzeros), _ptr(w_gateup.scales), _ptr(_want(out, _act_dtype(out_f16), "out")),
              ACT_F16 if out_f16 else ACT_BF16, B, w_gateup.K, I, w_gateup.group_size, _ptr(ws.buf), ws.nbytes, _stream())
    return out


def interleave_gate_up(gate: AwqWeight, up: AwqWeight) -> AwqWeight:
    """Two [K, I] weights -> one [K, 2I] weight with column 2i = gate_i, 2i+1 = up_i."""
    if (gate.K, gate.N, gate.group_size) != (up.K, up.N, up.group_size):
        raise _lib.AwqBackendError("gate and up must have the same shape and group size")
    K, I, G = gate.K, gate.N, gate.K // gate.group_size
    dev = gate.qweight.device
    qw = torch.empty((K, 2 * I // 8), dtype=torch.int32, device=dev)
    qz = torch.empty((G, 2 * I // 8), dtype=torch.int32, device=dev)
    sc = torch.empty((G, 2 * I), dtype=torch.bfloat16, device=dev)
    _lib.call("awq_b200_interleave_gate_up", _ptr(gate.qweight), _ptr(gate.qzeros), _ptr(gate.scales),
              _ptr(up.qweight), _ptr(up.qzeros), _ptr(up.scales), _ptr(qw), _ptr(qz), _ptr(sc), K, I,
              gate.group_size, _stream())
    return AwqWeight(qw, qz, sc, gate.group_size)


def rmsnorm(x, gamma, eps=1e-5, out=None, out_f16=False):
    _want(x, torch.bfloat16, "x")
    x2 = x.view(1, -1) if x.dim() == 1 else x
    if out is None:
        out = torch.empty(x2.shape, dtype=_act_dtype(out_f16), device=x.device)
    _lib.call("awq_b200_rmsnorm_act", _ptr(x2), _ptr(_want(gamma, torch.bfloat16, "gamma")), float(eps),
              _ptr(_want(out, _act_dtype(out_f16), "out")), ACT_F16 if out_f16 else ACT_BF16, x2.shape[0], x2.shape[1],
              _stream())
    return out


def add_rmsnorm(h, partial_sum, gamma=None, eps=1e-5, h_out=None, normed=None, normed_f16=False):
    """h_out = bf16(h + partial_sum); normed = rmsnorm(h_out, gamma) when gamma is given."""
    _want(h, torch.bfloat16, "h")
    _want(partial_sum, torch.float32, "partial_sum")
    if h_out is None:
        h_out = torch.empty_like(h)
    if gamma is not None and normed is None:
        normed = torch.empty(h.shape, dtype=_act_dtype(normed_f16), device=h.device)
    _lib.call("awq_b200_add_rmsnorm_act", _ptr(h), _ptr(partial_sum), _ptr(gamma), float(eps), _ptr(h_out),
              _ptr(normed), ACT_F16 if normed_f16 else ACT_BF16, h.shape[0], h.shape[1], _stream())
    return h_out, normed


def ffn_decode(x, w_gateup: AwqWeight, w_down: AwqWeight, ws: Workspace, gamma=None, eps=1e-5, residual=None,
               normed=None, inter=None, out=None):
    """out [B, H] = down(swiglu(gateup . norm(x))) (+ residual): one C-ABI call, three kernels.
    `normed` and `inter` are 16-bit scratch (the library keeps its intermediates there as fp16)."""
    x = _x2d(x, w_gateup.K)
    B, H, I = x.shape[0], w_gateup.K, w_gateup.N // 2
    if w_down.K != I or w_down.N != H:
        raise _lib.AwqBackendError(f"down weight must be [{I}, {H}], got [{w_down.K}, {w_down.N}]")
    dev = x.device
    if gamma is not None and normed is None:
        normed = torch.empty((B, H), dtype=torch.float16, device=dev)
    if inter is None:
        inter = torch.empty((B, I), dtype=torch.float16, device=dev)
    if out is None:
        out = torch.empty((B, H), dtype=torch.bfloat16, device=dev)
    _lib.call("awq_b200_ffn_decode_bf16", _ptr(x), _ptr(gamma), float(eps), _ptr(w_gateup.qweight),
              _ptr(w_gateup.qzeros), _ptr(w_gateup.scales), _ptr(w_down.qweight), _ptr(w_down.qzeros),
              _ptr(w_down.scales), _ptr(residual), _ptr(normed), _ptr(inter), _ptr(out), B, H, I, w_gateup.group_size,
              _ptr(ws.buf), ws.nbytes, _stream())
    return out


def gemv_f32_push(x, w: AwqWeight, ws: Workspace, peers, slot: int, x_f16=False):
    """This rank's f32 partial x @ w written to its send slot, every rank signalled
    (`peers`: mlir_air_b200.peer.PeerBuffers); B <= 8."""
    x = _x2d(x, w.K, x_f16)
    _lib.call("awq_b200_gemv_f32_push", _ptr(x), ACT_F16 if x_f16 else ACT_BF16, _ptr(w.qweight), _ptr(w.qzeros),
              _ptr(w.scales), peers.local_send(slot), x.shape[0], w.K, w.N, w.group_size, peers.flag_array(slot),
              peers.world, peers.rank, _ptr(ws.buf), ws.nbytes, _stream())


def tp_reduce_add_rmsnorm(h, peers, slot: int, ws: Workspace, gamma=None, eps=1e-5, h_out=None, normed=None,
                          normed_f16=False):
    """Wait for every rank's partial in `slot`, h_out = bf16(h + sum of the partials in rank order),
    and with gamma the RMSNorm of h_out."""
    _want(h, torch.bfloat16, "h")
    if h_out is None:
        h_out = torch.empty_like(h)
    if gamma is not None and normed is None:
        normed = torch.empty(h.shape, dtype=_act_dtype(normed_f16), device=h.device)
    _lib.call("awq_b200_tp_reduce_add_rmsnorm_act", _ptr(h), peers.send_array(slot), peers.local_flags(slot),
              peers.world, _ptr(gamma), float(eps), _ptr(h_out), _ptr(normed), ACT_F16 if normed_f16 else ACT_BF16,
              h.shape[0], h.shape[1], _ptr(ws.buf), _stream())
    return h_out, normed


class FFNStackPlan:
    """Tensor maps of a decode FFN layer stack in device memory, for ffn_stack_decode.
    `gateups`, `downs`: one AwqWeight per layer (gate/up interleaved [H, 2I], down [I, H]);
    `gammas`: one bf16 [H] tensor per layer.  Keeps references to the weights it describes."""

    def __init__(self, gateups: Sequence[AwqWeight], downs: Sequence[AwqWeight], gammas: Sequence[torch.Tensor]):
        import ctypes
        n = len(gateups)
        if n == 0 or len(downs) != n or len(gammas) != n:
            raise _lib.AwqBackendError("FFNStackPlan: one gate/up weight, one down weight and one gamma per layer")
        self.n_layers = n
        self.H, self.I, self.group_size = gateups[0].K, gateups[0].N // 2, gateups[0].group_size
        for gu, d, g in zip(gateups, downs, gammas):
            if (gu.K, gu.N, d.K, d.N, gu.group_size, d.group_size) != (self.H, 2 * self.I, self.I, self.H, self.group_size,
                                                                         self.group_size):
                raise _lib.AwqBackendError("FFNStackPlan: all layers must have the same shape and group size")
            _want(g, torch.bfloat16, "gamma")
            if g.numel() != self.H:
                raise _lib.AwqBackendError(f"FFNStackPlan: gamma must have {self.H} elements")
        self._keep = (list(gateups), list(downs), list(gammas))
        dev = gateups[0].qweight.device
        lib = _lib.load()
        self.nbytes = int(lib.awq_b200_ffn_stack_plan_bytes(n))
        self.buf = torch.empty(self.nbytes + 128, dtype=torch.uint8, device=dev)
        self.ptr = (self.buf.data_ptr() + 127) // 128 * 128
        arr = ctypes.c_void_p * n

        def ptrs(ts):
            return arr(*[t.data_ptr() for t in ts])

        with torch.cuda.device(dev):
            _lib.call("awq_b200_ffn_stack_plan", self.ptr, self.nbytes, n, ptrs([w.qweight for w in gateups]),
                      ptrs([w.qzeros for w in gateups]), ptrs([w.scales for w in gateups]), ptrs([w.qweight for w in downs]),
                      ptrs([w.qzeros for w in downs]), ptrs([w.scales for w in downs]), ptrs(list(gammas)), self.H, self.I,
                      self.group_size)

    def workspace_bytes(self) -> int:
        return int(_lib.load().awq_b200_ffn_stack_workspace_bytes(self.n_layers))


def set_ffn_stack_tuning(lookahead_units: int = -1, split_per_1024: int = -1):
    """Tuning of the one-launch stack kernel (negative = keep): units per half-CTA prefetched into
    L2 ahead of the ring; and 0 = a down unit waits for the whole gate/up phase, other = only for the
    sub-strips that produce its inputs (the default)."""
    _lib.call("awq_b200_set_ffn_stack_tuning", int(lookahead_units), int(split_per_1024))


def ffn_stack_decode(plan: FFNStackPlan, x, ws: Workspace, eps=1e-5, inter=None, out=None):
    """out [B, H] = the whole layer stack applied to x [B <= 8, H], ONE kernel launch."""
    x = _x2d(x, plan.H)
    B = x.shape[0]
    if inter is None:
        inter = torch.empty((B, plan.I), dtype=torch.float16, device=x.device)
    if out is None:
        out = torch.empty((B, plan.H), dtype=torch.bfloat16, device=x.device)
    _want(out, torch.bfloat16, "out")
    if inter.numel() < B * plan.I or inter.element_size() != 2:
        raise _lib.AwqBackendError("ffn_stack_decode: inter must hold B * I 16-bit elements")
    _lib.call("awq_b200_ffn_stack_decode_bf16", plan.ptr, plan.n_layers, _ptr(x), _ptr(out), _ptr(inter), float(eps), B,
              plan.H, plan.I, plan.group_size, _ptr(ws.buf), ws.nbytes, _stream())
    return out


def ffn_stack_tp_slot_bytes(H: int, n_ranks: int) -> int:
    return int(_lib.load().awq_b200_ffn_stack_tp_slot_bytes(int(H), int(n_ranks)))


def ffn_stack_decode_tp(plan: FFNStackPlan, x, ws: Workspace, peers, eps=1e-5, inter=None, out=None):
    """The one-launch stack on this rank's shards, with the partials exchanged through `peers`
    (mlir_air_b200.peer.PeerBuffers with two slots of ffn_stack_tp_slot_bytes(H, world) bytes, used by
    nothing else and always with the same number of layers)."""
    x = _x2d(x, plan.H)
    B = x.shape[0]
    if inter is None:
        inter = torch.empty((B, plan.I), dtype=torch.float16, device=x.device)
    if out is None:
        out = torch.empty((B, plan.H), dtype=torch.bfloat16, device=x.device)
    _want(out, torch.bfloat16, "out")
    if inter.numel() < B * plan.I or inter.element_size() != 2:
        raise _lib.AwqBackendError("ffn_stack_decode_tp: inter must hold B * I 16-bit elements")
    _lib.call("awq_b200_ffn_stack_decode_tp_bf16", plan.ptr, plan.n_layers, _ptr(x), _ptr(out), _ptr(inter), float(eps), B,
              plan.H, plan.I, plan.group_size, peers.base_array(), peers.stride, peers.recv_bytes, peers.world, peers.rank,
              _ptr(ws.buf), ws.nbytes, _stream())
    return out


def gemm(A, w: AwqWeight, out=None, residual=None, swiglu=False):
    """C [M, N] = A [M, K] @ W, f32 accumulate, bf16 out (prefill).  With `residual` [M, N] the sum is
    bf16(acc + residual); with `swiglu` W is gate/up-interleaved and C is [M, N/2]."""
    _want(A, torch.bfloat16, "A")
    if A.dim() != 2 or A.shape[1] != w.K:
        raise _lib.AwqBackendError(f"A must be [M, {w.K}], got {tuple(A.shape)}")
    if residual is not None or swiglu:
        n_out = w.N // 2 if swiglu else w.N
        if out is None:
            out = torch.empty((A.shape[0], n_out), dtype=torch.bfloat16, device=A.device)
        _want(out, torch.bfloat16, "out")
        if residual is not None:
            _want(residual, torch.bfloat16, "residual")
        _lib.call("awq_b200_gemm_fused_bf16", _ptr(A), _ptr(w.qweight), _ptr(w.qzeros), _ptr(w.scales), _ptr(residual),
                  _ptr(out), 1 if swiglu else 0, A.shape[0], w.K, w.N, w.group_size, _stream())
        return out
    if out is None:
        out = torch.empty((A.shape[0], w.N), dtype=torch.bfloat16, device=A.device)
    _lib.call("awq_b200_gemm_bf16", _ptr(A), _ptr(w.qweight), _ptr(w.qzeros), _ptr(w.scales), _ptr(out), A.shape[0],
              w.K, w.N, w.group_size, _stream())
    return out


class GemmDecodeWorkspace:
    """Caller-owned scratch of `gemm_decode` (the f32 sums of each SM's share of a tile) for up to `batch` rows and `N`
    columns.  One per stream: calls that share it must not overlap on the GPU."""

    def __init__(self, N: int, device="cuda", batch: int = 64, K: int = 0):
        """`K` > 0 also makes room for the split token rows of `gemm_decode(..., f8=True)` (up to 32 rows of K elements)."""
        self.batch, self.N, self.K = int(batch), int(N), int(K)
        lib = _lib.load()
        self.nbytes = int(lib.awq_b200_gemm_decode_workspace_bytes(self.batch, self.N))
        if self.K > 0:
            self.nbytes = max(self.nbytes, int(lib.awq_b200_gemm_decode_f8_workspace_bytes(min(self.batch, 32), self.K, self.N)))
        self.buf = torch.empty(self.nbytes, dtype=torch.uint8, device=device)

    def fits(self, M, N):
        return int(_lib.load().awq_b200_gemm_decode_workspace_bytes(int(M), int(N))) <= self.nbytes

    def fits_f8(self, M, K, N):
        return int(M) <= 32 and 0 < int(_lib.load().awq_b200_gemm_decode_f8_workspace_bytes(int(M), int(K), int(N))) <= self.nbytes


def gemm_decode(A, w: AwqWeight, ws: GemmDecodeWorkspace, out=None, residual=None, swiglu=False, f32_out=False, out_f16=False,
                f8=False):
    """C [M, N] = A [M, K] @ W for a decode batch of M <= 64 rows (weights streamed once, all SMs busy whatever the
    shape); `residual` / `swiglu` as in `gemm`; `f32_out`: the f32 sums themselves (a tensor-parallel partial).
    A may be bf16 or fp16 (the weights are then dequantised to fp16 too: 11 significant bits instead of 8);
    `out_f16` stores a plain or SwiGLU result as fp16 for a following fp16 product.  `f8` (up to 32 rows): the kernel that
    feeds the tensor core the packed nibbles and split token rows as fp8 and applies zero point and scale in f32."""
    if A.dtype not in (torch.bfloat16, torch.float16):
        raise _lib.AwqBackendError(f"A must be bf16 or fp16, got {A.dtype}")
    _want(A, A.dtype, "A")
    if A.dim() != 2 or A.shape[1] != w.K:
        raise _lib.AwqBackendError(f"A must be [M, {w.K}], got {tuple(A.shape)}")
    if f32_out and (residual is not None or swiglu or out_f16):
        raise _lib.AwqBackendError("gemm_decode: f32_out takes neither residual, swiglu nor out_f16")
    if out_f16 and residual is not None:
        raise _lib.AwqBackendError("gemm_decode: the residual add goes with a bf16 output")
    dt = torch.float32 if f32_out else _act_dtype(out_f16)
    if out is None:
        out = torch.empty((A.shape[0], w.N // 2 if swiglu else w.N), dtype=dt, device=A.device)
    _want(out, dt, "out")
    if residual is not None:
        _want(residual, torch.bfloat16, "residual")
    _lib.call("awq_b200_gemm_decode_f8" if f8 else "awq_b200_gemm_decode_act", _ptr(A), ACT_F16 if A.dtype == torch.float16 else ACT_BF16, _ptr(w.qweight),
              _ptr(w.qzeros), _ptr(w.scales), _ptr(residual), _ptr(out), OUT_F32 if f32_out else (ACT_F16 if out_f16 else ACT_BF16),
              1 if swiglu else 0, A.shape[0], w.K, w.N, w.group_size, _ptr(ws.buf), ws.nbytes, _stream())
    return out


def rope_halfsplit(x, lut, n_heads: int, head_dim: int, out=None):
    """Half-split RoPE of x [B, >= n_heads * head_dim] (a column slice of a wider projection output
    is fine: the row stride is passed on) with one LUT row [cos | sin] per token; in place by default."""
    _want(lut, torch.bfloat16, "lut")
    if out is None:
        out = x
    for name, t in (("x", x), ("out", out)):
        if not t.is_cuda or t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1 or \
                t.shape[1] < n_heads * head_dim:
            raise _lib.AwqBackendError(f"rope: {name} must be a CUDA bf16 [B, >= n_heads * head_dim] tensor with unit "
                                       "column stride")
    if out.shape[0] != x.shape[0] or lut.shape != (x.shape[0], head_dim):
        raise _lib.AwqBackendError(f"rope: out must have {x.shape[0]} rows and lut must be [{x.shape[0]}, {head_dim}]")
    # the stride of a one-row tensor is arbitrary (0 after numpy's None indexing): it is never used
    xs = x.stride(0) if x.shape[0] > 1 else n_heads * head_dim
    os_ = out.stride(0) if out.shape[0] > 1 else n_heads * head_dim
    _lib.call("awq_b200_rope_halfsplit_bf16", x.data_ptr(), xs, _ptr(lut), out.data_ptr(), os_, x.shape[0], n_heads,
              head_dim, _stream())
    return out


def linear_bf16(x, W, out=None):
    """y [M, N] = x [M, K] @ W[N, K]^T with un-quantised bf16 weights (the bf16 sibling path)."""
    _want(x, torch.bfloat16, "x")
    _want(W, torch.bfloat16, "W")
    x2 = x.view(1, -1) if x.dim() == 1 else x
    if out is None:
        out = torch.empty((x2.shape[0], W.shape[0]), dtype=torch.bfloat16, device=x.device)
    _lib.call("awq_b200_linear_bf16", _ptr(x2), _ptr(W), _ptr(out), x2.shape[0], x2.shape[1], W.shape[0], _stream())
    return out


def silu_mul(gate, up, out=None):
    """out = silu(gate) * up elementwise (bf16 in, f32 math, bf16 out)."""
    if out is None:
        out = torch.empty_like(gate)
    _lib.call("awq_b200_silu_mul_bf16", _ptr(_want(gate, torch.bfloat16, "gate")), _ptr(_want(up, torch.bfloat16, "up")),
              _ptr(out), gate.numel(), _stream())
    return out


def gemm_check():
    """Synchronise and raise if the tensor-core GEMM reported a device-side timeout."""
    _lib.call("awq_b200_gemm_check", _stream())


def repack_B_to_A(A_q, A_s, A_z, group_size=128) -> AwqWeight:
    """mlir-air logical layout (A_q u8 [M, K/2], A_s bf16 [G, M], A_z u8 [G, M]) -> layout A."""
    M, K = A_q.shape[0], A_q.shape[1] * 2
    G = K // group_size
    dev = A_q.device
    qw = torch.empty((K, M // 8), dtype=torch.int32, device=dev)
    qz = torch.empty((G, M // 8), dtype=torch.int32, device=dev)
    sc = torch.empty((G, M), dtype=torch.bfloat16, device=dev)
    _lib.call("awq_b200_repack_B_to_A", _ptr(_want(A_q, torch.uint8, "A_q")), _ptr(_want(A_s, torch.bfloat16, "A_s")),
              _ptr(_want(A_z, torch.uint8, "A_z")), _ptr(qw), _ptr(qz), _ptr(sc), M, K, group_size, _stream())
    return AwqWeight(qw, qz, sc, group_size)


def repack_A_to_B(w: AwqWeight):
    M, K, G = w.N, w.K, w.K // w.group_size
    dev = w.qweight.device
    A_q = torch.empty((M, K // 2), dtype=torch.uint8, device=dev)
    A_s = torch.empty((G, M), dtype=torch.bfloat16, device=dev)
    A_z = torch.empty((G, M), dtype=torch.uint8, device=dev)
    _lib.call("awq_b200_repack_A_to_B", _ptr(w.qweight), _ptr(w.qzeros), _ptr(w.scales), _ptr(A_q), _ptr(A_s),
              _ptr(A_z), M, K, w.group_size, _stream())
    return A_q, A_s, A_z


def repack_C_to_B(packed, M: int, K: int, group_size=128, m_tile=8, k_chunk=2048):
    """Per-tile packed buffer (uint8, tiles in (row block, k chunk) order: the reference's NPU layout
    for the GEMV and, with M = N and m_tile = N_TILE, for the GEMM) -> layout B on the device."""
    _want(packed, torch.uint8, "packed")
    G = K // group_size
    tile = m_tile * (k_chunk // 2) + 3 * (k_chunk // group_size) * m_tile
    if packed.numel() != (M // m_tile) * (K // k_chunk) * tile:
        raise _lib.AwqBackendError(f"packed buffer has {packed.numel()} bytes, expected {(M // m_tile) * (K // k_chunk)} "
                                   f"tiles of {tile}")
    dev = packed.device
    A_q = torch.empty((M, K // 2), dtype=torch.uint8, device=dev)
    A_s = torch.empty((G, M), dtype=torch.bfloat16, device=dev)
    A_z = torch.empty((G, M), dtype=torch.uint8, device=dev)
    _lib.call("awq_b200_repack_C_to_B", _ptr(packed), _ptr(A_q), _ptr(A_s), _ptr(A_z), M, K, group_size, m_tile, k_chunk,
              _stream())
    return A_q, A_s, A_z


def repack_C_to_A(packed, M: int, K: int, group_size=128, m_tile=8, k_chunk=2048) -> AwqWeight:
    """Per-tile packed buffer -> resident layout-A weight (two device passes, once per weight)."""
    return repack_B_to_A(*repack_C_to_B(packed, M, K, group_size, m_tile, k_chunk), group_size)
