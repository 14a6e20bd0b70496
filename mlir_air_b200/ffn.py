"""Weight-resident decode FFN layers and stacks, single GPU or tensor-parallel.

The reference keeps the weights of every layer resident in device buffers and only
moves activations per token (`KernelCache.load_and_run` with `static_input_indices`,
programming_examples/llms/shared/infra/cache.py:494-737); a layer is the LGU -> LD chain
of llms/llama32_1b_int4/multi_launch_builder/o_gemv_ffn_int4_multi.py:9-12:

    h <- bf16(h + down(swiglu(gateup . rmsnorm(h, gamma))))

Tensor parallelism follows the reference's output-row split across cores
(matvec_int4_packed.py:69-75) lifted to GPUs: gate/up is split over its output columns,
down over its input rows (group-of-128 granularity, uneven when the group count does not
divide), and the per-rank f32 partials of down are summed with one allreduce per layer.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import ops
from ._lib import AwqBackendError
from .ops import AwqWeight, Workspace


def tp_shard_bounds(intermediate: int, tp: int, group_size: int = 128) -> List[Tuple[int, int]]:
    """[i0, i1) of the intermediate dimension owned by each rank: whole quantisation groups,
    as even as possible (the first `groups % tp` ranks get one more group)."""
    if intermediate % group_size:
        raise AwqBackendError(f"intermediate {intermediate} is not a multiple of the group size {group_size}")
    groups = intermediate // group_size
    if tp < 1 or tp > groups:
        raise AwqBackendError(f"cannot split {groups} groups over {tp} ranks")
    base, extra = divmod(groups, tp)
    bounds, g0 = [], 0
    for r in range(tp):
        g1 = g0 + base + (1 if r < extra else 0)
        bounds.append((g0 * group_size, g1 * group_size))
        g0 = g1
    return bounds


def slice_gateup(qweight, qzeros, scales, i0: int, i1: int):
    """Columns [2 i0, 2 i1) of gate/up-interleaved [K, 2I] tensors (a column-parallel shard).
    Works on numpy arrays and on torch tensors."""
    if i0 % 4 or i1 % 4:
        raise AwqBackendError("gate/up shard bounds must be multiples of 4")
    return qweight[:, 2 * i0 // 8:2 * i1 // 8], qzeros[:, 2 * i0 // 8:2 * i1 // 8], scales[:, 2 * i0:2 * i1]


def slice_down(qweight, qzeros, scales, i0: int, i1: int, group_size: int = 128):
    """Rows [i0, i1) of [I, H] tensors (a row-parallel shard); bounds on group boundaries."""
    if i0 % group_size or i1 % group_size:
        raise AwqBackendError("down shard bounds must be multiples of the group size")
    return qweight[i0:i1], qzeros[i0 // group_size:i1 // group_size], scales[i0 // group_size:i1 // group_size]


def shard_gateup(w: AwqWeight, i0: int, i1: int) -> AwqWeight:
    return AwqWeight(*(t.contiguous() for t in slice_gateup(w.qweight, w.qzeros, w.scales, i0, i1)), w.group_size)


def shard_down(w: AwqWeight, i0: int, i1: int) -> AwqWeight:
    return AwqWeight(*(t.contiguous() for t in slice_down(w.qweight, w.qzeros, w.scales, i0, i1, w.group_size)),
                     w.group_size)


@dataclass
class FFNLayer:
    """One layer's resident weights (this rank's shard when tensor-parallel)."""
    gateup: AwqWeight            # [H, 2 I_local], gate/up column-interleaved
    down: AwqWeight              # [I_local, H]
    gamma: Optional[torch.Tensor] = None  # RMSNorm weight bf16 [H]

    @property
    def nbytes(self):
        return self.gateup.nbytes + self.down.nbytes


def random_layer(hidden: int, intermediate: int, seed: int, device="cuda", group_size: int = 128,
                 bounds: Optional[Tuple[int, int]] = None, with_gamma: bool = True) -> FFNLayer:
    """Random-init AWQ layer with the benchmark's distributions (nibbles and zeros uniform 0..15,
    scales ~U(0.001, 0.02), gamma ~ 1 + 0.1 N(0,1)), generated on the device.  With `bounds`
    only the [i0, i1) shard of the intermediate dimension is generated."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    i0, i1 = bounds if bounds is not None else (0, intermediate)
    il = i1 - i0

    def rnd(K, N):
        qw = torch.randint(-2 ** 31, 2 ** 31 - 1, (K, N // 8), dtype=torch.int32, device=device, generator=gen)
        qz = torch.randint(-2 ** 31, 2 ** 31 - 1, (K // group_size, N // 8), dtype=torch.int32, device=device,
                           generator=gen)
        s = (torch.rand((K // group_size, N), device=device, generator=gen) * 0.019 + 0.001).to(torch.bfloat16)
        return AwqWeight(qw, qz, s, group_size)

    gamma = None
    if with_gamma:
        gamma = (torch.randn(hidden, device=device, generator=gen) * 0.1 + 1.0).to(torch.bfloat16)
    return FFNLayer(rnd(hidden, 2 * il), rnd(il, hidden), gamma)


def _lib_call_workspace_init(ws: Workspace):
    from . import _lib
    _lib.call("awq_b200_workspace_init", ws.buf.data_ptr(), ws.nbytes, torch.cuda.current_stream().cuda_stream)
    torch.cuda.current_stream().synchronize()


class DecodeFFNStack:
    """A stack of decode FFN layers with resident weights.

    step(h)          device tensor in, device tensor out (eager launches)
    forward_host(x)  host array in, host array out: pinned H2D, one CUDA-graph replay of the
                     whole stack, D2H -- the call a serving loop makes per token batch.
    With `group` (a torch.distributed process group) the layers are this rank's shards and
    each layer ends in one exchange of the f32 down-projection partials: inside the one-launch
    kernel for batches it takes, an allreduce per layer otherwise.  `align_ranks`: the one-launch
    kernels of the ranks wait for one another with a limit of about a second, so a one-element
    allreduce is enqueued in front of each launch (also inside the captured graph); it makes the
    ranks' kernels start together however far apart the host threads are.
    """

    def __init__(self, layers: Sequence[FFNLayer], hidden: int, max_batch: int = 64, eps: float = 1e-5,
                 group=None, device="cuda", fused: bool = True, peer_push: bool = False, align_ranks: bool = True):
        self.layers = list(layers)
        self.hidden = hidden
        self.eps = eps
        self.group = group
        self.device = torch.device(device)
        self.tp = 1 if group is None else torch.distributed.get_world_size(group)
        self.max_batch = max_batch
        maxK = max([hidden] + [l.down.K for l in self.layers])
        maxN = max([hidden] + [l.gateup.N for l in self.layers])
        self.ws = Workspace(maxK, maxN, device=device)
        max_il = max(l.down.K for l in self.layers)
        # split-K sums of the batched-decode GEMM (batches of 9 to 64 rows)
        # (its size grows with N: the widest product decides; K: room for the split token rows of the fp8-operand kernel)
        self.gemm_ws = ops.GemmDecodeWorkspace(maxN, device=device, batch=min(max_batch, 64), K=maxK) \
            if max_batch >= self.GEMM_BATCH else None
        bf = dict(dtype=torch.bfloat16, device=device)
        self._h = [torch.zeros((max_batch, hidden), **bf) for _ in range(2)]  # zeros: a capture's warm-up run reads them
        # intermediates between the kernels of a layer are fp16 (the GEMV kernel's fastest input)
        self._normed = torch.empty((max_batch, hidden), dtype=torch.float16, device=device)
        self._inter = torch.empty((max_batch, max_il), dtype=torch.float16, device=device)
        self._partial = torch.empty((max_batch, hidden), dtype=torch.float32, device=device)
        self._graphs = {}
        # tensor parallel, optional: partials are read from the peers' send buffers (two slots used
        # alternately) instead of going through an allreduce call, for batches the push kernel takes;
        # off by default, NCCL's allreduce measured faster at 2 and 4 ranks
        self.peers = None
        if peer_push and self.tp > 1 and hidden % 128 == 0 and all(l.down.group_size == 128 and l.down.K % 128 == 0
                                                                    for l in self.layers):
            self.peers = self._peer_buffers_or_none(group, 8 * hidden * 4, device)
        # one launch for the whole stack where the fused kernel applies: one GPU, every layer with
        # a norm weight, one shape, group 128, batch <= 8 (larger batches take the per-layer kernels)
        self.plan = None
        self.plan_peers = None
        self._align = torch.zeros(1, dtype=torch.int32, device=device) if align_ranks and self.tp > 1 else None
        if fused and self._fusable():
            self.plan = ops.FFNStackPlan([l.gateup for l in self.layers], [l.down for l in self.layers],
                                         [l.gamma for l in self.layers])
            if self.plan.workspace_bytes() > self.ws.nbytes:
                self.plan = None
            elif self.tp > 1:  # the ranks exchange their partials inside the launch, through these buffers
                self.plan_peers = self._peer_buffers_or_none(group, ops.ffn_stack_tp_slot_bytes(hidden, self.tp), device)
                if self.plan_peers is None:
                    self.plan = None  # every rank falls back to the per-layer kernels + NCCL together
        self._pin_in = torch.empty((max_batch, hidden), dtype=torch.bfloat16).pin_memory() if torch.cuda.is_available() else None
        self._pin_out = torch.empty((max_batch, hidden), dtype=torch.bfloat16).pin_memory() if torch.cuda.is_available() else None

    @staticmethod
    def _peer_buffers_or_none(group, recv_bytes, device):
        """Peer-mapped buffers, or None on EVERY rank if mapping failed on any (the ranks must take the
        same path, so they agree through one allreduce)."""
        import warnings
        from .peer import PeerBuffers
        peers, err = None, None
        try:
            peers = PeerBuffers(group, 2, recv_bytes, device)
        except Exception as e:  # noqa: BLE001 -- whatever the mapping raised, the answer is the NCCL path
            err = e
        ok = torch.tensor([1 if peers is not None else 0], dtype=torch.int32, device=device)
        torch.distributed.all_reduce(ok, op=torch.distributed.ReduceOp.MIN, group=group)
        if int(ok.item()) == 0:
            warnings.warn(f"peer-mapped buffers are not available ({err!r}); tensor-parallel ranks use NCCL per layer")
            return None
        return peers

    def _fusable(self) -> bool:
        l0 = self.layers[0]
        il = l0.down.K
        if l0.gateup.group_size != 128 or self.hidden % 128 or il % 128:
            return False
        for l in self.layers:
            if l.gamma is None or l.gateup.K != self.hidden or l.gateup.N != 2 * il or l.down.K != il or \
                    l.down.N != self.hidden or l.gateup.group_size != 128 or l.down.group_size != 128:
                return False
        return True

    def uses_fused(self, batch: int) -> bool:
        return self.plan is not None and batch <= 8

    # From this batch on one GPU, a layer is two batched-decode tensor-core GEMMs (weights streamed once
    # per layer whatever the batch, SwiGLU / residual in the epilogue) instead of one GEMV pass per 8 rows
    # (9-16 rows: the same time as the two-tile GEMV pass at the 70B dimensions, 9 % less at the 7B ones).
    GEMM_BATCH = 9
    # Up to here the GEMM is the kernel that feeds the tensor core the packed nibbles and split token rows as fp8 (scale and
    # zero point in f32): 10 % faster than the 16-bit-operand kernel at 16 rows, 3 % at 32, and no weight is rounded.
    GEMM_F8_BATCH = 32
    # ... where a layer is large enough for its three launches per product to pay: measured on one box (us per layer,
    # 16-bit against fp8 operands, by weights per layer on this rank): 35 M 21.0 / 22.3 at 16 rows and 24.0 / 27.0 at 32;
    # 88 M 28.6 / 30.9 at 32; 135 M 33.4 / 32.6 and 36.6 / 38.3; 176 M 38.2 / 36.0 and 40.4 / 41.2; 352 M 60.3 / 54.7 and
    # 63.4 / 59.9; 705 M 104.4 / 89.6 and 111.3 / 99.4.
    GEMM_F8_MIN_WEIGHTS = {16: 120e6, 32: 250e6}

    def uses_gemm_f8(self, batch: int) -> bool:
        if not self.uses_gemm(batch) or batch > self.GEMM_F8_BATCH:
            return False
        weights = min(l.gateup.K * l.gateup.N + l.down.K * l.down.N for l in self.layers)
        if weights < self.GEMM_F8_MIN_WEIGHTS[16 if batch <= 16 else 32]:
            return False
        return all(self.gemm_ws.fits_f8(batch, w.K, w.N) for l in self.layers for w in (l.gateup, l.down))

    def uses_gemm(self, batch: int) -> bool:
        if batch < self.GEMM_BATCH or batch > 64 or self.gemm_ws is None:
            return False
        return all(l.gamma is not None and l.gateup.group_size == 128 and l.down.group_size == 128 and
                   l.gateup.K % 128 == 0 and l.down.K % 128 == 0 and l.gateup.N % 32 == 0 and l.down.N % 32 == 0
                   for l in self.layers)

    # kernels launched per step (this library's own), for accounting
    def launches_per_step(self, batch: int) -> int:
        if self.uses_fused(batch):
            return 1
        if self.uses_gemm(batch):
            # norm, and two launches (product, sum of the SMs' shares + epilogue) per GEMM, three with the split of the token
            # rows in front of the fp8-operand kernel; tensor parallel: the norm is fused with the residual add behind the
            # allreduce, plus the first layer's norm
            return (7 if self.uses_gemm_f8(batch) else 5) * len(self.layers) + (1 if self.tp > 1 else 0)
        passes = (batch + 7) // 8  # the decode kernels take 8 rows per launch
        n = len(self.layers)
        if self.tp == 1:
            return n * (1 + 2 * passes)
        return 1 + n * (2 * passes + 1)

    @property
    def weight_bytes(self):
        return sum(l.nbytes for l in self.layers)

    def _run(self, B: int):
        """Enqueue the whole stack on the current stream; input in _h[0][:B], returns the buffer
        holding the result."""
        h, other = self._h[0][:B], self._h[1][:B]
        normed, inter, partial = self._normed[:B], self._inter, self._partial[:B]
        if self.uses_fused(B):
            if self.tp > 1:
                if self._align is not None:
                    torch.distributed.all_reduce(self._align, group=self.group)
                return ops.ffn_stack_decode_tp(self.plan, h, self.ws, self.plan_peers, eps=self.eps, inter=inter, out=other)
            return ops.ffn_stack_decode(self.plan, h, self.ws, eps=self.eps, inter=inter, out=other)
        if self.uses_gemm(B) and self.tp > 1:
            # tensor parallel: gate/up shard -> SwiGLU, down shard -> f32 partial, allreduce, residual add fused with
            # the next layer's norm
            # activations between the kernels are fp16, as in the GEMV path: the products then run on fp16 operands
            f8 = self.uses_gemm_f8(B)
            ops.rmsnorm(h, self.layers[0].gamma, self.eps, out=normed, out_f16=True)
            for idx, l in enumerate(self.layers):
                il = l.down.K
                it = inter.view(-1)[:B * il].view(B, il)
                ops.gemm_decode(normed, l.gateup, self.gemm_ws, out=it, swiglu=True, out_f16=True, f8=f8)
                ops.gemm_decode(it, l.down, self.gemm_ws, out=partial, f32_out=True, f8=f8)
                torch.distributed.all_reduce(partial, group=self.group)
                nxt = self.layers[idx + 1].gamma if idx + 1 < len(self.layers) else None
                ops.add_rmsnorm(h, partial, nxt, self.eps, h_out=other, normed=normed if nxt is not None else None,
                                normed_f16=True)
                h, other = other, h
            return h
        if self.uses_gemm(B):
            f8 = self.uses_gemm_f8(B)
            for l in self.layers:
                il = l.down.K
                it = inter.view(-1)[:B * il].view(B, il)
                ops.rmsnorm(h, l.gamma, self.eps, out=normed, out_f16=True)
                ops.gemm_decode(normed, l.gateup, self.gemm_ws, out=it, swiglu=True, out_f16=True, f8=f8)
                ops.gemm_decode(it, l.down, self.gemm_ws, out=other, residual=h, f8=f8)
                h, other = other, h
            return h
        if self.tp == 1:
            for l in self.layers:
                il = l.down.K
                ops.ffn_decode(h, l.gateup, l.down, self.ws, gamma=l.gamma, eps=self.eps, residual=h,
                               normed=normed, inter=inter.view(-1)[:B * il].view(B, il), out=other)
                h, other = other, h
            return h
        # tensor-parallel: norm of the first layer, then per layer gate/up -> down partial ->
        # allreduce -> residual add fused with the next layer's norm
        x = h
        if self.layers[0].gamma is not None:
            ops.rmsnorm(h, self.layers[0].gamma, self.eps, out=normed, out_f16=True)
            x = normed
        push = self.peers is not None and B <= 8
        for idx, l in enumerate(self.layers):
            il = l.down.K
            it = inter.view(-1)[:B * il].view(B, il)
            ops.gateup_swiglu(x, l.gateup, self.ws, out=it, x_f16=x is normed, out_f16=True)
            nxt = self.layers[idx + 1].gamma if idx + 1 < len(self.layers) else None
            if push:
                ops.gemv_f32_push(it, l.down, self.ws, self.peers, idx & 1, x_f16=True)
                ops.tp_reduce_add_rmsnorm(h, self.peers, idx & 1, self.ws, nxt, self.eps, h_out=other,
                                          normed=normed if nxt is not None else None, normed_f16=True)
            else:
                ops.gemv(it, l.down, self.ws, out=partial, f32_out=True, x_f16=True)
                torch.distributed.all_reduce(partial, group=self.group)
                ops.add_rmsnorm(h, partial, nxt, self.eps, h_out=other, normed=normed if nxt is not None else None,
                                normed_f16=True)
            h, other = other, h
            x = normed if nxt is not None else h
        return h

    def step(self, h: torch.Tensor) -> torch.Tensor:
        """Eager: run the stack on a device tensor [B, H]; returns a new device tensor."""
        B = h.shape[0]
        if B > self.max_batch or h.shape[1] != self.hidden:
            raise AwqBackendError(f"input {tuple(h.shape)} does not fit [<= {self.max_batch}, {self.hidden}]")
        self._h[0][:B].copy_(h)
        return self._run(B).clone()

    def capture(self, B: int):
        """Capture the stack for batch B into a CUDA graph (after one eager warm-up run)."""
        if B in self._graphs:
            return self._graphs[B]
        keep = self._h[0][:B].clone()  # the warm-up run may end in the input buffer
        self._run(B)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out = self._run(B)
        self._h[0][:B].copy_(keep)
        self._graphs[B] = (g, out)
        return self._graphs[B]

    def replay(self, B: int):
        """Replay the captured stack on whatever _h[0][:B] currently holds; returns the result buffer."""
        g, out = self.capture(B)
        g.replay()
        return out

    def load_input(self, h: torch.Tensor):
        self._h[0][:h.shape[0]].copy_(h)

    def forward_host(self, x: np.ndarray) -> np.ndarray:
        """Host [B, H] bf16 (ml_dtypes) in, host [B, H] bf16 out."""
        from ml_dtypes import bfloat16
        B = x.shape[0]
        src = torch.from_numpy(np.ascontiguousarray(x).view(np.int16)).view(torch.bfloat16)
        self._pin_in[:B].copy_(src)
        self._h[0][:B].copy_(self._pin_in[:B], non_blocking=True)
        out = self.replay(B)
        self._pin_out[:B].copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self._pin_out[:B].view(torch.int16).numpy().view(bfloat16).copy()

    def resync(self):
        """Collective, tensor parallel only: after a failed step on any rank, bring the ranks' exchange buffers back to
        the same state (every rank must call it; nothing of this stack may be in flight)."""
        for peers in (self.plan_peers, self.peers):
            if peers is not None:
                peers.reset()
        with torch.cuda.device(self.device):
            _lib_call_workspace_init(self.ws)

    def check(self):
        self.ws.check()
        if self.gemm_ws is not None:
            ops.gemm_check()
