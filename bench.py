#!/usr/bin/env python
"""Headline benchmark: int4-AWQ decode-FFN tokens/s on the Llama-3-70B FFN stack.

    python bench.py --gpus N --steps K --warmup W            # this library, TP = N
    python bench.py --impl reference --gpus N ...            # the numpy golden path on host cores

Workload (the fifth configuration of the benchmark definition): hidden 8192, intermediate 28672, 80 random-init AWQ-int4
layers (group 128, scales ~U(0.001, 0.02)), residual add per layer, batch 8 tokens by default;
TP = N with one allreduce after each down projection.  One step = one pass of the whole stack
over one token batch.  Prints ONE JSON line (see the keys below).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "int4_decode_ffn_tokens_per_s"
UNIT = "tokens/s"
BYTES_PER_WEIGHT = 0.5 + 1.0 / 256 + 1.0 / 64  # qweight + qzeros + bf16 scales at group 128


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=80)
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--intermediate", type=int, default=28672)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-prefill", action="store_true", help="skip the prefill GEMM timing (extra key `prefill`)")
    ap.add_argument("--unfused", action="store_true", help="per-layer kernels instead of the one-launch stack kernel")
    ap.add_argument("--peer-exchange", action="store_true",
                    help="tensor parallel with the per-layer kernels: partials read from peer memory + flag words instead of an NCCL allreduce per layer")
    ap.add_argument("--no-replicas", action="store_true", help="N > 1: skip the data-parallel measurement (extra key `replicas`)")
    ap.add_argument("--sweep", action="store_true", help="time the batch sweep (extra key `batches`) on all layers instead of 16")
    ap.add_argument("--no-configs", action="store_true",
                    help="skip the extra keys dequant_cfg1 / gemv_cfg2 / ffn_cfg3 / batches (the other configurations of the benchmark definition)")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle comparison of the timed path (key `parity`)")
    return ap.parse_args()


# dram__bytes_read.sum + dram__bytes_write.sum per launch from the committed ncu summaries, keyed by
# (kernel, hidden, intermediate per rank, batch).  The stack kernel's figure is per layer (a 2-layer
# capture, halved) and is scaled by the layer count; shapes that were not captured report null.
NCU_TRAFFIC = {
    ("ffn_fused_kernel", 8192, 28672, 8): {"bytes_per_layer": 370109184, "source": "profiles/ffn_fused_70b_stack.md"},
    ("gemv_streamk_kernel<EPI_SWIGLU>", 8192, 28672, 8): {"bytes": 252018688, "source": "profiles/gemv_streamk_70b_ffn_layer.md"},
}


def workload_name(a):
    return (f"decode FFN stack, Llama-3-70B dims: hidden {a.hidden}, intermediate {a.intermediate}, "
            f"{a.layers} AWQ-int4 layers (group 128), batch {a.batch}, residual add per layer")


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


# --------------------------------------------------------------------------------------
# CPU golden path on a bounded sample (cpu_baseline and --impl reference)
# --------------------------------------------------------------------------------------
def cpu_sample_setup(a, cols=4096):
    """A column slice of one layer: gate/up restricted to `cols` intermediate columns and down to
    the same `cols` rows: exactly cols / intermediate of one layer's weights and flops."""
    import numpy as np
    from ml_dtypes import bfloat16
    from oracle import awq_oracle as O
    rng = np.random.default_rng(0)
    H, gs = a.hidden, 128

    def synth(K, N):
        return (O.pack_awq_int32(rng.integers(0, 16, (K, N), dtype=np.uint8)),
                O.pack_awq_int32(rng.integers(0, 16, (K // gs, N), dtype=np.uint8)),
                rng.uniform(0.001, 0.02, (K // gs, N)).astype(bfloat16))

    gate, up, down = synth(H, cols), synth(H, cols), synth(cols, H)
    x = rng.standard_normal((a.batch, H)).astype(bfloat16)
    gamma = (rng.standard_normal(H) * 0.1 + 1.0).astype(bfloat16)
    return dict(gate=gate, up=up, down=down, x=x, gamma=gamma, cols=cols)


def cpu_sample_run(a, s):
    from oracle import awq_oracle as O
    t0 = time.perf_counter()
    O.ffn_layer_A_ref(s["x"], s["gamma"], s["gate"], s["up"], s["down"], 128)
    return time.perf_counter() - t0


def cpu_tokens_per_s(a, sample_seconds, cols):
    layer_seconds = sample_seconds * (a.intermediate / cols)
    return a.batch / (layer_seconds * a.layers)


def cpu_threads():
    try:
        from threadpoolctl import threadpool_info
        n = max([p.get("num_threads", 1) for p in threadpool_info()] or [1])
        return int(n)
    except Exception:
        return os.cpu_count() or 1


def use_all_host_cores():
    """Give the BLAS pool every host core, whatever the launcher put in OMP_NUM_THREADS (torchrun
    sets it to 1).  Returns the object that keeps the limit alive."""
    try:
        import numpy  # noqa: F401  (loads BLAS so the pool exists)
        from threadpoolctl import threadpool_limits
        return threadpool_limits(limits=os.cpu_count() or 1)
    except Exception:
        return None


def run_reference(a):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    _pool = use_all_host_cores()  # noqa: F841
    s = cpu_sample_setup(a)
    for _ in range(min(a.warmup, 1)):
        cpu_sample_run(a, s)
    times = [cpu_sample_run(a, s) for _ in range(max(1, a.steps))]
    per = sum(times) / len(times)
    v = cpu_tokens_per_s(a, per, s["cols"])
    factor = (a.intermediate / s["cols"]) * a.layers
    sample = (f"numpy golden (dequant + f32 matmul + SwiGLU + residual) on {s['cols']}/{a.intermediate} of one layer's "
              f"columns per step; value and ms_per_step are EXTRAPOLATED by {factor:g} (x {a.intermediate / s['cols']:g} columns, "
              f"x {a.layers} layers)")
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": a.gpus, "steps": a.steps,
        "warmup": a.warmup, "ms_per_step": per * 1e3 * (a.intermediate / s["cols"]) * a.layers,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(a), "parallelism": "host cores"},
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": cpu_threads(), "kind": "port", "sample": sample,
                         "extrapolated": True, "extrapolation_factor": factor, "measured_ms_per_sample": per * 1e3},
        "extrapolated": True, "extrapolation_factor": factor, "measured_ms_per_sample": per * 1e3,
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------
# clocks sampler
# --------------------------------------------------------------------------------------
class ClockSampler:
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.samples = []
        self._stop = threading.Event()
        self._t = threading.Thread(target=self._loop, daemon=True)
        self.source = "nvidia-smi"

    def _nvml_loop(self):
        """Read-only NVML queries every 2 ms (a timed region of 100 ms gets tens of samples; one
        nvidia-smi process per sample gets one or two).  Returns False if NVML is not usable."""
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            reasons_of = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
            mx = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
            pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)
            reasons_of(h)
        except Exception:
            return False
        self.source = "nvml"
        bits = (0x8, 0x40, 0x20, 0x4)  # hw_slowdown, hw_thermal_slowdown, sw_thermal_slowdown, sw_power_cap
        while not self._stop.is_set():
            try:
                r = int(reasons_of(h))
                self.samples.append([str(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)), str(mx)] +
                                    ["Active" if r & b else "Not Active" for b in bits])
            except Exception:
                pass
            self._stop.wait(0.002)
        return True

    def _loop(self):
        if self._nvml_loop():
            return
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                f = [x.strip() for x in out.strip().split(",")]
                if len(f) >= 6:
                    self.samples.append(f)
            except Exception:
                pass
            self._stop.wait(0.05)

    def __enter__(self):
        self._t.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._t.join(timeout=6)

    def summary(self):
        sm = sorted(int(s[0]) for s in self.samples if s[0].isdigit())
        mx = [int(s[1]) for s in self.samples if s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.samples), "source": self.source}


# --------------------------------------------------------------------------------------
# this library
# --------------------------------------------------------------------------------------
def _dbg(msg):
    if os.environ.get("AWQ_BENCH_DEBUG"):
        print(f"[bench rank {os.environ.get('RANK', '0')}] {msg}", file=sys.stderr, flush=True)


# --------------------------------------------------------------------------------------
# the other configurations of the benchmark definition (extra keys) and the parity check
# --------------------------------------------------------------------------------------
def _graph_us(torch, enqueue, launches, reps=20, warm=3):
    """Device time per launch of `enqueue()` (which enqueues `launches` kernels on distinct data)
    captured in one CUDA graph and replayed `reps` times after `warm` replays."""
    enqueue()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        enqueue()
    for _ in range(warm):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * launches)


def _hbm_entry(us, nbytes, peak):
    gbs = nbytes / (us * 1e-6) / 1e9
    return {"us": us, "bytes": int(nbytes), "achieved_gbs": gbs, "frac_of_measured": gbs / peak, "frac_of_8TBs": gbs / 8000.0}


def time_other_configs(a, torch, ops, ffn, peak):
    """dequant 2048 x 2048, decode GEMV 4096 x 11008 (batch 1, 8), decode FFN 4096 / 11008 (batch 1, 4, 16):
    graph replays over weight copies totalling more than twice the L2, so every launch streams from HBM."""
    l2 = int(torch.cuda.get_device_properties(torch.cuda.current_device()).L2_cache_size)
    out = {"l2_bytes": l2, "timing": "CUDA graph of one launch per weight copy, copies total > 2 x L2, 20 replays after 3"}
    # ---- configuration 1: dequant of a 2048 x 2048 weight ----
    K = N = 2048
    per = K * N * BYTES_PER_WEIGHT + K * N * 2
    copies = int(2 * l2 // per) + 2
    ws_ = [ffn.random_layer(K, N // 2, seed=50 + i, with_gamma=False).gateup for i in range(copies)]
    outs = [torch.empty((K, N), dtype=torch.bfloat16, device="cuda") for _ in range(copies)]
    us = _graph_us(torch, lambda: [ops.dequant(w, o) for w, o in zip(ws_, outs)], copies)
    out["dequant_cfg1"] = dict(_hbm_entry(us, per, peak), workload="AWQ dequant 2048 x 2048 -> bf16", copies=copies,
                               kernel="dequant_kernel")
    del ws_, outs
    # ---- configuration 2: decode GEMV 4096 x 11008 ----
    K, N = 4096, 11008
    copies = int(2 * l2 // (K * N * BYTES_PER_WEIGHT)) + 2
    ws_ = [ffn.random_layer(K, N // 2, seed=80 + i, with_gamma=False).gateup for i in range(copies)]
    wsp = ops.Workspace(K, N)
    g2 = {}
    for B in (1, 8):
        x = torch.randn((B, K), device="cuda").to(torch.bfloat16)
        ys = [torch.empty((B, N), dtype=torch.bfloat16, device="cuda") for _ in range(copies)]
        us = _graph_us(torch, lambda: [ops.gemv(x, w, wsp, out=y) for w, y in zip(ws_, ys)], copies)
        g2[str(B)] = _hbm_entry(us, K * N * BYTES_PER_WEIGHT + B * K * 2 + B * N * 2, peak)
    wsp.check()
    out["gemv_cfg2"] = {"workload": "decode GEMV [B x 4096] x AWQ [4096 x 11008], one awq_b200_gemv_bf16 call per weight "
                                    "(one kernel launch each: at this size the bf16 activations are multiplied as they are)",
                        "copies": copies, "batch": g2}
    del ws_
    # ---- configuration 3: decode SwiGLU FFN 4096 / 11008 ----
    H, I = 4096, 11008
    per = 3 * H * I * BYTES_PER_WEIGHT
    nl = int(2 * l2 // per) + 2
    layers = [ffn.random_layer(H, I, seed=300 + i) for i in range(nl)]
    st = ffn.DecodeFFNStack(layers, H, max_batch=16)
    g3 = {}
    for B in (1, 4, 16):
        x = torch.randn((B, H), device="cuda").to(torch.bfloat16)
        st.capture(B)
        st.load_input(x)
        for _ in range(3):
            st.replay(B)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(20):
            st.replay(B)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (20 * nl)
        g3[str(B)] = dict(_hbm_entry(us, per + 4 * B * H * 2, peak), tokens_per_s=B / (us * 1e-6),
                          path="one launch of the stack kernel for all layers" if st.uses_fused(B) else
                          ("per layer: RMSNorm + two batched-decode GEMMs (" + ("fp8" if st.uses_gemm_f8(B) else "fp16") + " operands)"
                           if st.uses_gemm(B) else "per-layer kernels"))
    st.check()
    out["ffn_cfg3"] = {"workload": f"decode SwiGLU FFN hidden 4096 / intermediate 11008 with RMSNorm and residual, {nl} distinct "
                                   "layers back to back, time per layer", "layers": nl, "batch": g3}
    del st, layers
    torch.cuda.empty_cache()
    return out


def parity_check(a, torch, ops, ffn, group, rank, world):
    """The path the timed region uses (DecodeFFNStack with this run's group, exchange and kernels) on a
    small seeded stack whose weights also exist on the host, compared on rank 0 with the unsharded
    numpy oracle.  Outside every timed region."""
    import numpy as np
    from ml_dtypes import bfloat16
    from oracle import awq_oracle as O  # the checker only
    H, I, L, B, gs = 1024, 2816, 4, min(8, a.batch), 128
    i0, i1 = ffn.tp_shard_bounds(I, world)[rank]

    def synth(K, N, seed, lo=0.001, hi=0.02):
        r = np.random.default_rng(seed)
        return (O.pack_awq_int32(r.integers(0, 16, (K, N), dtype=np.uint8)),
                O.pack_awq_int32(r.integers(0, 16, (K // gs, N), dtype=np.uint8)), r.uniform(lo, hi, (K // gs, N)).astype(bfloat16))

    def dev16(v):
        return torch.from_numpy(np.ascontiguousarray(v).view(np.int16)).cuda().view(torch.bfloat16)

    full, layers = [], []
    for l in range(L):
        gate, up, down = synth(H, I, 900 + 10 * l), synth(H, I, 901 + 10 * l), synth(I, H, 902 + 10 * l, 0.0005, 0.004)
        gamma = (np.random.default_rng(903 + 10 * l).standard_normal(H) * 0.1 + 1.0).astype(bfloat16)
        full.append((gate, up, down, gamma))
        gu = ops.interleave_gate_up(ops.AwqWeight.from_numpy(*gate, gs), ops.AwqWeight.from_numpy(*up, gs))
        layers.append(ffn.FFNLayer(ffn.shard_gateup(gu, i0, i1), ffn.shard_down(ops.AwqWeight.from_numpy(*down, gs), i0, i1),
                                   dev16(gamma)))
    x = np.random.default_rng(899).standard_normal((B, H)).astype(bfloat16)
    st = ffn.DecodeFFNStack(layers, H, max_batch=32, group=group, fused=not a.unfused, peer_push=a.peer_exchange)
    # the stack chooses between the two batched-decode GEMMs by the size of a layer: check the one that the timed
    # configuration takes at 32 rows on this many ranks
    f8_min = dict(ffn.DecodeFFNStack.GEMM_F8_MIN_WEIGHTS)
    if 3 * a.hidden * a.intermediate / world >= f8_min[32]:
        f8_min = {16: 0, 32: 0}
    st.GEMM_F8_MIN_WEIGHTS = f8_min
    y_eager = st.step(dev16(x))
    st.load_input(dev16(x))
    y_graph = st.replay(B).clone()
    # the path the batch sweep times for 32 and 64 rows (RMSNorm + two batched-decode GEMMs per layer; fp8 operands at 32 rows), same
    # layers: end to end, and every layer on its own from the oracle's input of that layer; both are judged
    x32 = np.random.default_rng(898).standard_normal((32, H)).astype(bfloat16)
    y32 = st.step(dev16(x32))
    st.check()
    golden_in, y32_layers = [x32], []
    for gate, up, down, gamma in full[:-1]:
        golden_in.append(O.ffn_layer_A_ref(golden_in[-1], gamma, gate, up, down, gs))
    for l in range(L):
        one = ffn.DecodeFFNStack(layers[l:l + 1], H, max_batch=32, group=group, fused=not a.unfused, peer_push=a.peer_exchange)
        one.GEMM_F8_MIN_WEIGHTS = f8_min
        y32_layers.append(one.step(dev16(golden_in[l])))
        one.check()
        del one
    res = None
    if rank == 0:
        def oracle(v):
            for gate, up, down, gamma in full:
                v = O.ffn_layer_A_ref(v, gamma, gate, up, down, gs)
            return v
        host = lambda t: t.contiguous().view(torch.int16).cpu().numpy().view(bfloat16)  # noqa: E731
        ref = oracle(x)
        e1, e2 = O.rel_l2(host(y_eager), ref), O.rel_l2(host(y_graph), ref)
        e32 = O.rel_l2(host(y32), oracle(x32))
        e32_layers = [O.rel_l2(host(y32_layers[l]), O.ffn_layer_A_ref(golden_in[l], full[l][3], full[l][0], full[l][1], full[l][2], gs))
                      for l in range(L)]
        res = {"rel_l2": max(e1, e2), "rel_l2_eager": e1, "rel_l2_graph_replay": e2, "tolerance": 1e-2,
               "dims": f"hidden {H}, intermediate {I}, {L} layers, batch {B}, tp{world}",
               "path": ("one-launch stack kernel" + (" with the in-kernel exchange" if world > 1 else "")) if st.uses_fused(B)
               else "per-layer kernels", "oracle": "oracle.awq_oracle.ffn_layer_A_ref, unsharded",
               "batch_32": {"rel_l2": max(max(e32_layers), e32), "rel_l2_per_layer": e32_layers, "rel_l2_end_to_end": e32,
                            "judged": "the chain of all layers, and every layer from the oracle's input of that layer",
                            "path": ("per layer: RMSNorm + two batched-decode GEMMs (" + ("fp8" if st.uses_gemm_f8(32) else "fp16") + " operands)")
                            if st.uses_gemm(32) else "per-layer kernels"}}
    del st, layers
    return res



def run_ours(a):
    import numpy as np
    import torch
    import torch.distributed as dist
    from ml_dtypes import bfloat16

    from mlir_air_b200 import ffn, ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        group = dist.group.WORLD
    assert world == a.gpus or world == 1, f"--gpus {a.gpus} but WORLD_SIZE={world}"
    tp = world

    _dbg("process group ready")
    bounds = ffn.tp_shard_bounds(a.intermediate, tp)[rank]
    layers = [ffn.random_layer(a.hidden, a.intermediate, seed=1000 + l, bounds=bounds) for l in range(a.layers)]
    stack = ffn.DecodeFFNStack(layers, a.hidden, max_batch=max(64, a.batch), group=group, fused=not a.unfused,
                               peer_push=a.peer_exchange)
    B = a.batch
    rng = np.random.default_rng(0)
    x_host = rng.standard_normal((B, a.hidden)).astype(bfloat16)
    x_dev = torch.from_numpy(x_host.view(np.int16)).cuda().view(torch.bfloat16)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    _dbg("weights ready")

    def time_steps(batch, steps, warmup):
        # the input first: the eager run and the capture below read it (an uninitialised buffer may hold NaNs,
        # which the kernels report)
        stack.load_input(x_dev[:batch] if batch <= B else x_dev.repeat((batch + B - 1) // B, 1)[:batch])
        stack._run(batch)
        torch.cuda.synchronize()
        _dbg("eager run done")
        stack.capture(batch)
        _dbg("graph captured")
        for _ in range(max(3, warmup)):
            stack.replay(batch)
        sync_all()
        _dbg("warm-up replays done")
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            stack.replay(batch)
        e1.record()
        sync_all()
        return max_over_ranks(e0.elapsed_time(e1)) / steps

    # ---- device-resident throughput (the `value`) ----
    with ClockSampler(local) as clk:
        ms_step = time_steps(B, a.steps, a.warmup)
    clocks = clk.summary()
    stack.check()
    value = B / (ms_step * 1e-3)

    # ---- end to end through the public host API: pinned H2D + stack + D2H every step ----
    for _ in range(3):
        stack.forward_host(x_host)
    sync_all()
    t0 = time.perf_counter()
    for _ in range(a.steps):
        out_host = stack.forward_host(x_host)
    torch.cuda.synchronize()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3) / a.steps
    assert np.isfinite(out_host.astype(np.float32)).all(), "stack output is not finite"
    io_bytes = B * a.hidden * 2

    # ---- roofline of the dominant kernel (gate/up GEMV + SwiGLU), timed live: one launch per
    #      layer on distinct weights (no L2 reuse), captured in a graph so the host does not pace it
    il = bounds[1] - bounds[0]
    gu_bytes = a.hidden * 2 * il * BYTES_PER_WEIGHT + B * a.hidden * 2 + B * il * 2
    normed = torch.randn((B, a.hidden), device="cuda").to(torch.bfloat16)
    inter = torch.empty((B, il), dtype=torch.bfloat16, device="cuda")

    def gu_all():
        for l in layers:
            ops.gateup_swiglu(normed, l.gateup, stack.ws, out=inter)

    gu_all()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        gu_all()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 5
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    passes = (B + 7) // 8
    gu_us = e0.elapsed_time(e1) * 1e3 / (reps * len(layers) * passes)
    peak, peak_src = measured_peak_gbs()
    achieved = gu_bytes / passes / (gu_us * 1e-6) / 1e9
    gateup_kernel = {"bound": "hbm", "kernel": "gemv_streamk_kernel<EPI_SWIGLU> (gate/up GEMV + SwiGLU)",
                "achieved": achieved, "peak": peak, "peak_source": peak_src, "unit": "GB/s", "frac": achieved / peak,
                "frac_of_8TBs": achieved / 8000.0, "us_per_launch": gu_us, "bytes_per_launch": gu_bytes / passes,
                # dram__bytes_read.sum + dram__bytes_write.sum of one launch at this exact shape
                # (the committed ncu summary of that kernel); other shapes were not captured
                "traffic": (NCU_TRAFFIC.get(("gemv_streamk_kernel<EPI_SWIGLU>", a.hidden, il, B)) or {}).get("bytes"),
                "traffic_source": (NCU_TRAFFIC.get(("gemv_streamk_kernel<EPI_SWIGLU>", a.hidden, il, B)) or {}).get("source")}
    stack_bytes = stack.weight_bytes + a.layers * 4 * B * a.hidden * 2
    stack_gbs = stack_bytes / (ms_step * 1e-3) / 1e9
    if stack.uses_fused(B):
        # the timed region is ONE launch of the stack kernel: its roofline is the step's
        roofline = {"bound": "hbm", "kernel": "ffn_fused_kernel (all layers of the stack in one launch)",
                    "achieved": stack_gbs, "peak": peak, "peak_source": peak_src, "unit": "GB/s", "frac": stack_gbs / peak,
                    "frac_of_8TBs": stack_gbs / 8000.0, "us_per_launch": ms_step * 1e3, "bytes_per_launch": stack_bytes,
                    # dram bytes of a 2-layer launch scaled by the layer count
                    "traffic": (lambda t: t["bytes_per_layer"] * a.layers if t else None)(
                        NCU_TRAFFIC.get(("ffn_fused_kernel", a.hidden, il, B))),
                    "traffic_source": (NCU_TRAFFIC.get(("ffn_fused_kernel", a.hidden, il, B)) or {}).get("source")}
    else:
        roofline = gateup_kernel

    # ---- prefill int4 GEMM (the fourth configuration: 2048 x 4096 x 14336) on this GPU: extra key, not the headline ----
    prefill = None
    if not a.no_prefill:
        Mp, Kp, Np = 2048, 4096, 14336
        wp = ffn.random_layer(Kp, Np // 2, seed=7, with_gamma=False).gateup  # a [4096, 14336] AWQ weight
        Ap = torch.randn((Mp, Kp), device="cuda").to(torch.bfloat16)
        Cp = torch.empty((Mp, Np), dtype=torch.bfloat16, device="cuda")
        for _ in range(3):
            ops.gemm(Ap, wp, Cp)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            ops.gemm(Ap, wp, Cp)
        e1.record()
        torch.cuda.synchronize()
        ops.gemm_check()
        us = e0.elapsed_time(e1) * 100.0
        tf = 2.0 * Mp * Kp * Np / us / 1e6
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                pk = float(json.load(f)["bf16_tflops"])
        except Exception:
            pk = 1590.0
        prefill = {"workload": "int4 GEMM [2048 x 4096] x AWQ [4096 x 14336]", "us": us, "tflops": tf,
                   "frac_of_measured_bf16_peak": tf / pk, "frac_of_2250": tf / 2250.0,
                   "kernel": "gemm_tm_kernel (tcgen05, dequantised weights in tensor memory)"}
        del wp, Ap, Cp

    # ---- the other way to use N GPUs (extra key, not the headline): every rank holds the whole stack
    #      and decodes its own batch; no exchange at all, per-GPU work fixed ("weak" scaling) ----
    replicas = None
    if world > 1 and not a.no_replicas:
        full = [ffn.random_layer(a.hidden, a.intermediate, seed=1000 + l) for l in range(a.layers)]
        rstack = ffn.DecodeFFNStack(full, a.hidden, max_batch=max(8, B), fused=not a.unfused)
        rstack.load_input(x_dev)
        rstack.capture(B)
        rstack.load_input(x_dev)
        for _ in range(3):
            rstack.replay(B)
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.steps):
            rstack.replay(B)
        e1.record()
        sync_all()
        rms = max_over_ranks(e0.elapsed_time(e1)) / a.steps
        rstack.check()
        replicas = {"value": world * B / (rms * 1e-3), "unit": UNIT, "ms_per_step": rms, "scaling": "weak",
                    "global_batch": world * B, "parallelism": f"{world} replicas of the whole stack, no exchange"}
        del rstack, full

    # ---- the batch sweep of configuration 5 (1 / 8 / 32 / 64 tokens, and 16) on a shorter stack unless --sweep ----
    batches = None
    if not a.no_configs or a.sweep:
        nl = a.layers if a.sweep else min(a.layers, 16)
        sub = stack if nl == a.layers else ffn.DecodeFFNStack(layers[:nl], a.hidden, max_batch=64, group=group,
                                                              fused=not a.unfused, peer_push=a.peer_exchange)
        keep_stack = stack
        stack = sub
        batches = {"layers": nl, "note": "ms per step of a stack of `layers` layers; bytes = this rank's weights + activations"}
        for b in (1, 8, 16, 32, 64):
            ms = time_steps(b, max(3, a.steps // 2), 3)
            by = sub.weight_bytes + nl * 4 * b * a.hidden * 2
            batches[str(b)] = {"ms_per_step": ms, "us_per_layer": ms * 1e3 / nl, "tokens_per_s": b / (ms * 1e-3),
                               "achieved_gbs": by / (ms * 1e-3) / 1e9, "frac_of_measured": by / (ms * 1e-3) / 1e9 / peak,
                               "frac_of_8TBs": by / (ms * 1e-3) / 1e9 / 8000.0}
        sub.check()
        stack = keep_stack
        if sub is not stack:
            del sub

    # ---- configurations 1-3 of the benchmark definition on this GPU (rank 0 of a multi-GPU run skips them) ----
    other = None
    if not a.no_configs and world == 1:
        other = time_other_configs(a, torch, ops, ffn, peak)

    # ---- oracle parity of the timed path, outside the timed region, at every N ----
    parity = None
    if not a.no_parity:
        parity = parity_check(a, torch, ops, ffn, group, rank, world)

    def finish():
        """Leave without tearing the communicator down: destroying a process group while captured
        graphs still hold its collectives can block, and there is nothing left to clean up."""
        if world > 1:
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            sys.stdout.flush()
            sys.stderr.flush()
            os._exit(0)

    if rank != 0:
        finish()
        return

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": a.gpus, "steps": a.steps, "warmup": max(3, a.warmup),
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": workload_name(a), "parallelism": f"tp{tp}",
                   "exchange": ("none" if tp == 1 else
                                "inside the stack kernel: f32 partials stored into every rank's peer-mapped receive area as value+tag words, polled and added in rank order"
                                if stack.uses_fused(B) else
                                "peer loads from every rank's send buffer + flag words"
                                if stack.peers is not None and B <= 8 else "NCCL allreduce per layer"),
                   "l2": "inputs_exceed_l2 (weights streamed once per step)",
                   "launch": ("one CUDA graph per step: one launch of the stack kernel" if stack.uses_fused(B)
                              else "one CUDA graph per step")},
        "clocks": clocks,
        "e2e": {"value": B / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": io_bytes,
                "d2h_bytes_per_step": io_bytes},
        "gpu_launches": stack.launches_per_step(B) * a.steps,
        "roofline": roofline,
        "gateup_kernel": gateup_kernel,
        "stack_hbm": {"achieved": stack_gbs, "unit": "GB/s", "frac": stack_gbs / peak, "frac_of_8TBs": stack_gbs / 8000.0,
                      "bytes_per_step_per_gpu": stack_bytes},
    }
    if replicas:
        line["replicas"] = replicas
    if batches:
        line["batches"] = batches
    if other:
        line.update({k: v for k, v in other.items() if k.endswith(("cfg1", "cfg2", "cfg3"))})
        line["configs_timing"] = {"l2_bytes": other["l2_bytes"], "method": other["timing"]}
    if parity:
        line["parity"] = parity
    if prefill:
        line["prefill"] = prefill
    if a.gpus == 1 and not a.no_cpu_baseline:
        _pool = use_all_host_cores()  # noqa: F841
        s = cpu_sample_setup(a)
        cpu_sample_run(a, s)
        reps, t_acc = 0, 0.0
        while reps < 60 and t_acc < 12.0:  # about 12 s of host work
            t_acc += cpu_sample_run(a, s)
            reps += 1
        v = cpu_tokens_per_s(a, t_acc / reps, s["cols"])
        factor = (a.intermediate / s["cols"]) * a.layers
        line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cpu_threads(), "kind": "port",
                                "sample": f"numpy golden on {s['cols']}/{a.intermediate} of one layer's columns, mean of "
                                          f"{reps} runs; value EXTRAPOLATED by {factor:g} to {a.layers} whole layers",
                                "extrapolated": True, "extrapolation_factor": factor,
                                "measured_ms_per_sample": t_acc / reps * 1e3}
    print(json.dumps(line), flush=True)
    if parity and not max(parity["rel_l2"], parity["batch_32"]["rel_l2"]) <= parity["tolerance"]:
        print(f"parity check failed: rel-L2 {parity['rel_l2']:.3e} (batch 32: {parity['batch_32']['rel_l2']:.3e}) against the "
              f"oracle exceeds {parity['tolerance']}",
              file=sys.stderr, flush=True)
        if world > 1:
            torch.cuda.synchronize()
            dist.barrier()
            os._exit(3)
        sys.exit(3)
    finish()


def main():
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)


if __name__ == "__main__":
    main()
