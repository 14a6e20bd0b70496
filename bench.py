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
    ap.add_argument("--sweep", action="store_true", help="also time batch 1/8/32/64 (extra key `batches`)")
    return ap.parse_args()


# dram__bytes_read.sum + dram__bytes_write.sum per layer of the stack kernel at hidden 8192 / intermediate
# 28672 / batch 8: ncu capture of a 2-layer launch, halved (the committed ncu summary of that kernel)
FUSED_TRAFFIC_PER_LAYER = 370400128


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


def run_reference(a):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy  # noqa: F401  (loads BLAS so threadpool_info sees it)
    s = cpu_sample_setup(a)
    for _ in range(min(a.warmup, 1)):
        cpu_sample_run(a, s)
    times = [cpu_sample_run(a, s) for _ in range(max(1, a.steps))]
    per = sum(times) / len(times)
    v = cpu_tokens_per_s(a, per, s["cols"])
    sample = (f"numpy golden (dequant + f32 matmul + SwiGLU + residual) on {s['cols']}/{a.intermediate} of one layer's "
              f"columns per step, scaled to {a.layers} layers")
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": a.gpus, "steps": a.steps,
        "warmup": a.warmup, "ms_per_step": per * 1e3 * (a.intermediate / s["cols"]) * a.layers,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(a), "parallelism": "host cores"},
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": cpu_threads(), "kind": "port", "sample": sample},
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
        stack._run(batch)
        torch.cuda.synchronize()
        _dbg("eager run done")
        stack.capture(batch)
        _dbg("graph captured")
        stack.load_input(x_dev[:batch] if batch <= B else x_dev.repeat((batch + B - 1) // B, 1)[:batch])
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
                "traffic": 249810432 if (a.hidden, il, B) == (8192, 28672, 8) else None}
    stack_bytes = stack.weight_bytes + a.layers * 4 * B * a.hidden * 2
    stack_gbs = stack_bytes / (ms_step * 1e-3) / 1e9
    if stack.uses_fused(B):
        # the timed region is ONE launch of the stack kernel: its roofline is the step's
        roofline = {"bound": "hbm", "kernel": "ffn_fused_kernel (all layers of the stack in one launch)",
                    "achieved": stack_gbs, "peak": peak, "peak_source": peak_src, "unit": "GB/s", "frac": stack_gbs / peak,
                    "frac_of_8TBs": stack_gbs / 8000.0, "us_per_launch": ms_step * 1e3, "bytes_per_launch": stack_bytes,
                    # dram bytes of a 2-layer launch scaled by the layer count
                    "traffic": FUSED_TRAFFIC_PER_LAYER * a.layers
                    if FUSED_TRAFFIC_PER_LAYER and (a.hidden, il, B) == (8192, 28672, 8) else None}
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
                   "frac_of_measured_bf16_peak": tf / pk, "frac_of_2250": tf / 2250.0, "kernel": "gemm_tc_kernel (tcgen05)"}
        del wp, Ap, Cp

    # ---- the other way to use N GPUs (extra key, not the headline): every rank holds the whole stack
    #      and decodes its own batch; no exchange at all, per-GPU work fixed ("weak" scaling) ----
    replicas = None
    if world > 1 and not a.no_replicas:
        full = [ffn.random_layer(a.hidden, a.intermediate, seed=1000 + l) for l in range(a.layers)]
        rstack = ffn.DecodeFFNStack(full, a.hidden, max_batch=max(8, B), fused=not a.unfused)
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

    batches = None
    if a.sweep:
        batches = {}
        for b in (1, 8, 32, 64):
            ms = time_steps(b, max(3, a.steps // 2), 3)
            batches[str(b)] = {"ms_per_step": ms, "tokens_per_s": b / (ms * 1e-3)}

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
    if prefill:
        line["prefill"] = prefill
    if a.gpus == 1 and not a.no_cpu_baseline:
        s = cpu_sample_setup(a)
        cpu_sample_run(a, s)
        reps, t_acc = 0, 0.0
        while reps < 60 and t_acc < 12.0:  # about 12 s of host work
            t_acc += cpu_sample_run(a, s)
            reps += 1
        v = cpu_tokens_per_s(a, t_acc / reps, s["cols"])
        line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cpu_threads(), "kind": "port",
                                "sample": f"numpy golden on {s['cols']}/{a.intermediate} of one layer's columns, mean of "
                                          f"{reps} runs, scaled to {a.layers} layers"}
    print(json.dumps(line), flush=True)
    finish()


def main():
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)


if __name__ == "__main__":
    main()
