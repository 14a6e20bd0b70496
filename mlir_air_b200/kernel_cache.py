"""Weight-resident kernel invocation: the counterpart of the LLM drivers' KernelCache
(llms/shared/infra/cache.py:309-737).

The reference compiles each kernel once (`compile_and_cache`) and then calls `load_and_run(name,
backend_kwargs, *inputs, output_indices=..., static_input_indices=..., intermediate_indices=...,
bo_key=...)` per layer and token: buffers are kept per `bo_key`, arguments listed as static
(weights, LUTs) are written on the first call only, intermediates are never uploaded, and the
buffers named in `output_indices` (default: the last one) are read back.  Here there is nothing to
compile; an "artifact" is the KernelSpec the example's builder returns.  A static argument is turned
into its device form (layout-A weight on the GPU) on the first call for a `bo_key` and reused after
that, so a decode loop pays the unpacking and the upload of a layer's weights once, exactly as the
reference pays the BO write once.
"""
from __future__ import annotations

import time
from typing import Dict, Optional, Sequence

import numpy as np

from .backend import _INSTANCES, KernelSpec, _to_host
from ._lib import AwqBackendError


class Profiler:
    """Per-kernel wall time, the part of cache.py:70-160 the decode drivers read."""

    def __init__(self, enabled: bool = False):
        self.enabled = enabled
        self.kernel_s: Dict[str, float] = {}
        self.kernel_calls: Dict[str, int] = {}

    def record_kernel(self, name: str, duration: float):
        if self.enabled:
            self.kernel_s[name] = self.kernel_s.get(name, 0.0) + duration
            self.kernel_calls[name] = self.kernel_calls.get(name, 0) + 1

    def report(self) -> str:
        return "\n".join(f"{n}: {self.kernel_calls[n]} calls, {1e3 * t:.2f} ms" for n, t in sorted(self.kernel_s.items()))


class KernelCache:
    def __init__(self, cache_dir=None, verbose: bool = False, profiler: Optional[Profiler] = None):
        self.cache_dir = cache_dir  # accepted for interface parity: nothing is written to disk
        self.verbose = verbose
        self.profiler = profiler or Profiler(False)
        self.artifacts: Dict[str, KernelSpec] = {}
        self._resident: Dict[tuple, dict] = {}

    def compile_and_cache(self, name: str, mlir_module: KernelSpec, backend_kwargs=None, output_binary_name: str = "air"):
        if not isinstance(mlir_module, KernelSpec):
            raise AwqBackendError(f"expected a KernelSpec from the example's builder, got {type(mlir_module).__name__}")
        instance = (backend_kwargs or {}).get("instance_name") or mlir_module.instance_name
        if instance not in _INSTANCES:
            raise AwqBackendError(f"no B200 implementation registered for kernel instance '{instance}'")
        self.artifacts[name] = KernelSpec(instance, dict(mlir_module.params))

    def load_and_run(self, name: str, backend_kwargs, *inputs, output_indices: Optional[Sequence[int]] = None,
                     static_input_indices=None, intermediate_indices=None, bo_key: Optional[str] = None,
                     shared_nonstatic: bool = False, shared_alias=None):
        import torch
        if name not in self.artifacts:
            raise RuntimeError(f"Kernel '{name}' not found in cache. Available: {list(self.artifacts.keys())}")
        static = set(static_input_indices or ())
        if shared_alias:
            clash = sorted(set(shared_alias) & static)
            if clash:
                raise ValueError(f"shared_alias must not target static_input_indices {clash}: static BOs are "
                                 "per-bo_key, aliases are process-wide")
            oob = sorted(i for i in shared_alias if not 0 <= i < len(inputs))
            if oob:
                raise ValueError(f"shared_alias indices {oob} out of range for {len(inputs)} args")
            unnamed = sorted(i for i, n in shared_alias.items() if not isinstance(n, str) or not n)
            if unnamed:
                raise ValueError(f"shared_alias pool names must be non-empty strings; bad at arg indices {unnamed}")
        spec = self.artifacts[name]
        resident = self._resident.setdefault((name, bo_key if bo_key is not None else name), {})
        params = dict(spec.params, __static__=frozenset(static), __resident__=resident)
        args = [np.asarray(a) for a in inputs]
        t0 = time.time()
        outs, idx = _INSTANCES[spec.instance_name](params, args)
        torch.cuda.synchronize()
        self.profiler.record_kernel(name, time.time() - t0)
        produced = dict(zip(idx, outs))
        readback = {len(inputs) - 1} if output_indices is None else set(output_indices)
        missing = sorted(i for i in readback if i not in produced and not 0 <= i < len(inputs))
        if missing:
            raise ValueError(f"output_indices {missing} out of range for {len(inputs)} args")
        # buffers the kernel does not write come back as given (the reference reads the BO it uploaded)
        return tuple((_to_host(produced[i], args[i]) if i in produced else args[i].copy()) if i in readback
                     else np.empty(0, dtype=args[i].dtype) for i in range(len(args)))

    def resident_keys(self):
        """(kernel name, bo_key) pairs that hold device-resident static arguments."""
        return sorted(k for k, v in self._resident.items() if v)
