"""KernelCache.load_and_run semantics (llms/shared/infra/cache.py:494-737): static arguments are
turned into their device form once per bo_key, results match the uncached runner."""
import numpy as np
import pytest
from ml_dtypes import bfloat16


def test_validation_needs_no_gpu():
    from mlir_air_b200.backend import KernelSpec
    from mlir_air_b200.kernel_cache import KernelCache
    kc = KernelCache()
    with pytest.raises(RuntimeError):
        kc.load_and_run("nope", {}, np.zeros(1))
    with pytest.raises(Exception):
        kc.compile_and_cache("x", KernelSpec("not_an_instance", {}))
    kc.compile_and_cache("mv", KernelSpec("matvec_int4_packed", dict(M=64, K=512, GS=128, M_TILE=8, K_CHUNK=256, N_CORES=4,
                                                                     M_PER_LAUNCH=32)))
    a = [np.zeros(4, np.uint8), np.zeros(4, bfloat16), np.zeros(4, bfloat16)]
    with pytest.raises(ValueError):
        kc.load_and_run("mv", {}, *a, static_input_indices={0}, shared_alias={0: "pool"})
    with pytest.raises(ValueError):
        kc.load_and_run("mv", {}, *a, shared_alias={7: "pool"})
    with pytest.raises(ValueError):
        kc.load_and_run("mv", {}, *a, shared_alias={1: ""})


@pytest.mark.gpu
def test_static_weights_stay_resident_per_bo_key():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from golden_util import load
    from mlir_air_b200 import backend
    from mlir_air_b200.kernel_cache import KernelCache, Profiler
    from mlir_air_b200.programming_examples.matrix_vector_multiplication.int4_awq import matvec_int4_packed as mv
    from oracle import awq_oracle as O
    g = load("matvec_int4_packed_64x512")
    spec = mv.build_module(64, 512, 128, 8, 256, 4, 32)
    kc = KernelCache(profiler=Profiler(True))
    kc.compile_and_cache("o_gemv", spec, {"instance_name": "matvec_int4_packed"})
    from mlir_air_b200 import ops
    calls = {"n": 0}
    real = ops.repack_C_to_A  # the per-tile buffer is unpacked on the GPU (awq_b200_repack_C_to_B + _B_to_A)

    def counting(*a, **k):
        calls["n"] += 1
        return real(*a, **k)

    ops.repack_C_to_A = counting
    try:
        out = np.zeros(64, bfloat16)
        for layer in range(2):
            for token in range(3):
                x = np.random.default_rng(token).standard_normal(512).astype(bfloat16)
                res = kc.load_and_run("o_gemv", {}, g["packed"], x, out, static_input_indices={0}, intermediate_indices={2},
                                      bo_key=f"o_gemv_L{layer}")
                assert res[0].size == 0 and res[1].size == 0  # only the last buffer is read back by default
                assert O.rel_l2(res[2], O.gemv_ref(g["A_q"], g["A_s"], g["A_z"], x)) <= 1e-2
        assert calls["n"] == 2  # one unpack + upload per bo_key, not per call
        assert kc.resident_keys() == [("o_gemv", "o_gemv_L0"), ("o_gemv", "o_gemv_L1")]
        # without the static declaration every call converts again
        kc.load_and_run("o_gemv", {}, g["packed"], g["B"], out, output_indices=[2])
        kc.load_and_run("o_gemv", {}, g["packed"], g["B"], out, output_indices=[2])
        assert calls["n"] == 4
    finally:
        ops.repack_C_to_A = real
    assert "o_gemv: 8 calls" in kc.profiler.report()
