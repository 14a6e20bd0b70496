"""Host side of the example mirrors, without a GPU: every script's `-p` names a kernel instance
the backend implements, its compile-only mode exits 0, and tilings the reference's build_module
rejects are rejected here too."""
import importlib
import re

import pytest

PE = "mlir_air_b200.programming_examples."
SCRIPTS = [
    "dequant_awq.dequant_awq",
    "matrix_vector_multiplication.int4_awq.matvec_int4_packed",
    "matrix_vector_multiplication.int4_awq.matvec_int4_packed_add",
    "matrix_vector_multiplication.bf16.matvec",
    "decode_ffn_swiglu.matvec_int4_swiglu_rms",
    "decode_ffn_swiglu.matvec_swiglu_rms",
    "ffn_swiglu.decode.ffn_decode",
    "ffn_swiglu.prefill.ffn_prefill",
    "matrix_multiplication.int4_awq.matmul_int4_packed",
    "silu_and_mul.silu_and_mul",
    "llms.llama32_1b_int4.multi_launch_builder.rms_qkv_int4_rope_multi",
]


@pytest.mark.parametrize("script", SCRIPTS, ids=[s.split(".")[-1] for s in SCRIPTS])
def test_print_module_names_a_registered_instance(script, capsys):
    from mlir_air_b200.backend import _INSTANCES
    mod = importlib.import_module(PE + script)
    with pytest.raises(SystemExit) as e:
        mod.main(["-p"])
    assert e.value.code == 0
    out = capsys.readouterr().out
    m = re.search(r"b200\.kernel @(\w+)\(", out)
    assert m, out
    assert m.group(1) in _INSTANCES


@pytest.mark.parametrize("script", ["matrix_vector_multiplication.int4_awq.matvec_int4_packed",
                                    "decode_ffn_swiglu.matvec_swiglu_rms"])
def test_compile_only_needs_no_gpu(script):
    mod = importlib.import_module(PE + script)
    flag = "compile-and-xclbin" if script.endswith("matvec_swiglu_rms") else "compile-only"
    with pytest.raises(SystemExit) as e:
        mod.main(["--compile-mode", flag])
    assert e.value.code == 0


def test_bad_tilings_are_rejected():
    from mlir_air_b200.programming_examples.decode_ffn_swiglu import matvec_swiglu_rms as bf
    from mlir_air_b200.programming_examples.matrix_vector_multiplication.bf16 import matvec
    from mlir_air_b200.programming_examples.matrix_vector_multiplication.int4_awq import matvec_int4_packed as mv
    with pytest.raises(ValueError):
        bf.build_module(16384, 2048, n_cascade=1)       # a cascade needs two stages
    with pytest.raises(ValueError):
        bf.build_module(16384, 2048, tile_m=8)          # fewer than 16 outputs per tile
    with pytest.raises(ValueError):
        bf.build_module(16384 + 2, 2048)
    with pytest.raises(ValueError):
        matvec.build_module(2050, 8192)
    with pytest.raises(ValueError):
        mv.build_module(64, 512, 128, 8, 256, 4, 48)    # M_PER_LAUNCH does not divide M
