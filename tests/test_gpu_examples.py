"""The example scripts (same names and flags as mlir-air's) run end to end on the GPU through
B200Runner and print PASS!, exactly what the reference's lit tests FileCheck for."""
import subprocess
import sys
import os

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PE = "mlir_air_b200.programming_examples."

CASES = [
    ("dequant_awq.dequant_awq", []),                                              # N=1024, gs=128, herd 4
    ("dequant_awq.dequant_awq", ["--hf", "2048", "2048"]),                        # benchmark configuration 1
    ("matrix_vector_multiplication.int4_awq.matvec_int4_packed", []),            # 2048 x 2048 (lit shape)
    ("matrix_vector_multiplication.int4_awq.matvec_int4_packed", ["--k", "8192", "--k-chunk", "2048"]),
    ("matrix_vector_multiplication.int4_awq.matvec_int4_packed", ["--m", "1024", "--k", "512", "--batch", "8"]),
    ("matrix_vector_multiplication.int4_awq.matvec_int4_packed_add", []),
    ("decode_ffn_swiglu.matvec_int4_swiglu_rms", []),                             # M=16384, K=2048
    ("ffn_swiglu.decode.ffn_decode", []),                                         # dim 128, 4 cols, bf16
    ("ffn_swiglu.decode.ffn_decode", ["--int4", "--hidden", "1024", "--intermediate", "2816", "--batch", "4"]),
    ("ffn_swiglu.prefill.ffn_prefill", []),                                       # seq 16, dim 128
    ("matrix_multiplication.int4_awq.matmul_int4_packed", []),                    # 64 x 128 x 128
    ("matrix_multiplication.int4_awq.matmul_int4_packed", ["--m", "32", "--k", "2048", "--n", "2048"]),
    ("llms.llama32_1b_int4.awq_repacker", []),
    ("llms.llama32_1b_int4.multi_launch_builder.rms_qkv_int4_rope_multi", []),
    ("matrix_vector_multiplication.bf16.matvec", []),                            # 2048 x 8192, bf16 sibling
    ("matrix_vector_multiplication.bf16.matvec", ["--m", "512", "--k", "2048", "--perf-iters", "3"]),
    ("decode_ffn_swiglu.matvec_swiglu_rms", []),                                 # 16384 x 2048, bf16 fused sibling
    ("decode_ffn_swiglu.matvec_swiglu_rms", ["--m", "512", "--k", "1024"]),
    ("silu_and_mul.silu_and_mul", []),                                            # n = 65536   # emb 2048, kv 512, 32/8 heads of 64
]


@pytest.mark.parametrize("module,flags", CASES, ids=[f"{m.split('.')[-1]}{'-' + '_'.join(f) if f else ''}" for m, f in CASES])
def test_example_passes(module, flags):
    r = subprocess.run([sys.executable, "-m", PE + module, *flags], cwd=ROOT, capture_output=True, text=True, timeout=600)
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-2000:]
    assert "PASS" in out, out[-2000:]
