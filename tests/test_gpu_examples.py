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
    ("silu_and_mul.silu_and_mul", []),                                            # n = 65536
    ("ffn_swiglu.prefill.ffn_prefill", ["--int4", "--seq-len", "256", "--hidden", "1024", "--intermediate", "2816"]),
    ("llms.llama32_1b_int4.multi_launch_builder.o_gemv_ffn_int4_multi", []),     # emb 2048, hidden 8192: three stages
    ("llms.llama32_1b_int4.multi_launch_builder.o_gemv_ffn_int4_fused", []),     # the FFN in one launch
    ("llms.llama32_1b_int4.multi_launch_builder.o_gemv_ffn_int4_fused", ["--emb-dim", "1024", "--hidden-dim", "2048", "--k-chunk", "1024"]),
]


@pytest.mark.parametrize("module,flags", CASES, ids=[f"{m.split('.')[-1]}{'-' + '_'.join(f) if f else ''}" for m, f in CASES])
def test_example_passes(module, flags):
    r = subprocess.run([sys.executable, "-m", PE + module, *flags], cwd=ROOT, capture_output=True, text=True, timeout=600)
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-2000:]
    assert "PASS" in out, out[-2000:]


def test_tp_flag_of_the_decode_example():
    """`ffn_decode.py --int4 --tp 2`: two processes, one per GPU; skipped on a box with one GPU."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    r = subprocess.run([sys.executable, "-m", PE + "ffn_swiglu.decode.ffn_decode", "--int4", "--hidden", "1024", "--intermediate",
                        "2816", "--batch", "4", "--tp", "2"], cwd=ROOT, capture_output=True, text=True, timeout=600,
                       env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    out = r.stdout + r.stderr
    assert r.returncode == 0 and "PASS" in out, out[-2000:]


def test_post_attention_block_against_the_reference_fixture():
    """The 15- and 8-argument post-attention blocks through the backend on the inputs of the reference-generated
    fixture, against the reference's own outputs (rel-L2 <= 1e-2; res1 bit-close to the O-projection golden)."""
    import numpy as np
    from ml_dtypes import bfloat16
    from golden_util import load
    from mlir_air_b200.backend import B200Backend
    from mlir_air_b200.programming_examples.matrix_vector_multiplication.int4_awq.matvec_int4_packed import pack_inputs
    from mlir_air_b200.programming_examples.llms.llama32_1b_int4.multi_launch_builder import o_gemv_ffn_int4_fused as f
    from mlir_air_b200.programming_examples.llms.llama32_1b_int4.multi_launch_builder import o_gemv_ffn_int4_multi as m
    from oracle import awq_oracle as O
    g = load("o_gemv_ffn_int4_256x512")
    emb, hid = 256, 512
    pk = lambda k, M, K: pack_inputs(g[k + "_q"], g[k + "_s"], g[k + "_z"], M, K, 128, 8, 256, 4, M)  # noqa: E731
    wo, gu, wd = pk("wo", emb, emb), pk("gu", 2 * hid, emb), pk("wd", emb, hid)
    z = lambda n: np.zeros(n, dtype=bfloat16)  # noqa: E731
    be = B200Backend()
    inv = be.load(be.compile(f.build_o_gemv_ffn_int4_fused_module(emb, hid, 128, 8, 256, 4)))
    res = inv(wo, g["attn_out"], g["x_residual"], gu, g["ffn_norm_w"], wd, z(emb), z(emb))
    be.unload()
    assert O.rel_l2(res[7], g["res1"]) <= 4e-3 and O.rel_l2(res[6], g["fused_out"]) <= 1e-2
    rms = np.zeros((2, emb), dtype=bfloat16)
    rms[1] = g["ffn_norm_w"]
    inv = be.load(be.compile(m.build_o_gemv_ffn_int4_module(emb, hid, 128, 8, 256, 4)))
    res = inv(wo, g["attn_out"], z(emb), g["x_residual"], z(emb), z(emb), rms, gu, z(hid), np.zeros((1, 1), bfloat16), z(hid), z(hid), wd,
              z(emb), z(emb))
    be.unload()
    assert O.rel_l2(res[14], g["multi_out"]) <= 1e-2 and O.rel_l2(res[11], g["swiglu"]) <= 1e-2
    assert O.rel_l2(res[6].reshape(2, emb)[0], g["res1"]) <= 4e-3


def test_bf16_sibling_kernels_against_the_ffn_goldens():
    """awq_b200_linear_bf16 and awq_b200_silu_mul_bf16 directly against the stored goldens of the bf16 FFN examples
    (ffn_decode.py:306-313 at dim 128, ffn_prefill.py:315-322 at 16 x 128), rel-L2 <= 1e-2 on the final output."""
    from golden_util import load
    from gpu_util import to_dev, to_host
    from mlir_air_b200 import ops
    from oracle import awq_oracle as O
    for name in ("ffn_decode_128", "ffn_prefill_16x128"):
        g = load(name)
        x = to_dev(g["x"].reshape(-1, 128))
        gate, up = ops.linear_bf16(x, to_dev(g["W_gate"])), ops.linear_bf16(x, to_dev(g["W_up"]))
        out = to_host(ops.linear_bf16(ops.silu_mul(gate, up), to_dev(g["W_down"])))
        assert O.rel_l2(out.reshape(g["out"].shape), g["out"]) <= 1e-2, name
        xf = g["x"].reshape(-1, 128).astype("float32")
        assert O.rel_l2(to_host(gate), xf @ g["W_gate"].astype("float32").T) <= 1e-2, name
