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
    "llms.llama32_1b_int4.multi_launch_builder.o_gemv_ffn_int4_multi",
    "llms.llama32_1b_int4.multi_launch_builder.o_gemv_ffn_int4_fused",
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


def test_int4_ffn_flags_name_registered_instances(capsys):
    from mlir_air_b200.backend import _INSTANCES
    from mlir_air_b200.programming_examples.ffn_swiglu.decode import ffn_decode
    from mlir_air_b200.programming_examples.ffn_swiglu.prefill import ffn_prefill
    for mod, flags in ((ffn_prefill, ["--int4", "--hidden", "256", "--intermediate", "512", "--seq-len", "32", "-p"]),
                       (ffn_decode, ["--int4", "--hidden", "256", "--intermediate", "512", "-p"]),
                       (ffn_decode, ["--int4", "--hidden", "256", "--intermediate", "512", "--tp", "2", "-p"])):
        with pytest.raises(SystemExit) as e:
            mod.main(flags)
        assert e.value.code == 0
        m = re.search(r"b200\.kernel @(\w+)\(", capsys.readouterr().out)
        assert m and m.group(1) in _INSTANCES
    with pytest.raises(SystemExit) as e:  # --tp is a property of the int4 path
        ffn_decode.main(["--tp", "2"])
    assert e.value.code != 0


def test_post_attention_block_builders_reject_bad_tilings():
    from mlir_air_b200.programming_examples.llms.llama32_1b_int4.multi_launch_builder import o_gemv_ffn_int4_fused as f
    from mlir_air_b200.programming_examples.llms.llama32_1b_int4.multi_launch_builder import o_gemv_ffn_int4_multi as m
    assert m._packed_dims(2048, 2048, 128, 8, 2048, 8, 2048) == (256, 8576)  # tiles, bytes per tile
    with pytest.raises(ValueError):
        m.build_o_gemv_ffn_int4_module(emb_dim=2048 + 8)
    with pytest.raises(ValueError):
        f.build_module(K=2048, M_LA=1024, M_LGU=16384, K_LD=8192)  # res1 must double as the down projection's residual
    assert f.build_o_gemv_ffn_int4_fused_module(512, 1024, k_chunk=512).params["hidden_dim"] == 1024


def test_post_attention_block_goldens_match_the_reference_fixture():
    """lgu_cpu_reference, ld_cpu_reference and o_gemv_ffn_int4_reference as restated in the mirrors against what
    mlir-air's own functions returned on the same inputs (tests/golden/o_gemv_ffn_int4_256x512.npz)."""
    import numpy as np
    from golden_util import bits, load
    from mlir_air_b200.programming_examples import _common as C
    from mlir_air_b200.programming_examples.llms.llama32_1b_int4.multi_launch_builder import o_gemv_ffn_int4_fused as f
    from mlir_air_b200.programming_examples.llms.llama32_1b_int4.multi_launch_builder import o_gemv_ffn_int4_multi as m
    from ml_dtypes import bfloat16
    g = load("o_gemv_ffn_int4_256x512")
    sw = f.lgu_cpu_reference(g["gu_q"], g["gu_s"], g["gu_z"], g["res1"], g["ffn_norm_w"])
    assert np.array_equal(bits(sw), bits(g["swiglu"]))
    assert np.array_equal(bits(f.ld_cpu_reference(g["wd_q"], g["wd_s"], g["wd_z"], g["swiglu"], g["res1"])), bits(g["fused_out"]))
    deq = lambda k: C.dequant_B(g[k + "_q"], g[k + "_s"], g[k + "_z"]).astype(bfloat16)  # noqa: E731
    gu = deq("gu")
    out = m.o_gemv_ffn_int4_reference(deq("wo"), g["attn_out"], g["x_residual"], g["ffn_norm_w"], gu[0::2], gu[1::2], deq("wd"))
    assert np.array_equal(bits(out), bits(g["multi_out"]))
    # the seeded generator is the reference's
    q, s_, z, d = m._gen_int4_weights(256, 256, 128, 100)
    assert np.array_equal(q, g["wo_q"]) and np.array_equal(bits(s_), bits(g["wo_s"])) and np.array_equal(z, g["wo_z"])
