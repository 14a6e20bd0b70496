"""AutoAWQ checkpoint loader (the callable of llama32_1b_int4_weights.py:80-238): host half on CPU
against a synthetic checkpoint written here; device half on the GPU against the numpy oracle."""
import json
import os

import numpy as np
import pytest
from ml_dtypes import bfloat16

from mlir_air_b200.programming_examples.llms.llama32_1b_int4 import llama32_1b_int4_weights as W
from oracle import awq_oracle as O

H, I, KV, L, GS = 256, 512, 64, 2, 128
SHAPES = {"self_attn.q_proj": (H, H), "self_attn.k_proj": (H, KV), "self_attn.v_proj": (H, KV), "self_attn.o_proj": (H, H),
          "mlp.gate_proj": (H, I), "mlp.up_proj": (H, I), "mlp.down_proj": (I, H)}


def _synthetic_checkpoint(tmp_path, sharded=False, drop=None):
    """A 2-layer AutoAWQ-shaped checkpoint: int32 qweight / qzeros, fp16 scales (what AutoAWQ stores),
    bf16 norms.  Returns the path and the tensors by key."""
    from safetensors.numpy import save_file
    rng = np.random.default_rng(0)
    t = {"model.embed_tokens.weight": rng.standard_normal((32, H)).astype(bfloat16),
         "model.norm.weight": (1 + 0.1 * rng.standard_normal(H)).astype(bfloat16)}
    for i in range(L):
        base = f"model.layers.{i}"
        t[f"{base}.input_layernorm.weight"] = (1 + 0.1 * rng.standard_normal(H)).astype(bfloat16)
        t[f"{base}.post_attention_layernorm.weight"] = (1 + 0.1 * rng.standard_normal(H)).astype(bfloat16)
        for prefix, (K, N) in SHAPES.items():
            t[f"{base}.{prefix}.qweight"] = O.pack_awq_int32(rng.integers(0, 16, (K, N), dtype=np.uint8))
            t[f"{base}.{prefix}.qzeros"] = O.pack_awq_int32(rng.integers(0, 16, (K // GS, N), dtype=np.uint8))
            t[f"{base}.{prefix}.scales"] = rng.uniform(0.001, 0.02, (K // GS, N)).astype(np.float16)
    if drop:
        t.pop(drop)
    d = tmp_path / "ckpt"
    d.mkdir()
    if not sharded:
        save_file(t, str(d / "model.safetensors"))
    else:
        keys = sorted(t)
        parts = {"model-00001-of-00002.safetensors": keys[::2], "model-00002-of-00002.safetensors": keys[1::2]}
        for name, ks in parts.items():
            save_file({k: t[k] for k in ks}, str(d / name))
        with open(d / "model.safetensors.index.json", "w") as f:
            json.dump({"weight_map": {k: name for name, ks in parts.items() for k in ks}}, f)
    return str(d), t


@pytest.mark.parametrize("sharded", [False, True])
def test_read_checkpoint_host_half(tmp_path, sharded):
    path, t = _synthetic_checkpoint(tmp_path, sharded)
    ck = W.read_awq_checkpoint(path)
    assert len(ck["layers"]) == L
    assert np.array_equal(ck["embed_table"].view(np.int16), t["model.embed_tokens.weight"].view(np.int16))
    assert ck["lm_head"] is ck["embed_table"] or np.array_equal(ck["lm_head"].view(np.int16), ck["embed_table"].view(np.int16))
    for i, layer in enumerate(ck["layers"]):
        base = f"model.layers.{i}"
        for prefix, fld in W._HF_AWQ_LINEARS.items():
            qw, qz, sc = layer[fld]
            assert qw.dtype == np.int32 and np.array_equal(qw, t[f"{base}.{prefix}.qweight"])
            assert np.array_equal(qz, t[f"{base}.{prefix}.qzeros"])
            # fp16 scales rounded to bf16, as awq_repacker.py:74-78 does before every use
            assert sc.dtype == bfloat16
            assert np.array_equal(sc.view(np.int16), t[f"{base}.{prefix}.scales"].astype(bfloat16).view(np.int16))
        assert np.array_equal(layer["ffn_norm"].view(np.int16), t[f"{base}.post_attention_layernorm.weight"].view(np.int16))
    # one file given directly, FFN linears only
    if not sharded:
        ck2 = W.read_awq_checkpoint(os.path.join(path, "model.safetensors"), n_layers=1, with_attention=False)
        assert len(ck2["layers"]) == 1 and "wq" not in ck2["layers"][0] and "w_down" in ck2["layers"][0]


def test_read_checkpoint_errors(tmp_path):
    path, _ = _synthetic_checkpoint(tmp_path, drop="model.layers.1.mlp.up_proj.qzeros")
    with pytest.raises(KeyError):
        W.read_awq_checkpoint(path)
    with pytest.raises(FileNotFoundError):
        W.read_awq_checkpoint(str(tmp_path / "nowhere"))
    (tmp_path / "empty").mkdir()
    with pytest.raises(FileNotFoundError):
        W.read_awq_checkpoint(str(tmp_path / "empty"))
    with pytest.raises(ValueError):
        W.read_awq_checkpoint(path, n_layers=1, group_size=64)


@pytest.mark.gpu
def test_loaded_weights_on_the_gpu(tmp_path):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from gpu_util import to_host
    from mlir_air_b200 import ops
    path, t = _synthetic_checkpoint(tmp_path)
    w = W.load_weights_awq(path)
    assert len(w.layers) == L and w.hidden == H and w.intermediate == I
    x = np.random.default_rng(3).standard_normal((4, H)).astype(bfloat16)
    h = x
    for i, layer in enumerate(w.layers):
        base = f"model.layers.{i}"
        raw = {f: tuple(t[f"{base}.{p}.{s}"] for s in ("qweight", "qzeros", "scales")) for p, f in W._HF_AWQ_LINEARS.items()}
        # every linear dequantises bit-exactly to the reference's dense bf16 form
        for fld in ("wq", "wk", "wv", "wo", "w_down"):
            got = to_host(ops.dequant(getattr(layer, fld)))
            assert np.array_equal(got.view(np.int16), O.dequant_to_bf16(*raw[fld], GS).view(np.int16)), (i, fld)
        gu = to_host(ops.dequant(layer.w_gateup))
        assert np.array_equal(gu[:, 0::2].view(np.int16), O.dequant_to_bf16(*raw["w_gate"], GS).view(np.int16))
        assert np.array_equal(gu[:, 1::2].view(np.int16), O.dequant_to_bf16(*raw["w_up"], GS).view(np.int16))
        bf = lambda q: (q[0], q[1], q[2].astype(bfloat16))
        h = O.ffn_layer_A_ref(h, t[f"{base}.post_attention_layernorm.weight"], bf(raw["w_gate"]), bf(raw["w_up"]),
                              bf(raw["w_down"]), GS)
    stack = w.ffn_stack(max_batch=8)
    y = stack.forward_host(x)
    stack.check()
    assert O.rel_l2(y, h) <= 1e-2
