"""HuggingFace AutoAWQ Llama checkpoint -> device-resident layout-A weights for the decode kernels.

The callable of mlir-air's llms/llama32_1b_int4/llama32_1b_int4_weights.py: `load_weights_awq` (:80-238).
The reference turns every linear into two host layouts (a dense bf16 dequant for its bf16 prefill and
a per-tile packed BO for its decode ELFs, with gate/up row-interleaved, :173-205).  The CUDA kernels
read the checkpoint's own layout, so here a linear stays what the file holds -- `qweight int32
[in, out/8]`, `qzeros int32 [in/gs, out/8]`, `scales` rounded fp16 -> bf16 as awq_repacker.py:74-78
does -- and goes to the GPU as it is; gate and up are interleaved column-wise on the device
(awq_b200_interleave_gate_up), which is the layout-A view of the reference's row interleave.

    weights = load_weights_awq("/path/to/awq-checkpoint")        # directory or one .safetensors file
    stack = weights.ffn_stack()                                   # mlir_air_b200.ffn.DecodeFFNStack
    y = stack.forward_host(x)

`read_awq_checkpoint` is the host half alone (numpy, no GPU).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np
from ml_dtypes import bfloat16

# checkpoint prefix -> field, as in the reference (llama32_1b_int4_weights.py:60-68)
_HF_AWQ_LINEARS = {
    "self_attn.q_proj": "wq",
    "self_attn.k_proj": "wk",
    "self_attn.v_proj": "wv",
    "self_attn.o_proj": "wo",
    "mlp.gate_proj": "w_gate",
    "mlp.up_proj": "w_up",
    "mlp.down_proj": "w_down",
}


def _resolve_safetensor_files(model_path: str) -> List[str]:
    """A .safetensors file, or a directory holding model.safetensors.index.json / *.safetensors."""
    if os.path.isfile(model_path):
        return [model_path]
    if not os.path.isdir(model_path):
        raise FileNotFoundError(f"{model_path}: no such file or directory (there is no network: a local "
                                "AutoAWQ checkpoint is needed)")
    index = os.path.join(model_path, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index) as f:
            names = sorted(set(json.load(f)["weight_map"].values()))
        return [os.path.join(model_path, n) for n in names]
    files = sorted(f for f in os.listdir(model_path) if f.endswith(".safetensors"))
    if not files:
        raise FileNotFoundError(f"{model_path}: no .safetensors files")
    return [os.path.join(model_path, f) for f in files]


def _as_bf16(a: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a).astype(bfloat16))


def read_awq_checkpoint(model_path: str, n_layers: Optional[int] = None, group_size: int = 128,
                        with_attention: bool = True) -> Dict:
    """Host half: {"layers": [{"attn_norm", "ffn_norm", "wq": (qweight, qzeros, scales_bf16), ...}],
    "embed_table", "final_norm", "lm_head"} as numpy arrays; the optional tensors are None when the
    file does not hold them.  Raises KeyError for a checkpoint that is not AutoAWQ."""
    from safetensors import safe_open
    key_to_file = {}
    for path in _resolve_safetensor_files(model_path):
        with safe_open(path, framework="numpy") as f:
            for k in f.keys():
                key_to_file[k] = path

    def get(key, required=True):
        if key not in key_to_file:
            if required:
                raise KeyError(f"Missing tensor: {key} (is this an AutoAWQ checkpoint?)")
            return None
        with safe_open(key_to_file[key], framework="numpy") as f:
            return f.get_tensor(key)

    if n_layers is None:
        n_layers = 0
        while f"model.layers.{n_layers}.mlp.down_proj.qweight" in key_to_file:
            n_layers += 1
        if n_layers == 0:
            raise KeyError("Missing tensor: model.layers.0.mlp.down_proj.qweight (is this an AutoAWQ checkpoint?)")
    layers = []
    for i in range(n_layers):
        base = f"model.layers.{i}"
        layer = {"attn_norm": get(f"{base}.input_layernorm.weight", required=False),
                 "ffn_norm": get(f"{base}.post_attention_layernorm.weight")}
        for name in ("attn_norm", "ffn_norm"):
            if layer[name] is not None:
                layer[name] = _as_bf16(layer[name])
        for prefix, fld in _HF_AWQ_LINEARS.items():
            if not with_attention and prefix.startswith("self_attn"):
                continue
            qw = np.ascontiguousarray(get(f"{base}.{prefix}.qweight")).astype(np.int32, copy=False)
            qz = np.ascontiguousarray(get(f"{base}.{prefix}.qzeros")).astype(np.int32, copy=False)
            sc = get(f"{base}.{prefix}.scales")
            K, nb = qw.shape
            if K % group_size or qz.shape != (K // group_size, nb) or sc.shape != (K // group_size, 8 * nb):
                raise ValueError(f"{base}.{prefix}: qweight {qw.shape}, qzeros {qz.shape}, scales {sc.shape} do not "
                                 f"fit group size {group_size}")
            layer[fld] = (qw, qz, _as_bf16(sc))
        layers.append(layer)
    opt = {k: get(k, required=False) for k in ("model.embed_tokens.weight", "model.norm.weight", "lm_head.weight")}
    embed = opt["model.embed_tokens.weight"]
    lm_head = opt["lm_head.weight"] if opt["lm_head.weight"] is not None else embed  # tied embeddings (:228-229)
    return {"layers": layers,
            "embed_table": None if embed is None else _as_bf16(embed),
            "final_norm": None if opt["model.norm.weight"] is None else _as_bf16(opt["model.norm.weight"]),
            "lm_head": None if lm_head is None else _as_bf16(lm_head)}


@dataclass
class AwqLayerWeights:
    """One decoder layer on the device.  Linears are mlir_air_b200.ops.AwqWeight in layout A
    ([in, out]); `w_gateup` is gate and up interleaved column-wise ([hidden, 2 * intermediate])."""
    ffn_norm: "object"
    w_gateup: "object"
    w_down: "object"
    attn_norm: "object" = None
    wq: "object" = None
    wk: "object" = None
    wv: "object" = None
    wo: "object" = None


@dataclass
class AwqLlamaWeights:
    layers: List[AwqLayerWeights] = field(default_factory=list)
    embed_table: Optional[np.ndarray] = None  # host bf16 (the reference keeps these un-quantised)
    final_norm: Optional[np.ndarray] = None
    lm_head: Optional[np.ndarray] = None
    group_size: int = 128

    @property
    def hidden(self) -> int:
        return self.layers[0].w_gateup.K

    @property
    def intermediate(self) -> int:
        return self.layers[0].w_down.K

    def ffn_stack(self, max_batch: int = 64, eps: float = 1e-5, **kwargs):
        """The FFN halves of all layers as a resident decode stack."""
        from mlir_air_b200 import ffn
        return ffn.DecodeFFNStack([ffn.FFNLayer(l.w_gateup, l.w_down, l.ffn_norm) for l in self.layers], self.hidden,
                                  max_batch=max_batch, eps=eps, **kwargs)


def load_weights_awq(model_name_or_path: str, n_layers: Optional[int] = None, group_size: int = 128,
                     device="cuda", with_attention: bool = True) -> AwqLlamaWeights:
    """Load a local AutoAWQ Llama checkpoint onto `device`."""
    import torch
    from mlir_air_b200 import ops
    host = read_awq_checkpoint(model_name_or_path, n_layers, group_size, with_attention)

    def dev_norm(a):
        return None if a is None else torch.from_numpy(a.view(np.int16)).to(device).view(torch.bfloat16)

    out = AwqLlamaWeights(embed_table=host["embed_table"], final_norm=host["final_norm"], lm_head=host["lm_head"],
                          group_size=group_size)
    for i, h in enumerate(host["layers"]):
        lin = {k: ops.AwqWeight.from_numpy(*h[k], group_size, device=device) for k in _HF_AWQ_LINEARS.values() if k in h}
        gate, up = lin.pop("w_gate"), lin.pop("w_up")
        out.layers.append(AwqLayerWeights(ffn_norm=dev_norm(h["ffn_norm"]), attn_norm=dev_norm(h["attn_norm"]),
                                          w_gateup=ops.interleave_gate_up(gate, up), **lin))
        if (i + 1) % 4 == 0 or i == 0:
            print(f"  AWQ layer {i + 1}/{len(host['layers'])} loaded")
    return out
