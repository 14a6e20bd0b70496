"""Generate tests/golden/ffn_stack_70b.npz: the hidden state after each layer of a seeded two-layer
decode-FFN stack at the Llama-3-70B dimensions (hidden 8192, intermediate 28672, batch 8), computed by
the numpy oracle.  CPU only; needs nothing but this repository:

    python tests/golden/make_golden_stack70b.py

The oracle's layer function (oracle.awq_oracle.ffn_layer_A_ref: the chain of
matvec_int4_swiglu_rms.py:490-516 and matvec_int4_packed_add.py:302-319) is applied in column
chunks so that only a slice of a dequantised matrix exists at a time: the gate/up products of a
column chunk are independent, and the down projection is a sum over row chunks (f32, added in chunk
order).  The fixture stores the seeds and the outputs; tests regenerate the weights from the seeds
(tests/golden_util.py: stack70b_layer).
"""
import os
import sys

import numpy as np
from ml_dtypes import bfloat16

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))                   # tests/
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))  # repository root

from golden_util import STACK70B, stack70b_input, stack70b_layer  # noqa: E402
from oracle import awq_oracle as O  # noqa: E402


def layer_chunked(h, gate, up, down, gamma, gs, chunk=2048):
    """ffn_layer_A_ref with bounded memory; same rounding points."""
    I = gate[0].shape[1] * 8
    normed = np.stack([O.rmsnorm_ref(r, gamma) for r in h]).astype(np.float32)
    acc = np.zeros((h.shape[0], down[0].shape[1] * 8), dtype=np.float32)
    for c0 in range(0, I, chunk):
        c1 = min(I, c0 + chunk)
        sl = lambda w: (w[0][:, c0 // 8:c1 // 8], w[1][:, c0 // 8:c1 // 8], w[2][:, c0:c1])  # noqa: E731
        g = (normed @ O.dequant_f32(*sl(gate), gs)).astype(bfloat16).astype(np.float32)
        u = (normed @ O.dequant_f32(*sl(up), gs)).astype(bfloat16).astype(np.float32)
        t = (g * 0.5 * (np.tanh(g / 2.0) + 1.0) * u).astype(bfloat16).astype(np.float32)
        dsl = (down[0][c0:c1], down[1][c0 // gs:c1 // gs], down[2][c0 // gs:c1 // gs])
        acc += t @ O.dequant_f32(*dsl, gs)
    return (acc + h.astype(np.float32)).astype(bfloat16)


def main():
    cfg = STACK70B
    h = stack70b_input(cfg)
    outs = []
    for l in range(cfg["layers"]):
        gate, up, down, gamma = stack70b_layer(l, cfg)
        if l == 0:
            # the chunked form against the oracle's own function on a slice that fits in memory
            k = 1024
            small = tuple((w[0][:, :k // 8], w[1][:, :k // 8], w[2][:, :k]) for w in (gate, up))
            dsmall = (down[0][:k], down[1][:k // 128], down[2][:k // 128])
            a = layer_chunked(h, small[0], small[1], dsmall, gamma, 128, chunk=256)
            b = O.ffn_layer_A_ref(h, gamma, small[0], small[1], dsmall, 128)
            assert O.rel_l2(a, b) < 2e-3, O.rel_l2(a, b)
        h = layer_chunked(h, gate, up, down, gamma, cfg["group_size"])
        outs.append(h.view(np.uint16).copy())
        print(f"layer {l}: |h| = {np.linalg.norm(h.astype(np.float32)):.3f}", flush=True)
    np.savez_compressed(os.path.join(HERE, "ffn_stack_70b.npz"), h=np.stack(outs), __bf16__h=np.zeros(0),
                        **{k: np.int64(v) for k, v in cfg.items()})
    print("wrote ffn_stack_70b.npz")


if __name__ == "__main__":
    main()
