"""SwiGLU FFN prefill (GEMM form) on a B200.

Entry points of mlir-air's ffn_swiglu/prefill/ffn_prefill.py: `build_module(seq_len, dim, num_cols,
np_dtype)` (:40), the column-block weight packing (:295-301), command line (:255-271), golden (:315-322).
Default: the reference's square bf16 case.  `--int4` runs the prefill FFN on AWQ int4 weights (HF layout,
rectangular dims) as two tensor-core GEMMs with SwiGLU in the first one's epilogue:
    --int4 --seq-len 2048 --hidden 4096 --intermediate 11008
"""
import numpy as np
from ml_dtypes import bfloat16

from mlir_air_b200 import layouts
from mlir_air_b200.backend import KernelSpec
from mlir_air_b200.programming_examples import _common as C


def pack_weights(W, dim, dim_n, num_cols):
    """Partition c holds W[:, c * dim_n : (c + 1) * dim_n] row-major."""
    return layouts.pack_ffn_weights_prefill(W, dim, num_cols)


def build_module(seq_len, dim, num_cols, np_dtype=bfloat16):
    if dim % num_cols or dim % 8:
        raise ValueError("dim must be a multiple of num_cols and of 8")
    return KernelSpec("ffn_swiglu", dict(dim=dim, num_cols=num_cols, mode="prefill", seq_len=seq_len))


def cpu_reference(x, W_gate, W_up, W_down):
    xf = x.astype(np.float32)
    gate, up = xf @ W_gate.astype(np.float32).T, xf @ W_up.astype(np.float32).T
    inter = gate * (1.0 / (1.0 + np.exp(-gate))) * up
    return (inter @ W_down.astype(np.float32).T).astype(bfloat16)


def main(argv=None):
    ap = C.base_parser("run.py", "FFN SwiGLU prefill")
    ap.add_argument("--seq-len", type=int, default=16, dest="seq_len")
    ap.add_argument("--dim", type=int, default=128)
    ap.add_argument("--num-cols", type=int, default=4, dest="num_cols")
    ap.add_argument("--output-format", choices=["xclbin", "elf"], default="elf", dest="output_format")
    ap.add_argument("--int4", action="store_true", help="AWQ int4 weights (HF layout), rectangular dims")
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--intermediate", type=int, default=11008)
    args = ap.parse_args(argv)
    if args.int4:
        return _int4(args)
    S, dim, cols = args.seq_len, args.dim, args.num_cols
    spec = build_module(S, dim, cols, bfloat16)
    np.random.seed(0)
    x = (np.random.randn(S, dim) * 0.1).astype(bfloat16)
    Wg, Wu, Wd = ((np.random.randn(dim, dim) * 0.1).astype(bfloat16) for _ in range(3))
    # the kernel consumes B = W^T; partition c of B is (W^T)[:, c-block], which that example stores as
    # W[:, c-block] read row-major -- so the flat buffer round-trips to W itself
    packed = np.concatenate([pack_weights(W, dim, dim // cols, cols) for W in (Wg, Wu, Wd)]).astype(bfloat16)
    xf = x.astype(np.float32)
    g, u = xf @ Wg.astype(np.float32).T, xf @ Wu.astype(np.float32).T
    expected = [g.astype(bfloat16).reshape(-1), u.astype(bfloat16).reshape(-1),
                (g / (1 + np.exp(-g)) * u).astype(bfloat16).reshape(-1), cpu_reference(x, Wg, Wu, Wd).reshape(-1)]
    # rtol / atol are the reference's; the rel-L2 bound is what can actually fail at these magnitudes
    C.finish(args, spec, dict(instance_name="ffn_swiglu"), [x.reshape(-1), packed], expected, rtol=1e0, atol=0.5,
             max_rel_l2=1e-2)


def _int4(args):
    """x [seq, hidden] through gate/up (interleaved columns) + SwiGLU and down on AWQ weights; golden with the
    int4 examples' rounding points (matvec_int4_swiglu_rms.py:511-516 per row, matmul_int4_packed.py:97-105)."""
    from mlir_air_b200.programming_examples.ffn_swiglu.decode.ffn_decode import int4_ffn_inputs
    H, I, S = args.hidden, args.intermediate, args.seq_len
    spec = KernelSpec("ffn_swiglu_int4_prefill", dict(hidden=H, intermediate=I, GS=128, seq_len=S))
    x, gu, down, inter, out = int4_ffn_inputs(H, I, S)
    inputs = [x, gu[0], gu[1], gu[2], down[0], down[1], down[2]]
    C.finish(args, spec, dict(instance_name="ffn_swiglu_int4_prefill"), inputs, [inter, out], rtol=0.15, atol=0.5,
             min_correlation=0.999, max_rel_l2=1e-2)


if __name__ == "__main__":
    main()
