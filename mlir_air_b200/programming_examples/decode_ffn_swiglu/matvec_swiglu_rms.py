"""bf16 GEMV with RMSNorm on the input and SwiGLU on the output, on a B200: the un-quantised sibling of
matvec_int4_swiglu_rms.py, kept for A/B comparison against the int4 path.

Entry points of mlir-air's decode_ffn_swiglu/matvec_swiglu_rms.py: `build_module` (:97) and the command
line with its seeded inputs, golden and tolerances (:908-1020).  A holds gate and up rows interleaved
(row 2i = gate[i], row 2i+1 = up[i]); the second input is `[2, K]`, row 0 the vector to normalise and
row 1 the RMSNorm weight; the output has M/2 elements.
"""
import numpy as np
from ml_dtypes import bfloat16

from mlir_air_b200.backend import KernelSpec
from mlir_air_b200.programming_examples import _common as C


def build_module(m, k, tile_m=32, m_input=4, herd_cols=8, n_cascade=4, np_dtype_in=bfloat16, np_dtype_out=bfloat16):
    if np_dtype_in != bfloat16 or np_dtype_out != bfloat16:
        raise ValueError("only bf16 in / bf16 out is built")
    if n_cascade < 2 or k % n_cascade or (k // n_cascade) % 64:
        raise ValueError("n_cascade must be >= 2 and split K into chunks that are multiples of 64")
    if m % (tile_m * herd_cols) or tile_m % m_input or m_input % 2 or (tile_m // 2) % 16 or tile_m < 32:
        raise ValueError("M / tile_m / herd_cols / m_input do not tile (gate/up pairs, 16 outputs per tile)")
    return KernelSpec("matvec_swiglu_rms", dict(M=m, K=k, eps=1e-5))


def cpu_reference(input_a, input_rms, eps=1e-5):
    """The golden of the reference's command line (:981-992): RMSNorm rounded to bf16, f32 gate/up
    sums, SiLU through tanh, one bf16 rounding at the end."""
    k = input_a.shape[1]
    x = input_rms[0].astype(np.float32)
    w = input_rms[1].astype(np.float32)
    rstd = 1.0 / np.sqrt(float((x * x).sum()) / k + eps)
    normed = ((x * rstd) * w).astype(bfloat16).astype(np.float32)
    g = input_a[0::2].astype(np.float32) @ normed
    u = input_a[1::2].astype(np.float32) @ normed
    return ((g * 0.5 * (np.tanh(g / 2.0) + 1.0)) * u).astype(bfloat16)


def main(argv=None):
    ap = C.base_parser("matvec_swiglu_rms.py", "BF16 GEMV with fused RMSNorm input and SwiGLU output: swiglu = "
                       "silu(A_interleaved . rms_norm(B[0], B[1])); output is M/2.")
    ap.add_argument("--m", type=int, default=16384)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--tile-m", type=int, default=32, dest="tile_m")
    ap.add_argument("--m-input", type=int, default=4, dest="m_input")
    ap.add_argument("--herd-cols", type=int, default=8, dest="herd_cols")
    ap.add_argument("--n-cascade", type=int, default=4, dest="n_cascade")
    ap.add_argument("--output-format", choices=["xclbin", "elf"], default="elf", dest="output_format")
    ap.add_argument("--compile-mode", choices=["compile-and-run", "compile-and-xclbin"], default="compile-and-run",
                    dest="compile_mode")
    ap.add_argument("--debug-ir", action="store_true", dest="debug_ir")
    args = ap.parse_args(argv)
    spec = build_module(args.m, args.k, args.tile_m, args.m_input, args.herd_cols, args.n_cascade)
    if args.compile_mode == "compile-and-xclbin":
        args.compile_mode = "compile-only"
    np.random.seed(42)
    n_out = args.m // 2
    gate = (np.random.randn(n_out, args.k) * 0.02).astype(bfloat16)
    up = (np.random.randn(n_out, args.k) * 0.02).astype(bfloat16)
    input_a = np.empty((args.m, args.k), dtype=bfloat16)
    input_a[0::2] = gate
    input_a[1::2] = up
    input_vec = np.random.randn(args.k).astype(bfloat16)
    norm_weight = (np.random.randn(args.k) * 0.1 + 1.0).astype(bfloat16)
    input_rms = np.stack([input_vec, norm_weight], axis=0).astype(bfloat16)
    C.finish(args, spec, dict(instance_name="matvec_swiglu_rms"), [input_a, input_rms], [cpu_reference(input_a, input_rms)],
             rtol=0.08, atol=1e-2)


if __name__ == "__main__":
    main()
