"""bf16 matrix-vector multiplication  C[m] = sum_k A[m, k] B[k]  on a B200: the un-quantised sibling
of the int4 GEMV (and the form of the LM head, which AWQ checkpoints keep in bf16).

Entry points of mlir-air's matrix_vector_multiplication/bf16/matvec.py: `build_module` (:59) and the
command line with its seeded inputs and tolerances (:172-325).  f32 accumulate, one bf16 rounding.
"""
import numpy as np
from ml_dtypes import bfloat16

from mlir_air_b200.backend import KernelSpec
from mlir_air_b200.programming_examples import _common as C


def build_module(m, k, tile_m=4, m_input=1, herd_m=4, np_dtype_in=bfloat16, np_dtype_out=bfloat16, target="auto"):
    if np_dtype_in != bfloat16 or np_dtype_out != bfloat16:
        raise ValueError("only bf16 in / bf16 out is built")
    if m % (tile_m * herd_m) or tile_m % m_input:
        raise ValueError("m must be a multiple of tile_m * herd_m and tile_m of m_input")
    return KernelSpec("matvec_bf16", dict(M=m, K=k))


def main(argv=None):
    ap = C.base_parser("matvec.py", "Builds, runs, and tests the bf16 matrix-vector multiplication (GEMV) example")
    ap.add_argument("--m", type=int, default=2048)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--tile-m", "--tile-m-l2", type=int, default=4, dest="tile_m")
    ap.add_argument("--m-input", type=int, default=1)
    ap.add_argument("--herd-m", type=int, default=4)
    ap.add_argument("--output-format", choices=["xclbin", "elf"], default="xclbin", dest="output_format")
    ap.add_argument("--compile-mode", choices=["compile-and-run", "compile-and-xclbin"], default="compile-and-run",
                    dest="compile_mode")
    ap.add_argument("--debug-ir", action="store_true", dest="debug_ir")
    ap.add_argument("--perf-iters", type=int, default=0, dest="perf_iters")
    ap.add_argument("--target", type=str, default="auto")
    args = ap.parse_args(argv)
    if args.perf_iters < 0:
        ap.error("--perf-iters must be >= 0")
    spec = build_module(args.m, args.k, args.tile_m, args.m_input, args.herd_m, target=args.target)
    if args.compile_mode == "compile-and-xclbin":
        args.compile_mode = "compile-only"
    np.random.seed(42)
    input_a = (np.random.randn(args.m, args.k) * 4).astype(bfloat16)
    input_b = (np.random.randn(args.k) * 4).astype(bfloat16)
    output_c = np.dot(input_a.astype(np.float32), input_b.astype(np.float32)).astype(bfloat16)
    C.finish(args, spec, dict(instance_name="matvec_bf16", n_perf_iters=args.perf_iters,
                              perf_flops=(2.0 * args.m * args.k) if args.perf_iters > 0 else None),
             [input_a, input_b], [output_c], rtol=1.6e-2, atol=1e-3)


if __name__ == "__main__":
    main()
