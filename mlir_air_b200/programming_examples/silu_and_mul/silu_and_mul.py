"""SiLU-and-mul  out = silu(gate) * up  on bf16 vectors on a B200 (the activation of the un-quantised
SwiGLU FFN).

Entry points of mlir-air's silu_and_mul/silu_and_mul.py: `build_module` (:37), `silu_reference`
(:251) and the command line with its seeded inputs and tolerances (:255-364).  The golden is the
true sigmoid 1 / (1 + exp(-g)) in f32 with one bf16 rounding, which is what the kernel computes.
"""
import numpy as np
from ml_dtypes import bfloat16

from mlir_air_b200.backend import KernelSpec
from mlir_air_b200.programming_examples import _common as C


def build_module(n, tile_n, np_dtype_in=bfloat16, herd_x=8, herd_y=None):
    herd_y = 1 if herd_y is None else herd_y
    if np_dtype_in != bfloat16:
        raise ValueError("only bf16 is built")
    if n % (tile_n * herd_x * herd_y):
        raise ValueError(f"n ({n}) must be divisible by tile_n * total_tiles ({tile_n * herd_x * herd_y})")
    return KernelSpec("silu_and_mul", dict(n=n))


def silu_reference(x):
    x_f32 = np.asarray(x).astype(np.float32)
    return x_f32 * (1.0 / (1.0 + np.exp(-x_f32)))


def main(argv=None):
    ap = C.base_parser("silu_and_mul.py", "Builds, runs, and tests the SiLU-and-mul example")
    ap.add_argument("--n", type=int, default=65536, help="Total number of elements")
    ap.add_argument("--tile-n", type=int, default=1024, help="Tile size")
    ap.add_argument("--herd-x", type=int, default=8)
    ap.add_argument("--herd-y", type=int, default=None)
    ap.add_argument("--perf-iters", type=int, default=0, dest="perf_iters")
    ap.add_argument("--compile-mode", choices=["compile-only", "compile-and-run"], default="compile-and-run",
                    dest="compile_mode")
    ap.add_argument("--output-format", choices=["xclbin", "elf"], default="xclbin", dest="output_format")
    args = ap.parse_args(argv)
    if args.perf_iters < 0:
        ap.error("--perf-iters must be >= 0")
    spec = build_module(args.n, args.tile_n, bfloat16, herd_x=args.herd_x, herd_y=args.herd_y)
    rng = np.random.default_rng(0)
    gate = rng.standard_normal(args.n, dtype=np.float32).astype(bfloat16)
    up = rng.standard_normal(args.n, dtype=np.float32).astype(bfloat16)
    expected = (silu_reference(gate) * up.astype(np.float32)).astype(bfloat16)
    C.finish(args, spec, dict(instance_name="silu_and_mul", n_perf_iters=args.perf_iters), [gate, up], [expected],
             rtol=1.6e-2, atol=8e-2)


if __name__ == "__main__":
    main()
