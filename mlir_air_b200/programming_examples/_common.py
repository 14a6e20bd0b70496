"""Shared pieces of the example scripts: flag groups, seeded inputs, vectorised goldens."""
import argparse
import sys

import numpy as np
from ml_dtypes import bfloat16

from mlir_air_b200 import layouts
from mlir_air_b200.backend import B200Backend, B200Runner, KernelSpec


def base_parser(prog, description):
    ap = argparse.ArgumentParser(prog=prog, description=description)
    ap.add_argument("-v", "--verbose", action="store_true")
    ap.add_argument("-p", "--print-module-only", action="store_true")
    return ap


def add_compile_mode(ap, default_format="elf"):
    ap.add_argument("--output-format", choices=["xclbin", "elf"], default=default_format, dest="output_format")
    ap.add_argument("--compile-mode", choices=["compile-and-run", "compile-only"], default="compile-and-run",
                    dest="compile_mode")


def add_gemv_tiling(ap, m, k):
    ap.add_argument("--m", type=int, default=m)
    ap.add_argument("--k", type=int, default=k)
    ap.add_argument("--gs", type=int, default=128)
    ap.add_argument("--m-tile", type=int, default=8, dest="m_tile")
    ap.add_argument("--k-chunk", type=int, default=None, dest="k_chunk",
                    help="K per packed tile (default: min(K, 2048))")
    ap.add_argument("--n-cores", type=int, default=8, dest="n_cores")


def resolve_k_chunk(args):
    if args.k_chunk is None:
        args.k_chunk = min(args.k, 2048)
    return args.k_chunk


def seeded_layout_B(M, K, GS, seed=42):
    """np.random.seed(seed) inputs in the order the reference scripts draw them: nibbles,
    scales ~U(0.005, 0.02), zeros in {7, 8}.  Further draws continue the same stream."""
    np.random.seed(seed)
    unp = np.random.randint(0, 16, size=(M, K), dtype=np.uint8)
    A_q = (unp[:, 0::2] | (unp[:, 1::2] << 4)).astype(np.uint8)
    A_s = np.random.uniform(0.005, 0.02, size=(K // GS, M)).astype(bfloat16)
    A_z = np.random.randint(7, 9, size=(K // GS, M), dtype=np.uint8)
    return A_q, A_s, A_z


def dequant_B(A_q, A_s, A_z):
    """[M, K] f32 weights (nib - z) * s of a layout-B matrix."""
    nibs = layouts.nibbles_of_B(A_q).astype(np.int32)
    gs = nibs.shape[1] // A_s.shape[0]
    s = np.repeat(A_s.astype(np.float32), gs, axis=0).T
    z = np.repeat(A_z.astype(np.int32), gs, axis=0).T
    return (nibs - z) * s


def finish(args, spec, runner_kwargs, inputs, expected, **tol):
    """Common tail of every script: -p, compile-only, or run and check."""
    if args.print_module_only:
        print(spec)
        sys.exit(0)
    if getattr(args, "compile_mode", "compile-and-run") == "compile-only":
        backend = B200Backend(verbose=args.verbose, **runner_kwargs)
        backend.compile(spec)
        backend.unload()
        sys.exit(0)
    runner = B200Runner(verbose=args.verbose, **runner_kwargs)
    sys.exit(runner.run_test(spec, inputs=inputs, expected_outputs=expected, **tol))
