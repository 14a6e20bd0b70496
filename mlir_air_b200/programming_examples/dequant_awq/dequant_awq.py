"""AWQ-style int4 -> bf16 dequantisation on a B200.

Entry points of mlir-air's dequant_awq/dequant_awq.py: `packed_tile_bytes` (:59), `build_module` (:159),
`pack_inputs` (:259), command line and checks (:286-373), seeded inputs and golden (:382-396).
`--hf K N` switches to the HF AutoAWQ layout (qweight / qzeros / scales -> bf16 [K, N]).
"""
import sys

import numpy as np
from ml_dtypes import bfloat16

from mlir_air_b200 import layouts
from mlir_air_b200.backend import KernelSpec
from mlir_air_b200.programming_examples import _common as C

R_SUB = 64  # inner width of the reference's --direct-codegen body; only constrains its flag check


def packed_tile_bytes(n_tile, group_size):
    return layouts.dequant_tile_bytes(n_tile, group_size)


def pack_inputs(int4_vals, scales, zeros, n, group_size, herd_n):
    return layouts.pack_dequant_tiles(int4_vals, scales, zeros, n, group_size, herd_n)


def build_module(n, group_size, herd_n, direct_codegen=False):
    return KernelSpec("dequant", dict(n=n, group_size=group_size, herd_n=herd_n))


def main(argv=None):
    ap = C.base_parser("dequant_awq.py", "AWQ-style int4 to bf16 dequantization example")
    ap.add_argument("--n", type=int, default=1024, help="Number of elements")
    ap.add_argument("--group-size", type=int, default=128, dest="group_size")
    ap.add_argument("--herd-n", type=int, default=4, dest="herd_n")
    ap.add_argument("--device", choices=["npu1", "npu2"], default=None)
    ap.add_argument("--direct-codegen", action="store_true", dest="direct_codegen")
    ap.add_argument("--hf", type=int, nargs=2, metavar=("K", "N"), default=None,
                    help="dequantise a seeded HF-AutoAWQ weight [K, N] instead of the 1-D example")
    C.add_compile_mode(ap, default_format="xclbin")
    args = ap.parse_args(argv)
    if args.n <= 0 or args.group_size <= 0 or args.herd_n <= 0:
        ap.error("N, group_size and herd_n must be positive")
    if args.n % 2:
        ap.error("N must be even (2 int4 values per byte)")
    if args.direct_codegen and args.group_size % R_SUB:
        ap.error(f"--direct-codegen requires group_size multiple of {R_SUB}")
    if args.direct_codegen and args.device == "npu1":
        ap.error("--direct-codegen is AIE2P only (no npu1 support)")
    if args.group_size % 32:
        ap.error("group_size must be a multiple of 32 (kernel inner vector width)")
    if args.n % args.group_size or args.n % args.herd_n or (args.n // args.herd_n) % args.group_size:
        ap.error("N must be divisible by group_size and herd_n, and N / herd_n by group_size")
    if args.device == "npu1" and args.output_format == "elf":
        ap.error("--output-format=elf is not supported on npu1; use xclbin")

    if args.hf:
        return _hf_mode(args)
    spec = build_module(args.n, args.group_size, args.herd_n, args.direct_codegen)
    np.random.seed(0)
    ng = args.n // args.group_size
    int4_vals = np.random.randint(0, 16, args.n).astype(np.uint8)
    scales = np.random.uniform(0.01, 0.1, ng).astype(bfloat16)
    zeros = np.random.randint(7, 10, ng).astype(np.uint8)
    grp = np.arange(args.n) // args.group_size
    ref = ((int4_vals.astype(np.float32) - zeros.astype(np.float32)[grp]) * scales.astype(np.float32)[grp]).astype(bfloat16)
    packed = pack_inputs(int4_vals, scales, zeros, args.n, args.group_size, args.herd_n)
    C.finish(args, spec, dict(instance_name="dequant"), [packed], [ref], rtol=1e-1, atol=5e-2)


def _hf_mode(args):
    import torch
    from mlir_air_b200 import ops
    from mlir_air_b200.programming_examples.llms.llama32_1b_int4 import awq_repacker as R
    K, N = args.hf
    qw, qz, s, _, _ = R._gen_synthetic_awq(K, N, args.group_size, seed=0)
    out = ops.dequant(ops.AwqWeight.from_numpy(qw, qz, s, args.group_size))
    got = out.view(torch.int16).cpu().numpy().view(np.uint16)
    ok = np.array_equal(got, R.dequant_to_bf16(qw, qz, s, args.group_size).view(np.uint16))
    print("PASS!" if ok else "failed.")
    sys.exit(0 if ok else -1)


if __name__ == "__main__":
    main()
