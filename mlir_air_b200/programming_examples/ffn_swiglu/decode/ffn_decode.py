"""SwiGLU FFN decode (gate, up, silu*up, down) on a B200.

Entry points of mlir-air's ffn_swiglu/decode/ffn_decode.py: `transpose_32bit_words` (:39),
`build_module(dim, num_cols, np_dtype)` (:49), the flat [gate | up | down] weight packing (:287-299),
command line (:254-269) and golden (:306-313).  Default: the reference's square bf16 case.
`--int4` runs the same four stages on AWQ int4 weights with rectangular dims and a batch:
    --int4 --hidden 4096 --intermediate 11008 --batch 4
`--tp N` (with --int4) splits the layer over N GPUs of this node, one process per GPU: gate/up by columns,
down by rows on group boundaries, one allreduce of the f32 partial sums (NCCL), rank 0 checks the result.
"""
import sys

import numpy as np
from ml_dtypes import bfloat16

from mlir_air_b200 import layouts
from mlir_air_b200.backend import KernelSpec
from mlir_air_b200.programming_examples import _common as C

transpose_32bit_words = layouts.transpose_32bit_words


def pack_weights_partitioned(W, dim, dim_m, num_cols):
    return layouts.pack_ffn_weights_decode(W, dim, num_cols)


def build_module(dim, num_cols, np_dtype=bfloat16):
    if dim % num_cols or (dim // num_cols) % 16 or dim % 8:
        raise ValueError("dim / num_cols must be a multiple of 16 and dim a multiple of 8")
    return KernelSpec("ffn_swiglu", dict(dim=dim, num_cols=num_cols, mode="decode"))


def cpu_reference(x, W_gate, W_up, W_down):
    """All-f32 golden; weights are [out, in]; one bf16 rounding at the end."""
    xf = x.astype(np.float32)
    gate, up = xf @ W_gate.astype(np.float32).T, xf @ W_up.astype(np.float32).T
    inter = gate * (1.0 / (1.0 + np.exp(-gate))) * up
    return (inter @ W_down.astype(np.float32).T).astype(bfloat16)


def main(argv=None):
    ap = C.base_parser("run.py", "FFN SwiGLU decode")
    ap.add_argument("--dim", type=int, default=128)
    ap.add_argument("--num-cols", type=int, default=4, dest="num_cols")
    ap.add_argument("--output-format", choices=["xclbin", "elf"], default="elf", dest="output_format")
    ap.add_argument("--int4", action="store_true", help="AWQ int4 weights (HF layout), rectangular dims")
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--intermediate", type=int, default=11008)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel ranks (GPUs of this node), with --int4")
    args = ap.parse_args(argv)
    if args.tp > 1 and not args.int4:
        ap.error("--tp needs --int4")
    if args.int4:
        return _int4_tp(args) if args.tp > 1 else _int4(args)
    dim, cols = args.dim, args.num_cols
    spec = build_module(dim, cols, bfloat16)
    np.random.seed(0)
    x = (np.random.randn(dim) * 0.1).astype(bfloat16)
    Wg, Wu, Wd = ((np.random.randn(dim, dim) * 0.1).astype(bfloat16) for _ in range(3))
    packed = np.concatenate([pack_weights_partitioned(W, dim, dim // cols, cols) for W in (Wg, Wu, Wd)]).astype(bfloat16)
    bufs = [np.zeros(dim, dtype=bfloat16) for _ in range(3)]
    # the runner treats trailing arguments as outputs: gate / up / inter are checked loosely too
    xf = x.astype(np.float32)
    g, u = Wg.astype(np.float32) @ xf, Wu.astype(np.float32) @ xf
    expected = [g.astype(bfloat16), u.astype(bfloat16), (g / (1 + np.exp(-g)) * u).astype(bfloat16),
                cpu_reference(x, Wg, Wu, Wd)]
    # rtol / atol are the reference's; the rel-L2 bound is what can actually fail at these magnitudes
    C.finish(args, spec, dict(instance_name="ffn_swiglu"), [x, packed], expected, rtol=1e0, atol=0.5, max_rel_l2=1e-2)


def int4_ffn_inputs(H, I, B, gs=128):
    """Seeded AWQ FFN: x [B, H], gate/up interleaved (column 2i = gate_i, 2i + 1 = up_i) and down in HF layout,
    and the golden intermediate and output with the int4 examples' rounding points."""
    from mlir_air_b200.programming_examples.llms.llama32_1b_int4 import awq_repacker as R
    gate = R._gen_synthetic_awq(H, I, gs, seed=1)[:3]
    up = R._gen_synthetic_awq(H, I, gs, seed=2)[:3]
    down = R._gen_synthetic_awq(I, H, gs, seed=3)[:3]
    x = np.random.default_rng(0).standard_normal((B, H)).astype(bfloat16)
    # interleave gate/up columns on the host, once
    nib = np.empty((H, 2 * I), np.uint8)
    nib[:, 0::2], nib[:, 1::2] = R.unpack_awq_int32(gate[0]), R.unpack_awq_int32(up[0])
    zn = np.empty((H // gs, 2 * I), np.uint8)
    zn[:, 0::2], zn[:, 1::2] = R.unpack_awq_int32(gate[1]), R.unpack_awq_int32(up[1])
    sc = np.empty((H // gs, 2 * I), bfloat16)
    sc[:, 0::2], sc[:, 1::2] = gate[2].astype(bfloat16), up[2].astype(bfloat16)
    gu = (layouts.pack_awq_int32(nib), layouts.pack_awq_int32(zn), sc)
    xf = x.astype(np.float32)
    g = (xf @ R.dequant_f32(*gate, gs)).astype(bfloat16).astype(np.float32)
    u = (xf @ R.dequant_f32(*up, gs)).astype(bfloat16).astype(np.float32)
    inter = (g * 0.5 * (np.tanh(g / 2.0) + 1.0) * u).astype(bfloat16)
    out = (inter.astype(np.float32) @ R.dequant_f32(*down, gs)).astype(bfloat16)
    return x, gu, (down[0], down[1], down[2].astype(bfloat16)), inter, out


def _int4(args):
    H, I, B = args.hidden, args.intermediate, args.batch
    spec = KernelSpec("ffn_swiglu_int4", dict(hidden=H, intermediate=I, GS=128))
    x, gu, down, inter, out = int4_ffn_inputs(H, I, B)
    inputs = [x, gu[0], gu[1], gu[2], down[0], down[1], down[2]]
    C.finish(args, spec, dict(instance_name="ffn_swiglu_int4"), inputs, [inter, out], rtol=0.15, atol=0.5,
             min_correlation=0.999, max_rel_l2=1e-2)


def _tp_worker(rank, world, port, H, I, B, ret):
    """One tensor-parallel rank: its column shard of gate/up, its row shard of down, one allreduce."""
    import os
    import torch
    import torch.distributed as dist
    from mlir_air_b200 import ffn, ops
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        x, gu, down, _, out = int4_ffn_inputs(H, I, B)
        i0, i1 = ffn.tp_shard_bounds(I, world)[rank]
        wgu = ops.AwqWeight.from_numpy(*(np.ascontiguousarray(t) for t in ffn.slice_gateup(*gu, i0, i1)), 128)
        wd = ops.AwqWeight.from_numpy(*(np.ascontiguousarray(t) for t in ffn.slice_down(*down, i0, i1)), 128)
        ws = ops.Workspace(max(H, i1 - i0), max(2 * (i1 - i0), H))
        xd = torch.from_numpy(x.view(np.int16)).cuda().view(torch.bfloat16)
        inter = ops.gateup_swiglu(xd, wgu, ws, out_f16=True)
        partial = ops.gemv(inter, wd, ws, f32_out=True, x_f16=True)
        dist.all_reduce(partial)
        y, _ = ops.add_rmsnorm(torch.zeros_like(xd), partial)  # bf16(0 + sum of the ranks' partial sums)
        ws.check()
        if rank == 0:
            a = y.view(torch.int16).cpu().numpy().view(bfloat16).astype(np.float64)
            e = out.astype(np.float64)
            ret["rel_l2"] = float(np.linalg.norm(a - e) / np.linalg.norm(e))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _int4_tp(args):
    import socket
    import torch
    import torch.multiprocessing as mp
    if args.print_module_only:
        print(KernelSpec("ffn_swiglu_int4", dict(hidden=args.hidden, intermediate=args.intermediate, GS=128, tp=args.tp)))
        sys.exit(0)
    if not torch.cuda.is_available() or torch.cuda.device_count() < args.tp:
        print(f"--tp {args.tp} needs {args.tp} GPUs, found {torch.cuda.device_count() if torch.cuda.is_available() else 0}")
        sys.exit(2)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_tp_worker, args=(args.tp, port, args.hidden, args.intermediate, args.batch, ret), nprocs=args.tp, join=True)
        rel = ret.get("rel_l2")
    print(f"Output 0: rel-L2 {rel:.3e} (tp{args.tp}, gate/up column split, down row split, one allreduce)")
    ok = rel is not None and rel <= 1e-2
    print("PASS!" if ok else "failed.")
    sys.exit(0 if ok else -1)


if __name__ == "__main__":
    main()
