"""The C ABI without a GPU: every function declared in include/awq_b200.h is exported by the library
and bound in mlir_air_b200/_lib.py, and argument errors come back as status codes with a message
before anything touches the device."""
import ctypes
import os
import re

from mlir_air_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "awq_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(awq_b200_\w+)\s*\(", text)))


def test_header_library_and_binding_agree():
    names = _declared()
    assert len(names) >= 35
    lib = _lib.load()
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in the header but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes prototype"
    assert sorted(_lib.SIGNATURES) == names, "a bound symbol is missing from the header"
    assert lib.awq_b200_version() >= 100


def _err(rc):
    assert rc != 0
    msg = _lib.last_error()
    assert msg
    return rc, msg


def test_argument_errors_need_no_gpu():
    lib = _lib.load()
    p = ctypes.c_void_p(256)  # a non-null, 16-byte aligned value that is never dereferenced
    INV, UNS = _lib.AWQ_ERR_INVALID_ARGUMENT, _lib.AWQ_ERR_UNSUPPORTED
    # dequant / gemv: shapes
    assert _err(lib.awq_b200_dequant_bf16(p, p, p, p, 100, 64, 128, None))[0] == INV       # K not a multiple of the group
    assert _err(lib.awq_b200_gemv_bf16(p, p, p, p, None, p, 1, 256, 12, 128, p, 1 << 20, None))[0] == INV  # N % 8
    assert _err(lib.awq_b200_gemv_bf16(p, p, p, p, None, p, 65, 256, 64, 128, p, 1 << 20, None))[0] == INV  # batch > 64
    assert _err(lib.awq_b200_gemv_bf16(None, p, p, p, None, p, 1, 256, 64, 128, p, 1 << 20, None))[0] == INV  # null x
    # a misaligned output or residual is an argument error, not a device fault: the kernels move both in 16-byte pieces
    odd = ctypes.c_void_p(256 + 2)
    rc, msg = _err(lib.awq_b200_gemv_bf16(p, p, p, p, None, odd, 1, 256, 64, 128, p, 1 << 20, None))
    assert rc == INV and "output" in msg and "16-byte" in msg
    rc, msg = _err(lib.awq_b200_gemv_bf16(p, p, p, p, odd, p, 1, 256, 64, 128, p, 1 << 20, None))
    assert rc == INV and "residual" in msg
    assert _err(lib.awq_b200_gemv_f32(p, p, p, p, ctypes.c_void_p(256 + 8), 1, 256, 64, 128, p, 1 << 20, None))[0] == INV
    assert _err(lib.awq_b200_gateup_swiglu_bf16(p, p, p, p, odd, 1, 256, 64, 128, p, 1 << 20, None))[0] == INV
    assert _err(lib.awq_b200_gemv_bf16_static(p, p, p, p, None, odd, 1, 256, 64, 128, None))[0] == INV
    assert _err(lib.awq_b200_gemv_bf16_static(p, p, p, p, odd, p, 1, 256, 64, 128, None))[0] == INV
    # the limit of device-side waits
    assert _err(lib.awq_b200_set_wait_limit(-1))[0] == INV
    assert lib.awq_b200_set_wait_limit(1 << 20) == 0 and lib.awq_b200_set_wait_limit(0) == 0
    # rope
    rc, msg = _err(lib.awq_b200_rope_halfsplit_bf16(p, 256, p, p, 256, 1, 4, 40, None))
    assert rc == INV and "head_dim" in msg
    assert _err(lib.awq_b200_rope_halfsplit_bf16(p, 100, p, p, 256, 2, 4, 64, None))[0] == INV  # row stride too small
    # one-launch stack: plan and decode
    arr = (ctypes.c_void_p * 1)(256)
    assert _err(lib.awq_b200_ffn_stack_plan(p, 1 << 20, 0, arr, arr, arr, arr, arr, arr, arr, 512, 1024, 128))[0] == INV
    assert _err(lib.awq_b200_ffn_stack_plan(p, 1 << 20, 1, None, arr, arr, arr, arr, arr, arr, 512, 1024, 128))[0] == INV
    assert lib.awq_b200_ffn_stack_plan_bytes(3) == 3 * lib.awq_b200_ffn_stack_plan_bytes(1) > 0
    assert lib.awq_b200_ffn_stack_workspace_bytes(80) > lib.awq_b200_ffn_stack_workspace_bytes(1) > 0
    assert lib.awq_b200_ffn_stack_decode_bf16(p, 1, p, p, p, 1e-5, 0, 512, 1024, 128, p, 1 << 20, None) == 0  # empty batch
    assert _err(lib.awq_b200_ffn_stack_decode_bf16(None, 1, p, p, p, 1e-5, 1, 512, 1024, 128, p, 1 << 20, None))[0] == INV
    assert _err(lib.awq_b200_ffn_stack_decode_bf16(p, 1, p, p, p, 1e-5, 9, 512, 1024, 128, p, 1 << 20, None))[0] == UNS
    # tensor-parallel entry points
    assert _err(lib.awq_b200_ffn_stack_decode_tp_bf16(p, 1, p, p, p, 1e-5, 1, 512, 1024, 128, arr, 1 << 16, 1 << 15, 1, 0, p,
                                                      1 << 20, None))[0] == INV  # a single rank is not tensor parallel
    assert _err(lib.awq_b200_ffn_stack_decode_tp_bf16(p, 1, p, p, p, 1e-5, 1, 512, 1024, 128, arr, 64, 0, 2, 0, p, 1 << 20,
                                                      None))[0] == INV  # slots too small for the receive area
    # receive area of one slot: per rank and 64-column sub-strip of the hidden state 16 x 32 words of 8 bytes
    assert lib.awq_b200_ffn_stack_tp_slot_bytes(8192, 8) == 8 * (8192 // 64) * 16 * 32 * 8
    assert lib.awq_b200_ffn_stack_tp_slot_bytes(1000, 2) == 2 * 2 * 8 * 16 * 32 * 8  # strips of 512 columns, rounded up
    two = (ctypes.c_void_p * 2)(256, 512)
    need = lib.awq_b200_ffn_stack_tp_slot_bytes(512, 2)
    rc, msg = _err(lib.awq_b200_ffn_stack_decode_tp_bf16(p, 1, p, p, p, 1e-5, 1, 512, 1024, 128, two, need + 240, need - 16, 2, 0,
                                                         p, 1 << 20, None))
    assert rc == INV and "tp_slot_bytes" in msg
    assert _err(lib.awq_b200_gemv_f32_push(p, 0, p, p, p, p, 9, 256, 64, 128, arr, 2, 0, p, 1 << 20, None))[0] == INV
    assert _err(lib.awq_b200_tp_reduce_add_rmsnorm_act(p, arr, p, 9, None, 1e-5, p, None, 0, 1, 512, p, None))[0] == INV
    # fused GEMM epilogues
    rc, msg = _err(lib.awq_b200_gemm_fused_bf16(p, p, p, p, p, p, 1, 64, 256, 512, 128, None))
    assert rc == INV and "do not combine" in msg
    # batched-decode GEMMs: formats and epilogues that do not combine are refused before anything is launched
    for fn in (lib.awq_b200_gemm_decode_act, lib.awq_b200_gemm_decode_f8):
        assert _err(fn(p, 2, p, p, p, None, p, 0, 0, 16, 256, 512, 128, p, 1 << 24, None))[0] == INV  # a_format
        assert _err(fn(p, 0, p, p, p, None, p, 3, 0, 16, 256, 512, 128, p, 1 << 24, None))[0] == INV  # c_format
        assert _err(fn(p, 0, p, p, p, p, p, 0, 1, 16, 256, 512, 128, p, 1 << 24, None))[0] == INV    # SwiGLU + residual
        assert _err(fn(p, 0, p, p, p, p, p, 1, 0, 16, 256, 512, 128, p, 1 << 24, None))[0] == INV    # residual + fp16 output
        assert _err(fn(p, 0, p, p, p, None, p, 2, 1, 16, 256, 512, 128, p, 1 << 24, None))[0] == INV  # f32 sums + SwiGLU
        assert _err(fn(ctypes.c_void_p(258), 0, p, p, p, None, p, 0, 0, 16, 256, 512, 128, p, 1 << 24, None))[0] == INV  # misaligned rows
        assert fn(p, 0, p, p, p, None, p, 0, 0, 0, 256, 512, 128, p, 1 << 24, None) == 0  # empty batch
    # knobs
    assert _err(lib.awq_b200_set_decode_kernel(7))[0] == INV
    assert lib.awq_b200_set_decode_kernel(0) == 0 and lib.awq_b200_set_ffn_stack_tuning(-1, -1) == 0


def test_gemm_decode_f8_workspace_holds_split_rows_and_slots():
    """The fp8-operand GEMM's workspace = the split token rows (two bytes per element of the padded rows, their group sums,
    the rows' powers of two) in front of the 16-bit kernel's slots; it grows with K and N and is 0 for sizes it cannot be."""
    lib = _lib.load()
    for rows, m in ((16, 9), (16, 16), (32, 17), (32, 32)):
        for k in (128, 4096, 28672):
            g = k // 128
            split = g * 2 * rows * 128 + g * rows * 4 + rows * 4
            split = (split + 1023) // 1024 * 1024
            for n in (32, 8192, 57344):
                assert int(lib.awq_b200_gemm_decode_f8_workspace_bytes(m, k, n)) == \
                    split + int(lib.awq_b200_gemm_decode_workspace_bytes(m, n)), (m, k, n)
    assert lib.awq_b200_gemm_decode_f8_workspace_bytes(0, 128, 32) == 0
    assert lib.awq_b200_gemm_decode_f8_workspace_bytes(8, 64, 32) == 0


def test_gemm_decode_workspace_serves_every_narrower_product():
    """A workspace sized for N columns must also serve every product with fewer columns (a tensor-parallel rank runs its
    gate/up shard and the full-width down projection through one workspace): the size may not shrink when N grows."""
    lib = _lib.load()
    for rows in (16, 32, 64):
        prev = 0
        for n in range(32, 65536 + 1, 32):
            b = int(lib.awq_b200_gemm_decode_workspace_bytes(rows, n))
            assert b >= prev, (rows, n, b, prev)
            prev = b
