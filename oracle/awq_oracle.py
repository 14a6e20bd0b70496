"""NumPy restatement of mlir-air's int4-AWQ golden path.  TEST INFRASTRUCTURE ONLY.

Every function restates one reference function (cited by path:line inside the
mlir-air tree).  The restatements are pinned against outputs of the reference's
own Python functions, generated once by ``tests/golden/make_golden.py`` and stored
as ``tests/golden/*.npz``; ``tests/test_oracle_golden.py`` replays them.

Layouts
-------
A  (HF AutoAWQ "gemm"):  qweight int32 [K, N/8], qzeros int32 [K/gs, N/8],
   scales [K/gs, N];  nibble at bits [4i+3:4i] of word (k, j) is output column
   8j + AWQ_PACK_ORDER[i].
B  (mlir-air logical):   A_q uint8 [M=N, K/2] (low nibble = even k),
   A_s bf16 [K/gs, M], A_z uint8 [K/gs, M].
C  (per-tile packed BO): see ``pack_inputs_gemv`` / ``pack_inputs_gemm`` /
   ``pack_inputs_dequant``.
"""

from __future__ import annotations

import numpy as np
from ml_dtypes import bfloat16

# programming_examples/llms/llama32_1b_int4/awq_repacker.py:36-38
AWQ_PACK_ORDER = np.array([0, 2, 4, 6, 1, 3, 5, 7], dtype=np.int64)
AWQ_UNPACK_PERM = np.argsort(AWQ_PACK_ORDER)


# ---------------------------------------------------------------------------
# Layout A <-> nibbles
# ---------------------------------------------------------------------------
def unpack_awq_int32(packed: np.ndarray) -> np.ndarray:
    """int32 [..., N/8] -> uint8 nibbles [..., N].

    awq_repacker.py:41-54 (also awq_pack.py:66-76).  Done with uint32 shifts per
    nibble position instead of an (..., 8) int64 temporary; same result.
    """
    p = np.ascontiguousarray(packed).view(np.uint32)
    out = np.empty(p.shape[:-1] + (p.shape[-1], 8), dtype=np.uint8)
    for i in range(8):
        out[..., AWQ_PACK_ORDER[i]] = (p >> np.uint32(4 * i)) & np.uint32(0xF)
    return out.reshape(*p.shape[:-1], p.shape[-1] * 8)


def pack_awq_int32(nibs: np.ndarray) -> np.ndarray:
    """uint8 nibbles [..., N] -> int32 [..., N/8]; the packing loop of
    awq_repacker.py:155-162 (`_gen_synthetic_awq`)."""
    n = nibs.shape[-1]
    assert n % 8 == 0
    acc = np.zeros(nibs.shape[:-1] + (n // 8,), dtype=np.uint32)
    for i in range(8):
        col = int(AWQ_PACK_ORDER[i])
        acc |= (nibs[..., col::8].astype(np.uint32) & np.uint32(0xF)) << np.uint32(4 * i)
    return acc.view(np.int32)


def gen_synthetic_awq(K, N, group_size, seed=42):
    """awq_repacker.py:143-163: same rng call order, so same tensors for a seed."""
    rng = np.random.default_rng(seed)
    n_groups = K // group_size
    nibs = rng.integers(0, 16, size=(K, N), dtype=np.uint8)
    z_nibs = rng.integers(0, 16, size=(n_groups, N), dtype=np.uint8)
    scales = rng.uniform(0.005, 0.02, size=(n_groups, N)).astype(np.float16)
    return pack_awq_int32(nibs), pack_awq_int32(z_nibs), scales, nibs, z_nibs


def dequant_to_bf16(qweight, qzeros, scales, group_size):
    """Layout A -> dense bf16 [K, N];  awq_repacker.py:57-82.

    w = bf16_rne((q - z) * float(bf16(s))).  The f32 product is exact (|q-z| <= 15
    times an 8-bit significand), so there is exactly one rounding.
    """
    q = unpack_awq_int32(qweight)
    z = unpack_awq_int32(qzeros)
    K, N = q.shape
    n_groups = K // group_size
    if z.shape != (n_groups, N):
        raise ValueError(f"qzeros shape {z.shape} vs expected ({n_groups}, {N})")
    if scales.shape != (n_groups, N):
        raise ValueError(f"scales shape {scales.shape} vs expected ({n_groups}, {N})")
    s = scales.astype(bfloat16).astype(np.float32)
    out = np.empty((K, N), dtype=bfloat16)
    for g in range(n_groups):  # group by group: no [K, N] repeat temporaries
        sl = slice(g * group_size, (g + 1) * group_size)
        d = q[sl].astype(np.int32) - z[g].astype(np.int32)[None, :]
        out[sl] = (d.astype(np.float32) * s[g][None, :]).astype(bfloat16)
    return out


def dequant_f32(qweight, qzeros, scales, group_size):
    """(q - z) * s kept in f32 (no bf16 rounding): the weight the GEMV/GEMM goldens
    multiply by (matvec_int4_packed.py:283-286, matmul_int4_packed.py:97-103)."""
    q = unpack_awq_int32(qweight).astype(np.int32)
    z = unpack_awq_int32(qzeros).astype(np.int32)
    s = scales.astype(bfloat16).astype(np.float32)
    zk = np.repeat(z, group_size, axis=0)
    sk = np.repeat(s, group_size, axis=0)
    return ((q - zk) * sk).astype(np.float32)


# ---------------------------------------------------------------------------
# Layout A <-> B
# ---------------------------------------------------------------------------
def repack_hf_awq_linear(qweight, qzeros, scales, group_size):
    """A -> B;  awq_repacker.py:85-109."""
    q = unpack_awq_int32(qweight)
    z = unpack_awq_int32(qzeros)
    K, N = q.shape
    n_groups = K // group_size
    if z.shape != (n_groups, N) or scales.shape != (n_groups, N):
        raise ValueError("qzeros/scales shape mismatch")
    q_mn = np.ascontiguousarray(q.T)
    A_q = ((q_mn[:, 0::2] & 0x0F) | ((q_mn[:, 1::2] & 0x0F) << 4)).astype(np.uint8)
    A_s = np.ascontiguousarray(scales).astype(bfloat16)
    A_z = np.ascontiguousarray(z).astype(np.uint8)
    return A_q, A_s, A_z


def nibbles_from_B(A_q):
    """uint8 [M, K/2] -> nibbles [M, K] (low nibble = even k);
    matvec_int4_swiglu_rms.py:502-507."""
    M, Kh = A_q.shape
    nibs = np.empty((M, 2 * Kh), dtype=np.uint8)
    nibs[:, 0::2] = A_q & 0x0F
    nibs[:, 1::2] = (A_q >> 4) & 0x0F
    return nibs


def layout_B_to_A(A_q, A_s, A_z):
    """Inverse of ``repack_hf_awq_linear``: B -> A (scales stay bf16)."""
    nibs = nibbles_from_B(A_q)  # [M, K]
    qweight = pack_awq_int32(np.ascontiguousarray(nibs.T))
    qzeros = pack_awq_int32(np.ascontiguousarray(A_z))
    return qweight, qzeros, np.ascontiguousarray(A_s).astype(bfloat16)


# ---------------------------------------------------------------------------
# Layout B -> C (per-tile packed BOs) and back
# ---------------------------------------------------------------------------
def gemv_tile_bytes(M_TILE, K_CHUNK, GS):
    n_gpc = K_CHUNK // GS
    q_bytes = M_TILE * (K_CHUNK // 2)
    s_bytes = n_gpc * M_TILE * 2
    z_bytes = n_gpc * M_TILE
    return q_bytes, s_bytes, z_bytes, q_bytes + s_bytes + z_bytes


def _gemv_tile_coords(M, K, M_TILE, K_CHUNK, N_CORES, M_PER_LAUNCH):
    """Tile order (launch, core, outer, kc) of matvec_int4_packed.py:77-87."""
    m_pc = M_PER_LAUNCH // N_CORES
    for lj in range(M // M_PER_LAUNCH):
        for c in range(N_CORES):
            for outer in range(m_pc // M_TILE):
                row = lj * M_PER_LAUNCH + c * m_pc + outer * M_TILE
                for kc in range(K // K_CHUNK):
                    yield row, kc


def pack_inputs_gemv(A_q, A_s, A_z, M, K, GS, M_TILE, K_CHUNK, N_CORES, M_PER_LAUNCH):
    """B -> C for the GEMV examples;  matvec_int4_packed.py:57-103."""
    n_gpc = K_CHUNK // GS
    q_bytes, s_bytes, _, tile_bytes = gemv_tile_bytes(M_TILE, K_CHUNK, GS)
    coords = list(_gemv_tile_coords(M, K, M_TILE, K_CHUNK, N_CORES, M_PER_LAUNCH))
    packed = np.zeros((len(coords), tile_bytes), dtype=np.uint8)
    for t, (row, kc) in enumerate(coords):
        qc = kc * (K_CHUNK // 2)
        g0 = kc * n_gpc
        p = packed[t]
        p[:q_bytes] = np.ascontiguousarray(A_q[row:row + M_TILE, qc:qc + K_CHUNK // 2]).reshape(-1)
        p[q_bytes:q_bytes + s_bytes] = (
            np.ascontiguousarray(A_s[g0:g0 + n_gpc, row:row + M_TILE]).view(np.uint8).reshape(-1))
        p[q_bytes + s_bytes:] = np.ascontiguousarray(A_z[g0:g0 + n_gpc, row:row + M_TILE]).reshape(-1)
    return packed


def unpack_inputs_gemv(packed, M, K, GS, M_TILE, K_CHUNK, N_CORES, M_PER_LAUNCH):
    """C -> B: inverse of ``pack_inputs_gemv``."""
    n_gpc = K_CHUNK // GS
    q_bytes, s_bytes, _, tile_bytes = gemv_tile_bytes(M_TILE, K_CHUNK, GS)
    packed = np.asarray(packed, dtype=np.uint8).reshape(-1, tile_bytes)
    A_q = np.zeros((M, K // 2), dtype=np.uint8)
    A_s = np.zeros((K // GS, M), dtype=bfloat16)
    A_z = np.zeros((K // GS, M), dtype=np.uint8)
    for t, (row, kc) in enumerate(_gemv_tile_coords(M, K, M_TILE, K_CHUNK, N_CORES, M_PER_LAUNCH)):
        qc = kc * (K_CHUNK // 2)
        g0 = kc * n_gpc
        p = packed[t]
        A_q[row:row + M_TILE, qc:qc + K_CHUNK // 2] = p[:q_bytes].reshape(M_TILE, K_CHUNK // 2)
        A_s[g0:g0 + n_gpc, row:row + M_TILE] = (
            np.ascontiguousarray(p[q_bytes:q_bytes + s_bytes]).view(bfloat16).reshape(n_gpc, M_TILE))
        A_z[g0:g0 + n_gpc, row:row + M_TILE] = p[q_bytes + s_bytes:].reshape(n_gpc, M_TILE)
    return A_q, A_s, A_z


def pack_inputs_gemm(W_q, W_s, W_z, M, K, N, GS, N_TILE, K_CHUNK):
    """B -> C for the prefill GEMM;  matmul_int4_packed.py:57-86.
    Result [N/N_TILE, K/K_CHUNK, tile_bytes]."""
    n_gpc = K_CHUNK // GS
    q_bytes, s_bytes, _, tile_bytes = gemv_tile_bytes(N_TILE, K_CHUNK, GS)
    packed = np.zeros((N // N_TILE, K // K_CHUNK, tile_bytes), dtype=np.uint8)
    for no in range(N // N_TILE):
        c0 = no * N_TILE
        for ko in range(K // K_CHUNK):
            qc = ko * (K_CHUNK // 2)
            g0 = ko * n_gpc
            p = packed[no, ko]
            p[:q_bytes] = np.ascontiguousarray(W_q[c0:c0 + N_TILE, qc:qc + K_CHUNK // 2]).reshape(-1)
            p[q_bytes:q_bytes + s_bytes] = (
                np.ascontiguousarray(W_s[g0:g0 + n_gpc, c0:c0 + N_TILE]).view(np.uint8).reshape(-1))
            p[q_bytes + s_bytes:] = np.ascontiguousarray(W_z[g0:g0 + n_gpc, c0:c0 + N_TILE]).reshape(-1)
    return packed


def unpack_inputs_gemm(packed, K, N, GS, N_TILE, K_CHUNK):
    """C -> B: inverse of ``pack_inputs_gemm``."""
    n_gpc = K_CHUNK // GS
    q_bytes, s_bytes, _, tile_bytes = gemv_tile_bytes(N_TILE, K_CHUNK, GS)
    packed = np.asarray(packed, dtype=np.uint8).reshape(N // N_TILE, K // K_CHUNK, tile_bytes)
    W_q = np.zeros((N, K // 2), dtype=np.uint8)
    W_s = np.zeros((K // GS, N), dtype=bfloat16)
    W_z = np.zeros((K // GS, N), dtype=np.uint8)
    for no in range(N // N_TILE):
        c0 = no * N_TILE
        for ko in range(K // K_CHUNK):
            qc = ko * (K_CHUNK // 2)
            g0 = ko * n_gpc
            p = packed[no, ko]
            W_q[c0:c0 + N_TILE, qc:qc + K_CHUNK // 2] = p[:q_bytes].reshape(N_TILE, K_CHUNK // 2)
            W_s[g0:g0 + n_gpc, c0:c0 + N_TILE] = (
                np.ascontiguousarray(p[q_bytes:q_bytes + s_bytes]).view(bfloat16).reshape(n_gpc, N_TILE))
            W_z[g0:g0 + n_gpc, c0:c0 + N_TILE] = p[q_bytes + s_bytes:].reshape(n_gpc, N_TILE)
    return W_q, W_s, W_z


def dequant_tile_bytes(n_tile, group_size):
    """dequant_awq/dequant_awq.py:59-69."""
    ng = n_tile // group_size
    q_bytes, s_bytes, z_bytes = n_tile // 2, 2 * ng, ng
    return q_bytes, s_bytes, z_bytes, (q_bytes + s_bytes + z_bytes + 3) & ~3


def pack_inputs_dequant(int4_vals, scales, zeros, n, group_size, herd_n):
    """1-D dequant example packing;  dequant_awq/dequant_awq.py:259-278."""
    n_tile = n // herd_n
    ng = n_tile // group_size
    q_bytes, s_bytes, z_bytes, tile_bytes = dequant_tile_bytes(n_tile, group_size)
    pq = (int4_vals[0::2] | (int4_vals[1::2] << 4)).astype(np.uint8)
    packed = np.zeros((herd_n, tile_bytes), dtype=np.uint8)
    for ty in range(herd_n):
        bo = packed[ty]
        bo[:q_bytes] = pq[ty * n_tile // 2:(ty + 1) * n_tile // 2]
        bo[q_bytes:q_bytes + s_bytes] = np.ascontiguousarray(scales[ty * ng:(ty + 1) * ng]).view(np.uint8)
        bo[q_bytes + s_bytes:q_bytes + s_bytes + z_bytes] = zeros[ty * ng:(ty + 1) * ng]
    return packed


def dequant_1d(int4_vals, scales, zeros, group_size):
    """Golden of the 1-D dequant example;  dequant_awq/dequant_awq.py:391-396."""
    g = np.arange(int4_vals.shape[0]) // group_size
    d = int4_vals.astype(np.float32) - zeros.astype(np.float32)[g]
    return (d * scales.astype(np.float32)[g]).astype(bfloat16)


# ---------------------------------------------------------------------------
# Goldens on layout B (the examples' cpu_reference functions)
# ---------------------------------------------------------------------------
def dequant_B_f32(A_q, A_s, A_z):
    """[M, K] f32 (nib - z) * s;  matvec_int4_swiglu_rms.py:501-510."""
    nibs = nibbles_from_B(A_q).astype(np.int32)
    gs = nibs.shape[1] // A_s.shape[0]
    s = np.repeat(A_s.astype(np.float32), gs, axis=0)
    z = np.repeat(A_z.astype(np.int32), gs, axis=0)
    return ((nibs - z.T) * s.T).astype(np.float32)


def gemv_ref(A_q, A_s, A_z, B):
    """D = bf16(dequant @ B), f32 accumulate;  matvec_int4_packed.py:272-287
    (vectorised; the scalar loop there differs only in f32 summation order)."""
    return (dequant_B_f32(A_q, A_s, A_z) @ B.astype(np.float32)).astype(bfloat16)


def gemv_add_ref(A_q, A_s, A_z, B, R):
    """D = bf16(dequant @ B + R), one rounding;  matvec_int4_packed_add.py:302-319."""
    acc = dequant_B_f32(A_q, A_s, A_z) @ B.astype(np.float32)
    return (acc + R.astype(np.float32)).astype(bfloat16)


def rmsnorm_ref(x, w, eps=1e-5):
    """bf16(x * rsqrt(mean(x^2) + eps) * w);  matvec_int4_swiglu_rms.py:496-500."""
    xf = x.astype(np.float32)
    wf = w.astype(np.float32)
    mean_sq = float((xf * xf).sum()) / xf.shape[-1]
    rstd = 1.0 / np.sqrt(mean_sq + eps)
    return ((xf * rstd) * wf).astype(bfloat16)


def swiglu_pair_ref(raw_f32):
    """raw [2I] (gate/up row-interleaved) -> bf16 [I];
    matvec_int4_swiglu_rms.py:512-516: raw -> bf16 -> silu via tanh -> bf16."""
    r = raw_f32.astype(bfloat16).astype(np.float32)
    gate, up = r[..., 0::2], r[..., 1::2]
    silu = gate * 0.5 * (np.tanh(gate / 2.0) + 1.0)
    return (silu * up).astype(bfloat16)


def swiglu_rms_ref(A_q, A_s, A_z, RMS_in, eps=1e-5):
    """RMSNorm -> interleaved gate/up GEMV -> SwiGLU;  matvec_int4_swiglu_rms.py:490-516."""
    normed = rmsnorm_ref(RMS_in[0], RMS_in[1], eps).astype(np.float32)
    return swiglu_pair_ref(dequant_B_f32(A_q, A_s, A_z) @ normed)


def gemm_ref(W_q, W_s, W_z, A):
    """C = bf16(A_f32 @ W_dq_f32);  matmul_int4_packed.py:89-105."""
    return (A.astype(np.float32) @ dequant_B_f32(W_q, W_s, W_z).T).astype(bfloat16)


def ffn_bf16_ref(x, W_gate, W_up, W_down):
    """All-f32 SwiGLU FFN on bf16 weights;  ffn_swiglu/decode/ffn_decode.py:306-313 (x [dim])
    and ffn_swiglu/prefill/ffn_prefill.py:315-322 (x [seq, dim]); W are [out, in]."""
    xf = x.astype(np.float32)
    gate = xf @ W_gate.astype(np.float32).T
    up = xf @ W_up.astype(np.float32).T
    inter = gate * (1.0 / (1.0 + np.exp(-gate))) * up
    return (inter @ W_down.astype(np.float32).T).astype(bfloat16)


def transpose_32bit_words(A, M, K):
    """ffn_swiglu/decode/ffn_decode.py:39-45."""
    if M % 16 != 0:
        raise ValueError(f"M must be divisible by 16; got M={M}.")
    if K % 8 != 0:
        raise ValueError(f"K must be divisible by 8; got K={K}.")
    return A.reshape(M, K // 2, 2).transpose(1, 0, 2).reshape(-1)


def pack_ffn_weights_decode(W, dim, dim_m, num_cols):
    """`pack_weights_partitioned`, ffn_swiglu/decode/ffn_decode.py:287-292."""
    return np.concatenate([
        transpose_32bit_words(W[c * dim_m:(c + 1) * dim_m, :], dim_m, dim) for c in range(num_cols)])


def pack_ffn_weights_prefill(W, dim, dim_n, num_cols):
    """`pack_weights`, ffn_swiglu/prefill/ffn_prefill.py:295-301."""
    return np.concatenate([W[:, c * dim_n:(c + 1) * dim_n].reshape(-1) for c in range(num_cols)])


# ---------------------------------------------------------------------------
# Goldens on layout A (the layout the CUDA library consumes)
# ---------------------------------------------------------------------------
def gemv_A_ref(x, qweight, qzeros, scales, group_size, residual=None):
    """y[B, N] = bf16(x_f32 @ ((q - z) s)_f32 (+ residual)); the layout-A form of
    matvec_int4_packed.py:272-287 / matvec_int4_packed_add.py:302-319 (batched as in
    matmul_int4_packed.py:104-105)."""
    acc = np.atleast_2d(x).astype(np.float32) @ dequant_f32(qweight, qzeros, scales, group_size)
    if residual is not None:
        acc = acc + np.atleast_2d(residual).astype(np.float32)
    return acc.astype(bfloat16)


def gateup_swiglu_A_ref(x, gate, up, group_size, gamma=None, eps=1e-5):
    """Layout-A form of matvec_int4_swiglu_rms.py:490-516 with separate gate / up
    matrices (each a (qweight, qzeros, scales) triple); x [B, K]."""
    x = np.atleast_2d(x)
    if gamma is not None:
        x = np.stack([rmsnorm_ref(r, gamma, eps) for r in x])
    xf = x.astype(np.float32)
    g = (xf @ dequant_f32(*gate, group_size)).astype(bfloat16).astype(np.float32)
    u = (xf @ dequant_f32(*up, group_size)).astype(bfloat16).astype(np.float32)
    silu = g * 0.5 * (np.tanh(g / 2.0) + 1.0)
    return (silu * u).astype(bfloat16)


def ffn_A_ref(x, gate, up, down, group_size, gamma=None, eps=1e-5, residual=None):
    """Decode FFN on AWQ weights: down(swiglu(gate x, up x)) (+ residual), with the
    rounding points of matvec_int4_swiglu_rms.py:511-516 and
    matvec_int4_packed_add.py:313-319."""
    t = gateup_swiglu_A_ref(x, gate, up, group_size, gamma, eps)
    return gemv_A_ref(t, *down, group_size, residual=residual)


def ffn_layer_A_ref(h, gamma, gate, up, down, group_size, eps=1e-5):
    """One layer of the decode stack: h <- bf16(h + down(swiglu(gateup . rmsnorm(h, gamma))));
    the LGU -> LD chain of o_gemv_ffn_int4_multi.py:9-12 without the O projection."""
    return ffn_A_ref(h, gate, up, down, group_size, gamma=gamma, eps=eps, residual=h)


def rms_norm_1d_ref(x, weight, eps=1e-5):
    """bf16(x / sqrt(mean(x^2) + eps) * w): the RMSNorm golden of the QKV block
    (rms_qkv_int4_rope_multi.py:527-530); x may be [K] or [B, K]."""
    xf = np.asarray(x).astype(np.float32)
    rms = np.sqrt(np.mean(xf ** 2, axis=-1, keepdims=True) + np.float32(eps))
    return (xf / rms * np.asarray(weight).astype(np.float32)).astype(bfloat16)


def rope_lut_ref(head_dim, rope_base, seq_len, dtype=bfloat16):
    """[seq_len, head_dim] rows [cos(pos f_i) | sin(pos f_i)], f_i = base^(-2i / head_dim), formed in
    f64 (llama32_1b/llama32_1b_weights.py:395-440)."""
    inv_freq = 1.0 / (float(rope_base) ** (np.arange(0, head_dim, 2, dtype=np.float64) / head_dim))
    ang = np.outer(np.arange(seq_len, dtype=np.float64), inv_freq)
    return np.concatenate([np.cos(ang), np.sin(ang)], axis=1).astype(dtype)


def rope_halfsplit_ref(x_flat, lut_flat, head_dim):
    """Half-split RoPE over consecutive heads of head_dim values, one LUT row per head
    (rms_qkv_int4_rope_multi.py:533-551): f32 arithmetic, one bf16 rounding."""
    half = head_dim // 2
    x = np.asarray(x_flat).astype(np.float32).reshape(-1, head_dim)
    lut = np.asarray(lut_flat).astype(np.float32).reshape(-1, head_dim)
    c, s_ = lut[:, :half], lut[:, half:]
    x1, x2 = x[:, :half], x[:, half:]
    out = np.empty_like(x)
    out[:, :half] = x1 * c - x2 * s_
    out[:, half:] = x1 * s_ + x2 * c
    return out.astype(bfloat16).reshape(np.asarray(x_flat).shape)


def rms_qkv_rope_A_ref(x, norm_w, wq, wk, wv, lut_rows, n_heads, n_kv_heads, head_dim, group_size, eps=1e-5):
    """The QKV block for a batch: normed = rmsnorm(x); q, k, v = bf16(normed @ W) with layout-A weights;
    RoPE on q and k with one LUT row per token.  Returns (q_roped, k_roped, v)."""
    normed = rms_norm_1d_ref(x, norm_w, eps)
    q, k, v = (gemv_A_ref(normed, *w, group_size) for w in (wq, wk, wv))
    B = normed.shape[0]
    lut_rows = np.asarray(lut_rows).reshape(B, head_dim)
    q_r = rope_halfsplit_ref(q, np.repeat(lut_rows, n_heads, axis=0), head_dim)
    k_r = rope_halfsplit_ref(k, np.repeat(lut_rows, n_kv_heads, axis=0), head_dim)
    return q_r, k_r, v


def rel_l2(actual, expected):
    a = np.asarray(actual).astype(np.float64).ravel()
    e = np.asarray(expected).astype(np.float64).ravel()
    return float(np.linalg.norm(a - e) / max(np.linalg.norm(e), 1e-30))
