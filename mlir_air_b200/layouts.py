"""Host-side (numpy) converters between the three weight layouts of the int4-AWQ path.

A  HF AutoAWQ: qweight int32 [K, N/8], qzeros int32 [K/gs, N/8], scales [K/gs, N]
   (llms/llama32_1b_int4/awq_repacker.py:33-54)
B  mlir-air logical: A_q uint8 [M, K/2] (low nibble = even k), A_s bf16 [K/gs, M], A_z uint8 [K/gs, M]
   (matrix_vector_multiplication/int4_awq/matvec_int4_packed.py:346-350)
C  per-tile packed buffer objects built for the NPU's DMA
   (matvec_int4_packed.py:57-103, matmul_int4_packed.py:57-86, dequant_awq.py:259-278)

These run once per weight; they are whole-array reshapes, not per-tile Python loops.  The
device-side A <-> B converters are in the CUDA library (awq_b200_repack_*).
"""
from __future__ import annotations

import numpy as np
from ml_dtypes import bfloat16

AWQ_PACK_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)


def unpack_awq_int32(packed: np.ndarray) -> np.ndarray:
    """int32 [..., n] -> uint8 nibbles [..., 8 n] in column order."""
    words = np.ascontiguousarray(packed).view(np.uint32)
    cols = np.empty(words.shape + (8,), dtype=np.uint8)
    for pos, col in enumerate(AWQ_PACK_ORDER):
        cols[..., col] = (words >> np.uint32(4 * pos)) & np.uint32(15)
    return cols.reshape(words.shape[:-1] + (words.shape[-1] * 8,))


def pack_awq_int32(nibbles: np.ndarray) -> np.ndarray:
    """uint8 nibbles [..., 8 n] -> int32 [..., n]."""
    nb = np.asarray(nibbles)
    if nb.shape[-1] % 8:
        raise ValueError("last axis must be a multiple of 8")
    grouped = nb.reshape(nb.shape[:-1] + (nb.shape[-1] // 8, 8)).astype(np.uint32) & np.uint32(15)
    words = np.zeros(grouped.shape[:-1], dtype=np.uint32)
    for pos, col in enumerate(AWQ_PACK_ORDER):
        words |= grouped[..., col] << np.uint32(4 * pos)
    return words.view(np.int32)


def nibbles_of_B(A_q: np.ndarray) -> np.ndarray:
    out = np.empty((A_q.shape[0], A_q.shape[1] * 2), dtype=np.uint8)
    out[:, 0::2] = A_q & 15
    out[:, 1::2] = A_q >> 4
    return out


def A_to_B(qweight, qzeros, scales, group_size):
    """What repack_hf_awq_linear produces (awq_repacker.py:85-109)."""
    q = unpack_awq_int32(qweight)
    z = unpack_awq_int32(qzeros)
    if z.shape != (q.shape[0] // group_size, q.shape[1]) or scales.shape != z.shape:
        raise ValueError("qzeros / scales do not match qweight and group_size")
    qt = np.ascontiguousarray(q.T)
    return (qt[:, 0::2] | (qt[:, 1::2] << 4)).astype(np.uint8), np.asarray(scales).astype(bfloat16), z


def B_to_A(A_q, A_s, A_z):
    return (pack_awq_int32(np.ascontiguousarray(nibbles_of_B(A_q).T)), pack_awq_int32(A_z),
            np.ascontiguousarray(A_s).astype(bfloat16))


# ---------------------------------------------------------------------------------------
# layout C: GEMV tiles, ordered (launch, core, outer, k-chunk); each tile is
# [Q: M_TILE x K_CHUNK/2 bytes | S: n_gpc x M_TILE bf16 | Z: n_gpc x M_TILE bytes]
# ---------------------------------------------------------------------------------------
def gemv_tile_bytes(M_TILE, K_CHUNK, GS):
    n_gpc = K_CHUNK // GS
    q, s, z = M_TILE * (K_CHUNK // 2), 2 * n_gpc * M_TILE, n_gpc * M_TILE
    return q, s, z, q + s + z


def _check_gemv_tiling(M, K, GS, M_TILE, K_CHUNK, N_CORES, M_PER_LAUNCH):
    if M % M_PER_LAUNCH or M_PER_LAUNCH % N_CORES or (M_PER_LAUNCH // N_CORES) % M_TILE:
        raise ValueError("M, M_PER_LAUNCH, N_CORES and M_TILE do not tile")
    if K % K_CHUNK or K_CHUNK % GS:
        raise ValueError("K, K_CHUNK and GS do not tile")


def pack_gemv_tiles(A_q, A_s, A_z, M, K, GS, M_TILE, K_CHUNK, N_CORES, M_PER_LAUNCH):
    """B -> C.  (launch, core, outer) enumerate consecutive blocks of M_TILE rows, so the tile
    order is simply (row block, k chunk)."""
    _check_gemv_tiling(M, K, GS, M_TILE, K_CHUNK, N_CORES, M_PER_LAUNCH)
    rb, kd, n_gpc = M // M_TILE, K // K_CHUNK, K_CHUNK // GS
    q = np.asarray(A_q, dtype=np.uint8).reshape(rb, M_TILE, kd, K_CHUNK // 2).transpose(0, 2, 1, 3)
    s = np.ascontiguousarray(np.asarray(A_s).astype(bfloat16)).view(np.uint16).reshape(kd, n_gpc, rb, M_TILE)
    z = np.asarray(A_z, dtype=np.uint8).reshape(kd, n_gpc, rb, M_TILE).transpose(2, 0, 1, 3)
    s_bytes = np.ascontiguousarray(s.transpose(2, 0, 1, 3)).view(np.uint8)
    return np.concatenate([q.reshape(rb * kd, -1), s_bytes.reshape(rb * kd, -1), z.reshape(rb * kd, -1)], axis=1)


def unpack_gemv_tiles(packed, M, K, GS, M_TILE, K_CHUNK, N_CORES, M_PER_LAUNCH):
    """C -> B."""
    _check_gemv_tiling(M, K, GS, M_TILE, K_CHUNK, N_CORES, M_PER_LAUNCH)
    rb, kd, n_gpc = M // M_TILE, K // K_CHUNK, K_CHUNK // GS
    qb, sb, _, tb = gemv_tile_bytes(M_TILE, K_CHUNK, GS)
    t = np.asarray(packed, dtype=np.uint8).reshape(rb, kd, tb)
    A_q = t[:, :, :qb].reshape(rb, kd, M_TILE, K_CHUNK // 2).transpose(0, 2, 1, 3).reshape(M, K // 2)
    s = np.ascontiguousarray(t[:, :, qb:qb + sb]).view(np.uint16).reshape(rb, kd, n_gpc, M_TILE)
    A_s = np.ascontiguousarray(s.transpose(1, 2, 0, 3)).reshape(K // GS, M).view(bfloat16)
    A_z = t[:, :, qb + sb:].reshape(rb, kd, n_gpc, M_TILE).transpose(1, 2, 0, 3).reshape(K // GS, M)
    return np.ascontiguousarray(A_q), A_s, np.ascontiguousarray(A_z)


# GEMM tiles: [N / N_TILE, K / K_CHUNK, tile_bytes], same per-tile structure
def pack_gemm_tiles(W_q, W_s, W_z, K, N, GS, N_TILE, K_CHUNK):
    if N % N_TILE or K % K_CHUNK or K_CHUNK % GS:
        raise ValueError("N, K, N_TILE, K_CHUNK and GS do not tile")
    flat = pack_gemv_tiles(W_q, W_s, W_z, N, K, GS, N_TILE, K_CHUNK, 1, N)
    return flat.reshape(N // N_TILE, K // K_CHUNK, -1)


def unpack_gemm_tiles(packed, K, N, GS, N_TILE, K_CHUNK):
    return unpack_gemv_tiles(np.asarray(packed).reshape(-1, gemv_tile_bytes(N_TILE, K_CHUNK, GS)[3]), N, K, GS,
                             N_TILE, K_CHUNK, 1, N)


# 1-D dequant example: [herd_n, tile_bytes], tile = [Q n_tile/2 | S 2 ng | Z ng | pad to 4]
def dequant_tile_bytes(n_tile, group_size):
    ng = n_tile // group_size
    q, s, z = n_tile // 2, 2 * ng, ng
    return q, s, z, (q + s + z + 3) & ~3


def pack_dequant_tiles(int4_vals, scales, zeros, n, group_size, herd_n):
    n_tile = n // herd_n
    ng = n_tile // group_size
    qb, sb, zb, tb = dequant_tile_bytes(n_tile, group_size)
    out = np.zeros((herd_n, tb), dtype=np.uint8)
    v = np.asarray(int4_vals, dtype=np.uint8)
    out[:, :qb] = (v[0::2] | (v[1::2] << 4)).reshape(herd_n, qb)
    out[:, qb:qb + sb] = np.ascontiguousarray(np.asarray(scales).astype(bfloat16)).view(np.uint8).reshape(herd_n, sb)
    out[:, qb + sb:qb + sb + zb] = np.asarray(zeros, dtype=np.uint8).reshape(herd_n, ng)
    return out


def unpack_dequant_tiles(packed, n, group_size, herd_n):
    """-> (packed nibble bytes [n/2], scales bf16 [n/gs], zeros uint8 [n/gs])"""
    n_tile = n // herd_n
    qb, sb, zb, tb = dequant_tile_bytes(n_tile, group_size)
    t = np.asarray(packed, dtype=np.uint8).reshape(herd_n, tb)
    return (np.ascontiguousarray(t[:, :qb]).reshape(-1), np.ascontiguousarray(t[:, qb:qb + sb]).reshape(-1).view(bfloat16),
            np.ascontiguousarray(t[:, qb + sb:qb + sb + zb]).reshape(-1))


def interleave_rows_gate_up(gate_B, up_B):
    """Row-interleave two layout-B weights (row 2i = gate_i, 2i+1 = up_i), as
    llama32_1b_int4_weights.py:173-205 does for the fused gate/up GEMV."""
    out = []
    for g, u, axis in ((gate_B[0], up_B[0], 0), (gate_B[1], up_B[1], 1), (gate_B[2], up_B[2], 1)):
        shape = list(g.shape)
        shape[axis] *= 2
        m = np.empty(shape, dtype=g.dtype)
        if axis == 0:
            m[0::2], m[1::2] = g, u
        else:
            m[:, 0::2], m[:, 1::2] = g, u
        out.append(m)
    return tuple(out)


# ---------------------------------------------------------------------------------------
# bf16 FFN examples: one flat buffer [gate | up | down], each matrix cut into `num_cols`
# partitions (ffn_swiglu/decode/ffn_decode.py:39-45,287-299; ffn_swiglu/prefill/ffn_prefill.py:295-301)
# ---------------------------------------------------------------------------------------
def transpose_32bit_words(A, M, K):
    """A[M, K] row-major -> 32-bit-word-transposed: pairs of k stay together, rows vary fastest."""
    if M % 16:
        raise ValueError(f"M must be divisible by 16; got M={M}.")
    if K % 8:
        raise ValueError(f"K must be divisible by 8; got K={K}.")
    return A.reshape(M, K // 2, 2).transpose(1, 0, 2).reshape(-1)


def pack_ffn_weights_decode(W, dim, num_cols):
    dim_m = dim // num_cols
    return np.concatenate([transpose_32bit_words(W[c * dim_m:(c + 1) * dim_m, :], dim_m, dim) for c in range(num_cols)])


def unpack_ffn_weights_decode(flat, dim, num_cols):
    dim_m = dim // num_cols
    parts = np.asarray(flat).reshape(num_cols, dim // 2, dim_m, 2)
    return np.ascontiguousarray(parts.transpose(0, 2, 1, 3)).reshape(dim, dim)


def pack_ffn_weights_prefill(W, dim, num_cols):
    dim_n = dim // num_cols
    return np.concatenate([W[:, c * dim_n:(c + 1) * dim_n].reshape(-1) for c in range(num_cols)])


def unpack_ffn_weights_prefill(flat, dim, num_cols):
    dim_n = dim // num_cols
    parts = np.asarray(flat).reshape(num_cols, dim, dim_n)
    return np.ascontiguousarray(parts.transpose(1, 0, 2)).reshape(dim, dim)
