// Pieces shared by the stream-K decode kernels (single product and fused FFN layer stack): unit
// geometry, workspace layout, nibble decode, MMA wrappers, epilogues.
#pragma once

#include <cuda_fp16.h>

#include "awq_common.cuh"
#include "awq_ptx.cuh"

namespace awq {

constexpr int SK_STRIP = 512;                 // columns per unit
constexpr int SK_BOX_COLS = 256;              // columns per 128-byte-wide TMA box
constexpr int SK_GROUP = 128;
constexpr int SK_CONSUMER_WARPS = SK_STRIP / 64;
constexpr int SK_THREADS = SK_CONSUMER_WARPS * 32 + 32;
constexpr int SK_CTAS_PER_SM = 2;
constexpr int SK_STAGES = 3;
constexpr int SK_WBOX_BYTES = SK_GROUP * 128;          // 128 k rows x 32 packed words
constexpr int SK_W_BYTES = (SK_STRIP / SK_BOX_COLS) * SK_WBOX_BYTES;
constexpr int SK_X_BYTES = 2 * 1024;                   // two boxes of 8 batch rows x 64 k (bf16)
constexpr int SK_S_BYTES = SK_STRIP * 2;
constexpr int SK_Z_BYTES = SK_STRIP / 8 * 4;
constexpr int SK_TX_BYTES = SK_W_BYTES + SK_X_BYTES + SK_S_BYTES + SK_Z_BYTES;
constexpr int SK_OFF_X = SK_W_BYTES;
constexpr int SK_OFF_S = SK_OFF_X + SK_X_BYTES;
constexpr int SK_OFF_Z = SK_OFF_S + SK_S_BYTES;
constexpr int SK_STAGE_BYTES = 36 * 1024;         // + 256 B of norm weights in the fused stack kernel
constexpr int SK_BAR_BYTES = 2 * SK_STAGES * 8 + 16;
constexpr int SK_SMEM_BYTES = SK_STAGES * SK_STAGE_BYTES + SK_BAR_BYTES + 1024;
constexpr int SK_ACC_WORDS = 16 * 32;                  // one 64-column sub-strip: 16 sums per lane, [sum][lane]
constexpr int SK_STRIP_WORDS = SK_CONSUMER_WARPS * SK_ACC_WORDS;
static_assert(SK_TX_BYTES <= SK_STAGE_BYTES, "stage too small");
static_assert(SK_CTAS_PER_SM * (SK_SMEM_BYTES + 1024) <= 228 * 1024, "shared memory budget");

// Workspace: [0, 256) header (int error flag, counter of the peer push); then, from SK_WS_ACCUM
// on, the split-K accumulators: one 64-bit word per (strip, warp, batch row, column), strip v at a
// fixed offset (up to SK_MAX_STRIPS).  All words are zero between launches (the warp that
// completes a sum takes it out and leaves zero), and the offsets do not depend on the shape, so
// one workspace serves products of different shapes back to back.
constexpr size_t SK_WS_HEADER = 256;
constexpr int SK_MAX_STRIPS = 504;  // N up to 258,048 columns
constexpr size_t SK_WS_ACCUM = 16384;
constexpr size_t SK_WS_END = SK_WS_ACCUM + (size_t)SK_MAX_STRIPS * SK_STRIP_WORDS * 8;
// behind the accumulators: the state of the one-launch stack kernel (awq_ffn_fused.cu), then room to convert
// activations to fp16
constexpr size_t SK_WS_FUSED_STATE = 5u << 20;
constexpr size_t SK_WS_XH = SK_WS_END + SK_WS_FUSED_STATE;
constexpr int SK_MAX_CTAS = 1023;

// ---- split-K hand-over: value and progress in ONE 64-bit atomic ------------------------------
// A partial sum travels as a fixed-point integer (2^-20 resolution) in the low 54 bits of a word
// and the number of k groups it covers in the high 10 bits, so a single atom.add carries both: the
// word's group count says when the sum is complete, and no fence, counter or ordering between
// separate memory operations is needed.  Integer addition is associative, so the total does not
// depend on the order in which the contributions arrive: results are bit-reproducible.
// Every contribution adds groups * 2^43 so that the value field never goes negative;
// |partial sum| must stay below 2^43 * 2^-20 = 8.39e6 (it is clamped and flagged otherwise), and a
// product may have at most 1023 groups.
constexpr int SK_FX_COUNT_SHIFT = 54;
constexpr unsigned long long SK_FX_VALUE_MASK = (1ull << SK_FX_COUNT_SHIFT) - 1;
constexpr long long SK_FX_BIAS = 1ll << 43;
constexpr float SK_FX_SCALE = 1048576.f;  // 2^20
constexpr float SK_FX_LIMIT = 8.38e6f;
constexpr int SK_MAX_GROUPS = 1023;

__device__ __forceinline__ unsigned long long sk_fx_encode(float v, int groups, bool &clamped) {
    if (!(fabsf(v) <= SK_FX_LIMIT)) {  // also NaN
        clamped = true;
        v = v != v ? 0.f : copysignf(SK_FX_LIMIT, v);
    }
    const long long fx = __float2ll_rn(v * SK_FX_SCALE) + (long long)groups * SK_FX_BIAS;
    return ((unsigned long long)groups << SK_FX_COUNT_SHIFT) + (unsigned long long)fx;
}
__device__ __forceinline__ float sk_fx_decode(unsigned long long word, int G) {
    const long long fx = (long long)(word & SK_FX_VALUE_MASK) - (long long)G * SK_FX_BIAS;
    return (float)fx * (1.f / SK_FX_SCALE);
}
__device__ __forceinline__ unsigned long long ld_relaxed_gpu_u64(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// Hand this warp's partial sums of a sub-strip (own[h][j], `seg_groups` of the product's G groups)
// to the sub-strip's accumulator words at `sub`.  Returns true in exactly one contributor per use
// of the accumulator: the one whose add completed word 0 of lane 0.  It then holds the complete
// sums in `own` (the other words are normally complete too; where another contributor's adds are
// still on their way it re-reads them, bounded by `wait_limit` cycles) and has left the words zero.
__device__ __forceinline__ bool sk_handover(unsigned long long *sub, float (&own)[2][8], int seg_groups, int G, int lane,
                                            long long wait_limit, int *err_flag) {
    unsigned long long *w = sub + lane;
    unsigned long long tot[16];
    bool clamped = false;
#pragma unroll
    for (int i = 0; i < 16; ++i) tot[i] = sk_fx_encode(own[i >> 3][i & 7], seg_groups, clamped);
#pragma unroll
    for (int i = 0; i < 16; ++i) tot[i] += atomicAdd(w + 32 * i, tot[i]);
    if (clamped) atomicExch(err_flag, 7);
    const int pilot = __shfl_sync(0xffffffffu, (int)(tot[0] >> SK_FX_COUNT_SHIFT), 0);
    if (pilot != G) return false;
    bool complete = true;
#pragma unroll
    for (int i = 0; i < 16; ++i) complete = complete && (int)(tot[i] >> SK_FX_COUNT_SHIFT) == G;
    if (!__all_sync(0xffffffffu, complete)) {
        const long long t0 = clock64();
        bool all, late;
        do {
            complete = true;
#pragma unroll
            for (int i = 0; i < 16; ++i)
                if ((int)(tot[i] >> SK_FX_COUNT_SHIFT) != G) {
                    tot[i] = ld_relaxed_gpu_u64(w + 32 * i);
                    complete = complete && (int)(tot[i] >> SK_FX_COUNT_SHIFT) == G;
                }
            all = __all_sync(0xffffffffu, complete);
            // the lanes must leave together: one lane's clock decides for the warp
            late = __shfl_sync(0xffffffffu, clock64() - t0 > wait_limit ? 1 : 0, 0) != 0;
        } while (!all && !late);
        if (!all) {
            if (lane == 0) atomicExch(err_flag, 8);
            return false;
        }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        w[32 * i] = 0ull;  // nobody else touches the word before its next use
        own[i >> 3][i & 7] = sk_fx_decode(tot[i], G);
    }
    return true;
}

// CTA that owns unit x when U units are split over C CTAs as [c U / C, (c + 1) U / C).
__host__ __device__ __forceinline__ long long sk_owner(long long x, long long C, long long U) {
    return ((x + 1) * C + U - 1) / U - 1;
}

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t v, uint32_t mask, uint32_t magic) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(v), "r"(mask), "r"(magic));
    return r;
}

// R holds one 16-bit half of a packed word for k (low 16 bits) and for k + 1 (high 16 bits):
// four nibbles each.  Output e is the pair (nibble e at k, nibble e at k + 1) as 16-bit floats.
//   bf16: 128 + n for every e (three shifts).
//   fp16: 1024 + n for e = 0, 2 and 1024 + 16 n for e = 1, 3 (one shift); the factor 16 and the
//         different offset are undone in the per-group fix-up.
template <bool XH>
__device__ __forceinline__ void decode4(uint32_t R, uint32_t (&o)[4]) {
    if (XH) {
        const uint32_t T = R >> 8;
        o[0] = lop3_and_or(R, 0x000F000Fu, 0x64006400u);
        o[1] = lop3_and_or(R, 0x00F000F0u, 0x64006400u);
        o[2] = lop3_and_or(T, 0x000F000Fu, 0x64006400u);
        o[3] = lop3_and_or(T, 0x00F000F0u, 0x64006400u);
    } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) o[e] = lop3_and_or(R >> (4 * e), 0x000F000Fu, 0x43004300u);
    }
}

template <bool XH>
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    if (XH) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
            "{%0, %1, %2, %3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
        mma_bf16_16816(d, a0, a1, a2, a3, b0, b1);
    }
}

// bf16-rounded value -> fp16 bits.  Nothing is clamped: a value beyond the fp16 range becomes an infinity and a
// NaN stays a NaN, so an overflow inside a chain of kernels shows in the output (and trips the range check of
// the split-K hand-over) instead of turning into a plausible finite number.
__device__ __forceinline__ uint16_t bf16_value_to_f16_bits(float v) { return __half_as_ushort(__float2half_rn(v)); }

// One lane's share of a finished strip after the lane exchange: batch row b, and for each
// 32-column half h of the warp's 64 columns, 8 consecutive columns starting at n + 32 h.
template <int EPI>
__device__ __forceinline__ void sk_epilogue(const float (&own)[2][8], const uint16_t *__restrict__ residual,
                                            void *__restrict__ y_, int B, int N, int n, int b, int out_f16) {
    if (b >= B) return;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int nh = n + 32 * h;
        if (nh >= N) continue;
        const float(&v)[8] = own[h];
        if (EPI == EPI_SWIGLU) {
            uint16_t o[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                o[i] = swiglu_bits(v[2 * i], v[2 * i + 1]);
                if (out_f16) o[i] = bf16_value_to_f16_bits(bf16_bits_to_f32(o[i]));
            }
            *reinterpret_cast<uint2 *>(reinterpret_cast<uint16_t *>(y_) + (size_t)b * (N >> 1) + (nh >> 1)) =
                make_uint2((uint32_t)o[0] | ((uint32_t)o[1] << 16), (uint32_t)o[2] | ((uint32_t)o[3] << 16));
        } else if (EPI == EPI_F32 || EPI == EPI_F32_PUSH) {
            float4 *dst = reinterpret_cast<float4 *>(reinterpret_cast<float *>(y_) + (size_t)b * N + nh);
            dst[0] = make_float4(v[0], v[1], v[2], v[3]);
            dst[1] = make_float4(v[4], v[5], v[6], v[7]);
        } else {
            float r[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (residual) {
                const uint4 rv = *reinterpret_cast<const uint4 *>(residual + (size_t)b * N + nh);
                const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    r[2 * i] = bf16x2_lo(rw[i]);
                    r[2 * i + 1] = bf16x2_hi(rw[i]);
                }
            }
            uint32_t o[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) o[i] = pack_bf16x2(v[2 * i] + r[2 * i], v[2 * i + 1] + r[2 * i + 1]);
            *reinterpret_cast<uint4 *>(reinterpret_cast<uint16_t *>(y_) + (size_t)b * N + nh) =
                make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
}


// After a warp has stored a finished sub-strip with EPI_F32_PUSH.  Sub-strips are counted on this
// GPU first (`local_done`, zero between launches); the warp that finishes the launch's last one makes
// everything visible to the other GPUs with ONE system-scope fence (the fence is cumulative: it
// orders the other warps' stores, which it has observed through the counter, too) and adds 1 to its
// entry of every rank's arrival counters.  A system-scope fence per sub-strip costs 9 us per launch.
__device__ __forceinline__ void sk_push_signal(const PeerPush &push, int *local_done, int total, int lane) {
    __threadfence();
    __syncwarp();
    int last = 0;
    if (lane == 0) last = atomicAdd(local_done, 1) == total - 1;
    last = __shfl_sync(0xffffffffu, last, 0);
    if (!last) return;
    __threadfence_system();
    if (lane == 0) *local_done = 0;
    if (lane < push.n) atomicAdd_system(push.flag[lane] + push.rank, 1u);
}

// Per-lane geometry of a consumer warp.  Warp w owns strip columns [64 w, 64 w + 64): two
// 16-byte chunks (A, B) of every box row.  ldmatrix.trans hands lane (g8, t4) 16-bit half g8 of
// chunk A / B for rows 2 t4 and 2 t4 + 1 already paired in one register: half g8 = packed word
// g8 / 2, even (low half) or odd (high half) columns.  MMA row g8 is that lane's chunk-A column,
// row g8 + 8 its chunk-B column.
struct SkLane {
    int g8, t4, odd;
    int lm, lr;       // ldmatrix: matrix index, row within the matrix
    int colw;         // first strip column of this lane's 8-column blocks (+32 for chunk B)
    uint32_t w_off, z_off, s_off;
    __device__ __forceinline__ SkLane(int warp, int lane) {
        g8 = lane >> 2;
        t4 = lane & 3;
        odd = g8 & 1;
        lm = lane >> 3;
        lr = lane & 7;
        const uint32_t w_chunk = 2 * (warp & 3) + (lm >> 1);
        w_off = (warp >> 2) * SK_WBOX_BYTES + ((lm & 1) * 8 + lr) * 128 + ((w_chunk ^ lr) << 4);
        colw = warp * 64 + (g8 >> 1) * 8;
        z_off = SK_OFF_Z + (colw >> 3) * 4 + odd * 2;
        s_off = SK_OFF_S + (colw + odd) * 2;
    }
};

// One unit (512 columns x one group of 128 k) from the stage at shared address `st`: adds this
// warp's 64 columns x 8 batch rows into res and releases the stage through `empty_bar`.
template <bool XH>
__device__ __forceinline__ void sk_consume_unit(uint32_t st, const SkLane &L, float (&res)[4][4], uint32_t empty_bar,
                                                int lane) {
    const int lm = L.lm, lr = L.lr;
    const uint32_t w_off = L.w_off, z_off = L.z_off, s_off = L.s_off;
    const uint32_t ONES = XH ? 0x3C003C00u : 0x3F803F80u;
    float acc[4][4];
    float sx[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int e = 0; e < 4; ++e)
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[e][q] = 0.f;

#pragma unroll
    for (int p = 0; p < 4; ++p) {
        // activations for k-steps 2p and 2p+1: 16-byte chunk q = 4p + matrix index
        const int q = 4 * p + lm;
        uint32_t bx[4];
        ldmatrix_x4(bx, st + SK_OFF_X + (q >> 3) * 1024 + lr * 128 + (((q & 7) ^ lr) << 4));
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            uint32_t R[4];  // chunk A rows 0-7, chunk A rows 8-15, chunk B rows 0-7, chunk B rows 8-15
            ldmatrix_x4_trans(R, st + (2 * p + h) * 2048 + w_off);
            const uint32_t b0 = bx[2 * h], b1 = bx[2 * h + 1];
            mma_16816<XH>(sx, ONES, ONES, ONES, ONES, b0, b1);
            uint32_t a_lo[4], a_hi[4], b_lo[4], b_hi[4];
            decode4<XH>(R[0], a_lo);
            decode4<XH>(R[1], a_hi);
            decode4<XH>(R[2], b_lo);
            decode4<XH>(R[3], b_hi);
#pragma unroll
            for (int e = 0; e < 4; ++e) mma_16816<XH>(acc[e], a_lo[e], b_lo[e], a_hi[e], b_hi[e], b0, b1);
        }
    }

    // group fix-up: res += s * (acc - c * sum_x); the zero point (and, for fp16, the decode
    // offset and the factor 16 of odd nibbles) live in c and s
    const uint32_t zA = lds_u16(st + z_off), zB = lds_u16(st + z_off + 16);
    uint32_t sA[4], sB[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        sA[e] = lds_u16(st + s_off + 4 * e);
        sB[e] = lds_u16(st + s_off + 64 + 4 * e);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty_bar);  // all of this warp's reads of the slot are done
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        // 128 + z as f32: bits 0x43000000 | z << 16
        float cA = __uint_as_float(((zA << (16 - 4 * e)) & 0x000F0000u) | 0x43000000u);
        float cB = __uint_as_float(((zB << (16 - 4 * e)) & 0x000F0000u) | 0x43000000u);
        float fA = __uint_as_float(sA[e] << 16), fB = __uint_as_float(sB[e] << 16);
        if (XH) {
            if (e & 1) {
                cA = fmaf(cA, 16.f, -1024.f);  // 1024 + 16 z
                cB = fmaf(cB, 16.f, -1024.f);
                fA *= 0.0625f;
                fB *= 0.0625f;
            } else {
                cA += 896.f;  // 1024 + z
                cB += 896.f;
            }
        }
        res[e][0] = fmaf(fA, fmaf(-cA, sx[0], acc[e][0]), res[e][0]);
        res[e][1] = fmaf(fA, fmaf(-cA, sx[1], acc[e][1]), res[e][1]);
        res[e][2] = fmaf(fB, fmaf(-cB, sx[0], acc[e][2]), res[e][2]);
        res[e][3] = fmaf(fB, fmaf(-cB, sx[1], acc[e][3]), res[e][3]);
    }
}

// Lanes g8 and g8 ^ 1 hold the even / odd columns of the same 8-column blocks for batch rows 2t
// and 2t + 1: swap so that each owns one batch row (2 t4 + odd) and 8 consecutive columns per
// 32-column half.
__device__ __forceinline__ void sk_lane_exchange(const float (&res)[4][4], int odd, float (&own)[2][8]) {
#pragma unroll
    for (int e = 0; e < 4; ++e)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float keep = odd ? res[e][2 * h + 1] : res[e][2 * h];
            const float send = odd ? res[e][2 * h] : res[e][2 * h + 1];
            const float recv = __shfl_xor_sync(0xffffffffu, send, 4);
            own[h][2 * e] = odd ? recv : keep;
            own[h][2 * e + 1] = odd ? keep : recv;
        }
}

}  // namespace awq
