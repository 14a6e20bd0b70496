// Batched-decode GEMM for up to 32 token rows with the packed nibbles themselves as the tensor core's operand
// (same product and epilogues as awq_gemm_decode.cu: the batched-decode golden of
// matrix_multiplication/int4_awq/matmul_int4_packed.py:97-105 with M = batch).
//
// What bounds awq_gemm_decode.cu is the tensor pipe, not the dequant arithmetic: with the weights as the MMA's M-side
// operand in tensor memory, an instruction costs about 64 cycles however few token rows there are (the time to read
// 128 x 32 bytes of weights), and 16-bit weights need 16 of them per unit of 128 k: 1,050 to 1,180 cycles where the
// unit's share of HBM time is 760.  Here a weight stays one byte:
//
//  * A nibble q in the low half of a byte IS the e4m3 number q * 2^-9 (the subnormals and the first binade of a
//    floating-point format are linear in the bit pattern).  The dequant warps only regroup bits: ldmatrix.trans as
//    before, two PRMT to bring the same byte of four k into one register, AND / shift-AND to split its two nibbles:
//    half an instruction per weight, no arithmetic.  tcgen05.mma kind::f8f6f4 multiplies 32 k per instruction, so a
//    unit takes 8 instructions, not 16.
//  * The token rows come as e4m3 too, split by a small kernel in front (act_split_kernel): the row is scaled by a power
//    of two so that its largest magnitude lies in [128, 256), then x = hi + lo / 16 with hi = e4m3(x) and
//    lo = e4m3(16 (x - hi)).  A bf16 value has 8 significant bits and each piece carries 4, so the split is exact for
//    every element within 2^-14 of the row's largest (smaller ones keep an absolute error below 2^-22 of it).  The two
//    pieces are separate MMA columns (N = 2 x rows); inside a 32-k step the k order of both operands is permuted the
//    same way, which costs nothing and lets ldmatrix read conflict-free.
//  * Zero point and scale never touch the weights.  A unit is one quantisation group, so per weight column n they are
//    constants of the unit: the MMA leaves P[n, m] = sum_k q x per unit in a fresh accumulator, and eight "promote"
//    warps (a thread per weight column) fold it into f32 registers:
//        acc[m] += s (512 P_hi + 32 P_lo - z Sx[m]),   Sx[m] = sum over the group of the split x (from the split kernel)
//    which is exactly sum_k (q - z) s x with the scale applied in f32, as the oracle does: this path rounds no weight.
//  * Everything else as in awq_gemm_decode.cu: stream-K over (256-column tile, 128 k) units, TMA ring, the sums of a
//    CTA's share of a tile go to its slot of the workspace and the fix-up launch adds them up (undoing the row's power
//    of two) and applies the epilogue.
//
//   warp 0       producer (TMA: packed words, scales, zeros; split token rows and their group sums)
//   warp 1       MMA issuer: 8 tcgen05.mma (M 128, N 2 x rows, K 32) per unit into one of two accumulator sets
//   warps 2-9    regroup the nibbles into tensor memory (a warp: 32 weight columns x 128 k)
//   warps 10-17  promote (a warp: 32 weight columns x all token rows): tcgen05.ld of the unit's sums, three FMAs per
//                (column, row); their arrival also frees the unit's input stage
// Tensor memory: two accumulator sets of 4 x rows columns, the rest weight buffers of 64 columns (six up to 16 rows, four
// with 32).  Every wait is bounded.
#include <cudaTypedefs.h>
#include <cuda_fp8.h>

#include <mutex>

#include "awq_common.cuh"
#include "awq_gemm_decode.cuh"
#include "awq_ptx.cuh"
#include "awq_streamk.cuh"
#include "awq_tcgen05.cuh"

namespace awq {

constexpr int F8_REGROUP_WARPS = 8, F8_REGROUP_WARP0 = 2;
constexpr int F8_ABUF_COLS = 64;  // a weight buffer: two 128-column halves x 128 k bytes = 2 x 32 TMEM columns
constexpr int F8_MAX_ROWS = 32;
constexpr uint32_t F8_TMEM_COLS = 512;

template <int NB>
struct F8Cfg {
    static constexpr int X_BYTES = 2 * NB * DG_GROUP;  // both pieces of every token row, 128 k of one byte
    static constexpr int SX_OFF = DG_S_BYTES + DG_Z_BYTES;  // the rows' group sums sit behind scales and zeros
    static constexpr int SX_BYTES = NB * 4;
    static constexpr int STAGE_BYTES = X_BYTES + DG_W_BYTES + 1024;
    static constexpr int RING_BUDGET = 220 * 1024;
    static constexpr int STAGES = RING_BUDGET / STAGE_BYTES < 8 ? RING_BUDGET / STAGE_BYTES : 8;
    static constexpr int ACC_COLS = 4 * NB;  // two halves x (hi, lo) x rows
    static constexpr int ABUF = ((int)F8_TMEM_COLS - 2 * ACC_COLS) / F8_ABUF_COLS;  // weight buffers: 6 up to 16 rows, 4 with 32
    static constexpr int ACC_COL0 = ABUF * F8_ABUF_COLS;
    // a promote warp: 32 weight columns x all token rows.  (Measured: a second set of eight warps for rows 16-31 made the
    // kernel 9 % slower, 120 against 110 us per 70B layer: the waiting warps' polls cost more than the shorter chain wins.)
    static constexpr int PROMOTE_WARPS = 8;
    // Up to 16 rows the regroup warps' chain per unit (wait, ldmatrix, bit operations, tensor-memory stores, wait, arrive)
    // is the longest.  (Measured there: a second group of eight regroup warps, the two taking alternate units, 103
    // against 94 us per 70B layer; the one group taking two units per round of waits 110 against 90.)
    static constexpr int PROMOTE_WARP0 = F8_REGROUP_WARP0 + F8_REGROUP_WARPS;
    static constexpr int THREADS = (PROMOTE_WARP0 + PROMOTE_WARPS) * 32;  // 576
    static constexpr int NUM_BARS = 3 * STAGES + 2 * ABUF + 4;
    static constexpr int OFF_BARS = STAGES * STAGE_BYTES;
    static constexpr int SMEM_BYTES = OFF_BARS + NUM_BARS * 8 + 16 + 1024;
    // kind::f8f6f4: f32 accumulate, both operands e4m3 (format 0), K-major, M 128, N 2 NB
    static constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)((2 * NB) >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    static_assert(ACC_COL0 + 2 * ACC_COLS <= (int)F8_TMEM_COLS, "tensor memory budget");
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
    static_assert(STAGE_BYTES % 1024 == 0 && X_BYTES % 1024 == 0, "swizzled tiles need 1024-byte alignment");
    static_assert(SX_OFF + SX_BYTES <= 1024, "scales, zeros and group sums share one KB");
};

__device__ int g_gemm_f8_error;  // 0 = ok; set when a bounded wait gave up

__device__ __forceinline__ void f8_umma_ta(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// (d0, d1) += a * (b0, b1): one packed FMA for two token rows
__device__ __forceinline__ void f8_fma2(float &d0, float &d1, float a, float b0, float b1) {
    asm("{\n\t.reg .b64 ra, rb, rc;\n\t"
        "mov.b64 ra, {%2, %2};\n\tmov.b64 rb, {%3, %4};\n\tmov.b64 rc, {%0, %1};\n\t"
        "fma.rn.f32x2 rc, ra, rb, rc;\n\t"
        "mov.b64 {%0, %1}, rc;\n\t}"
        : "+f"(d0), "+f"(d1)
        : "f"(a), "f"(b0), "f"(b1));
}
__device__ __forceinline__ uint32_t f8_prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

// Where element k (0..31 inside a 32-k step) of a token row goes: byte 8 t + 2 i + b of the step for k = 8 i + 2 t + b.
// The regroup warps produce the weights in that order (lane t of a quad holds, after ldmatrix, k = 8 i + 2 t + b of
// matrix i, and tcgen05.st takes bytes 8 t .. 8 t + 7 of the step from it).
__host__ __device__ __forceinline__ int f8_k_slot(int k) {
    const int i = k >> 3, t = (k >> 1) & 3, b = k & 1;
    return 8 * t + 2 * i + b;
}

// ---------------------------------------------------------------------------------------------------------------------
// Split of the token rows.  F8_SPLIT_BLOCKS blocks per (padded) token row: each finds the row's largest magnitude itself (the
// row comes from L2) and splits its share of the groups.  Output, for rows = 16 or 32 MMA rows:
//   x8   [K / 128][2 rows][128] bytes: row m = hi piece of token m, row rows + m = lo piece, k permuted inside 32-k steps
//   sx   [K / 128][rows] f32: sum over the group of hi + lo / 16 (in the row's scaled units)
//   inv  [rows] f32: the power of two that undoes the row's scaling
// Rows from M on are written as zeros.
constexpr int F8_SPLIT_BLOCKS = 8;
template <bool XH>
__global__ void __launch_bounds__(256)
act_split_kernel(const uint16_t *__restrict__ x, int M, int K, int rows, uint8_t *__restrict__ x8, float *__restrict__ sx,
                 float *__restrict__ inv) {
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x, G = K / DG_GROUP, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    auto f32_of = [](uint32_t bits16) { return XH ? __half2float(__ushort_as_half((uint16_t)bits16)) : bf16_bits_to_f32(bits16 & 0xFFFFu); };
    __shared__ float red[8];
    auto value = [&](int k) {
        const uint16_t v = x[(size_t)m * K + k];
        return XH ? __half2float(__ushort_as_half(v)) : bf16_bits_to_f32(v);
    };
    float scale = 0.f;
    if (m < M) {
        float mx = 0.f;
        const uint4 *row = reinterpret_cast<const uint4 *>(x + (size_t)m * K);  // K is a multiple of 128, the row 16-byte aligned
        for (int v = threadIdx.x; v < K / 8; v += 256) {
            const uint4 q = row[v];
            const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) mx = fmaxf(mx, fmaxf(fabsf(f32_of(w4[j] & 0xFFFFu)), fabsf(f32_of(w4[j] >> 16))));
        }
        for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (lane == 0) red[warp] = mx;
        __syncthreads();
        mx = red[0];
        for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red[w]);
        // largest magnitude into [128, 256); an all-zero (or non-finite) row is left as it is
        int e = 0;
        if (mx > 0.f && mx < 3.0e38f) frexpf(mx, &e);  // mx = f 2^e, 0.5 <= f < 1
        e = e < -100 ? -100 : e;  // (a row of nothing but denormals: keep the power of two finite)
        scale = (mx > 0.f && mx < 3.0e38f) ? exp2f((float)(8 - e)) : 1.f;
        if (threadIdx.x == 0 && blockIdx.y == 0) inv[m] = 1.f / scale;
    } else if (threadIdx.x == 0 && blockIdx.y == 0) {
        inv[m] = 0.f;
    }
    for (int g = blockIdx.y * 8 + warp; g < G; g += 8 * F8_SPLIT_BLOCKS) {
        uint8_t *hi_row = x8 + ((size_t)g * 2 * rows + m) * DG_GROUP, *lo_row = hi_row + (size_t)rows * DG_GROUP;
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int kk = 32 * j + lane;  // k inside the group: step j, element `lane`
            uint8_t hi = 0, lo = 0;
            if (m < M) {
                const float v = value(g * DG_GROUP + kk) * scale;
                hi = (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
                const float hf = __half2float(__half(__nv_cvt_fp8_to_halfraw(hi, __NV_E4M3)));
                lo = (uint8_t)__nv_cvt_float_to_fp8(16.f * (v - hf), __NV_SATFINITE, __NV_E4M3);
                const float lf = __half2float(__half(__nv_cvt_fp8_to_halfraw(lo, __NV_E4M3)));
                sum += hf + 0.0625f * lf;
            }
            const int pos = 32 * j + f8_k_slot(lane);
            hi_row[pos] = hi;
            lo_row[pos] = lo;
        }
        for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) sx[(size_t)g * rows + m] = sum;
    }
}

// ---------------------------------------------------------------------------------------------------------------------
template <int NB>
__global__ void __launch_bounds__(F8Cfg<NB>::THREADS, 1)
gemm_decode_f8_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmSx,
                      const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmS,
                      const __grid_constant__ CUtensorMap tmZ, int M, int N, int K, int tiles, float *__restrict__ slots,
                      int slots_per_tile, long long wait_limit) {
    using Cfg = F8Cfg<NB>;
    constexpr int STAGES = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + Cfg::OFF_BARS;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem_gen + Cfg::OFF_BARS + Cfg::NUM_BARS * 8);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };                   // packed words, scales, zeros landed in stage s
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };       // MMA, regroup and promote warps done with stage s
    auto xfull_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };   // its token rows and group sums landed
    auto ready_bar = [&](int b) { return bar_base + 8u * (3 * STAGES + b); };   // weight buffer b written
    auto bfree_bar = [&](int b) { return bar_base + 8u * (3 * STAGES + Cfg::ABUF + b); };      // MMA done with weight buffer b
    auto acc_full = [&](int b) { return bar_base + 8u * (3 * STAGES + 2 * Cfg::ABUF + b); };   // a unit's sums complete
    auto acc_empty = [&](int b) { return bar_base + 8u * (3 * STAGES + 2 * Cfg::ABUF + 2 + b); };  // and promoted
    auto stage_addr = [&](int s) { return smem_base + (uint32_t)s * Cfg::STAGE_BYTES; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr uint32_t W_TX_BYTES = DG_W_BYTES + DG_S_BYTES + DG_Z_BYTES;
    constexpr uint32_t X_TX_BYTES = Cfg::X_BYTES + Cfg::SX_BYTES;
    const int KB = K / DG_GROUP;  // units per tile

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(xfull_bar(s), 1);
            mbar_init(empty_bar(s), Cfg::PROMOTE_WARPS);  // the promote warps are the last to need a stage
        }
        for (int b = 0; b < Cfg::ABUF; ++b) {
            mbar_init(ready_bar(b), F8_REGROUP_WARPS);
            mbar_init(bfree_bar(b), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full(b), 1);
            mbar_init(acc_empty(b), Cfg::PROMOTE_WARPS);
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        dg_tmem_alloc(smem_u32(tmem_slot), F8_TMEM_COLS);
        dg_tmem_relinquish();
    }
    dg_fence_before();
    __syncthreads();
    dg_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();

    if (warp == 0) {
        // ------------------------------ producer ------------------------------
        if (elect_one()) {
            tma_prefetch_desc(&tmX);
            tma_prefetch_desc(&tmSx);
            tma_prefetch_desc(&tmW);
            tma_prefetch_desc(&tmS);
            tma_prefetch_desc(&tmZ);
        }
        const uint64_t stream_policy = l2_policy_evict_first();
        auto load_weights = [&](int s, int n0, int g) {
            const uint32_t st = stage_addr(s) + Cfg::X_BYTES, bar = full_bar(s);
            if (elect_one()) {
                mbar_expect_tx(bar, W_TX_BYTES);
                tma_load_2d_hint(st, &tmW, n0 / 8, g * DG_GROUP, bar, stream_policy);
                tma_load_2d(st + DG_W_BYTES, &tmS, n0, g, bar);
                tma_load_2d(st + DG_W_BYTES + DG_S_BYTES, &tmZ, n0 / 8, g, bar);
            }
            __syncwarp();
        };
        auto load_rows = [&](int s, int g) {
            if (elect_one()) {
                mbar_expect_tx(xfull_bar(s), X_TX_BYTES);
                tma_load_2d(stage_addr(s), &tmX, 0, g * 2 * NB, xfull_bar(s));
                tma_load_2d(stage_addr(s) + Cfg::X_BYTES + DG_W_BYTES + Cfg::SX_OFF, &tmSx, 0, g, xfull_bar(s));
            }
            __syncwarp();
        };
        // The weights do not depend on the previous kernel in the stream (the split of the token rows): fill the ring with
        // them first.
        UnitWalk w(tiles, KB);
        int it = 0;
        for (UnitWalk f = w; f.valid() && it < STAGES; ++f.u, ++it) load_weights(it, f.tile() * DG_BN, f.kb());
        pdl_wait();
        it = 0;
        for (UnitWalk f = w; f.valid() && it < STAGES; ++f.u, ++it) load_rows(it, f.kb());
        for (w.u += it; w.valid(); ++w.u, ++it) {
            const int s = it % STAGES, round = it / STAGES;
            if (!mbar_wait_bounded_warp(empty_bar(s), (round - 1) & 1, wait_limit)) {
                if (lane == 0) atomicExch(&g_gemm_f8_error, 1);
                break;
            }
            load_weights(s, w.tile() * DG_BN, w.kb());
            load_rows(s, w.kb());
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        int it = 0;
        for (UnitWalk w(tiles, KB); w.valid(); ++w.u, ++it) {
            const int s = it % STAGES, round = it / STAGES;
            const int ab = it % Cfg::ABUF, around = it / Cfg::ABUF;
            const int b = it & 1, use = it >> 1;
            // token rows landed, weight buffer written, accumulator set promoted: three lanes wait side by side
            if (!mbar_wait_multi_warp(use >= 1 ? 3 : 2, xfull_bar(s), round & 1, ready_bar(ab), around & 1, acc_empty(b), (use - 1) & 1,
                                      wait_limit)) {
                if (lane == 0) atomicExch(&g_gemm_f8_error, 2);
                break;
            }
            dg_fence_after();
            const uint32_t d_tmem = tmem_base + Cfg::ACC_COL0 + (uint32_t)b * Cfg::ACC_COLS;
            const uint32_t a_tmem = tmem_base + (uint32_t)ab * F8_ABUF_COLS;
            const uint64_t x_desc = dg_desc_sw128(stage_addr(s));  // K-major 128-byte rows, 32 bytes further per step
            if (elect_one()) {
#pragma unroll
                for (int ks = 0; ks < DG_GROUP / 32; ++ks) {
#pragma unroll
                    for (int h = 0; h < 2; ++h)  // the tile's two halves of 128 weight columns
                        f8_umma_ta(d_tmem + h * (2 * NB), a_tmem + h * (F8_ABUF_COLS / 2) + 8 * ks, x_desc + (uint64_t)(2 * ks),
                                   Cfg::IDESC, ks ? 1u : 0u);
                }
                dg_umma_commit(bfree_bar(ab));
                dg_umma_commit(acc_full(b));
            }
            __syncwarp();
        }
    } else if (warp >= F8_REGROUP_WARP0 && warp < Cfg::PROMOTE_WARP0) {
        // ------------------------------ regroup ------------------------------
        // warp w: TMEM lanes 32 (w % 4) .. + 31 of one 128-column half, all 128 k
        const int rw = warp - F8_REGROUP_WARP0;
        const int q = warp & 3;   // TMEM lanes 32 q .. 32 q + 31 (a warp may only touch its own quarter)
        const int h = (rw >> 2) & 1;  // which 128-column half of the tile
        const int chunk = 4 * h + q;  // the warp's 32 columns are one 16-byte chunk (4 packed words) of a 128-byte row
        // ldmatrix.x4.trans: matrix i = rows k = 8 i .. 8 i + 7 of the call's 32 k (conflict-free under the 128-byte
        // swizzle); lane (g = lane / 4, t = lane % 4) then holds half word g of k = 8 i + 2 t, + 1 in register i.
        const int mi = lane >> 3, rr = lane & 7;
        const uint32_t w_off = (uint32_t)(8 * mi + rr) * 128 + (uint32_t)((chunk ^ rr) << 4);  // + 32 * 128 per call
        UnitWalk w(tiles, KB);
        const int n_units = w.u1 - w.u;
        for (int it = 0; it < n_units; ++it) {
            const int s = it % STAGES, round = it / STAGES;
            const int ab = it % Cfg::ABUF, around = it / Cfg::ABUF;
            // the unit's words landed: fetch them, and only then wait for the MMA to be done with the weight buffer they go to
            if (!mbar_wait_bounded(full_bar(s), round & 1, wait_limit)) {
                if (lane == 0) atomicExch(&g_gemm_f8_error, 3);
                break;
            }
            const uint32_t st = stage_addr(s) + Cfg::X_BYTES;
            uint32_t r[4][4];
#pragma unroll
            for (int c = 0; c < 4; ++c) ldmatrix_x4_trans(r[c], st + w_off + c * 32 * 128);
            // all the bit work first; only the stores need the weight buffer, i.e. the MMA to be done with it
            uint32_t lo[2][8], hi[2][8];
#pragma unroll
            for (int c = 0; c < 4; ++c) {  // 32-k step c of the unit
                // byte 0 / byte 1 of the half word at the step's bytes 8 t .. 8 t + 3 (lo) and 8 t + 4 .. 8 t + 7 (hi)
                const uint32_t b0lo = f8_prmt(r[c][0], r[c][1], 0x6420u), b1lo = f8_prmt(r[c][0], r[c][1], 0x7531u);
                const uint32_t b0hi = f8_prmt(r[c][2], r[c][3], 0x6420u), b1hi = f8_prmt(r[c][2], r[c][3], 0x7531u);
                // nibble e of the half word = column 2 e + (g & 1) of its packed word; TMEM lanes g, g + 8, g + 16, g + 24
                const int p = c >> 1, d = c & 1;
                lo[p][4 * d] = b0lo & 0x0F0F0F0Fu, lo[p][4 * d + 1] = b0hi & 0x0F0F0F0Fu;
                lo[p][4 * d + 2] = (b0lo >> 4) & 0x0F0F0F0Fu, lo[p][4 * d + 3] = (b0hi >> 4) & 0x0F0F0F0Fu;
                hi[p][4 * d] = b1lo & 0x0F0F0F0Fu, hi[p][4 * d + 1] = b1hi & 0x0F0F0F0Fu;
                hi[p][4 * d + 2] = (b1lo >> 4) & 0x0F0F0F0Fu, hi[p][4 * d + 3] = (b1hi >> 4) & 0x0F0F0F0Fu;
            }
            if (around > 0 && !mbar_wait_bounded(bfree_bar(ab), (around - 1) & 1, wait_limit)) {
                if (lane == 0) atomicExch(&g_gemm_f8_error, 3);
                break;
            }
            dg_fence_after();
            const uint32_t a_tmem = tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(ab * F8_ABUF_COLS + h * (F8_ABUF_COLS / 2));
#pragma unroll
            for (int p = 0; p < 2; ++p) {  // 32-k steps 2 p and 2 p + 1: one store per 16 TMEM lanes for both
                dg_tmem_st_16x256b_x2(a_tmem + 16 * p, lo[p]);
                dg_tmem_st_16x256b_x2(a_tmem + (16u << 16) + 16 * p, hi[p]);
            }
            dg_tmem_st_wait();
            dg_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(ready_bar(ab));
        }
    } else if (warp >= Cfg::PROMOTE_WARP0) {
        // ------------------------------ promote ------------------------------
        // thread = one weight column: TMEM lane 32 q + lane of half h
        const int pw = warp - Cfg::PROMOTE_WARP0;
        const int q = warp & 3, h = pw >> 2;
        const int col = 128 * h + 32 * q + dg_lane_column(lane);  // column inside the tile
        const int z_shift = 4 * (((col & 1) << 2) | ((col & 7) >> 1));  // nibble of column c of a packed word: PERM[c]
        float acc[NB];
#pragma unroll
        for (int i = 0; i < NB; ++i) acc[i] = 0.f;
        pdl_wait();  // the previous kernel in the stream may still be reading the slots
        int it = 0;
        UnitWalk w(tiles, KB);
        while (w.valid()) {
            const int tile = w.tile(), n_seg = w.left_in_tile();
            bool ok = true;
            for (int i = 0; i < n_seg && ok; ++i, ++it, ++w.u) {
                const int s = it % STAGES;
                const int b = it & 1, use = it >> 1;
                // (the unit's sums being complete implies that its stage landed: the MMA read it)
                if (!mbar_wait_bounded(acc_full(b), use & 1, wait_limit)) {
                    if (lane == 0) atomicExch(&g_gemm_f8_error, 4);
                    ok = false;
                    break;
                }
                dg_fence_after();
                const uint32_t sz = stage_addr(s) + Cfg::X_BYTES + DG_W_BYTES;
                const float sc = bf16_bits_to_f32((lds32(sz + 2 * (col & ~1)) >> (16 * (col & 1))) & 0xFFFFu);
                const float z = (float)((lds32(sz + DG_S_BYTES + 4 * (col >> 3)) >> z_shift) & 0xFu);
                const float c_hi = 512.f * sc, c_lo = 32.f * sc, c_z = -sc * z;  // a nibble reads as q 2^-9, lo as 16 (x - hi)
                const uint32_t t_acc = tmem_base + ((uint32_t)(32 * q) << 16) + Cfg::ACC_COL0 + (uint32_t)(b * Cfg::ACC_COLS + h * (2 * NB));
                // 16 token rows at a time (all 32 at once spill); the accumulator set goes back to the MMA as soon as its last
                // sums are in registers, before the arithmetic on them
#pragma unroll
                for (int m0 = 0; m0 < NB; m0 += 16) {
                    uint32_t p_hi[16], p_lo[16];
                    dg_tmem_ld_32x32b_x16(t_acc + (uint32_t)m0, p_hi);
                    dg_tmem_ld_32x32b_x16(t_acc + (uint32_t)(NB + m0), p_lo);
                    dg_tmem_ld_wait();
                    if (m0 + 16 == NB) {
                        dg_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(acc_empty(b));
                    }
#pragma unroll
                    for (int j = 0; j < 16; j += 4) {
                        const uint4 sxv = lds128(sz + Cfg::SX_OFF + 4 * (m0 + j));
                        const float sx4[4] = {__uint_as_float(sxv.x), __uint_as_float(sxv.y), __uint_as_float(sxv.z), __uint_as_float(sxv.w)};
#pragma unroll
                        for (int jj = 0; jj < 4; jj += 2) {
                            float &a0 = acc[m0 + j + jj], &a1 = acc[m0 + j + jj + 1];
                            f8_fma2(a0, a1, c_z, sx4[jj], sx4[jj + 1]);
                            f8_fma2(a0, a1, c_lo, __uint_as_float(p_lo[j + jj]), __uint_as_float(p_lo[j + jj + 1]));
                            f8_fma2(a0, a1, c_hi, __uint_as_float(p_hi[j + jj]), __uint_as_float(p_hi[j + jj + 1]));
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty_bar(s));  // scales, zeros and group sums of the stage have been read
            }
            if (!ok) break;
            // the segment's sums go into this CTA's slot among the tile's contributors (N is a multiple of 32: a warp's 32
            // columns are all inside the matrix or all outside)
            const int me = (int)blockIdx.x - dg_first_cta(tile, KB, tiles);
            const bool inside = tile * DG_BN + 128 * h + 32 * q < N;
#pragma unroll
            for (int m = 0; m < NB; ++m) {
                if (inside && m < M) __stcg(dg_slot_word<NB>(slots, slots_per_tile, tile, me, m, col), acc[m]);
                acc[m] = 0.f;
            }
        }
    }

    dg_fence_before();
    __syncthreads();
    if (warp == 1) {
        dg_fence_after();
        dg_tmem_dealloc(tmem_base, F8_TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------------------------------
bool gemm_decode_f8_supported(int M, int K, int N, int group_size) {
    return M <= F8_MAX_ROWS && gemm_decode_supported(M, K, N, group_size);
}

// Split token rows, their group sums and the rows' powers of two, in front of the slots.
static size_t f8_split_bytes(int M, int K) {
    const size_t rows = dg_rows(M), G = K / DG_GROUP;
    const size_t b = G * 2 * rows * DG_GROUP + G * rows * 4 + rows * 4;
    return (b + 1023) / 1024 * 1024;
}
size_t gemm_decode_f8_workspace_bytes(int M, int K, int N) {
    if (M < 1 || N < 1 || K < DG_GROUP) return 0;
    return f8_split_bytes(M, K) + gemm_decode_workspace_bytes(M, N);
}

template <int NB>
static int launch_f8(const CUtensorMap &tmX, const CUtensorMap &tmSx, const CUtensorMap &tmW, const CUtensorMap &tmS,
                     const CUtensorMap &tmZ, int M, int N, int K, int tiles, float *slots, int spt, int *ctas_out, cudaStream_t stream) {
    using Cfg = F8Cfg<NB>;
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(gemm_decode_f8_kernel<NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    });
    if (attr_err != cudaSuccess) return check_cuda(attr_err, "decode gemm (fp8 operands): shared memory attribute");
    const int sms = dg_sm_count();
    const long long U = (long long)tiles * (K / DG_GROUP);
    const int ctas = (long long)sms < U ? sms : (int)U;
    *ctas_out = ctas;
    return check_cuda(launch_pdl(gemm_decode_f8_kernel<NB>, dim3(ctas), dim3(Cfg::THREADS), Cfg::SMEM_BYTES, stream, tmX, tmSx, tmW, tmS, tmZ,
                                 M, N, K, tiles, slots, spt, wait_limit_cycles()),
                      "decode gemm (fp8 operands) launch");
}

int launch_gemm_decode_f8(const uint16_t *A, int a_f16, const int32_t *qweight, const int32_t *qzeros, const uint16_t *scales,
                          uint16_t *C, int M, int K, int N, cudaStream_t stream, int epilogue, const uint16_t *residual, int c_f16,
                          void *workspace, size_t workspace_bytes) {
    const size_t need = gemm_decode_f8_workspace_bytes(M, K, N);
    if (!workspace || workspace_bytes < need)
        return set_error(AWQ_ERR_WORKSPACE, "gemm_decode_f8: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    const int G = K / DG_GROUP, nb = N / 8, rows = dg_rows(M);
    const int tiles = (N + DG_BN - 1) / DG_BN;
    uint8_t *x8 = reinterpret_cast<uint8_t *>(workspace);
    float *sx = reinterpret_cast<float *>(x8 + (size_t)G * 2 * rows * DG_GROUP);
    float *inv = sx + (size_t)G * rows;
    float *slots = reinterpret_cast<float *>(x8 + f8_split_bytes(M, K));
    int rc;
    if (a_f16)
        rc = check_cuda(launch_pdl(act_split_kernel<true>, dim3(rows, F8_SPLIT_BLOCKS), dim3(256), 0, stream, A, M, K, rows, x8, sx, inv), "act split launch");
    else
        rc = check_cuda(launch_pdl(act_split_kernel<false>, dim3(rows, F8_SPLIT_BLOCKS), dim3(256), 0, stream, A, M, K, rows, x8, sx, inv), "act split launch");
    if (rc) return rc;
    CUtensorMap tmX, tmSx, tmW, tmS, tmZ;
    if ((rc = encode_tensor_map_2d(&tmX, CU_TENSOR_MAP_DATA_TYPE_UINT8, x8, DG_GROUP, (uint64_t)G * 2 * rows, DG_GROUP, DG_GROUP,
                                   2 * rows, CU_TENSOR_MAP_SWIZZLE_128B)))
        return rc;
    if ((rc = encode_tensor_map_2d(&tmSx, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, sx, rows, G, (uint64_t)rows * 4, rows, 1,
                                   CU_TENSOR_MAP_SWIZZLE_NONE)))
        return rc;
    if ((rc = encode_tensor_map_2d(&tmW, CU_TENSOR_MAP_DATA_TYPE_INT32, qweight, nb, K, (uint64_t)nb * 4, DG_BN / 8, DG_GROUP,
                                   CU_TENSOR_MAP_SWIZZLE_128B)))
        return rc;
    if ((rc = encode_tensor_map_2d(&tmS, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, scales, N, G, (uint64_t)N * 2, DG_BN, 1,
                                   CU_TENSOR_MAP_SWIZZLE_NONE)))
        return rc;
    if ((rc = encode_tensor_map_2d(&tmZ, CU_TENSOR_MAP_DATA_TYPE_INT32, qzeros, nb, G, (uint64_t)nb * 4, DG_BN / 8, 1,
                                   CU_TENSOR_MAP_SWIZZLE_NONE)))
        return rc;
    const int spt = dg_slots_per_tile(tiles);
    int ctas = 0;
    rc = rows == 16 ? launch_f8<16>(tmX, tmSx, tmW, tmS, tmZ, M, N, K, tiles, slots, spt, &ctas, stream)
                    : launch_f8<32>(tmX, tmSx, tmW, tmS, tmZ, M, N, K, tiles, slots, spt, &ctas, stream);
    if (rc) return rc;
    return launch_gemm_decode_fixup(rows, C, residual, epilogue, c_f16, 1.f, inv, M, N, G, tiles, ctas, slots, spt, stream);
}

int gemm_decode_f8_check(cudaStream_t stream) {
    int flag = 0;
    int rc = check_cuda(cudaStreamSynchronize(stream), "gemm_decode_f8_check sync");
    if (rc) return rc;
    rc = check_cuda(cudaMemcpyFromSymbol(&flag, g_gemm_f8_error, sizeof(int)), "gemm_decode_f8_check read");
    if (rc) return rc;
    if (flag != 0) {
        int zero = 0;
        cudaMemcpyToSymbol(g_gemm_f8_error, &zero, sizeof(int));
        return set_error(AWQ_ERR_DEVICE_TIMEOUT, "gemm_decode_f8: a device-side wait gave up (role %d)", flag);
    }
    return AWQ_OK;
}

}  // namespace awq
