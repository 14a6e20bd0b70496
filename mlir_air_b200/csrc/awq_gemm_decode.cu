// Batched-decode GEMM  C[M, N] = A[M, K] @ W  for AWQ int4 weights, 9 <= M <= 128 token rows
// (the batched-decode golden of matrix_multiplication/int4_awq/matmul_int4_packed.py:97-105 with M = batch),
// with the decode block's epilogues: bf16, bf16 + residual, SwiGLU over interleaved gate/up column pairs.
//
// With this few rows the product is bound by streaming the weights (0.52 B each, used once), like the GEMV,
// but there are too many rows for mma.sync to keep up, so the multiplies go to tcgen05.  A dequantised bf16
// tile in shared memory, as in the prefill kernel (awq_gemm_tc.cu), costs 4 bytes of shared-memory traffic per
// weight (2 written, 2 read by the MMA): more shared-memory cycles per SM than the weights' share of HBM time.
// So here the dequantised weights never touch shared memory:
//
//  * The operands are swapped: the weights are the MMA's M side (128 weight columns per instruction), the
//    token rows its N side (16 to 64, the batch rounded up), and the M-side operand is read from TENSOR MEMORY.
//    The dequant warps fetch the packed words with ldmatrix.trans (a register then holds the nibbles of four
//    columns at k and k + 1), turn each nibble pair into (q - z) s as a bf16 pair with one LOP3 and two
//    bf16x2 operations, and write the pairs into tensor memory with tcgen05.st.16x256b: a weight column per
//    TMEM lane, 64 TMEM columns per 128 k.  Which lane holds which column is a fixed permutation inside each
//    group of 32 columns (the one the nibble order gives for free); the epilogue undoes it.
//  * An instruction costs in proportion to the batch, and the accumulator has a weight column per TMEM lane
//    and a token row per TMEM column.
//  * Work unit = (256-column tile, 128 k = one quantisation group).  The units, tile-major, are cut into one
//    contiguous range per SM (stream-K), so every SM streams the same number of bytes whatever the shape: a
//    range covers the end of one tile, some whole tiles and the start of another.
//  * Four TMA copies per unit (token rows, 16 KB of packed words, scales, zeros) into a ring of 6 to 8 stages.
//  * The main kernel does no epilogue arithmetic.  Every segment (a CTA's units of one tile) writes its sums
//    (f32, plain coalesced stores) into the slot of the workspace that belongs to its position among the
//    tile's contributors, and a second, small kernel (gemm_decode_fixup_kernel, every SM, one thread per four
//    columns of a row) adds the slots of each tile in their fixed order and applies the epilogue.  No atomics,
//    no counters, nothing to zero, and the result does not depend on the order of arrival.  (Measured first:
//    the contributor that completes a tile finishing it inside the main kernel.  Four warps pulling five
//    contributors' sums with the few loads their registers allow kept the whole GPU waiting 20 to 50 us at
//    the end of a down projection, and the SwiGLU of a whole tile took the epilogue warp 26 us of issue
//    slots that the dequant warps, the bottleneck, share.)
//
//   warp 0      producer (one elected lane): TMA loads into the input ring
//   warp 1      MMA issuer (one elected lane): 16 tcgen05.mma (M 128, N = padded batch, K 16, A from tensor memory)
//               per unit; tcgen05.commit frees the input stage and the weight buffer, and at the end of a
//               segment hands the accumulator over
//   warps 4-19  dequant: two groups of eight take alternate units; in a group warp w owns TMEM lanes 32 (w % 4) .. + 31
//               of one 128-column half
//   warps 20-23 drain: tcgen05.ld (each warp its 32 TMEM lanes of both halves) and stores into the slot; two
//               accumulators alternate, so a segment drains while the next one runs
//
// Tensor memory (512 columns): two or three weight buffers of 128 columns, two accumulators of 2 x batch columns.
// Every wait is bounded; on expiry the kernel records an error and all roles drain, so the tensor memory is
// always released.
#include <cudaTypedefs.h>
#include <cuda_bf16.h>

#include <mutex>

#include "awq_common.cuh"
#include "awq_gemm_decode.cuh"
#include "awq_ptx.cuh"
#include "awq_streamk.cuh"
#include "awq_tcgen05.cuh"

namespace awq {

constexpr int DG_ABUF_COLS = 2 * (DG_GROUP / 2);        // a weight buffer in tensor memory: two 128-column halves x 128 k
                                                        // as bf16 pairs = 128 TMEM columns
constexpr int DG_SZ_BYTES = 1024;                       // scales, then zeros
constexpr int DG_DEQUANT_WARPS = 16;
constexpr int DG_DEQUANT_WARP0 = 4, DG_EPI_WARP0 = DG_DEQUANT_WARP0 + DG_DEQUANT_WARPS;
constexpr int DG_THREADS = (DG_EPI_WARP0 + 4) * 32;  // 768
constexpr uint32_t DG_TMEM_COLS = 512;
constexpr int DG_MAX_ROWS = 64;

// NB = token rows the MMA sees (its N): the batch rounded up to 16, 32 or 64.
template <int NB>
struct DgCfg {
    static constexpr int A_BYTES = 2 * NB * DG_BK * 2;  // two tiles of token rows x 64 k, 128-byte rows
    static constexpr int STAGE_BYTES = A_BYTES + DG_W_BYTES + DG_SZ_BYTES;
    static constexpr int RING_BUDGET = 220 * 1024;
    static constexpr int STAGES = RING_BUDGET / STAGE_BYTES < 8 ? RING_BUDGET / STAGE_BYTES : 8;
    static constexpr int ABUF = (int)(DG_TMEM_COLS - 4 * NB) / DG_ABUF_COLS;  // weight buffers: 3 up to 32 rows, 2 with 64
    static constexpr int ACC_COL0 = ABUF * DG_ABUF_COLS;                      // accumulators start behind them
    static constexpr int NUM_BARS = 3 * STAGES + 2 * ABUF + 4;
    static constexpr int OFF_BARS = STAGES * STAGE_BYTES;
    static constexpr int SMEM_BYTES = OFF_BARS + NUM_BARS * 8 + 16 + 1024;
    // f32 accumulate, A (weights, tensor memory) and B (token rows) K-major, M 128, N NB; both operands bf16 (format 1) or both
    // fp16 (format 0)
    static constexpr uint32_t IDESC_F16 = (1u << 4) | ((uint32_t)(NB >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    static constexpr uint32_t IDESC_BF16 = IDESC_F16 | (1u << 7) | (1u << 10);
    static_assert(ABUF >= 2 && ACC_COL0 + 4 * NB <= (int)DG_TMEM_COLS, "tensor memory budget");
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
    static_assert(STAGE_BYTES % 1024 == 0, "swizzled tiles need 1024-byte alignment");
    static_assert(STAGES >= 3, "input ring too shallow");
};

__device__ int g_gemm_dec_error;  // 0 = ok; set when a bounded wait gave up

// XH: the token rows are fp16 and so are the dequantised weights (11 significant bits instead of 8: what the decode stack
// uses between its kernels, like the GEMV kernels); otherwise both are bf16.
template <int NB, bool XH>
__global__ void __launch_bounds__(DG_THREADS, 1)
gemm_decode_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW,
                   const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmZ,
                   int M, int N, int K, int tiles, float *__restrict__ slots, int slots_per_tile, long long wait_limit) {
    using Cfg = DgCfg<NB>;
    constexpr int STAGES = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + Cfg::OFF_BARS;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem_gen + Cfg::OFF_BARS + Cfg::NUM_BARS * 8);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };                     // packed words, scales, zeros landed in stage s
    auto xfull_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + 2 * Cfg::ABUF + 4 + s); };  // its token rows landed
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };         // MMA and dequant done with input stage s
    auto ready_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };     // weight buffer b dequantised
    auto bfree_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + Cfg::ABUF + b); };       // MMA done with weight buffer b
    auto acc_full = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 * Cfg::ABUF + b); };    // segment complete
    auto acc_empty = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 * Cfg::ABUF + 2 + b); };  // accumulator drained
    auto stage_addr = [&](int s) { return smem_base + (uint32_t)s * Cfg::STAGE_BYTES; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr uint32_t W_TX_BYTES = DG_W_BYTES + DG_S_BYTES + DG_Z_BYTES;
    const int KB = K / DG_GROUP;  // units per tile

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(xfull_bar(s), 1);
            mbar_init(empty_bar(s), 1 + DG_DEQUANT_WARPS / 2);  // the MMA's commit and the eight dequant warps of the unit's group
        }
        for (int b = 0; b < Cfg::ABUF; ++b) {
            mbar_init(ready_bar(b), DG_DEQUANT_WARPS / 2);
            mbar_init(bfree_bar(b), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full(b), 1);
            mbar_init(acc_empty(b), 4);
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        dg_tmem_alloc(smem_u32(tmem_slot), DG_TMEM_COLS);
        dg_tmem_relinquish();
    }
    dg_fence_before();
    __syncthreads();
    dg_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();

    if (warp == 0) {
        // ------------------------------ producer ------------------------------
        // the whole warp walks the units; one elected lane issues the unit's four copies
        if (elect_one()) {
            tma_prefetch_desc(&tmA);
            tma_prefetch_desc(&tmW);
            tma_prefetch_desc(&tmS);
            tma_prefetch_desc(&tmZ);
        }
        const uint64_t stream_policy = l2_policy_evict_first();
        auto load_weights = [&](int s, int n0, int g) {
            const uint32_t st = stage_addr(s) + Cfg::A_BYTES, bar = full_bar(s);
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
                mbar_expect_tx(xfull_bar(s), Cfg::A_BYTES);
                tma_load_3d(stage_addr(s), &tmA, 0, 0, 2 * g, xfull_bar(s));
            }
            __syncwarp();
        };
        // The weights do not depend on the previous kernel in the stream: fill the ring with them, and only then wait for
        // that kernel, whose output the token rows are.
        UnitWalk w(tiles, KB);
        int it = 0;
        for (UnitWalk f = w; f.valid() && it < STAGES; ++f.u, ++it) load_weights(it, f.tile() * DG_BN, f.kb());
        pdl_wait();
        it = 0;
        for (UnitWalk f = w; f.valid() && it < STAGES; ++f.u, ++it) load_rows(it, f.kb());
        for (w.u += it; w.valid(); ++w.u, ++it) {
            const int s = it % STAGES, round = it / STAGES;
            if (!mbar_wait_bounded_warp(empty_bar(s), (round - 1) & 1, wait_limit)) {
                if (lane == 0) atomicExch(&g_gemm_dec_error, 1);
                break;
            }
            load_weights(s, w.tile() * DG_BN, w.kb());
            load_rows(s, w.kb());
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        // the whole warp walks the units and waits; one elected lane issues
        int it = 0, seg_it = 0;
        bool ok = true;
        UnitWalk w(tiles, KB);
        while (w.valid() && ok) {
            const int n_seg = w.left_in_tile();  // this segment: n_seg units of one tile
            const int b = seg_it & 1, use = seg_it >> 1;
            if (use >= 1 && !mbar_wait_bounded_warp(acc_empty(b), (use - 1) & 1, wait_limit)) {
                if (lane == 0) atomicExch(&g_gemm_dec_error, 2);
                break;
            }
            dg_fence_after();
            const uint32_t d_tmem = tmem_base + Cfg::ACC_COL0 + (uint32_t)b * (2 * NB);
            for (int i = 0; i < n_seg; ++i, ++it, ++w.u) {
                const int s = it % STAGES, round = it / STAGES;
                const int ab = it % Cfg::ABUF, around = it / Cfg::ABUF;
                // token rows landed and weight buffer written: two lanes wait side by side
                if (!mbar_wait_multi_warp(2, xfull_bar(s), round & 1, ready_bar(ab), around & 1, 0, 0, wait_limit)) {
                    if (lane == 0) atomicExch(&g_gemm_dec_error, 3);
                    ok = false;
                    break;
                }
                dg_fence_after();
                const uint32_t a_tmem = tmem_base + (uint32_t)ab * DG_ABUF_COLS;
                // token rows: K-major 128-byte rows, two tiles of 64 k, 32 bytes further in the row per step
                const uint64_t x_desc = dg_desc_sw128(stage_addr(s));
                const uint32_t acc0 = i ? 1u : 0u;
                if (elect_one()) {
#pragma unroll
                    for (int k16 = 0; k16 < DG_GROUP / 16; ++k16) {
#pragma unroll
                        for (int h = 0; h < 2; ++h)  // the tile's two halves of 128 weight columns
                            dg_umma_bf16_ta(d_tmem + h * NB, a_tmem + h * (DG_GROUP / 2) + 8 * k16,
                                            x_desc + (uint64_t)((k16 >> 2) * ((Cfg::A_BYTES / 2) >> 4) + 2 * (k16 & 3)), XH ? Cfg::IDESC_F16 : Cfg::IDESC_BF16,
                                            k16 ? 1u : acc0);
                    }
                    dg_umma_commit(empty_bar(s));
                    dg_umma_commit(bfree_bar(ab));
                }
                __syncwarp();
            }
            if (ok && elect_one()) dg_umma_commit(acc_full(b));
            __syncwarp();
            ++seg_it;
        }
    } else if (warp >= DG_DEQUANT_WARP0 && warp < DG_EPI_WARP0) {
        // ------------------------------ dequant ------------------------------
        // Two groups of eight warps take alternate units, so that one group computes while the other waits for its loads
        // and its tensor-memory stores; inside a group warp w owns TMEM lanes 32 (w % 4) .. + 31 of one 128-column half,
        // all 128 k.
        const int dw = warp - DG_DEQUANT_WARP0;
        const int grp = dw >> 3;
        const int q = warp & 3;        // TMEM lanes 32 q .. 32 q + 31 (a warp may only touch its own quarter)
        const int h = (dw >> 2) & 1;   // which 128-column half of the tile
        const int g = lane >> 2;       // ldmatrix.trans: lane (g, t = lane % 4) gets 16-bit column g of the chunk, rows 2t and 2t + 1
        const int chunk = 4 * h + q;   // the warp's 32 columns are one 16-byte chunk (4 packed words) of a 128-byte row
        // Row addresses of the four 8 x 8 matrices of one ldmatrix.x4: matrix m = 2 sp + x serves k16 step sp of the call's
        // 32 k and holds rows k = 16 sp + 4 j + 2 x + {0, 1} (j = 0..3), so that lane (g, t) receives the k pair 2t + x:
        // TMEM columns 2t and 2t + 1 of the step are what tcgen05.st.16x256b takes from this lane.
        const int mi = lane >> 3, rr = lane & 7;
        const int k_lane = 16 * (mi >> 1) + 4 * (rr >> 1) + 2 * (mi & 1) + (rr & 1);  // + 32 c for call c
        const uint32_t w_off = (uint32_t)k_lane * 128 + (uint32_t)((chunk ^ (k_lane & 7)) << 4);  // 128B swizzle; k + 32 c keeps k & 7
        UnitWalk w(tiles, KB);
        const int n_units = w.u1 - w.u;
        for (int it = grp; it < n_units; it += 2) {
            const int s = it % STAGES, round = it / STAGES;
            const int ab = it % Cfg::ABUF, around = it / Cfg::ABUF;
            if (!mbar_wait_bounded(full_bar(s), round & 1, wait_limit)) {
                if (lane == 0) atomicExch(&g_gemm_dec_error, 4);
                break;
            }
            const uint32_t st = stage_addr(s) + Cfg::A_BYTES;  // packed words, then scales, then zeros
            // this lane's four columns (nibbles e of its half word: columns 2e + (g & 1) of the word): 128 + z and the scale,
            // each twice (k, k + 1)
            const uint32_t zw = lds32(st + DG_W_BYTES + DG_S_BYTES + (4 * chunk + (g >> 1)) * 4) >> (16 * (g & 1));
            const uint4 sv = lds128(st + DG_W_BYTES + (32 * chunk + 8 * (g >> 1)) * 2);
            const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
            uint32_t zz[4], ss[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                zz[e] = ((zw >> (4 * e)) & 0xFu) * 0x00010001u + (XH ? 0x64006400u : 0x43004300u);  // 1024 + z / 128 + z
                asm("prmt.b32 %0, %1, %1, %2;" : "=r"(ss[e]) : "r"(sw[e]), "r"((g & 1) ? 0x3232u : 0x1010u));
                if (XH) {  // the scale as fp16 (exact for scales of 2^-14 and more)
                    const uint32_t hbits = bf16_value_to_f16_bits(__uint_as_float(ss[e] << 16));
                    ss[e] = hbits * 0x00010001u;
                }
            }
            uint32_t r[4][4];
#pragma unroll
            for (int c = 0; c < 4; ++c) ldmatrix_x4_trans(r[c], st + w_off + c * 32 * 128);
            if (around > 0 && !mbar_wait_bounded(bfree_bar(ab), (around - 1) & 1, wait_limit)) {
                if (lane == 0) atomicExch(&g_gemm_dec_error, 4);
                break;
            }
            dg_fence_after();
            const uint32_t a_tmem = tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(ab * DG_ABUF_COLS + h * (DG_GROUP / 2));
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int sp = 0; sp < 2; ++sp) {  // k16 step 2c + sp of the unit
                    const uint32_t lo = r[c][2 * sp], hi = r[c][2 * sp + 1];  // k pairs 2t and 2t + 1
                    uint32_t v[8];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        if (XH) {  // (1024 + q) - (1024 + z) and the product, each exact or rounded once, in fp16
                            v[2 * e] = dg_f16x2_mul(dg_f16x2_sub(lop3_and_or(lo >> (4 * e), 0x000F000Fu, 0x64006400u), zz[e]), ss[e]);
                            v[2 * e + 1] = dg_f16x2_mul(dg_f16x2_sub(lop3_and_or(hi >> (4 * e), 0x000F000Fu, 0x64006400u), zz[e]), ss[e]);
                        } else {
                            v[2 * e] = dg_bf16x2_mul(dg_bf16x2_sub(nib2_to_bf16x2_biased(lo >> (4 * e)), zz[e]), ss[e]);
                            v[2 * e + 1] = dg_bf16x2_mul(dg_bf16x2_sub(nib2_to_bf16x2_biased(hi >> (4 * e)), zz[e]), ss[e]);
                        }
                    }
                    // lanes g and g + 8 hold nibbles 0 and 1, lanes g + 16 and g + 24 nibbles 2 and 3
                    dg_tmem_st_16x256b(a_tmem + 8 * (2 * c + sp), v[0], v[1], v[2], v[3]);
                    dg_tmem_st_16x256b(a_tmem + (16u << 16) + 8 * (2 * c + sp), v[4], v[5], v[6], v[7]);
                }
            dg_tmem_st_wait();
            dg_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(ready_bar(ab));
                mbar_arrive(empty_bar(s));  // this warp has read the stage's words, scales and zeros
            }
        }
    } else if (warp >= DG_EPI_WARP0) {
        // ------------------------------ drain ------------------------------
        const int q = warp & 3;  // this warp's 32 TMEM lanes: columns 32 q + lane of each 128-column half
        pdl_wait();  // the previous kernel in the stream may still be reading the slots
        int seg_it = 0;
        UnitWalk w(tiles, KB);
        while (w.valid()) {
            const int tile = w.tile(), n_seg = w.left_in_tile();
            w.u += n_seg;
            const int b = seg_it & 1, use = seg_it >> 1;
            ++seg_it;
            const int n0 = tile * DG_BN;
            if (!mbar_wait_bounded(acc_full(b), use & 1, wait_limit)) {
                if (lane == 0) atomicExch(&g_gemm_dec_error, 5);
                break;
            }
            dg_fence_after();
            const uint32_t t_acc = tmem_base + ((uint32_t)(32 * q) << 16) + Cfg::ACC_COL0 + (uint32_t)b * (2 * NB);
            // N is a multiple of 32: a warp's 32 columns are all inside the matrix or all outside
            const bool in0 = n0 + 32 * q < N, in1 = n0 + 128 + 32 * q < N;
            // the segment's sums go into this CTA's slot among the tile's contributors
            const int me = (int)blockIdx.x - dg_first_cta(tile, KB, tiles);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (!(h ? in1 : in0)) continue;
                const int col = 128 * h + 32 * q + dg_lane_column(lane);
#pragma unroll 1
                for (int m0 = 0; m0 < M; m0 += 16) {
                    uint32_t r[16];
                    dg_tmem_ld_32x32b_x16(t_acc + (uint32_t)(h * NB + m0), r);
                    dg_tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        if (m0 + i < M) __stcg(dg_slot_word<NB>(slots, slots_per_tile, tile, me, m0 + i, col), __uint_as_float(r[i]));
                }
            }
            dg_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty(b));
        }
    }

    dg_fence_before();
    __syncthreads();
    if (warp == 1) {
        dg_fence_after();
        dg_tmem_dealloc(tmem_base, DG_TMEM_COLS);
    }
}

// Second pass: one thread per four columns of a token row adds the slots of the tile's contributors in their order and
// applies the epilogue.  A block takes four token rows of one tile.  `main_ctas` is the main kernel's grid size (the
// ranges of its CTAs decide who contributed to which tile).
template <int NB>
__global__ void __launch_bounds__(256)
gemm_decode_fixup_kernel(uint16_t *__restrict__ C, const uint16_t *__restrict__ R, int epi, int c_f16, float sum_scale,
                         const float *__restrict__ row_scale, int M, int N, int KB, int tiles, int main_ctas,
                         const float *__restrict__ slots, int slots_per_tile) {
    pdl_launch_dependents();
    pdl_wait();
    const int row_chunks = (M + 3) >> 2;
    const int tile = blockIdx.x / row_chunks, m = 4 * (blockIdx.x - tile * row_chunks) + (threadIdx.x >> 6);
    const int col = 4 * (threadIdx.x & 63), n = tile * DG_BN + col;
    if (m >= M || n >= N) return;
    const long long U = (long long)tiles * KB;
    const int first = (int)((((long long)tile * KB + 1) * main_ctas + U - 1) / U) - 1;
    const int last = (int)((((long long)(tile + 1) * KB) * main_ctas + U - 1) / U) - 1;
    const float *src = slots + (((size_t)tile * slots_per_tile) * NB + m) * DG_BN + col;
    float4 sum = __ldcg(reinterpret_cast<const float4 *>(src));
    for (int c = 1; c <= last - first; ++c) {
        const float4 v = __ldcg(reinterpret_cast<const float4 *>(src + (size_t)c * NB * DG_BN));
        sum.x += v.x, sum.y += v.y, sum.z += v.z, sum.w += v.w;
    }
    if (row_scale) {  // powers of two that the main kernel's operands left out: exact
        const float f = sum_scale * row_scale[m];
        sum.x *= f, sum.y *= f, sum.z *= f, sum.w *= f;
    }
    if (epi == GEMM_EPI_F32) {  // a tensor-parallel rank's partial sums, to be added up across the ranks
        *reinterpret_cast<float4 *>(reinterpret_cast<float *>(C) + (size_t)m * N + n) = sum;
    } else if (epi == GEMM_EPI_SWIGLU) {
        uint32_t o0 = swiglu_bits(sum.x, sum.y), o1 = swiglu_bits(sum.z, sum.w);
        if (c_f16) {  // the bf16 value, in the fp16 form the next product reads
            o0 = bf16_value_to_f16_bits(bf16_bits_to_f32((uint16_t)o0));
            o1 = bf16_value_to_f16_bits(bf16_bits_to_f32((uint16_t)o1));
        }
        *reinterpret_cast<uint32_t *>(C + (size_t)m * (N >> 1) + (n >> 1)) = o0 | (o1 << 16);
    } else {
        if (epi == GEMM_EPI_RESIDUAL) {
            const uint2 rv = *reinterpret_cast<const uint2 *>(R + (size_t)m * N + n);
            sum.x += bf16x2_lo(rv.x), sum.y += bf16x2_hi(rv.x), sum.z += bf16x2_lo(rv.y), sum.w += bf16x2_hi(rv.y);
        }
        if (c_f16) {
            const uint32_t o0 = (uint32_t)bf16_value_to_f16_bits(sum.x) | ((uint32_t)bf16_value_to_f16_bits(sum.y) << 16);
            const uint32_t o1 = (uint32_t)bf16_value_to_f16_bits(sum.z) | ((uint32_t)bf16_value_to_f16_bits(sum.w) << 16);
            *reinterpret_cast<uint2 *>(C + (size_t)m * N + n) = make_uint2(o0, o1);
        } else {
            *reinterpret_cast<uint2 *>(C + (size_t)m * N + n) = make_uint2(pack_bf16x2(sum.x, sum.y), pack_bf16x2(sum.z, sum.w));
        }
    }
}

// ---------------------------------------------------------------------------------------------
bool gemm_decode_supported(int M, int K, int N, int group_size) {
    return group_size == DG_GROUP && K % DG_GROUP == 0 && N % 32 == 0 && M >= 1 && M <= DG_MAX_ROWS && K > 0 &&
           N > 0 && (N + DG_BN - 1) / DG_BN <= DG_MAX_TILES && device_is_sm100();
}

int dg_rows(int M) { return M <= 16 ? 16 : (M <= 32 ? 32 : 64); }

int dg_sm_count() {
    const int sms = device_sm_count();
    return sms > 0 ? sms : 148;
}
// Slots a tile needs: the most CTAs whose ranges can reach into one tile.
int dg_slots_per_tile(int tiles) { return dg_sm_count() / tiles + 2; }

// The slots of every tile.  tiles x slots_per_tile <= SMs + 2 tiles: that bound is what is asked for, so that a workspace
// sized for some N also serves every smaller N (tiles x (SMs / tiles + 2) itself does not grow monotonically with N).
size_t gemm_decode_workspace_bytes(int M, int N) {
    if (M < 1 || N < 1) return 0;
    const size_t tiles = (size_t)(N + DG_BN - 1) / DG_BN;
    return ((size_t)dg_sm_count() + 2 * tiles) * DG_BN * dg_rows(M) * 4;
}

template <int NB, bool XH>
static int launch_dg(const CUtensorMap &tmA, const CUtensorMap &tmW, const CUtensorMap &tmS, const CUtensorMap &tmZ, uint16_t *C,
                     const uint16_t *residual, int epilogue, int c_f16, int M, int N, int K, int tiles, void *workspace,
                     cudaStream_t stream) {
    using Cfg = DgCfg<NB>;
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(gemm_decode_kernel<NB, XH>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    });
    if (attr_err != cudaSuccess) return check_cuda(attr_err, "decode gemm: shared memory attribute");
    const int sms = dg_sm_count();
    const long long U = (long long)tiles * (K / DG_GROUP);
    const int ctas = (long long)sms < U ? sms : (int)U;
    float *slots = reinterpret_cast<float *>(workspace);
    const int spt = dg_slots_per_tile(tiles);
    int rc = check_cuda(launch_pdl(gemm_decode_kernel<NB, XH>, dim3(ctas), dim3(DG_THREADS), Cfg::SMEM_BYTES, stream, tmA, tmW, tmS, tmZ, M, N, K,
                                   tiles, slots, spt, wait_limit_cycles()),
                        "decode gemm launch");
    if (rc) return rc;
    return launch_gemm_decode_fixup(NB, C, residual, epilogue, c_f16, 1.f, nullptr, M, N, K / DG_GROUP, tiles, ctas, slots, spt, stream);
}

int launch_gemm_decode_fixup(int rows, uint16_t *C, const uint16_t *residual, int epilogue, int c_f16, float sum_scale,
                             const float *row_scale, int M, int N, int KB, int tiles, int main_ctas, const float *slots,
                             int slots_per_tile, cudaStream_t stream) {
    const int blocks = tiles * ((M + 3) / 4);
#define DG_FIXUP(NBV)                                                                                                          \
    launch_pdl(gemm_decode_fixup_kernel<NBV>, dim3(blocks), dim3(256), 0, stream, C, residual, epilogue, c_f16, sum_scale, row_scale, \
               M, N, KB, tiles, main_ctas, slots, slots_per_tile)
    return check_cuda(rows == 16 ? DG_FIXUP(16) : (rows == 32 ? DG_FIXUP(32) : DG_FIXUP(64)), "decode gemm fix-up launch");
#undef DG_FIXUP
}

int launch_gemm_decode(const uint16_t *A, const int32_t *qweight, const int32_t *qzeros, const uint16_t *scales, uint16_t *C, int M,
                       int K, int N, cudaStream_t stream, int epilogue, const uint16_t *residual, void *workspace,
                       size_t workspace_bytes, int a_f16, int c_f16) {
    const size_t need = gemm_decode_workspace_bytes(M, N);
    if (!workspace || workspace_bytes < need)
        return set_error(AWQ_ERR_WORKSPACE, "gemm_decode: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    const int G = K / DG_GROUP, nb = N / 8, rows = dg_rows(M);
    const int tiles = (N + DG_BN - 1) / DG_BN;
    CUtensorMap tmA, tmW, tmS, tmZ;
    int rc;
    // token rows as (64 k, rows, K / 64): one copy brings the two 64-k tiles of a unit
    if ((rc = encode_tensor_map_3d(&tmA, a_f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, A, DG_BK, M, K / DG_BK, (uint64_t)K * 2, DG_BK * 2, DG_BK,
                                   rows, 2, CU_TENSOR_MAP_SWIZZLE_128B)))
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
#define DG_LAUNCH(NBV, XHV) launch_dg<NBV, XHV>(tmA, tmW, tmS, tmZ, C, residual, epilogue, c_f16, M, N, K, tiles, workspace, stream)
    if (a_f16) return rows == 16 ? DG_LAUNCH(16, true) : (rows == 32 ? DG_LAUNCH(32, true) : DG_LAUNCH(64, true));
    return rows == 16 ? DG_LAUNCH(16, false) : (rows == 32 ? DG_LAUNCH(32, false) : DG_LAUNCH(64, false));
#undef DG_LAUNCH
}

int gemm_decode_check(cudaStream_t stream) {
    int flag = 0;
    int rc = check_cuda(cudaStreamSynchronize(stream), "gemm_decode_check sync");
    if (rc) return rc;
    rc = check_cuda(cudaMemcpyFromSymbol(&flag, g_gemm_dec_error, sizeof(int)), "gemm_decode_check read");
    if (rc) return rc;
    if (flag != 0) {
        int zero = 0;
        cudaMemcpyToSymbol(g_gemm_dec_error, &zero, sizeof(int));
        return set_error(AWQ_ERR_DEVICE_TIMEOUT,
                         "decode gemm: a device-side wait gave up (role %d: 1 producer, 2/3 MMA issuer, 4 dequant, 5 epilogue); "
                         "re-initialise the workspace", flag);
    }
    return AWQ_OK;
}

}  // namespace awq
