// Prefill GEMM  C[M, N] = bf16(A[M, K] @ W)  with the dequantised weights in TENSOR MEMORY.
//
// The first tensor-core kernel (awq_gemm_tc.cu) dequantises a 256-column x 64-k block of weights into a bf16
// tile in shared memory, which 2 x 4 MMAs then read together with the token rows: per k-block shared memory
// moves 176 KB (1,408 wavefronts) where the tensor pipe needs 1,024 cycles.  Here the operands are swapped as
// in the batched-decode kernel (awq_gemm_decode.cu): the weights are the MMA's M side and are written by the
// dequant warps straight into tensor memory (ldmatrix.trans -> LOP3 / bf16x2 -> tcgen05.st), the token rows
// are its N side and the only thing the MMA reads from shared memory (about 700 wavefronts per k-block).
//
//   tile       256 weight columns (two 128-lane halves) x up to 192 token rows (a multiple of 16 chosen per launch so
//              that waves x rows is smallest); accumulators 2 x 192 TMEM columns
//   unit       one k-block of 64: four copies (token rows 24 KB, packed words 8 KB, scales, zeros), ring of 6
//   TMEM       512 columns: two weight buffers of 64 (2 halves x 32 columns = 64 k), one accumulator set of 384
//   warp 0     producer (one elected lane)
//   warp 1     MMA issuer (one elected lane): 8 tcgen05.mma (M 128, N = rows, K 16, A from tensor memory) per unit
//   warps 4-19 dequant: two groups of eight take alternate units (one computes while the other waits for its loads and
//              its tensor-memory stores); in a group warp w owns TMEM lanes 32 (w % 4) .. + 31 of one half
//   warps 20-27 epilogue at the end of a tile: tcgen05.ld, bf16, stores (a weight column per lane; two warps per TMEM
//              lane quarter, one for each half of the tile)
//
// Tiles are dealt round-robin to one CTA per SM.  There is one accumulator set, so the MMA issuer waits for
// the epilogue of the previous tile (about 13 % of a tile's time); loads and dequantisation of the next tile run on
// meanwhile.  Measured with a clock64 timeline: in the main loop the issuing warp is never idle and a unit's eight
// MMAs (128 x 160 x 16) take about 930 cycles, 69 % of the nominal rate, which is also what cuBLAS reaches on this
// part; a second issuing warp (one per half) and 32-bit packed epilogue stores changed nothing and are not kept.
// Every wait is bounded; on expiry the kernel records an error and all roles drain, so the tensor memory is
// always released.
#include <cudaTypedefs.h>
#include <cuda_bf16.h>

#include <mutex>

#include "awq_common.cuh"
#include "awq_ptx.cuh"
#include "awq_tcgen05.cuh"

namespace awq {

int encode_tensor_map_2d(CUtensorMap *map, int dtype, const void *base, uint64_t dim0, uint64_t dim1,
                         uint64_t stride1_bytes, uint32_t box0, uint32_t box1, int swizzle);

constexpr int TM_BN = 256, TM_BK = 64, TM_GROUP = 128;
constexpr int TM_ROWS = 192;                           // most token rows per tile (the MMA's N; a launch may use fewer)
constexpr int TM_A_BYTES = TM_ROWS * TM_BK * 2;        // 24 KB: token rows x 64 k, 128-byte rows
constexpr int TM_W_BYTES = TM_BK * (TM_BN / 8) * 4;    // 8 KB of packed words
constexpr int TM_S_BYTES = TM_BN * 2;
constexpr int TM_Z_BYTES = TM_BN / 8 * 4;
constexpr int TM_STAGE_BYTES = TM_A_BYTES + TM_W_BYTES + 1024;
constexpr int TM_STAGES = 6;
constexpr int TM_ABUF = 2;
constexpr int TM_ABUF_COLS = 2 * (TM_BK / 2);          // two halves x 64 k as bf16 pairs: 64 TMEM columns
constexpr int TM_ACC_COL0 = TM_ABUF * TM_ABUF_COLS;    // 128
constexpr uint32_t TM_TMEM_COLS = 512;
constexpr int TM_DEQUANT_WARPS = 16;
constexpr int TM_DEQUANT_WARP0 = 4, TM_EPI_WARP0 = TM_DEQUANT_WARP0 + TM_DEQUANT_WARPS;
constexpr int TM_EPI_WARPS = 8;                      // two per TMEM lane quarter: one for each 128-column half
constexpr int TM_THREADS = (TM_EPI_WARP0 + TM_EPI_WARPS) * 32;  // 896
constexpr int TM_NUM_BARS = 2 * TM_STAGES + 2 * TM_ABUF + 2;
constexpr int TM_OFF_BARS = TM_STAGES * TM_STAGE_BYTES;
constexpr int TM_SMEM_BYTES = TM_OFF_BARS + TM_NUM_BARS * 8 + 16 + 1024;
// f32 accumulate, bf16 x bf16, A (weights, tensor memory) and B (token rows) K-major, M 128; N (the tile's rows) is added at run time
constexpr uint32_t TM_IDESC_BASE = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(128 >> 4) << 24);
static_assert(TM_ACC_COL0 + 2 * TM_ROWS <= (int)TM_TMEM_COLS, "tensor memory budget");
static_assert(TM_SMEM_BYTES <= 227 * 1024, "shared memory budget");
static_assert(TM_STAGE_BYTES % 1024 == 0, "swizzled tiles need 1024-byte alignment");

__device__ int g_gemm_tm_error;  // 0 = ok; set when a bounded wait gave up

__global__ void __launch_bounds__(TM_THREADS, 1)
gemm_tm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW,
               const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmZ, uint16_t *__restrict__ C,
               const uint16_t *__restrict__ R, int epi, int M, int N, int K, int tile_rows, int row_tiles, int col_tiles,
               long long wait_limit) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + TM_OFF_BARS;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem_gen + TM_OFF_BARS + TM_NUM_BARS * 8);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };                                 // TMA landed in stage s
    auto empty_bar = [&](int s) { return bar_base + 8u * (TM_STAGES + s); };                  // MMA and dequant done with stage s
    auto ready_bar = [&](int b) { return bar_base + 8u * (2 * TM_STAGES + b); };              // weight buffer b dequantised
    auto bfree_bar = [&](int b) { return bar_base + 8u * (2 * TM_STAGES + TM_ABUF + b); };    // MMA done with weight buffer b
    const uint32_t acc_full = bar_base + 8u * (2 * TM_STAGES + 2 * TM_ABUF);                  // tile complete
    const uint32_t acc_empty = acc_full + 8u;                                                 // accumulators drained
    auto stage_addr = [&](int s) { return smem_base + (uint32_t)s * TM_STAGE_BYTES; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t TX_BYTES = (uint32_t)tile_rows * TM_BK * 2 + TM_W_BYTES + TM_S_BYTES + TM_Z_BYTES;
    const uint32_t idesc = TM_IDESC_BASE | ((uint32_t)(tile_rows >> 3) << 17);
    const int KB = K / TM_BK;
    const int n_tiles = row_tiles * col_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TM_STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1 + TM_DEQUANT_WARPS / 2);  // the MMA's commit and the eight dequant warps of the unit's group
        }
        for (int b = 0; b < TM_ABUF; ++b) {
            mbar_init(ready_bar(b), TM_DEQUANT_WARPS / 2);
            mbar_init(bfree_bar(b), 1);
        }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, TM_EPI_WARPS);
        mbar_fence_init();
    }
    if (warp == 1) {
        dg_tmem_alloc(smem_u32(tmem_slot), TM_TMEM_COLS);
        dg_tmem_relinquish();
    }
    dg_fence_before();
    __syncthreads();
    dg_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------ producer ------------------------------
        if (elect_one()) {
            tma_prefetch_desc(&tmA);
            tma_prefetch_desc(&tmW);
            tma_prefetch_desc(&tmS);
            tma_prefetch_desc(&tmZ);
        }
        int it = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
            const int m0 = (t % row_tiles) * tile_rows, n0 = (t / row_tiles) * TM_BN;
            for (int kb = 0; kb < KB; ++kb, ++it) {
                const int s = it % TM_STAGES, round = it / TM_STAGES;
                if (round > 0 && !mbar_wait_bounded_warp(empty_bar(s), (round - 1) & 1, wait_limit)) {
                    if (lane == 0) atomicExch(&g_gemm_tm_error, 1);
                    ok = false;
                    break;
                }
                const uint32_t st = stage_addr(s), bar = full_bar(s);
                const int g = (kb * TM_BK) / TM_GROUP;
                if (elect_one()) {
                    mbar_expect_tx(bar, TX_BYTES);
                    tma_load_2d(st, &tmA, kb * TM_BK, m0, bar);
                    tma_load_2d(st + TM_A_BYTES, &tmW, n0 / 8, kb * TM_BK, bar);
                    tma_load_2d(st + TM_A_BYTES + TM_W_BYTES, &tmS, n0, g, bar);
                    tma_load_2d(st + TM_A_BYTES + TM_W_BYTES + TM_S_BYTES, &tmZ, n0 / 8, g, bar);
                }
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        int it = 0, tile_it = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++tile_it) {
            if (tile_it >= 1 && !mbar_wait_bounded(acc_empty, (tile_it - 1) & 1, wait_limit)) {
                if (lane == 0) atomicExch(&g_gemm_tm_error, 2);
                break;
            }
            dg_fence_after();
            const uint32_t d_tmem = tmem_base + TM_ACC_COL0;
            for (int kb = 0; kb < KB; ++kb, ++it) {
                const int s = it % TM_STAGES, round = it / TM_STAGES;
                const int ab = it % TM_ABUF, around = it / TM_ABUF;
                // (all lanes poll: the issuing warp is the critical one here, and a wait that is already over costs a
                // single try_wait this way)
                if (!mbar_wait_bounded(full_bar(s), round & 1, wait_limit) || !mbar_wait_bounded(ready_bar(ab), around & 1, wait_limit)) {
                    if (lane == 0) atomicExch(&g_gemm_tm_error, 3);
                    ok = false;
                    break;
                }
                dg_fence_after();
                const uint32_t a_tmem = tmem_base + (uint32_t)ab * TM_ABUF_COLS;
                const uint64_t x_desc = dg_desc_sw128(stage_addr(s));  // token rows: K-major 128-byte rows
                const uint32_t acc0 = kb ? 1u : 0u;
                if (elect_one()) {
#pragma unroll
                    for (int k16 = 0; k16 < TM_BK / 16; ++k16)
#pragma unroll
                        for (int h = 0; h < 2; ++h)  // the tile's two halves of 128 weight columns
                            dg_umma_bf16_ta(d_tmem + h * TM_ROWS, a_tmem + h * (TM_BK / 2) + 8 * k16, x_desc + (uint64_t)(2 * k16), idesc,
                                            k16 ? 1u : acc0);
                    dg_umma_commit(empty_bar(s));
                    dg_umma_commit(bfree_bar(ab));
                }
                __syncwarp();
            }
            if (ok && elect_one()) dg_umma_commit(acc_full);
            __syncwarp();
        }
    } else if (warp >= TM_DEQUANT_WARP0 && warp < TM_EPI_WARP0) {
        // ------------------------------ dequant ------------------------------
        // Two groups of eight warps take alternate units (group = unit % 2 = weight buffer), so that one group computes
        // while the other waits for its loads and its tensor-memory stores; inside a group warp w owns TMEM lanes
        // 32 (w % 4) .. + 31 of one 128-column half, all 64 k.
        const int dw = warp - TM_DEQUANT_WARP0;
        const int grp = dw >> 3;
        const int q = warp & 3;        // TMEM lanes 32 q .. 32 q + 31 (a warp may only touch its own quarter)
        const int h = (dw >> 2) & 1;   // which 128-column half of the tile
        const int g = lane >> 2;       // ldmatrix.trans: lane (g, t = lane % 4) gets 16-bit column g of the chunk, rows 2t and 2t + 1
        const int chunk = 4 * h + q;   // the warp's 32 columns are one 16-byte chunk (4 packed words) of a 128-byte row
        // Row addresses of the four 8 x 8 matrices of an ldmatrix.x4: matrix m = 2 sp + x serves k16 step sp of the call's
        // 32 k and holds rows k = 16 sp + 4 j + 2 x + {0, 1} (j = 0..3), so that lane (g, t) receives the k pair 2t + x
        const int mi = lane >> 3, rr = lane & 7;
        const int k_lane = 16 * (mi >> 1) + 4 * (rr >> 1) + 2 * (mi & 1) + (rr & 1);  // + 32 for the second call
        const uint32_t w_off = (uint32_t)k_lane * 128 + (uint32_t)((chunk ^ (k_lane & 7)) << 4);  // 128B swizzle; k + 32 keeps k & 7
        int my_tiles = 0;
        for (int t = blockIdx.x; t < n_tiles; t += gridDim.x) ++my_tiles;
        const int n_units = my_tiles * KB;
        const int ab = grp;
        for (int it = grp; it < n_units; it += 2) {
            const int s = it % TM_STAGES, round = it / TM_STAGES;
            const int around = it >> 1;
            if (!mbar_wait_bounded(full_bar(s), round & 1, wait_limit)) {
                if (lane == 0) atomicExch(&g_gemm_tm_error, 4);
                break;
            }
            const uint32_t st = stage_addr(s) + TM_A_BYTES;  // packed words, then scales, then zeros
            const uint32_t zw = lds32(st + TM_W_BYTES + TM_S_BYTES + (4 * chunk + (g >> 1)) * 4) >> (16 * (g & 1));
            const uint4 sv = lds128(st + TM_W_BYTES + (32 * chunk + 8 * (g >> 1)) * 2);
            const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
            uint32_t zz[4], ss[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                zz[e] = ((zw >> (4 * e)) & 0xFu) * 0x00010001u + 0x43004300u;
                asm("prmt.b32 %0, %1, %1, %2;" : "=r"(ss[e]) : "r"(sw[e]), "r"((g & 1) ? 0x3232u : 0x1010u));
            }
            uint32_t r[2][4];
            ldmatrix_x4_trans(r[0], st + w_off);
            ldmatrix_x4_trans(r[1], st + w_off + 32 * 128);
            if (around > 0 && !mbar_wait_bounded(bfree_bar(ab), (around - 1) & 1, wait_limit)) {
                if (lane == 0) atomicExch(&g_gemm_tm_error, 4);
                break;
            }
            dg_fence_after();
            const uint32_t a_tmem = tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(ab * TM_ABUF_COLS + h * (TM_BK / 2));
#pragma unroll
            for (int c = 0; c < 2; ++c)
#pragma unroll
                for (int sp = 0; sp < 2; ++sp) {  // k16 step 2c + sp of the unit
                    const uint32_t lo = r[c][2 * sp], hi = r[c][2 * sp + 1];  // k pairs 2t and 2t + 1
                    uint32_t v[8];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        v[2 * e] = dg_bf16x2_mul(dg_bf16x2_sub(nib2_to_bf16x2_biased(lo >> (4 * e)), zz[e]), ss[e]);
                        v[2 * e + 1] = dg_bf16x2_mul(dg_bf16x2_sub(nib2_to_bf16x2_biased(hi >> (4 * e)), zz[e]), ss[e]);
                    }
                    dg_tmem_st_16x256b(a_tmem + 8 * (2 * c + sp), v[0], v[1], v[2], v[3]);
                    dg_tmem_st_16x256b(a_tmem + (16u << 16) + 8 * (2 * c + sp), v[4], v[5], v[6], v[7]);
                }
            dg_tmem_st_wait();
            dg_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(ready_bar(ab));
                mbar_arrive(empty_bar(s));
            }
        }
    } else if (warp >= TM_EPI_WARP0) {
        // ------------------------------ epilogue ------------------------------
        const int q = warp & 3;                         // this warp's 32 TMEM lanes: columns 32 q + (permuted lane) ...
        const int h = ((warp - TM_EPI_WARP0) >> 2) & 1;  // ... of this 128-column half
        int tile_it = 0;
        for (int t = blockIdx.x; t < n_tiles; t += gridDim.x, ++tile_it) {
            const int m_base = (t % row_tiles) * tile_rows, n0 = (t / row_tiles) * TM_BN;
            if (!mbar_wait_bounded(acc_full, tile_it & 1, wait_limit)) {
                if (lane == 0) atomicExch(&g_gemm_tm_error, 5);
                break;
            }
            dg_fence_after();
            const uint32_t t_acc = tmem_base + ((uint32_t)(32 * q) << 16) + TM_ACC_COL0 + (uint32_t)(h * TM_ROWS);
            const int rows = M - m_base < tile_rows ? M - m_base : tile_rows;
            if (n0 + 128 * h + 32 * q < N) {  // N is a multiple of 32: the warp's columns are all in or all out
                const int n = n0 + 128 * h + 32 * q + dg_lane_column(lane);
                // 32 token rows per tensor-memory load (the accumulator has 192 columns whatever the tile's rows, so a load
                // may run past the rows that were multiplied; what it brings from there is not stored)
#pragma unroll 1
                for (int mc = 0; mc < rows; mc += 32) {
                    uint32_t r[32];
                    dg_tmem_ld_32x32b_x32(t_acc + (uint32_t)mc, r);
                    dg_tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int m = m_base + mc + i;
                        if (mc + i >= rows) break;  // warp-uniform
                        const float v = __uint_as_float(r[i]);
                        if (epi == GEMM_EPI_SWIGLU) {
                            const float up = __shfl_down_sync(0xffffffffu, v, 1);
                            if (!(lane & 1)) C[(size_t)m * (N >> 1) + (n >> 1)] = swiglu_bits(v, up);
                        } else if (epi == GEMM_EPI_RESIDUAL) {
                            C[(size_t)m * N + n] = f32_to_bf16_bits(v + bf16_bits_to_f32(R[(size_t)m * N + n]));
                        } else {
                            C[(size_t)m * N + n] = f32_to_bf16_bits(v);
                        }
                    }
                }
            }
            dg_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty);
        }
    }

    dg_fence_before();
    __syncthreads();
    if (warp == 1) {
        dg_fence_after();
        dg_tmem_dealloc(tmem_base, TM_TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------
bool gemm_tm_supported(int M, int K, int N, int group_size) {
    return group_size == TM_GROUP && K % TM_GROUP == 0 && N % 32 == 0 && M >= 1 && K > 0 && N > 0 && device_is_sm100();
}

int launch_gemm_tm(const uint16_t *A, const int32_t *qweight, const int32_t *qzeros, const uint16_t *scales, uint16_t *C, int M, int K,
                   int N, cudaStream_t stream, int epilogue, const uint16_t *residual) {
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] { attr_err = cudaFuncSetAttribute(gemm_tm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TM_SMEM_BYTES); });
    if (attr_err != cudaSuccess) return check_cuda(attr_err, "tensor-memory gemm: shared memory attribute");
    const int G = K / TM_GROUP, nb = N / 8;
    int sms = device_sm_count();
    if (sms <= 0) sms = 148;
    // Rows per tile: tiles are dealt round-robin, so the time is waves x (time of a tile), and a tile's time grows with its
    // rows (the MMA's N) above a floor (the dequantisation of its weights): take the multiple of 16 that minimises it.
    const int col_tiles = (N + TM_BN - 1) / TM_BN;
    int tile_rows = TM_ROWS;
    long long best = -1;
    for (int r = TM_ROWS; r >= 64; r -= 16) {
        const long long t = (long long)((M + r - 1) / r) * col_tiles, waves = (t + sms - 1) / sms;
        const long long cost = waves * (r < 128 ? 128 + 32 : r + 32);
        if (best < 0 || cost < best) best = cost, tile_rows = r;
    }
    const int row_tiles = (M + tile_rows - 1) / tile_rows;
    CUtensorMap tmA, tmW, tmS, tmZ;
    int rc;
    if ((rc = encode_tensor_map_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, A, K, M, (uint64_t)K * 2, TM_BK, tile_rows,
                                   CU_TENSOR_MAP_SWIZZLE_128B)))
        return rc;
    if ((rc = encode_tensor_map_2d(&tmW, CU_TENSOR_MAP_DATA_TYPE_INT32, qweight, nb, K, (uint64_t)nb * 4, TM_BN / 8, TM_BK,
                                   CU_TENSOR_MAP_SWIZZLE_128B)))
        return rc;
    if ((rc = encode_tensor_map_2d(&tmS, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, scales, N, G, (uint64_t)N * 2, TM_BN, 1,
                                   CU_TENSOR_MAP_SWIZZLE_NONE)))
        return rc;
    if ((rc = encode_tensor_map_2d(&tmZ, CU_TENSOR_MAP_DATA_TYPE_INT32, qzeros, nb, G, (uint64_t)nb * 4, TM_BN / 8, 1,
                                   CU_TENSOR_MAP_SWIZZLE_NONE)))
        return rc;
    const long long tiles = (long long)row_tiles * col_tiles;
    const int ctas = tiles < sms ? (int)tiles : sms;
    gemm_tm_kernel<<<ctas, TM_THREADS, TM_SMEM_BYTES, stream>>>(tmA, tmW, tmS, tmZ, C, residual, epilogue, M, N, K, tile_rows, row_tiles, col_tiles,
                                                                wait_limit_cycles());
    return check_cuda(cudaGetLastError(), "tensor-memory gemm launch");
}

int gemm_tm_check(cudaStream_t stream) {
    int flag = 0;
    int rc = check_cuda(cudaStreamSynchronize(stream), "gemm_tm_check sync");
    if (rc) return rc;
    rc = check_cuda(cudaMemcpyFromSymbol(&flag, g_gemm_tm_error, sizeof(int)), "gemm_tm_check read");
    if (rc) return rc;
    if (flag != 0) {
        int zero = 0;
        cudaMemcpyToSymbol(g_gemm_tm_error, &zero, sizeof(int));
        return set_error(AWQ_ERR_DEVICE_TIMEOUT,
                         "tensor-memory gemm: a device-side wait gave up (role %d: 1 producer, 2/3 MMA issuer, 4 dequant, 5 epilogue)", flag);
    }
    return AWQ_OK;
}

}  // namespace awq
