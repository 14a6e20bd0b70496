// Prefill GEMM  C[M, N] = A[M, K] @ W  for AWQ int4 weights on the 5th-generation tensor cores.
//
// Compute-bound (2 M K N flops against 0.52 B per weight), so the weights are dequantised once
// per CTA tile into shared memory as bf16 -- bit-exactly bf16_rne((q - z) s), the same value the
// dequant kernel writes -- and fed to tcgen05.mma with the accumulator in tensor memory.
//
//   tile        MT x 128 (M) x 256 (N) per CTA with MT = 2 (MT = 1 when M <= 128): the two 128-row
//               accumulators share one dequantised B tile, which halves the dequant work per
//               flop; k-block 64.  Scheduling: the CTAs are split evenly over the M blocks and each
//               owns a contiguous range of 64-column atoms of its M block, walked in sub-tiles
//               of up to 4 atoms (256 columns), so no SM waits for a partial last wave; CTAs
//               of different M blocks walk the same columns at the same time (weights from L2)
//   warp 0      producer: TMA loads of the A tile (128 x 64 bf16, 128B swizzle), the packed
//               words (64 k rows x 32 words), scales and zeros of the k-block
//   warps 4-11  dequant: warp w owns k rows 8w .. 8w+7, lane j packed word j (8 columns); a word
//               unpacks to four bf16 pairs of adjacent columns (128 + q) by LOP3, exact
//               (v - (128 + z)) * s in bf16x2, and goes out as ONE 16-byte store: the B tile is
//               kept N-major ("MN-major", 128B swizzle), which is the order the AWQ word already
//               has, so nothing is transposed (all shared-memory accesses bank-conflict free)
//   warp 1      MMA issuer (one thread): 4 x MT tcgen05.mma.kind::f16 (M 128, N 256, K 16) per
//               k-block into 256-column TMEM accumulators (512 columns: MT = 1 double-buffers them,
//               MT = 2 uses both for one tile); tcgen05.commit releases the stage and, after the
//               last k-block, hands the accumulators to the epilogue
//   warps 12-15 epilogue: tcgen05.ld (each warp its 32 TMEM lanes), f32 -> bf16, global stores;
//               with MT = 1 it overlaps the next tile's main loop
//
// Every mbarrier wait is bounded; on expiry the kernel records an error and all roles drain, so
// the tensor memory is always released.
#include <cudaTypedefs.h>
#include <cuda_bf16.h>

#include <mutex>

#include "awq_common.cuh"
#include "awq_ptx.cuh"

namespace awq {

int encode_tensor_map_2d(CUtensorMap *map, int dtype, const void *base, uint64_t dim0, uint64_t dim1,
                         uint64_t stride1_bytes, uint32_t box0, uint32_t box1, int swizzle);

constexpr int TC_BM = 128, TC_BN = 256, TC_BK = 64, TC_GROUP = 128;
constexpr int TC_STAGES = 3;
constexpr int TC_PREFETCH = 12;  // k-blocks of packed words requested into L2 ahead of the ring
constexpr int TC_A_BYTES = 2 * TC_BM * TC_BK * 2;    // 32 KB: room for two 128-row A tiles
constexpr int TC_B_BYTES = TC_BN * TC_BK * 2;        // 32 KB
constexpr int TC_W_BYTES = TC_BK * (TC_BN / 8) * 4;  // 8 KB of packed words
constexpr int TC_S_BYTES = TC_BN * 2;
constexpr int TC_Z_BYTES = TC_BN / 8 * 4;
constexpr int TC_OFF_B = TC_A_BYTES;
constexpr int TC_OFF_W = TC_OFF_B + TC_B_BYTES;
constexpr int TC_OFF_S = TC_OFF_W + TC_W_BYTES;
constexpr int TC_OFF_Z = TC_OFF_S + TC_S_BYTES;
constexpr int TC_STAGE_BYTES = 73 * 1024;
constexpr int TC_TABLE_BYTES = 0;
constexpr int TC_B_NATOM_BYTES = 8 * 1024;  // B tile: 64-column atoms 8 KB apart, 8-row k atoms 1 KB apart
constexpr int TC_NUM_BARS = 3 * TC_STAGES + 4;
constexpr int TC_SMEM_BYTES = TC_STAGES * TC_STAGE_BYTES + TC_TABLE_BYTES + TC_NUM_BARS * 8 + 16 + 1024;
constexpr int TC_THREADS = 512;
constexpr int TC_DEQUANT_WARP0 = 4, TC_EPI_WARP0 = 12;
constexpr uint32_t TC_TMEM_COLS = 512;
static_assert(TC_OFF_Z + TC_Z_BYTES <= TC_STAGE_BYTES, "stage too small");
static_assert(TC_SMEM_BYTES <= 227 * 1024, "shared memory budget");

__device__ int g_gemm_error;  // 0 = ok; set when a bounded wait gave up

// ---- tcgen05 wrappers -----------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// D[tmem] (+)= A[smem] * B[smem], bf16 inputs, f32 accumulate
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The mbarrier gets one arrival when every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap *map, int x, int y) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];" ::"l"(map), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major tile of 128-byte rows, 128B swizzle, 8-row atoms 1024 B apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);  // start address
    d |= (uint64_t)1 << 16;                        // leading byte offset (unused with swizzle, K-major)
    d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset between 8-row atoms
    d |= (uint64_t)1 << 46;                        // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                        // 128-byte swizzle
    return d;
}
// N-major ("MN-major") tile with 128B swizzle: atoms of 64 columns (128 B) x 8 k rows; `lbo`
// bytes between atoms along N, `sbo` bytes between atoms along K.
__device__ __forceinline__ uint64_t umma_desc_sw128_nmajor(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// Instruction descriptor without its N field (bits 17-22 = N / 8, set per sub-tile): f32
// accumulate, bf16 x bf16, A K-major, B N-major, M 128.
constexpr uint32_t TC_IDESC_BASE = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(TC_BM >> 4) << 24);

__device__ __forceinline__ uint32_t bf16x2_sub(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

// The same walk over a CTA's sub-tiles for every warp role.  CTA (ml, p) of ML x P: M blocks
// ml, ml + ML, ...; in each, atoms [p NA / P, (p + 1) NA / P) in steps of up to 4 (full-width
// sub-tiles first: 13 atoms -> 4, 4, 4, 1 measured faster than 4, 3, 3, 3).
struct TileWalk {
    int ML, m_blocks, a0, a1, mb, a;
    __device__ __forceinline__ TileWalk(int ml_count, int p_count, int m_block_count, int atoms) {
        ML = ml_count;
        m_blocks = m_block_count;
        const int p = blockIdx.x / ML;
        a0 = (int)((long long)p * atoms / p_count);
        a1 = (int)((long long)(p + 1) * atoms / p_count);
        mb = blockIdx.x % ML;
        a = a0;
    }
    __device__ __forceinline__ bool valid() const { return mb < m_blocks && a0 < a1; }
    __device__ __forceinline__ int atoms() const { return a1 - a < 4 ? a1 - a : 4; }
    __device__ __forceinline__ void next() {
        a += atoms();
        if (a >= a1) {
            a = a0;
            mb += ML;
        }
    }
};

template <int MT>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW,
               const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmZ,
               uint16_t *__restrict__ C, const uint16_t *__restrict__ R, int epi, int M, int N, int K, int ML, int P,
               long long wait_limit) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + TC_STAGES * TC_STAGE_BYTES + TC_TABLE_BYTES;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem_gen + TC_STAGES * TC_STAGE_BYTES + TC_TABLE_BYTES +
                                                       TC_NUM_BARS * 8);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };                       // TMA landed
    auto ready_bar = [&](int s) { return bar_base + 8u * (TC_STAGES + s); };        // B tile dequantised
    auto empty_bar = [&](int s) { return bar_base + 8u * (2 * TC_STAGES + s); };    // MMA done with the stage
    auto acc_full = [&](int b) { return bar_base + 8u * (3 * TC_STAGES + b); };     // accumulator complete
    auto acc_empty = [&](int b) { return bar_base + 8u * (3 * TC_STAGES + 2 + b); };  // accumulator drained

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int NBUF = 2 / MT;  // accumulator buffers
    constexpr uint32_t TX_BYTES = MT * TC_BM * TC_BK * 2 + TC_W_BYTES + TC_S_BYTES + TC_Z_BYTES;
    const int m_blocks = (M + MT * TC_BM - 1) / (MT * TC_BM), n_atoms = (N + 63) / 64;
    const int k_blocks = K / TC_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(ready_bar(s), 8);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full(b), 1);
            mbar_init(acc_empty(b), 4);
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), TC_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------ producer ------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&tmA);
            tma_prefetch_desc(&tmW);
            tma_prefetch_desc(&tmS);
            tma_prefetch_desc(&tmZ);
            int it = 0;
            bool ok = true;
            for (TileWalk tw(ML, P, m_blocks, n_atoms); tw.valid() && ok; tw.next()) {
                const int m0 = tw.mb * (MT * TC_BM), n0 = tw.a * 64;
                // With few rows (decode batches) the packed words come from HBM, not L2, and three 8 KB
                // boxes in flight per SM cannot cover that latency: ask L2 for them TC_PREFETCH k-blocks ahead.
                for (int kb = 0; kb < TC_PREFETCH && kb < k_blocks; ++kb) tma_prefetch_l2_2d(&tmW, n0 / 8, kb * TC_BK);
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    if (kb + TC_PREFETCH < k_blocks) tma_prefetch_l2_2d(&tmW, n0 / 8, (kb + TC_PREFETCH) * TC_BK);
                    const int s = it % TC_STAGES, round = it / TC_STAGES;
                    if (round > 0 && !mbar_wait_bounded(empty_bar(s), (round - 1) & 1, wait_limit)) {
                        atomicExch(&g_gemm_error, 1);
                        ok = false;
                        break;
                    }
                    const uint32_t st = smem_base + s * TC_STAGE_BYTES;
                    const int g = (kb * TC_BK) / TC_GROUP;
                    mbar_expect_tx(full_bar(s), TX_BYTES);
                    tma_load_2d(st, &tmA, kb * TC_BK, m0, full_bar(s));  // MT * 128 rows in one box
                    tma_load_2d(st + TC_OFF_W, &tmW, n0 / 8, kb * TC_BK, full_bar(s));
                    tma_load_2d(st + TC_OFF_S, &tmS, n0, g, full_bar(s));
                    tma_load_2d(st + TC_OFF_Z, &tmZ, n0 / 8, g, full_bar(s));
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            int it = 0, tile_it = 0;
            bool ok = true;
            for (TileWalk tw(ML, P, m_blocks, n_atoms); tw.valid() && ok; tw.next(), ++tile_it) {
                const uint32_t idesc = TC_IDESC_BASE | ((uint32_t)(tw.atoms() * 64 >> 3) << 17);
                const int b = tile_it % NBUF, use = tile_it / NBUF;  // buffer and how often it was used before
                if (use >= 1 && !mbar_wait_bounded(acc_empty(b), (use - 1) & 1, wait_limit)) {
                    atomicExch(&g_gemm_error, 2);
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)b * TC_BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % TC_STAGES, round = it / TC_STAGES;
                    if (!mbar_wait_bounded(full_bar(s), round & 1, wait_limit) || !mbar_wait_bounded(ready_bar(s), round & 1, wait_limit)) {
                        atomicExch(&g_gemm_error, 3);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t st = smem_base + s * TC_STAGE_BYTES;
                    const uint64_t a_desc = umma_desc_sw128(st);
                    const uint64_t b_desc = umma_desc_sw128_nmajor(st + TC_OFF_B, TC_B_NATOM_BYTES, 1024);
#pragma unroll
                    for (int k4 = 0; k4 < TC_BK / 16; ++k4)  // A: 32 bytes further in the row; B: two k atoms further
#pragma unroll
                        for (int a = 0; a < MT; ++a)  // second 128 rows of A: 16 KB further, next 256 TMEM columns
                            umma_bf16(d_tmem + a * TC_BN, a_desc + 2 * k4 + a * (16384 >> 4), b_desc + (2048 >> 4) * k4,
                                      idesc, (kb | k4) ? 1u : 0u);
                    umma_commit(empty_bar(s));
                }
                if (ok) umma_commit(acc_full(b));
            }
        }
    } else if (warp >= TC_DEQUANT_WARP0 && warp < TC_EPI_WARP0) {
        // ------------------------------ dequant ------------------------------
        const int w = warp - TC_DEQUANT_WARP0;  // k atom: rows 8w .. 8w+7 of the k-block
        int it = 0;
        bool ok = true;
        for (TileWalk tw(ML, P, m_blocks, n_atoms); tw.valid() && ok; tw.next()) {
            // a sub-tile of 1 / 2 / 3-4 atoms has 8 / 16 / 32 packed words per row: the warp takes
            // 4 / 2 / 1 rows at a time so that narrow sub-tiles cost proportionally less
            const int words = tw.atoms() * 8;
            const int rows_at_once = words <= 8 ? 4 : (words <= 16 ? 2 : 1);
            const int lanes_per_row = 32 / rows_at_once;
            const int j = lane % lanes_per_row;     // packed word: tile columns 8j .. 8j+7
            const int r_sub = lane / lanes_per_row;
            const bool active = j < words;
            for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                const int s = it % TC_STAGES, round = it / TC_STAGES;
                if ((round > 0 && !mbar_wait_bounded(empty_bar(s), (round - 1) & 1, wait_limit)) ||
                    !mbar_wait_bounded(full_bar(s), round & 1, wait_limit)) {
                    if (lane == 0) atomicExch(&g_gemm_error, 4);
                    ok = false;
                    break;
                }
                const uint32_t st = smem_base + s * TC_STAGE_BYTES;
                if (active) {
                // this word's eight columns: 128 + z as bf16 pairs, and the scale pairs as stored
                const uint32_t zw = lds32(st + TC_OFF_Z + j * 4);
                const uint4 sv = lds128(st + TC_OFF_S + j * 16);
                const uint32_t ss[4] = {sv.x, sv.y, sv.z, sv.w};
                uint32_t zz[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) zz[e] = nib2_to_bf16x2_biased(zw >> (4 * e));
                const uint32_t w_src = st + TC_OFF_W + (8 * w) * 128 + (j & 3) * 4;
                const uint32_t b_dst = st + TC_OFF_B + (j >> 3) * TC_B_NATOM_BYTES + w * 1024;
#pragma unroll
                for (int i = 0; i < 8; ++i) {  // row k = 8w + r: its swizzle key is r
                    if (i * rows_at_once >= 8) break;
                    const int r = i * rows_at_once + r_sub;
                    const uint32_t word = lds32(w_src + r * 128 + (((j >> 2) ^ r) << 4));
                    uint32_t o[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e)  // nibbles e and e + 4 are columns 2e and 2e + 1
                        o[e] = bf16x2_mul(bf16x2_sub(nib2_to_bf16x2_biased(word >> (4 * e)), zz[e]), ss[e]);
                    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(b_dst + r * 128 + (((j & 7) ^ r) << 4)),
                                 "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3])
                                 : "memory");
                }
                }
                fence_async_smem();  // make the generic-proxy stores visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) mbar_arrive(ready_bar(s));
            }
        }
    } else if (warp >= TC_EPI_WARP0) {
        // ------------------------------ epilogue ------------------------------
        const int q = warp & 3;  // this warp's 32 TMEM lanes
        int tile_it = 0;
        for (TileWalk tw(ML, P, m_blocks, n_atoms); tw.valid(); tw.next(), ++tile_it) {
            const int b = tile_it % NBUF, use = tile_it / NBUF;
            const int m0 = tw.mb * (MT * TC_BM), n0 = tw.a * 64;
            const int chunks = tw.atoms() * 2;  // 32-column chunks in this sub-tile
            if (!mbar_wait_bounded(acc_full(b), use & 1, wait_limit)) {
                if (lane == 0) atomicExch(&g_gemm_error, 5);
                break;
            }
            tc_fence_after();
#pragma unroll 1
            for (int ac = 0; ac < MT * chunks; ++ac) {
                const int a = ac / chunks, c = ac % chunks;
                const int m = m0 + a * TC_BM + 32 * q + lane;
                uint32_t r[32];
                tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)((b + a) * TC_BN + 32 * c), r);
                tmem_ld_wait();
                const int n = n0 + 32 * c;
                if (m < M && n < N) {  // N is a multiple of 32: a 32-column chunk is all inside or all outside
                    if (epi == GEMM_EPI_SWIGLU) {
                        // columns 2i / 2i + 1 are gate_i / up_i: bf16 sums, SwiGLU, bf16 (the decode kernel's
                        // rounding points); 16 outputs per lane into C [M, N / 2]
                        uint32_t o[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            o[i] = (uint32_t)swiglu_bits(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1])) |
                                   ((uint32_t)swiglu_bits(__uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3])) << 16);
                        uint4 *dst = reinterpret_cast<uint4 *>(C + (size_t)m * (N >> 1) + (n >> 1));
                        dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
                        dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
                    } else {
                        uint32_t o[16];
                        if (epi == GEMM_EPI_RESIDUAL) {  // the residual joins the f32 sum before the one rounding
                            const uint4 *rs = reinterpret_cast<const uint4 *>(R + (size_t)m * N + n);
#pragma unroll
                            for (int i4 = 0; i4 < 4; ++i4) {
                                const uint4 rv = rs[i4];
                                const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                                for (int e = 0; e < 4; ++e)
                                    o[4 * i4 + e] = pack_bf16x2(__uint_as_float(r[8 * i4 + 2 * e]) + bf16x2_lo(rw[e]),
                                                                __uint_as_float(r[8 * i4 + 2 * e + 1]) + bf16x2_hi(rw[e]));
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 16; ++i)
                                o[i] = pack_bf16x2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
                        }
                        uint4 *dst = reinterpret_cast<uint4 *>(C + (size_t)m * N + n);
#pragma unroll
                        for (int i = 0; i < 4; ++i) dst[i] = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty(b));
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TC_TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------
bool gemm_tc_supported(int M, int K, int N, int group_size) {
    return group_size == TC_GROUP && K % TC_GROUP == 0 && N % 32 == 0 && M >= 1 && K > 0 && N > 0 && device_is_sm100();
}

int launch_gemm_tc(const uint16_t *A, const int32_t *qweight, const int32_t *qzeros, const uint16_t *scales,
                   uint16_t *C, int M, int K, int N, int group_size, cudaStream_t stream, int epilogue,
                   const uint16_t *residual) {
    (void)group_size;
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(gemm_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES);
        if (attr_err == cudaSuccess)
            attr_err = cudaFuncSetAttribute(gemm_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES);
    });
    if (attr_err != cudaSuccess) return check_cuda(attr_err, "tensor-core gemm: shared memory attribute");
    const int G = K / TC_GROUP, nb = N / 8;
    CUtensorMap tmA, tmW, tmS, tmZ;
    int rc;
    const int mt = M > TC_BM ? 2 : 1;  // 128-row accumulators per tile
    if ((rc = encode_tensor_map_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, A, K, M, (uint64_t)K * 2, TC_BK, mt * TC_BM,
                                   CU_TENSOR_MAP_SWIZZLE_128B)))
        return rc;
    if ((rc = encode_tensor_map_2d(&tmW, CU_TENSOR_MAP_DATA_TYPE_INT32, qweight, nb, K, (uint64_t)nb * 4, TC_BN / 8, TC_BK,
                                   CU_TENSOR_MAP_SWIZZLE_128B)))
        return rc;
    if ((rc = encode_tensor_map_2d(&tmS, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, scales, N, G, (uint64_t)N * 2, TC_BN, 1,
                                   CU_TENSOR_MAP_SWIZZLE_NONE)))
        return rc;
    if ((rc = encode_tensor_map_2d(&tmZ, CU_TENSOR_MAP_DATA_TYPE_INT32, qzeros, nb, G, (uint64_t)nb * 4, TC_BN / 8, 1,
                                   CU_TENSOR_MAP_SWIZZLE_NONE)))
        return rc;
    // CTAs: ML lanes over the M blocks times P column ranges per M block
    const int m_blocks = (M + mt * TC_BM - 1) / (mt * TC_BM), n_atoms = (N + 63) / 64;
    int sms = device_sm_count();
    if (sms <= 0) sms = 148;
    const int ML = m_blocks < sms ? m_blocks : sms;
    int P = sms / ML;
    if (P > n_atoms) P = n_atoms;
    if (P < 1) P = 1;
    const int ctas = ML * P;
    if (mt == 2)
        gemm_tc_kernel<2><<<ctas, TC_THREADS, TC_SMEM_BYTES, stream>>>(tmA, tmW, tmS, tmZ, C, residual, epilogue, M, N, K, ML, P,
                                                                       wait_limit_cycles());
    else
        gemm_tc_kernel<1><<<ctas, TC_THREADS, TC_SMEM_BYTES, stream>>>(tmA, tmW, tmS, tmZ, C, residual, epilogue, M, N, K, ML, P,
                                                                       wait_limit_cycles());
    return check_cuda(cudaGetLastError(), "tensor-core gemm launch");
}

int gemm_tc_check(cudaStream_t stream) {
    int flag = 0;
    int rc = check_cuda(cudaStreamSynchronize(stream), "gemm_check sync");
    if (rc) return rc;
    rc = check_cuda(cudaMemcpyFromSymbol(&flag, g_gemm_error, sizeof(int)), "gemm_check read");
    if (rc) return rc;
    if (flag != 0) {
        int zero = 0;
        cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int));
        return set_error(AWQ_ERR_DEVICE_TIMEOUT,
                         "prefill gemm: a device-side wait gave up (role %d: 1 producer, 2/3 MMA issuer, 4 dequant, "
                         "5 epilogue)", flag);
    }
    return AWQ_OK;
}

}  // namespace awq
