// Decode GEMV / gate-up SwiGLU for 9 to 32 batch rows per weight pass.
//
// The 8-row stream-K kernel (awq_gemv_streamk.cu) spends its time on the nibble decode (integer
// ALU); the MMAs are cheap.  For more rows the decoded fragments are therefore reused: a unit's
// weights are decoded once and multiplied with T = 2 or 4 activation tiles of 8 rows, each tile with
// its own accumulators.  That costs registers (36 per tile and thread), so this variant runs one CTA
// of 8 consumer warps per SM with a 5-stage ring instead of two CTAs with 3 stages.  With T = 4 there
// is no producer warp: a ninth warp would put three warps on one of the SM's four schedulers and cap
// every thread at 168 registers, so lane 0 of consumer warp 0 issues the TMA copies itself, between
// its units, whenever a stage has been released (and blocks for a release only when the unit it is
// about to consume has not been requested yet).
// Units, stage layout (with T activation tiles), decode, split-K hand-over (one 64-bit atomic per
// sum carrying value and progress) and epilogues are those of the 8-row kernel; strip v, tile t
// uses accumulator slot v T + t.  fp16 activations only (bf16 inputs are converted by the caller).
#include <cudaTypedefs.h>
#include <cuda_fp16.h>

#include <mutex>

#include "awq_common.cuh"
#include "awq_ptx.cuh"
#include "awq_streamk.cuh"

namespace awq {

int encode_tensor_map_2d(CUtensorMap *map, int dtype, const void *base, uint64_t dim0, uint64_t dim1,
                         uint64_t stride1_bytes, uint32_t box0, uint32_t box1, int swizzle);

template <int T>
struct MbCfg {
    static constexpr int X_BYTES = T * SK_X_BYTES;  // T tiles of [8 rows x 128 k]
    static constexpr int OFF_X = SK_W_BYTES;
    static constexpr int OFF_S = OFF_X + X_BYTES;
    static constexpr int OFF_Z = OFF_S + SK_S_BYTES;
    static constexpr int TX_BYTES = SK_W_BYTES + X_BYTES + SK_S_BYTES + SK_Z_BYTES;
    static constexpr int STAGE_BYTES = (OFF_Z + SK_Z_BYTES + 1023) / 1024 * 1024;
    static constexpr int STAGES = 5;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 2 * STAGES * 8 + 16 + 1024;
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
};

template <int T>
__host__ __device__ constexpr bool mb_fold() { return T > 2; }  // the producer's work is folded into consumer warp 0
template <int T>
__host__ __device__ constexpr int mb_threads() { return mb_fold<T>() ? SK_CONSUMER_WARPS * 32 : SK_THREADS; }

template <int EPI, int T>
__global__ void __launch_bounds__(mb_threads<T>(), 1)
gemv_streamk_mb_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                       const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmZ,
                       const uint16_t *__restrict__ residual, void *__restrict__ y_, int B, int N, int G, int V,
                       int out_f16, unsigned long long *__restrict__ accum, int *__restrict__ err_flag,
                       long long wait_limit) {
    using Cfg = MbCfg<T>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = smem_base + Cfg::STAGES * Cfg::STAGE_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (Cfg::STAGES + s); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long U = (long long)V * G, C = gridDim.x, c = blockIdx.x;
    const long long u0 = c * U / C, u1 = (c + 1) * U / C;
    const int n_units = (int)(u1 - u0);
    const int v_first = (int)(u0 / G), g_first = (int)(u0 % G);

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), SK_CONSUMER_WARPS);
        }
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    constexpr bool FOLD = mb_fold<T>();
    const uint64_t stream_policy = l2_policy_evict_first();
    auto load_weights = [&](int slot, int v, int g) {
        const uint32_t st = smem_base + slot * Cfg::STAGE_BYTES;
        const uint32_t bar = full_bar(slot);
        mbar_expect_tx(bar, Cfg::TX_BYTES);
#pragma unroll
        for (int bx = 0; bx < SK_STRIP / SK_BOX_COLS; ++bx)
            tma_load_2d_hint(st + bx * SK_WBOX_BYTES, &tmW, (v * SK_STRIP + bx * SK_BOX_COLS) / 8, g * SK_GROUP, bar,
                             stream_policy);
#pragma unroll
        for (int bx = 0; bx < SK_STRIP / SK_BOX_COLS; ++bx)
            tma_load_2d(st + Cfg::OFF_S + bx * SK_BOX_COLS * 2, &tmS, v * SK_STRIP + bx * SK_BOX_COLS, g, bar);
        tma_load_2d(st + Cfg::OFF_Z, &tmZ, v * (SK_STRIP / 8), g, bar);
    };
    auto load_activations = [&](int slot, int g) {  // rows beyond B read as zero
        const uint32_t st = smem_base + slot * Cfg::STAGE_BYTES;
#pragma unroll
        for (int t = 0; t < T; ++t) {
            tma_load_2d(st + Cfg::OFF_X + t * SK_X_BYTES, &tmX, g * SK_GROUP, 8 * t, full_bar(slot));
            tma_load_2d(st + Cfg::OFF_X + t * SK_X_BYTES + 1024, &tmX, g * SK_GROUP + 64, 8 * t, full_bar(slot));
        }
    };
    // what the issuing thread has requested so far: unit number, its strip / group, ring position
    int iss_n = 0, iss_v = v_first, iss_g = g_first, iss_slot = 0, iss_round = 0;
    auto issue_prologue = [&]() {
        // weights first (they do not depend on the previous kernel), then its output
        tma_prefetch_desc(&tmW);
        tma_prefetch_desc(&tmX);
        tma_prefetch_desc(&tmS);
        tma_prefetch_desc(&tmZ);
        const int n_first = n_units < Cfg::STAGES ? n_units : Cfg::STAGES;
        int v = v_first, g = g_first;
        for (int i = 0; i < n_first; ++i) {
            load_weights(i, v, g);
            if (++g == G) { g = 0; ++v; }
        }
        pdl_wait();
        int g2 = g_first;
        for (int i = 0; i < n_first; ++i) {
            load_activations(i, g2);
            if (++g2 == G) g2 = 0;
        }
        iss_n = n_first;
        iss_v = v;
        iss_g = g;
        iss_slot = n_first % Cfg::STAGES;
        iss_round = n_first / Cfg::STAGES;
    };
    // request the next unit into its stage; `must`: block (bounded) until the stage is released
    auto issue_next = [&](bool must) -> bool {
        const uint32_t parity = (uint32_t)(iss_round - 1) & 1u;
        if (must) {
            if (!mbar_wait_bounded(empty_bar(iss_slot), parity, wait_limit)) {
                atomicExch(err_flag, 1);
                return false;
            }
        } else if (!mbar_try_wait(empty_bar(iss_slot), parity)) {
            return false;
        }
        load_weights(iss_slot, iss_v, iss_g);
        load_activations(iss_slot, iss_g);
        ++iss_n;
        if (++iss_g == G) { iss_g = 0; ++iss_v; }
        if (++iss_slot == Cfg::STAGES) { iss_slot = 0; ++iss_round; }
        return true;
    };

    if (!FOLD && warp == SK_CONSUMER_WARPS) {
        // ------------------------------ producer warp ------------------------------
        if (lane == 0) {
            issue_prologue();
            while (iss_n < n_units && issue_next(true)) {
            }
        }
        return;
    }
    if (FOLD && threadIdx.x == 0) issue_prologue();
    pdl_wait();  // consumers read and write global memory the previous kernel may still be using

    // ------------------------------ consumers ------------------------------
    const SkLane L(warp, lane);
    const int g8 = L.g8, t4 = L.t4, odd = L.odd, colw = L.colw, lm = L.lm, lr = L.lr;
    const uint32_t z_off = L.z_off - SK_OFF_Z + Cfg::OFF_Z, s_off = L.s_off - SK_OFF_S + Cfg::OFF_S;
    const uint32_t ONES = 0x3C003C00u;
    bool failed = false;

    float res[T][4][4];
    int cur_v = -1, seg_groups = 0;

    // Finish the strip segment this warp has been accumulating (strip cur_v), tile by tile.
    auto flush = [&]() {
        const int v = cur_v;
        const int n = v * SK_STRIP + colw;
#pragma unroll
        for (int t = 0; t < T; ++t) {
            if (8 * t >= B) continue;  // uniform: a tile without rows has nothing to hand over
            float own[2][8];
            sk_lane_exchange(res[t], odd, own);
            const int b = 8 * t + 2 * t4 + odd;
            if (seg_groups != G &&
                !sk_handover(accum + ((size_t)(v * T + t) * SK_CONSUMER_WARPS + warp) * SK_ACC_WORDS, own, seg_groups, G, lane,
                             wait_limit, err_flag))
                continue;
            if (!failed) sk_epilogue<EPI>(own, residual, y_, B, N, n, b, out_f16);
        }
    };

    int v = v_first, g = g_first, slot = 0, round = 0;
    for (int i = 0; i < n_units; ++i) {
        if (v != cur_v) {
            if (cur_v >= 0) flush();
            cur_v = v;
            seg_groups = 0;
#pragma unroll
            for (int t = 0; t < T; ++t)
#pragma unroll
                for (int e = 0; e < 4; ++e)
#pragma unroll
                    for (int q = 0; q < 4; ++q) res[t][e][q] = 0.f;
        }
        ++seg_groups;
        if (FOLD && threadIdx.x == 0 && !failed) {
            // refill whatever has been released; the unit about to be consumed must have been requested
            while (iss_n < n_units && issue_next(iss_n <= i)) {
            }
        }
        if (!failed && !mbar_wait_bounded(full_bar(slot), round & 1, wait_limit)) {
            failed = true;
            if (lane == 0) atomicExch(err_flag, 2);
        }
        if (!failed) {
            const uint32_t st = smem_base + slot * Cfg::STAGE_BYTES;
            float acc[T][4][4];
            float sx[T][4];
#pragma unroll
            for (int t = 0; t < T; ++t) {
#pragma unroll
                for (int q = 0; q < 4; ++q) sx[t][q] = 0.f;
#pragma unroll
                for (int e = 0; e < 4; ++e)
#pragma unroll
                    for (int q = 0; q < 4; ++q) acc[t][e][q] = 0.f;
            }
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                // activations for k-steps 2p and 2p+1 of every tile: 16-byte chunk q = 4p + matrix index
                const int q = 4 * p + lm;
                uint32_t bx[T][4];
#pragma unroll
                for (int t = 0; t < T; ++t)
                    ldmatrix_x4(bx[t], st + Cfg::OFF_X + t * SK_X_BYTES + (q >> 3) * 1024 + lr * 128 + (((q & 7) ^ lr) << 4));
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t R[4];
                    ldmatrix_x4_trans(R, st + (2 * p + h) * 2048 + L.w_off);
                    uint32_t a_lo[4], a_hi[4], b_lo[4], b_hi[4];
                    decode4<true>(R[0], a_lo);
                    decode4<true>(R[1], a_hi);
                    decode4<true>(R[2], b_lo);
                    decode4<true>(R[3], b_hi);
#pragma unroll
                    for (int t = 0; t < T; ++t) {  // the decoded fragments serve every tile
                        const uint32_t b0 = bx[t][2 * h], b1 = bx[t][2 * h + 1];
                        mma_16816<true>(sx[t], ONES, ONES, ONES, ONES, b0, b1);
#pragma unroll
                        for (int e = 0; e < 4; ++e) mma_16816<true>(acc[t][e], a_lo[e], b_lo[e], a_hi[e], b_hi[e], b0, b1);
                    }
                }
            }
            // group fix-up: res += s * (acc - c * sum_x), as in the 8-row kernel (fp16 decode offsets)
            const uint32_t zA = lds_u16(st + z_off), zB = lds_u16(st + z_off + 16);
            uint32_t sA[4], sB[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                sA[e] = lds_u16(st + s_off + 4 * e);
                sB[e] = lds_u16(st + s_off + 64 + 4 * e);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar(slot));  // all of this warp's reads of the slot are done
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float cA = __uint_as_float(((zA << (16 - 4 * e)) & 0x000F0000u) | 0x43000000u);
                float cB = __uint_as_float(((zB << (16 - 4 * e)) & 0x000F0000u) | 0x43000000u);
                float fA = __uint_as_float(sA[e] << 16), fB = __uint_as_float(sB[e] << 16);
                if (e & 1) {
                    cA = fmaf(cA, 16.f, -1024.f);  // 1024 + 16 z
                    cB = fmaf(cB, 16.f, -1024.f);
                    fA *= 0.0625f;
                    fB *= 0.0625f;
                } else {
                    cA += 896.f;  // 1024 + z
                    cB += 896.f;
                }
#pragma unroll
                for (int t = 0; t < T; ++t) {
                    res[t][e][0] = fmaf(fA, fmaf(-cA, sx[t][0], acc[t][e][0]), res[t][e][0]);
                    res[t][e][1] = fmaf(fA, fmaf(-cA, sx[t][1], acc[t][e][1]), res[t][e][1]);
                    res[t][e][2] = fmaf(fB, fmaf(-cB, sx[t][0], acc[t][e][2]), res[t][e][2]);
                    res[t][e][3] = fmaf(fB, fmaf(-cB, sx[t][1], acc[t][e][3]), res[t][e][3]);
                }
            }
        }
        if (++g == G) { g = 0; ++v; }
        if (++slot == Cfg::STAGES) { slot = 0; ++round; }
    }
    if (cur_v >= 0) flush();
}

// ---------------------------------------------------------------------------------------
template <int EPI, int T>
static int launch_mb(const GemvArgs &a, const uint16_t *x, const uint16_t *residual, void *y, int B) {
    using Cfg = MbCfg<T>;
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(gemv_streamk_mb_kernel<EPI, T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        Cfg::SMEM_BYTES);
    });
    if (attr_err != cudaSuccess) return check_cuda(attr_err, "multi-row gemv: shared memory attribute");
    const int G = a.K / SK_GROUP, V = (a.N + SK_STRIP - 1) / SK_STRIP, nb = a.N / 8;
    CUtensorMap tmW, tmX, tmS, tmZ;
    int rc;
    if ((rc = encode_tensor_map_2d(&tmW, CU_TENSOR_MAP_DATA_TYPE_INT32, a.qweight, nb, a.K, (uint64_t)nb * 4, 32, SK_GROUP,
                                   CU_TENSOR_MAP_SWIZZLE_128B)))
        return rc;
    if ((rc = encode_tensor_map_2d(&tmX, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, x, a.K, B, (uint64_t)a.K * 2, 64, 8,
                                   CU_TENSOR_MAP_SWIZZLE_128B)))
        return rc;
    if ((rc = encode_tensor_map_2d(&tmS, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a.scales, a.N, G, (uint64_t)a.N * 2, SK_BOX_COLS, 1,
                                   CU_TENSOR_MAP_SWIZZLE_NONE)))
        return rc;
    if ((rc = encode_tensor_map_2d(&tmZ, CU_TENSOR_MAP_DATA_TYPE_INT32, a.qzeros, nb, G, (uint64_t)nb * 4, SK_STRIP / 8, 1,
                                   CU_TENSOR_MAP_SWIZZLE_NONE)))
        return rc;
    const long long U = (long long)V * G;
    int ctas = device_sm_count();
    if (ctas <= 0) ctas = 148;
    if ((long long)ctas > U) ctas = (int)U;
    uint8_t *ws = reinterpret_cast<uint8_t *>(a.workspace);
    return check_cuda(launch_pdl(gemv_streamk_mb_kernel<EPI, T>, dim3(ctas), dim3(mb_threads<T>()), Cfg::SMEM_BYTES, a.stream, tmW,
                                 tmX, tmS, tmZ, residual, y, B, a.N, G, V, a.out_format == ACT_F16 ? 1 : 0,
                                 reinterpret_cast<unsigned long long *>(ws + SK_WS_ACCUM), reinterpret_cast<int *>(ws),
                                 wait_limit_cycles()),
                      "multi-row gemv launch");
}

template <int T>
static int launch_mb_epi(const GemvArgs &a, const uint16_t *x, const uint16_t *residual, void *y, int B) {
    switch (a.epilogue) {
        case EPI_BF16: return launch_mb<EPI_BF16, T>(a, x, residual, y, B);
        case EPI_F32: return launch_mb<EPI_F32, T>(a, x, nullptr, y, B);
        case EPI_SWIGLU: return launch_mb<EPI_SWIGLU, T>(a, x, nullptr, y, B);
        default: return set_error(AWQ_ERR_UNSUPPORTED, "multi-row gemv: epilogue %d", a.epilogue);
    }
}

// Can B rows (9 <= B <= 32) go through one pass of this kernel?
bool gemv_streamk_mb_supported(const GemvArgs &a, int B) {
    const int V = (a.N + SK_STRIP - 1) / SK_STRIP;
    const int T = B > 16 ? 4 : 2;
    return B > 8 && B <= 32 && !a.deterministic && a.epilogue != EPI_F32_PUSH && V * T <= SK_MAX_STRIPS &&
           a.workspace_bytes >= SK_WS_END && a.K / SK_GROUP <= SK_MAX_GROUPS;
}

// x: fp16 [B, K] (already converted), 9 <= B <= 32.
int launch_gemv_streamk_mb(const GemvArgs &a, const uint16_t *x, const uint16_t *residual, void *y, int B) {
    return B > 16 ? launch_mb_epi<4>(a, x, residual, y, B) : launch_mb_epi<2>(a, x, residual, y, B);
}

}  // namespace awq
