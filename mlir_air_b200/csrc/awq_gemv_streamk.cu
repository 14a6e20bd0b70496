// Decode GEMV / fused gate-up SwiGLU for AWQ int4 weights: TMA-fed, tensor-core, stream-K.
//
//   y[B, N] = x[B, K] @ W,   W[k, n] = (q - z) * s,   B <= 8 per launch.
//
// HBM-bound (0.52 B per weight, each weight used once), so the design is about keeping
// bytes in flight and spending well under two issue slots per weight:
//
//  * Work unit = one 512-column strip x one quantisation group of 128 k: two 16 KB boxes of
//    packed words, 2 KB of activations, 1 KB of scales and 256 B of zeros, fetched by one
//    producer thread with seven TMA tensor copies into a 3-deep shared-memory ring.  Two CTAs
//    run per SM.  Units are numbered strip-major; CTA c of C takes the contiguous range
//    [c U / C, (c + 1) U / C) (stream-K), so all SMs stream the same number of bytes whatever
//    the shape.
//  * Each of the eight consumer warps owns 64 columns of the strip for the CTA's whole range,
//    so no warp ever needs another warp's sums: there is no block-level barrier after set-up.
//    A lane reads one packed word (8 columns) from four k rows with bank-conflict-free LDS.32
//    from the 128B-swizzled box, pairs rows k/k+1 with two PRMT, and turns nibbles into bf16
//    pairs (128 + q) with one LOP3 each: that is directly the A fragment of
//    mma.sync.m16n8k16 (rows = 16 output columns, k = 16).  The activations are the B
//    fragment (ldmatrix from swizzled smem).
//  * The zero point and scale never touch the inner loop:
//        sum_k (q - z) s x = s (sum_k (128 + q) x  -  (128 + z) sum_k x)
//    per group; sum_k x comes from one extra MMA with an all-ones A fragment.
//  * At the end of a strip segment a warp that covered the whole strip applies the epilogue
//    from registers.  Otherwise it stores its f32 partial to the workspace and bumps the
//    counter of its 64-column sub-strip; the warp that arrives last sums all partials in CTA
//    order (deterministic) and applies the epilogue.  Nothing waits on another CTA.
//
// Epilogues: bf16 (+ residual), f32 (tensor-parallel partial), SwiGLU over interleaved
// gate/up column pairs (matvec_int4_swiglu_rms.py:511-516 rounding points).
#include <cudaTypedefs.h>

#include <mutex>

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
constexpr int SK_STAGE_BYTES = 36 * 1024;
constexpr int SK_BAR_BYTES = 2 * SK_STAGES * 8 + 16;
constexpr int SK_SMEM_BYTES = SK_STAGES * SK_STAGE_BYTES + SK_BAR_BYTES + 1024;
constexpr int SK_PARTIAL_FLOATS = 8 * SK_STRIP;        // one slot: [warp][batch 8][64 columns]
static_assert(SK_TX_BYTES <= SK_STAGE_BYTES, "stage too small");
static_assert(SK_CTAS_PER_SM * (SK_SMEM_BYTES + 1024) <= 228 * 1024, "shared memory budget");

// Workspace: [0, 256) header (int error flag), then a fixed region of sub-strip counters (one per
// 64 columns), then partial slots.  The layout does not depend on the shape, so one workspace
// can serve products of different shapes back to back (the counters are all zero between
// launches).
constexpr size_t SK_WS_HEADER = 256;
constexpr int SK_MAX_STRIPS = 504;  // N up to 258,048 columns
constexpr size_t SK_WS_PARTIALS = SK_WS_HEADER + (size_t)SK_MAX_STRIPS * SK_CONSUMER_WARPS * 4;  // 16 KB
constexpr int SK_MAX_CTAS = 2048;

size_t gemv_streamk_workspace_bytes(int K, int N) {
    (void)K;
    const size_t V = (size_t)(N + SK_STRIP - 1) / SK_STRIP;
    int sms = device_sm_count();
    if (sms <= 0) sms = 148;
    return SK_WS_PARTIALS + (V + (size_t)sms * SK_CTAS_PER_SM) * SK_PARTIAL_FLOATS * 4;
}

// Leading bytes of a workspace (error flag + counters) that must be zero before a launch.
size_t gemv_streamk_workspace_clear_bytes() { return SK_WS_PARTIALS; }

// CTA that owns unit x when U units are split over C CTAs as [c U / C, (c + 1) U / C).
__host__ __device__ __forceinline__ long long sk_owner(long long x, long long C, long long U) {
    return ((x + 1) * C + U - 1) / U - 1;
}

// One lane's share of a finished strip: 8 consecutive columns (n .. n+7) for batch rows 2t and
// 2t+1.  v[e][0..3] = (col 2e, row 2t), (col 2e, row 2t+1), (col 2e+1, row 2t), (col 2e+1, row 2t+1).
template <int EPI>
__device__ __forceinline__ void sk_epilogue(const float (&v)[4][4], const uint16_t *__restrict__ residual,
                                            void *__restrict__ y_, int B, int N, int n, int row0) {
    if (n >= N) return;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int b = row0 + h;
        if (b >= B) continue;
        if (EPI == EPI_SWIGLU) {
            uint32_t o[2];
#pragma unroll
            for (int e = 0; e < 4; e += 2)
                o[e >> 1] = (uint32_t)swiglu_bits(v[e][h], v[e][2 + h]) |
                            ((uint32_t)swiglu_bits(v[e + 1][h], v[e + 1][2 + h]) << 16);
            *reinterpret_cast<uint2 *>(reinterpret_cast<uint16_t *>(y_) + (size_t)b * (N >> 1) + (n >> 1)) =
                make_uint2(o[0], o[1]);
        } else if (EPI == EPI_F32) {
            float4 *dst = reinterpret_cast<float4 *>(reinterpret_cast<float *>(y_) + (size_t)b * N + n);
            dst[0] = make_float4(v[0][h], v[0][2 + h], v[1][h], v[1][2 + h]);
            dst[1] = make_float4(v[2][h], v[2][2 + h], v[3][h], v[3][2 + h]);
        } else {
            float r[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (residual) {
                const uint4 rv = *reinterpret_cast<const uint4 *>(residual + (size_t)b * N + n);
                const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    r[2 * e] = bf16x2_lo(rw[e]);
                    r[2 * e + 1] = bf16x2_hi(rw[e]);
                }
            }
            uint32_t o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) o[e] = pack_bf16x2(v[e][h] + r[2 * e], v[e][2 + h] + r[2 * e + 1]);
            *reinterpret_cast<uint4 *>(reinterpret_cast<uint16_t *>(y_) + (size_t)b * N + n) =
                make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
}

template <int EPI>
__global__ void __launch_bounds__(SK_THREADS, SK_CTAS_PER_SM)
gemv_streamk_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                    const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmZ,
                    const uint16_t *__restrict__ residual, void *__restrict__ y_, int B, int N, int G,
                    int V, float *__restrict__ partials, int *__restrict__ counters,
                    int *__restrict__ err_flag) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = smem_base + SK_STAGES * SK_STAGE_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (SK_STAGES + s); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long U = (long long)V * G, C = gridDim.x, c = blockIdx.x;
    const long long u0 = c * U / C, u1 = (c + 1) * U / C;
    const int n_units = (int)(u1 - u0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < SK_STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), SK_CONSUMER_WARPS);
        }
        mbar_fence_init();
    }
    __syncthreads();

    if (warp == SK_CONSUMER_WARPS) {
        // ------------------------------ producer ------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&tmW);
            tma_prefetch_desc(&tmX);
            tma_prefetch_desc(&tmS);
            tma_prefetch_desc(&tmZ);
            const uint64_t stream_policy = l2_policy_evict_first();
            for (int i = 0; i < n_units; ++i) {
                const int slot = i % SK_STAGES, round = i / SK_STAGES;
                if (round > 0 && !mbar_wait_bounded(empty_bar(slot), (round - 1) & 1)) {
                    atomicExch(err_flag, 1);
                    break;
                }
                const long long u = u0 + i;
                const int v = (int)(u / G), g = (int)(u % G);
                const uint32_t st = smem_base + slot * SK_STAGE_BYTES;
                const uint32_t bar = full_bar(slot);
                mbar_expect_tx(bar, SK_TX_BYTES);
#pragma unroll
                for (int bx = 0; bx < SK_STRIP / SK_BOX_COLS; ++bx)
                    tma_load_2d_hint(st + bx * SK_WBOX_BYTES, &tmW, (v * SK_STRIP + bx * SK_BOX_COLS) / 8, g * SK_GROUP,
                                     bar, stream_policy);
                tma_load_2d(st + SK_OFF_X, &tmX, g * SK_GROUP, 0, bar);
                tma_load_2d(st + SK_OFF_X + 1024, &tmX, g * SK_GROUP + 64, 0, bar);
#pragma unroll
                for (int bx = 0; bx < SK_STRIP / SK_BOX_COLS; ++bx)
                    tma_load_2d(st + SK_OFF_S + bx * SK_BOX_COLS * 2, &tmS, v * SK_STRIP + bx * SK_BOX_COLS, g, bar);
                tma_load_2d(st + SK_OFF_Z, &tmZ, v * (SK_STRIP / 8), g, bar);
            }
        }
        return;
    }

    // ------------------------------ consumers ------------------------------
    // Warp w owns strip columns [64 w, 64 w + 64); lane (g8, t4) owns packed word g8 of them.
    const int g8 = lane >> 2, t4 = lane & 3;
    const uint32_t w_box = (warp >> 2) * SK_WBOX_BYTES;          // which 256-column box
    const uint32_t chunk = 2 * (warp & 3) + (g8 >> 2);           // 16-byte chunk inside a box row
    // Rows 2t and 2t+1 of a 16-row k-step; rows +8 share the swizzle (row & 7 unchanged).
    const uint32_t offA = w_box + (2 * t4) * 128 + ((chunk ^ (2 * t4)) << 4) + (g8 & 3) * 4;
    const uint32_t offB = w_box + (2 * t4 + 1) * 128 + ((chunk ^ (2 * t4 + 1)) << 4) + (g8 & 3) * 4;
    const int xm = lane >> 3, xb = lane & 7;  // ldmatrix: matrix index, batch row
    const uint32_t ONES = 0x3F803F80u;
    const int col0 = warp * 64 + g8 * 8;      // first of this lane's 8 strip columns
    bool failed = false;

    float res[4][4];
    int cur_v = -1;

    // Finish the strip segment this warp has been accumulating (strip cur_v).
    auto flush = [&]() {
        const int v = cur_v;
        const int n = v * SK_STRIP + col0;
        const long long c_lo = sk_owner((long long)v * G, C, U);
        const long long c_hi = sk_owner((long long)(v + 1) * G - 1, C, U);
        if (c_hi == c_lo) {
            if (!failed) sk_epilogue<EPI>(res, residual, y_, B, N, n, 2 * t4);
            return;
        }
        // [slot][warp][batch row][64 columns]
        float *mine = partials + (size_t)(c + v) * SK_PARTIAL_FLOATS + warp * 512 + g8 * 8;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float4 *dst = reinterpret_cast<float4 *>(mine + (2 * t4 + h) * 64);
            dst[0] = make_float4(res[0][h], res[0][2 + h], res[1][h], res[1][2 + h]);
            dst[1] = make_float4(res[2][h], res[2][2 + h], res[3][h], res[3][2 + h]);
        }
        __threadfence();
        __syncwarp();
        int old = 0;
        if (lane == 0) old = atomicAdd(&counters[v * SK_CONSUMER_WARPS + warp], 1);
        old = __shfl_sync(0xffffffffu, old, 0);
        if (old != (int)(c_hi - c_lo)) return;
        __threadfence();
        float sum[4][4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
#pragma unroll
            for (int q = 0; q < 4; ++q) sum[e][q] = 0.f;
        for (long long cc = c_lo; cc <= c_hi; ++cc) {
            const float *src = partials + (size_t)(cc + v) * SK_PARTIAL_FLOATS + warp * 512 + g8 * 8;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float4 a = __ldcg(reinterpret_cast<const float4 *>(src + (2 * t4 + h) * 64));
                const float4 b = __ldcg(reinterpret_cast<const float4 *>(src + (2 * t4 + h) * 64) + 1);
                sum[0][h] += a.x; sum[0][2 + h] += a.y; sum[1][h] += a.z; sum[1][2 + h] += a.w;
                sum[2][h] += b.x; sum[2][2 + h] += b.y; sum[3][h] += b.z; sum[3][2 + h] += b.w;
            }
        }
        __syncwarp();
        if (lane == 0) counters[v * SK_CONSUMER_WARPS + warp] = 0;  // ready for the next launch
        if (!failed) sk_epilogue<EPI>(sum, residual, y_, B, N, n, 2 * t4);
    };

    for (int i = 0; i < n_units; ++i) {
        const long long u = u0 + i;
        const int v = (int)(u / G);
        if (v != cur_v) {
            if (cur_v >= 0) flush();
            cur_v = v;
#pragma unroll
            for (int e = 0; e < 4; ++e)
#pragma unroll
                for (int q = 0; q < 4; ++q) res[e][q] = 0.f;
        }
        const int slot = i % SK_STAGES, round = i / SK_STAGES;
        if (!failed && !mbar_wait_bounded(full_bar(slot), round & 1)) {
            failed = true;
            if (lane == 0) atomicExch(err_flag, 2);
        }
        if (failed) continue;
        const uint32_t st = smem_base + slot * SK_STAGE_BYTES;

        float acc[4][4];
        float sx[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int e = 0; e < 4; ++e)
#pragma unroll
            for (int q = 0; q < 4; ++q) acc[e][q] = 0.f;

#pragma unroll
        for (int p = 0; p < 4; ++p) {
            // activations for k-steps 2p and 2p+1: 16-byte chunk q = 4p + matrix index
            const int q = 4 * p + xm;
            uint32_t bx[4];
            ldmatrix_x4(bx, st + SK_OFF_X + (q >> 3) * 1024 + xb * 128 + (((q & 7) ^ xb) << 4));
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t rb = st + (2 * p + h) * 2048;
                const uint32_t w0 = lds32(rb + offA);
                const uint32_t w1 = lds32(rb + offB);
                const uint32_t w2 = lds32(rb + 1024 + offA);
                const uint32_t w3 = lds32(rb + 1024 + offB);
                const uint32_t b0 = bx[2 * h], b1 = bx[2 * h + 1];
                mma_bf16_16816(sx, ONES, ONES, ONES, ONES, b0, b1);
                // low halves hold nibbles 0-3 (columns 0,2,4,6), high halves nibbles 4-7
                // (columns 1,3,5,7); pair rows k and k+1 of the same column in one register
                const uint32_t lo01 = __byte_perm(w0, w1, 0x5410);
                const uint32_t hi01 = __byte_perm(w0, w1, 0x7632);
                const uint32_t lo23 = __byte_perm(w2, w3, 0x5410);
                const uint32_t hi23 = __byte_perm(w2, w3, 0x7632);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    // MMA row g8 = column 2e of the lane's word, row g8 + 8 = column 2e + 1
                    mma_bf16_16816(acc[e], nib2_to_bf16x2_biased(lo01 >> (4 * e)),
                                   nib2_to_bf16x2_biased(hi01 >> (4 * e)), nib2_to_bf16x2_biased(lo23 >> (4 * e)),
                                   nib2_to_bf16x2_biased(hi23 >> (4 * e)), b0, b1);
                }
            }
        }

        // group fix-up: res += s * (acc - (128 + z) * sum_x)
        const uint32_t zw = lds32(st + SK_OFF_Z + (col0 >> 3) * 4);
        const uint4 sv = lds128(st + SK_OFF_S + col0 * 2);
        const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(slot));  // all of this warp's reads of the slot are done
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const uint32_t zz = nib2_to_bf16x2_biased(zw >> (4 * e));
            const float z_even = bf16x2_lo(zz), z_odd = bf16x2_hi(zz);
            const float s_even = bf16x2_lo(sw[e]), s_odd = bf16x2_hi(sw[e]);
            res[e][0] = fmaf(s_even, fmaf(-z_even, sx[0], acc[e][0]), res[e][0]);
            res[e][1] = fmaf(s_even, fmaf(-z_even, sx[1], acc[e][1]), res[e][1]);
            res[e][2] = fmaf(s_odd, fmaf(-z_odd, sx[0], acc[e][2]), res[e][2]);
            res[e][3] = fmaf(s_odd, fmaf(-z_odd, sx[1], acc[e][3]), res[e][3]);
        }
    }
    if (cur_v >= 0) flush();
}

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
static PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
    });
    return fn;
}

int encode_tensor_map_2d(CUtensorMap *map, int dtype, const void *base, uint64_t dim0, uint64_t dim1,
                         uint64_t stride1_bytes, uint32_t box0, uint32_t box1, int swizzle) {
    PFN_cuTensorMapEncodeTiled_v12000 fn = get_encode_fn();
    if (!fn) return set_error(AWQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {dim0, dim1};
    cuuint64_t strides[1] = {stride1_bytes};
    cuuint32_t box[2] = {box0, box1};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, (CUtensorMapDataType)dtype, 2, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, (CUtensorMapSwizzle)swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return set_error(AWQ_ERR_CUDA, "cuTensorMapEncodeTiled failed (CUresult %d; dims %llu x %llu, stride %llu)",
                         (int)r, (unsigned long long)dim0, (unsigned long long)dim1,
                         (unsigned long long)stride1_bytes);
    return AWQ_OK;
}

bool gemv_streamk_supported(const GemvArgs &a) {
    return a.group_size == SK_GROUP && a.K % SK_GROUP == 0 && a.N % 32 == 0 && a.B >= 1 && a.K > 0 && a.N > 0 &&
           aligned16(a.x) && aligned16(a.qweight) && aligned16(a.qzeros) && aligned16(a.scales) &&
           (a.N + SK_STRIP - 1) / SK_STRIP <= SK_MAX_STRIPS && device_is_sm100();
}

template <int EPI>
static int launch_one(const GemvArgs &a, const uint16_t *x, const uint16_t *residual, void *y, int B) {
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(gemv_streamk_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        SK_SMEM_BYTES);
    });
    if (attr_err != cudaSuccess) return check_cuda(attr_err, "stream-K gemv: shared memory attribute");

    const int G = a.K / SK_GROUP, V = (a.N + SK_STRIP - 1) / SK_STRIP, nb = a.N / 8;
    CUtensorMap tmW, tmX, tmS, tmZ;
    int rc;
    if ((rc = encode_tensor_map_2d(&tmW, CU_TENSOR_MAP_DATA_TYPE_INT32, a.qweight, nb, a.K, (uint64_t)nb * 4, 32,
                                   SK_GROUP, CU_TENSOR_MAP_SWIZZLE_128B)))
        return rc;
    if ((rc = encode_tensor_map_2d(&tmX, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, x, a.K, B, (uint64_t)a.K * 2, 64, 8,
                                   CU_TENSOR_MAP_SWIZZLE_128B)))
        return rc;
    if ((rc = encode_tensor_map_2d(&tmS, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a.scales, a.N, G, (uint64_t)a.N * 2,
                                   SK_BOX_COLS, 1, CU_TENSOR_MAP_SWIZZLE_NONE)))
        return rc;
    if ((rc = encode_tensor_map_2d(&tmZ, CU_TENSOR_MAP_DATA_TYPE_INT32, a.qzeros, nb, G, (uint64_t)nb * 4,
                                   SK_STRIP / 8, 1, CU_TENSOR_MAP_SWIZZLE_NONE)))
        return rc;

    const long long U = (long long)V * G;
    int ctas = device_sm_count() * SK_CTAS_PER_SM;
    if (ctas > SK_MAX_CTAS) ctas = SK_MAX_CTAS;
    if ((long long)ctas > U) ctas = (int)U;
    uint8_t *ws = reinterpret_cast<uint8_t *>(a.workspace);
    int *err_flag = reinterpret_cast<int *>(ws);
    int *counters = reinterpret_cast<int *>(ws + SK_WS_HEADER);
    float *partials = reinterpret_cast<float *>(ws + SK_WS_PARTIALS);
    gemv_streamk_kernel<EPI><<<ctas, SK_THREADS, SK_SMEM_BYTES, a.stream>>>(tmW, tmX, tmS, tmZ, residual, y, B, a.N,
                                                                           G, V, partials, counters, err_flag);
    return check_cuda(cudaGetLastError(), "stream-K gemv launch");
}

int launch_gemv_streamk(const GemvArgs &a) {
    if (!a.workspace || a.workspace_bytes < gemv_streamk_workspace_bytes(a.K, a.N))
        return set_error(AWQ_ERR_WORKSPACE, "gemv: workspace of %zu bytes needed, %zu given",
                         gemv_streamk_workspace_bytes(a.K, a.N), a.workspace_bytes);
    // more than 8 batch rows: one pass over the weights per 8 rows
    for (int b0 = 0; b0 < a.B; b0 += 8) {
        const int B = a.B - b0 < 8 ? a.B - b0 : 8;
        const uint16_t *x = a.x + (size_t)b0 * a.K;
        const uint16_t *res = a.residual ? a.residual + (size_t)b0 * a.N : nullptr;
        int rc;
        switch (a.epilogue) {
            case EPI_BF16:
                rc = launch_one<EPI_BF16>(a, x, res, reinterpret_cast<uint16_t *>(a.y) + (size_t)b0 * a.N, B);
                break;
            case EPI_F32:
                rc = launch_one<EPI_F32>(a, x, nullptr, reinterpret_cast<float *>(a.y) + (size_t)b0 * a.N, B);
                break;
            default:
                rc = launch_one<EPI_SWIGLU>(a, x, nullptr,
                                            reinterpret_cast<uint16_t *>(a.y) + (size_t)b0 * (a.N / 2), B);
                break;
        }
        if (rc) return rc;
    }
    return AWQ_OK;
}

}  // namespace awq
