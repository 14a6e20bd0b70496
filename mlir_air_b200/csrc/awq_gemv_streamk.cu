// Decode GEMV / fused gate-up SwiGLU for AWQ int4 weights: TMA-fed, tensor-core, stream-K.
//
//   y[B, N] = x[B, K] @ W,   W[k, n] = (q - z) * s,   B <= 8 per launch.
//
// HBM-bound (0.52 B per weight, each weight used once), so the design is about keeping
// bytes in flight and spending about one issue slot per weight:
//
//  * Work unit = one 256-column strip x one quantisation group of 128 k: a 16 KB box of
//    packed words, 2 KB of activations, 512 B of scales and 128 B of zeros, fetched by one
//    producer thread with four TMA tensor copies into a 10-deep shared-memory ring (about
//    190 KB in flight per SM).  Units are numbered strip-major; CTA c of C takes the
//    contiguous range [c U / C, (c + 1) U / C) (stream-K), so all SMs stream the same number
//    of bytes whatever the shape.
//  * Eight consumer warps take units round-robin.  A lane reads four 16-byte chunks
//    (4 packed words x 4 k rows) with bank-conflict-free LDS.128 from the 128B-swizzled box,
//    pairs rows k/k+1 with two PRMT, and turns nibbles into bf16 pairs (128 + q) with one
//    LOP3 each: that is directly the A fragment of mma.sync.m16n8k16 (rows = 16 output
//    columns, k = 16).  The activations are the B fragment (ldmatrix from swizzled smem).
//  * The zero point and scale never touch the inner loop:
//        sum_k (q - z) s x = s (sum_k (128 + q) x  -  (128 + z) sum_k x)
//    per group; sum_k x comes from one extra MMA with an all-ones A fragment.
//  * At the end of a strip segment the eight warps' f32 partials are summed in shared
//    memory in a fixed order.  If the CTA covered the whole strip it applies the epilogue;
//    otherwise it stores its partial to the workspace and bumps the strip's counter, and
//    the CTA that arrives last sums all partials in CTA order (deterministic) and applies
//    the epilogue.  Nothing waits on another CTA.
//
// Epilogues: bf16 (+ residual), f32 (tensor-parallel partial), SwiGLU over interleaved
// gate/up column pairs (matvec_int4_swiglu_rms.py:511-516 rounding points).
#include <cudaTypedefs.h>

#include <mutex>

#include "awq_common.cuh"
#include "awq_ptx.cuh"

namespace awq {

constexpr int SK_STRIP = 256;
constexpr int SK_GROUP = 128;
constexpr int SK_CONSUMER_WARPS = 8;
constexpr int SK_CONSUMER_THREADS = SK_CONSUMER_WARPS * 32;
constexpr int SK_THREADS = SK_CONSUMER_THREADS + 32;
constexpr int SK_STAGES = 10;
constexpr int SK_W_BYTES = SK_GROUP * 128;  // 128 k rows x 32 packed words
constexpr int SK_X_BYTES = 2 * 1024;        // two boxes of 8 batch rows x 64 k (bf16)
constexpr int SK_S_BYTES = SK_STRIP * 2;
constexpr int SK_Z_BYTES = SK_STRIP / 8 * 4;
constexpr int SK_TX_BYTES = SK_W_BYTES + SK_X_BYTES + SK_S_BYTES + SK_Z_BYTES;
constexpr int SK_OFF_X = SK_W_BYTES;
constexpr int SK_OFF_S = SK_OFF_X + SK_X_BYTES;
constexpr int SK_OFF_Z = SK_OFF_S + SK_S_BYTES;
constexpr int SK_STAGE_BYTES = 19 * 1024;
constexpr int SK_RED_PITCH = 260;  // floats per batch row of a reduction slot
constexpr int SK_RED_SLOT = 8 * SK_RED_PITCH;
constexpr int SK_RED_BYTES = 4 * SK_RED_SLOT * 4;
constexpr int SK_BAR_BYTES = 2 * SK_STAGES * 8 + 16;
constexpr int SK_SMEM_BYTES = SK_STAGES * SK_STAGE_BYTES + SK_RED_BYTES + SK_BAR_BYTES + 1024;
constexpr int SK_PARTIAL_FLOATS = 8 * SK_STRIP;
static_assert(SK_TX_BYTES <= SK_STAGE_BYTES, "stage too small");
static_assert(SK_SMEM_BYTES <= 227 * 1024, "shared memory budget");

// Workspace: [0, 256) header (int error flag), then a fixed region of strip counters, then
// partial slots.  The layout does not depend on the shape, so one workspace can serve
// products of different shapes back to back (the counters are all zero between launches).
constexpr size_t SK_WS_HEADER = 256;
constexpr int SK_MAX_STRIPS = 4032;  // N up to 1,032,192 columns
constexpr size_t SK_WS_PARTIALS = SK_WS_HEADER + (size_t)SK_MAX_STRIPS * 4;  // 16 KB
constexpr int SK_MAX_CTAS = 1024;

size_t gemv_streamk_workspace_bytes(int K, int N) {
    (void)K;
    const size_t V = (size_t)(N + SK_STRIP - 1) / SK_STRIP;
    int sms = device_sm_count();
    if (sms <= 0) sms = 148;
    return SK_WS_PARTIALS + (V + (size_t)sms) * SK_PARTIAL_FLOATS * 4;
}

// Leading bytes of a workspace (error flag + strip counters) that must be zero before a launch.
size_t gemv_streamk_workspace_clear_bytes() { return SK_WS_PARTIALS; }

// Conflict-free position of (batch row b, strip column col) inside a reduction slot, both for
// the MMA accumulator layout (lanes vary in col / 32 and b) and for column-contiguous readers.
__device__ __forceinline__ int sk_red_idx(int b, int col) {
    return b * SK_RED_PITCH + (col & ~31) + ((col + (col >> 5)) & 31);
}

// CTA that owns unit x when U units are split over C CTAs as [c U / C, (c + 1) U / C).
__host__ __device__ __forceinline__ long long sk_owner(long long x, long long C, long long U) {
    return ((x + 1) * C + U - 1) / U - 1;
}

template <int EPI>
__global__ void __launch_bounds__(SK_THREADS, 1)
gemv_streamk_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                    const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmZ,
                    const uint16_t *__restrict__ residual, void *__restrict__ y_, int B, int N, int G,
                    int V, float *__restrict__ partials, int *__restrict__ counters,
                    int *__restrict__ err_flag) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    float *red = reinterpret_cast<float *>(smem_gen + SK_STAGES * SK_STAGE_BYTES);
    const uint32_t bar_base = smem_base + SK_STAGES * SK_STAGE_BYTES + SK_RED_BYTES;
    int *s_flag = reinterpret_cast<int *>(smem_gen + SK_STAGES * SK_STAGE_BYTES + SK_RED_BYTES +
                                          2 * SK_STAGES * 8);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (SK_STAGES + s); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long U = (long long)V * G, C = gridDim.x, c = blockIdx.x;
    const long long u0 = c * U / C, u1 = (c + 1) * U / C;
    const int n_units = (int)(u1 - u0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < SK_STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
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
                mbar_expect_tx(full_bar(slot), SK_TX_BYTES);
                tma_load_2d_hint(st, &tmW, v * (SK_STRIP / 8), g * SK_GROUP, full_bar(slot), stream_policy);
                tma_load_2d(st + SK_OFF_X, &tmX, g * SK_GROUP, 0, full_bar(slot));
                tma_load_2d(st + SK_OFF_X + 1024, &tmX, g * SK_GROUP + 64, 0, full_bar(slot));
                tma_load_2d(st + SK_OFF_S, &tmS, v * SK_STRIP, g, full_bar(slot));
                tma_load_2d(st + SK_OFF_Z, &tmZ, v * (SK_STRIP / 8), g, full_bar(slot));
            }
        }
        return;
    }

    // ------------------------------ consumers ------------------------------
    const int g8 = lane >> 2, t4 = lane & 3;
    // Rows 2t and 2t+1 of a 16-row k-step; rows +8 share the swizzle (row & 7 unchanged).
    const uint32_t offA = (2 * t4) * 128 + ((g8 ^ (2 * t4)) << 4);
    const uint32_t offB = (2 * t4 + 1) * 128 + ((g8 ^ (2 * t4 + 1)) << 4);
    const int xm = lane >> 3, xb = lane & 7;  // ldmatrix: matrix index, batch row
    const uint32_t ONES = 0x3F803F80u;
    const int tid = threadIdx.x;  // 0..255: strip column owned in the epilogue
    bool failed = false;

    int i_begin = 0;
    while (i_begin < n_units) {
        const long long ub = u0 + i_begin;
        const int v = (int)(ub / G);
        const int i_end = (int)min((long long)n_units, (long long)(v + 1) * G - u0);

        float res[16][4];
#pragma unroll
        for (int m = 0; m < 16; ++m)
#pragma unroll
            for (int e = 0; e < 4; ++e) res[m][e] = 0.f;

        // first local unit index >= i_begin that is congruent to this warp modulo 8
        int i = i_begin + ((warp - i_begin) & (SK_CONSUMER_WARPS - 1));
        for (; i < i_end; i += SK_CONSUMER_WARPS) {
            const int slot = i % SK_STAGES, round = i / SK_STAGES;
            // A parity wait cannot tell phase r from phase r - 2.  The slot's previous round belongs
            // to another warp, so first see that round released (then the full barrier is in phase
            // r or later and its parity is unambiguous).
            if (!failed && round > 0 && !mbar_wait_bounded(empty_bar(slot), (round - 1) & 1)) {
                failed = true;
                if (lane == 0) atomicExch(err_flag, 3);
            }
            if (!failed && !mbar_wait_bounded(full_bar(slot), round & 1)) {
                failed = true;
                if (lane == 0) atomicExch(err_flag, 2);
            }
            if (failed) continue;
            const uint32_t st = smem_base + slot * SK_STAGE_BYTES;

            float acc[16][4];
            float sx[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int m = 0; m < 16; ++m)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[m][e] = 0.f;

#pragma unroll 1
            for (int p = 0; p < 4; ++p) {
                // activations for k-steps 2p and 2p+1: 16-byte chunk q = 4p + matrix index
                const int q = 4 * p + xm;
                uint32_t bx[4];
                ldmatrix_x4(bx, st + SK_OFF_X + (q >> 3) * 1024 + xb * 128 + (((q & 7) ^ xb) << 4));
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint32_t rb = st + (2 * p + h) * 2048;
                    const uint4 w0 = lds128(rb + offA);
                    const uint4 w1 = lds128(rb + offB);
                    const uint4 w2 = lds128(rb + 1024 + offA);
                    const uint4 w3 = lds128(rb + 1024 + offB);
                    const uint32_t b0 = bx[2 * h], b1 = bx[2 * h + 1];
                    mma_bf16_16816(sx, ONES, ONES, ONES, ONES, b0, b1);
                    const uint32_t q0[4] = {w0.x, w0.y, w0.z, w0.w};
                    const uint32_t q1[4] = {w1.x, w1.y, w1.z, w1.w};
                    const uint32_t q2[4] = {w2.x, w2.y, w2.z, w2.w};
                    const uint32_t q3[4] = {w3.x, w3.y, w3.z, w3.w};
#pragma unroll
                    for (int cb = 0; cb < 4; ++cb) {
                        // low halves hold nibbles 0-3 (columns 0,2,4,6), high halves nibbles 4-7
                        // (columns 1,3,5,7); pair rows k and k+1 of the same column in one register
                        const uint32_t lo01 = __byte_perm(q0[cb], q1[cb], 0x5410);
                        const uint32_t hi01 = __byte_perm(q0[cb], q1[cb], 0x7632);
                        const uint32_t lo23 = __byte_perm(q2[cb], q3[cb], 0x5410);
                        const uint32_t hi23 = __byte_perm(q2[cb], q3[cb], 0x7632);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            // MMA row g8 = column 8cb + 2e, row g8 + 8 = column 8cb + 2e + 1
                            mma_bf16_16816(acc[cb * 4 + e], nib2_to_bf16x2_biased(lo01 >> (4 * e)),
                                           nib2_to_bf16x2_biased(hi01 >> (4 * e)),
                                           nib2_to_bf16x2_biased(lo23 >> (4 * e)),
                                           nib2_to_bf16x2_biased(hi23 >> (4 * e)), b0, b1);
                        }
                    }
                }
            }

            // group fix-up: res += s * (acc - (128 + z) * sum_x)
            const uint4 zv = lds128(st + SK_OFF_Z + g8 * 16);
            const uint32_t zw[4] = {zv.x, zv.y, zv.z, zv.w};
#pragma unroll
            for (int cb = 0; cb < 4; ++cb) {
                const uint4 sv = lds128(st + SK_OFF_S + g8 * 64 + cb * 16);
                const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const uint32_t zz = nib2_to_bf16x2_biased(zw[cb] >> (4 * e));
                    const float z_even = bf16x2_lo(zz), z_odd = bf16x2_hi(zz);
                    const float s_even = bf16x2_lo(sw[e]), s_odd = bf16x2_hi(sw[e]);
                    float(&a)[4] = acc[cb * 4 + e];
                    float(&r)[4] = res[cb * 4 + e];
                    r[0] = fmaf(s_even, fmaf(-z_even, sx[0], a[0]), r[0]);
                    r[1] = fmaf(s_even, fmaf(-z_even, sx[1], a[1]), r[1]);
                    r[2] = fmaf(s_odd, fmaf(-z_odd, sx[0], a[2]), r[2]);
                    r[3] = fmaf(s_odd, fmaf(-z_odd, sx[1], a[3]), r[3]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar(slot));
        }

        // ---- sum the eight warps' partials (fixed order), one strip column per thread ----
        if (warp < 4) {
            float *slot = red + warp * SK_RED_SLOT;
#pragma unroll
            for (int m = 0; m < 16; ++m) {
                const int col = 32 * g8 + 8 * (m >> 2) + 2 * (m & 3);
                slot[sk_red_idx(2 * t4, col)] = res[m][0];
                slot[sk_red_idx(2 * t4 + 1, col)] = res[m][1];
                slot[sk_red_idx(2 * t4, col + 1)] = res[m][2];
                slot[sk_red_idx(2 * t4 + 1, col + 1)] = res[m][3];
            }
        }
        named_bar_sync(1, SK_CONSUMER_THREADS);
        if (warp >= 4) {
            float *slot = red + (warp - 4) * SK_RED_SLOT;
#pragma unroll
            for (int m = 0; m < 16; ++m) {
                const int col = 32 * g8 + 8 * (m >> 2) + 2 * (m & 3);
                slot[sk_red_idx(2 * t4, col)] += res[m][0];
                slot[sk_red_idx(2 * t4 + 1, col)] += res[m][1];
                slot[sk_red_idx(2 * t4, col + 1)] += res[m][2];
                slot[sk_red_idx(2 * t4 + 1, col + 1)] += res[m][3];
            }
        }
        named_bar_sync(1, SK_CONSUMER_THREADS);
        float val[8];
#pragma unroll
        for (int b = 0; b < 8; ++b) {
            const int idx = sk_red_idx(b, tid);
            val[b] = ((red[idx] + red[SK_RED_SLOT + idx]) + red[2 * SK_RED_SLOT + idx]) + red[3 * SK_RED_SLOT + idx];
        }
        named_bar_sync(1, SK_CONSUMER_THREADS);

        // ---- strips shared between CTAs: last arriver sums the partials in CTA order ----
        const long long c_lo = sk_owner((long long)v * G, C, U);
        const long long c_hi = sk_owner((long long)(v + 1) * G - 1, C, U);
        bool do_epilogue = true;
        if (c_hi > c_lo) {
            float *mine = partials + (size_t)(c + v) * SK_PARTIAL_FLOATS;
#pragma unroll
            for (int b = 0; b < 8; ++b)
                if (b < B) mine[b * SK_STRIP + tid] = val[b];
            __threadfence();
            named_bar_sync(1, SK_CONSUMER_THREADS);
            if (tid == 0) {
                const int old = atomicAdd(&counters[v], 1);
                *s_flag = (old == (int)(c_hi - c_lo)) ? 1 : 0;
            }
            named_bar_sync(1, SK_CONSUMER_THREADS);
            do_epilogue = (*s_flag != 0);
            if (do_epilogue) {
                __threadfence();
#pragma unroll
                for (int b = 0; b < 8; ++b) {
                    float s = 0.f;
                    if (b < B)
                        for (long long cc = c_lo; cc <= c_hi; ++cc)
                            s += __ldcg(partials + (size_t)(cc + v) * SK_PARTIAL_FLOATS + b * SK_STRIP + tid);
                    val[b] = s;
                }
                if (tid == 0) counters[v] = 0;  // leave the workspace ready for the next launch
            }
        }

        if (do_epilogue && !failed) {
            const int n = v * SK_STRIP + tid;
            if (EPI == EPI_SWIGLU) {
                uint16_t *out = reinterpret_cast<uint16_t *>(y_);
#pragma unroll
                for (int b = 0; b < 8; ++b) {
                    const float other = __shfl_xor_sync(0xffffffffu, val[b], 1);
                    if (b < B && n < N && !(tid & 1)) out[(size_t)b * (N >> 1) + (n >> 1)] = swiglu_bits(val[b], other);
                }
            } else if (n < N) {
#pragma unroll
                for (int b = 0; b < 8; ++b) {
                    if (b >= B) continue;
                    if (EPI == EPI_F32) {
                        reinterpret_cast<float *>(y_)[(size_t)b * N + n] = val[b];
                    } else {
                        float s = val[b];
                        if (residual) s += bf16_bits_to_f32(residual[(size_t)b * N + n]);
                        reinterpret_cast<uint16_t *>(y_)[(size_t)b * N + n] = f32_to_bf16_bits(s);
                    }
                }
            }
        }
        i_begin = i_end;
    }
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
                                   SK_STRIP, 1, CU_TENSOR_MAP_SWIZZLE_NONE)))
        return rc;
    if ((rc = encode_tensor_map_2d(&tmZ, CU_TENSOR_MAP_DATA_TYPE_INT32, a.qzeros, nb, G, (uint64_t)nb * 4, 32, 1,
                                   CU_TENSOR_MAP_SWIZZLE_NONE)))
        return rc;

    const long long U = (long long)V * G;
    int ctas = device_sm_count();
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
