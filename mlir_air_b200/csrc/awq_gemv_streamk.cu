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
//    ldmatrix.trans on the 128B-swizzled box hands lane (g, t) the 16-bit half g of a 16-byte
//    chunk for k rows 2t and 2t + 1 already paired in one register; one LOP3 per nibble pair turns
//    that into the A fragment of mma.sync.m16n8k16 (rows = 16 output columns, k = 16).  The
//    activations are the B fragment (ldmatrix from swizzled smem).
//  * The zero point and scale never touch the inner loop:
//        sum_k (q - z) s x = s (sum_k (128 + q) x  -  (128 + z) sum_k x)
//    per group; sum_k x comes from one extra MMA with an all-ones A fragment.
//  * At the end of a strip segment a warp that covered the whole strip applies the epilogue
//    from registers.  Otherwise it adds its partial sums to the sub-strip's 64-bit accumulator
//    words, each add carrying the value (fixed point) and the number of k groups it covers in one
//    atomic (awq_streamk.cuh: sk_handover); the warp whose add completes the count has the
//    total and applies the epilogue.  No fence, no counter, nothing waits on another CTA, and
//    the result does not depend on the order of the adds.
//
// Epilogues: bf16 (+ residual), f32 (tensor-parallel partial), SwiGLU over interleaved
// gate/up column pairs (matvec_int4_swiglu_rms.py:511-516 rounding points).
#include <cudaTypedefs.h>
#include <cuda_fp16.h>

#include <mutex>

#include "awq_common.cuh"
#include "awq_ptx.cuh"
#include "awq_streamk.cuh"

namespace awq {

// Leading bytes of a workspace (error flag, counters, accumulators of the strips a product of N
// columns uses) that must be zero before a launch.
size_t gemv_streamk_workspace_clear_bytes(int N) {
    return SK_WS_ACCUM + (size_t)((N + SK_STRIP - 1) / SK_STRIP) * SK_STRIP_WORDS * 8;
}

template <int EPI, bool XH>
__global__ void __launch_bounds__(SK_THREADS, SK_CTAS_PER_SM)
gemv_streamk_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                    const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmZ,
                    const uint16_t *__restrict__ residual, void *__restrict__ y_, int B, int N, int G,
                    int V, int out_f16, unsigned long long *__restrict__ accum, int *__restrict__ err_flag,
                    const PeerPush push, long long wait_limit) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = smem_base + SK_STAGES * SK_STAGE_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (SK_STAGES + s); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long U = (long long)V * G, C = gridDim.x, c = blockIdx.x;
    const long long u0 = c * U / C, u1 = (c + 1) * U / C;
    const int n_units = (int)(u1 - u0);
    const int v_first = (int)(u0 / G), g_first = (int)(u0 % G);

    if (threadIdx.x == 0) {
        for (int s = 0; s < SK_STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), SK_CONSUMER_WARPS);
        }
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == SK_CONSUMER_WARPS) {
        // ------------------------------ producer ------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&tmW);
            tma_prefetch_desc(&tmX);
            tma_prefetch_desc(&tmS);
            tma_prefetch_desc(&tmZ);
            const uint64_t stream_policy = l2_policy_evict_first();
            auto load_weights = [&](int slot, int v, int g) {
                const uint32_t st = smem_base + slot * SK_STAGE_BYTES;
                const uint32_t bar = full_bar(slot);
                mbar_expect_tx(bar, SK_TX_BYTES);
#pragma unroll
                for (int bx = 0; bx < SK_STRIP / SK_BOX_COLS; ++bx)
                    tma_load_2d_hint(st + bx * SK_WBOX_BYTES, &tmW, (v * SK_STRIP + bx * SK_BOX_COLS) / 8, g * SK_GROUP,
                                     bar, stream_policy);
#pragma unroll
                for (int bx = 0; bx < SK_STRIP / SK_BOX_COLS; ++bx)
                    tma_load_2d(st + SK_OFF_S + bx * SK_BOX_COLS * 2, &tmS, v * SK_STRIP + bx * SK_BOX_COLS, g, bar);
                tma_load_2d(st + SK_OFF_Z, &tmZ, v * (SK_STRIP / 8), g, bar);
            };
            auto load_activations = [&](int slot, int g) {
                const uint32_t st = smem_base + slot * SK_STAGE_BYTES;
                tma_load_2d(st + SK_OFF_X, &tmX, g * SK_GROUP, 0, full_bar(slot));
                tma_load_2d(st + SK_OFF_X + 1024, &tmX, g * SK_GROUP + 64, 0, full_bar(slot));
            };
            // The weights do not depend on the previous kernel: fill the ring with them first, and
            // only then wait for the previous kernel (whose output is this kernel's activations).
            const int n_first = n_units < SK_STAGES ? n_units : SK_STAGES;
            int v = v_first, g = g_first;
            for (int i = 0; i < n_first; ++i) {
                load_weights(i, v, g);
                if (++g == G) { g = 0; ++v; }
            }
            pdl_wait();
            g = g_first;
            for (int i = 0; i < n_first; ++i) {
                load_activations(i, g);
                if (++g == G) g = 0;
            }
            int slot = 0, round = 1;
            for (int i = n_first; i < n_units; ++i) {
                if (!mbar_wait_bounded(empty_bar(slot), (round - 1) & 1, wait_limit)) {
                    atomicExch(err_flag, 1);
                    break;
                }
                load_weights(slot, v, g);
                load_activations(slot, g);
                if (++g == G) { g = 0; ++v; }
                if (++slot == SK_STAGES) { slot = 0; ++round; }
            }
        }
        return;
    }
    pdl_wait();  // consumers read and write global memory the previous kernel may still be using

    // ------------------------------ consumers ------------------------------
    // Warp w owns strip columns [64 w, 64 w + 64): two 16-byte chunks (A, B) of every box row.
    // ldmatrix.trans hands lane (g8, t4) 16-bit half g8 of chunk A / B for rows 2 t4 and 2 t4 + 1
    // already paired in one register: half g8 = packed word g8 / 2, even (low half) or odd
    // (high half) columns.  MMA row g8 is that lane's chunk-A column, row g8 + 8 its chunk-B column.
    const SkLane lane_geo(warp, lane);
    const int g8 = lane_geo.g8, t4 = lane_geo.t4, odd = lane_geo.odd, colw = lane_geo.colw;
    bool failed = false;

    float res[4][4];
    int cur_v = -1, seg_groups = 0;  // strip being accumulated, k groups of it added so far

    // Finish the strip segment this warp has been accumulating (strip cur_v).
    auto flush = [&]() {
        const int v = cur_v;
        float own[2][8];
        sk_lane_exchange(res, odd, own);
        const int b = 2 * t4 + odd;
        const int n = v * SK_STRIP + colw;
        if (seg_groups != G &&
            !sk_handover(accum + ((size_t)v * SK_CONSUMER_WARPS + warp) * SK_ACC_WORDS, own, seg_groups, G, lane, wait_limit,
                         err_flag))
            return;
        if (!failed) sk_epilogue<EPI>(own, residual, y_, B, N, n, b, out_f16);
        if (EPI == EPI_F32_PUSH && !failed) sk_push_signal(push, err_flag + 8, V * SK_CONSUMER_WARPS, lane);
    };

    int v = v_first, g = g_first, slot = 0, round = 0;
    for (int i = 0; i < n_units; ++i) {
        if (v != cur_v) {
            if (cur_v >= 0) flush();
            cur_v = v;
            seg_groups = 0;
#pragma unroll
            for (int e = 0; e < 4; ++e)
#pragma unroll
                for (int q = 0; q < 4; ++q) res[e][q] = 0.f;
        }
        ++seg_groups;
        if (!failed && !mbar_wait_bounded(full_bar(slot), round & 1, wait_limit)) {
            failed = true;
            if (lane == 0) atomicExch(err_flag, 2);
        }
        if (!failed) {
            sk_consume_unit<XH>(smem_base + slot * SK_STAGE_BYTES, lane_geo, res, empty_bar(slot), lane);
        }
        if (++g == G) { g = 0; ++v; }
        if (++slot == SK_STAGES) { slot = 0; ++round; }
    }
    if (cur_v >= 0) flush();
}

// x bf16 -> fp16 (a value beyond the fp16 range becomes an infinity and is reported through the error flag)
__global__ void cvt_bf16_to_f16_kernel(const uint16_t *__restrict__ x, uint16_t *__restrict__ xh, size_t n,
                                       int *__restrict__ err_flag) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = bf16_bits_to_f32(x[i]);
    if (fabsf(v) > 65504.f && !(v != v)) atomicExch(err_flag, 4);
    xh[i] = bf16_value_to_f16_bits(v);
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

// Tiled tensor map of rank 2 or 3 (dim2 == 0: rank 2).  dim0 is contiguous; stride1 / stride2 are the byte strides
// of dim1 / dim2 (multiples of 16, in any order of size).
int encode_tensor_map_3d(CUtensorMap *map, int dtype, const void *base, uint64_t dim0, uint64_t dim1, uint64_t dim2,
                         uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0, uint32_t box1, uint32_t box2,
                         int swizzle) {
    PFN_cuTensorMapEncodeTiled_v12000 fn = get_encode_fn();
    if (!fn) return set_error(AWQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const int rank = dim2 ? 3 : 2;
    cuuint64_t dims[3] = {dim0, dim1, dim2};
    cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
    cuuint32_t box[3] = {box0, box1, box2};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, (CUtensorMapDataType)dtype, rank, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, (CUtensorMapSwizzle)swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return set_error(AWQ_ERR_CUDA, "cuTensorMapEncodeTiled failed (CUresult %d; dims %llu x %llu x %llu, strides %llu, %llu)",
                         (int)r, (unsigned long long)dim0, (unsigned long long)dim1, (unsigned long long)dim2,
                         (unsigned long long)stride1_bytes, (unsigned long long)stride2_bytes);
    return AWQ_OK;
}

int encode_tensor_map_2d(CUtensorMap *map, int dtype, const void *base, uint64_t dim0, uint64_t dim1,
                         uint64_t stride1_bytes, uint32_t box0, uint32_t box1, int swizzle) {
    return encode_tensor_map_3d(map, dtype, base, dim0, dim1, 0, stride1_bytes, 0, box0, box1, 1, swizzle);
}

// A rank signals once per EPI_F32_PUSH launch, when its last sub-strip is stored.
int gemv_push_arrivals_per_rank(int N) {
    (void)N;
    return 1;
}

bool gemv_streamk_supported(const GemvArgs &a) {
    return a.group_size == SK_GROUP && a.K % SK_GROUP == 0 && a.K / SK_GROUP <= SK_MAX_GROUPS && a.N % 32 == 0 && a.B >= 1 &&
           a.K > 0 && a.N > 0 &&
           aligned16(a.x) && aligned16(a.qweight) && aligned16(a.qzeros) && aligned16(a.scales) &&
           (a.N + SK_STRIP - 1) / SK_STRIP <= SK_MAX_STRIPS && device_is_sm100();
}

// Scratch without the activation-conversion buffer: the header and the accumulators of the strips.
size_t gemv_streamk_scratch_bytes(int N, bool deterministic) {
    (void)deterministic;  // the hand-over adds integers: every mode is reproducible
    return SK_WS_ACCUM + (size_t)((N + SK_STRIP - 1) / SK_STRIP) * SK_STRIP_WORDS * 8;
}

size_t gemv_streamk_workspace_bytes(int B, int K, int N) {
    // header + accumulators of every strip a product may use + room for B rows of activations converted to fp16
    const size_t rows = B < 1 ? 1 : (B > 64 ? 64 : B);
    (void)N;
    return SK_WS_XH + rows * (size_t)(K > 0 ? K : 0) * 2;
}

template <int EPI, bool XH>
static int launch_one(const GemvArgs &a, const uint16_t *x, const uint16_t *residual, void *y, int B) {
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(gemv_streamk_kernel<EPI, XH>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        SK_SMEM_BYTES);
    });
    if (attr_err != cudaSuccess) return check_cuda(attr_err, "stream-K gemv: shared memory attribute");

    const int G = a.K / SK_GROUP, V = (a.N + SK_STRIP - 1) / SK_STRIP, nb = a.N / 8;
    CUtensorMap tmW, tmX, tmS, tmZ;
    int rc;
    if ((rc = encode_tensor_map_2d(&tmW, CU_TENSOR_MAP_DATA_TYPE_INT32, a.qweight, nb, a.K, (uint64_t)nb * 4, 32,
                                   SK_GROUP, CU_TENSOR_MAP_SWIZZLE_128B)))
        return rc;
    if ((rc = encode_tensor_map_2d(&tmX, XH ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, x,
                                   a.K, B, (uint64_t)a.K * 2, 64, 8, CU_TENSOR_MAP_SWIZZLE_128B)))
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
    unsigned long long *accum = reinterpret_cast<unsigned long long *>(ws + SK_WS_ACCUM);
    return check_cuda(launch_pdl(gemv_streamk_kernel<EPI, XH>, dim3(ctas), dim3(SK_THREADS), SK_SMEM_BYTES, a.stream, tmW,
                                 tmX, tmS, tmZ, residual, y, B, a.N, G, V, a.out_format == ACT_F16 ? 1 : 0, accum, err_flag,
                                 a.push ? *a.push : PeerPush{}, wait_limit_cycles()),
                      "stream-K gemv launch");
}

template <bool XH>
static int launch_passes(const GemvArgs &a, const uint16_t *x_all) {
    // more than 8 batch rows: up to 32 rows per pass over the weights with the multi-row kernel
    // (fp16 activations, f32-atomic reduction), else one pass per 8 rows
    int B = 0;
    for (int b0 = 0; b0 < a.B; b0 += B) {
        const int left = a.B - b0;
        const uint16_t *x = x_all + (size_t)b0 * a.K;
        const uint16_t *res = a.residual ? a.residual + (size_t)b0 * a.N : nullptr;
        int rc;
        B = left < 32 ? left : 32;
        if (XH && B > 8 && gemv_streamk_mb_supported(a, B)) {
            void *yb = a.epilogue == EPI_F32      ? (void *)(reinterpret_cast<float *>(a.y) + (size_t)b0 * a.N)
                       : a.epilogue == EPI_SWIGLU ? (void *)(reinterpret_cast<uint16_t *>(a.y) + (size_t)b0 * (a.N / 2))
                                                  : (void *)(reinterpret_cast<uint16_t *>(a.y) + (size_t)b0 * a.N);
            if ((rc = launch_gemv_streamk_mb(a, x, a.epilogue == EPI_BF16 ? res : nullptr, yb, B))) return rc;
            continue;
        }
        B = left < 8 ? left : 8;
        switch (a.epilogue) {
            case EPI_BF16:
                rc = launch_one<EPI_BF16, XH>(a, x, res, reinterpret_cast<uint16_t *>(a.y) + (size_t)b0 * a.N, B);
                break;
            case EPI_F32:
                rc = launch_one<EPI_F32, XH>(a, x, nullptr, reinterpret_cast<float *>(a.y) + (size_t)b0 * a.N, B);
                break;
            case EPI_F32_PUSH:  // one pass only: the receivers expect one launch worth of arrivals
                rc = a.B <= 8 && a.push ? launch_one<EPI_F32_PUSH, XH>(a, x, nullptr, a.y, B)
                                        : set_error(AWQ_ERR_UNSUPPORTED, "gemv push: at most 8 batch rows");
                break;
            default:
                rc = launch_one<EPI_SWIGLU, XH>(a, x, nullptr,
                                                reinterpret_cast<uint16_t *>(a.y) + (size_t)b0 * (a.N / 2), B);
                break;
        }
        if (rc) return rc;
    }
    return AWQ_OK;
}

int launch_gemv_streamk(const GemvArgs &a) {
    const bool convert = a.x_format == ACT_BF16 && !a.native_bf16;
    const size_t xh_off = SK_WS_XH;  // the conversion buffer sits behind the accumulators of every possible strip and the stack kernel's state
    const size_t need = convert ? xh_off + (size_t)a.B * a.K * 2 : gemv_streamk_scratch_bytes(a.N, a.deterministic);
    if (!a.workspace || a.workspace_bytes < need)
        return set_error(AWQ_ERR_WORKSPACE, "gemv: workspace of %zu bytes needed, %zu given", need, a.workspace_bytes);
    if (a.x_format == ACT_F16) return launch_passes<true>(a, a.x);
    if (a.native_bf16) return launch_passes<false>(a, a.x);
    // bf16 activations: convert once to fp16 in the workspace, then take the fp16 path
    uint8_t *ws = reinterpret_cast<uint8_t *>(a.workspace);
    uint16_t *xh = reinterpret_cast<uint16_t *>(ws + xh_off);
    const size_t n = (size_t)a.B * a.K;
    int rc = check_cuda(launch_pdl(cvt_bf16_to_f16_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, a.stream, a.x,
                                   xh, n, reinterpret_cast<int *>(ws)),
                        "activation conversion launch");
    if (rc) return rc;
    return launch_passes<true>(a, xh);
}

}  // namespace awq
