// Generic CUDA-core kernels: the any-shape decode GEMV / prefill GEMM (used where the
// specialised kernels' shape rules do not hold, and as an independent cross-check in the
// tests), RMSNorm, residual-add + RMSNorm, and the once-per-weight layout converters.
#include <cuda_fp16.h>

#include "awq_common.cuh"
#include "awq_ptx.cuh"

namespace awq {

// =====================================================================================
// Generic decode GEMV.  Block = 32 packed word columns (256 output columns) x 8 k-slices;
// a warp reads 128 contiguous bytes of one k row.  f32 weights (q - z) * s, f32 accumulate,
// k-slices reduced through shared memory in a fixed order.
// =====================================================================================
constexpr int GV_TB = 4;  // batch rows per pass

template <int EPI>
__global__ void __launch_bounds__(256)
gemv_generic_kernel(const uint16_t *__restrict__ x, const uint32_t *__restrict__ qweight,
                    const uint32_t *__restrict__ qzeros, const uint16_t *__restrict__ scales,
                    const uint16_t *__restrict__ residual, void *__restrict__ y_, int B, int K,
                    int N, int group_size, int x_f16, int out_f16) {
    __shared__ float red[8][GV_TB][256];
    const int nb = N >> 3;
    const int cx = threadIdx.x & 31, ky = threadIdx.x >> 5;
    const int j = blockIdx.x * 32 + cx;
    const bool active = j < nb;
    for (int b0 = 0; b0 < B; b0 += GV_TB) {
        float acc[GV_TB][8];
#pragma unroll
        for (int b = 0; b < GV_TB; ++b)
#pragma unroll
            for (int c = 0; c < 8; ++c) acc[b][c] = 0.f;
        if (active) {
            int cur_group = -1;
            float s[8];
            int z[8];
            for (int k = ky; k < K; k += 8) {
                const int g = k / group_size;
                if (g != cur_group) {
                    cur_group = g;
                    const uint32_t zw = qzeros[(size_t)g * nb + j];
                    const uint4 sv = *reinterpret_cast<const uint4 *>(scales + (size_t)g * N + 8 * j);
                    const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        z[c] = (int)awq_nibble(zw, c);
                        s[c] = (c & 1) ? bf16x2_hi(sw[c >> 1]) : bf16x2_lo(sw[c >> 1]);
                    }
                }
                const uint32_t qw = __ldg(qweight + (size_t)k * nb + j);
                float w[8];
#pragma unroll
                for (int c = 0; c < 8; ++c) w[c] = (float)((int)awq_nibble(qw, c) - z[c]) * s[c];
#pragma unroll
                for (int b = 0; b < GV_TB; ++b) {
                    if (b0 + b < B) {
                        const uint16_t xb = x[(size_t)(b0 + b) * K + k];
                        const float xv = x_f16 ? __half2float(__ushort_as_half(xb)) : bf16_bits_to_f32(xb);
#pragma unroll
                        for (int c = 0; c < 8; ++c) acc[b][c] = fmaf(w[c], xv, acc[b][c]);
                    }
                }
            }
        }
#pragma unroll
        for (int b = 0; b < GV_TB; ++b)
#pragma unroll
            for (int c = 0; c < 8; ++c) red[ky][b][cx * 8 + c] = acc[b][c];
        __syncthreads();
        const int col = threadIdx.x;
        const int n = blockIdx.x * 256 + col;
#pragma unroll
        for (int b = 0; b < GV_TB; ++b) {
            float sum = 0.f;
#pragma unroll
            for (int q = 0; q < 8; ++q) sum += red[q][b][col];
            const int bb = b0 + b;
            if (EPI == EPI_SWIGLU) {
                const float other = __shfl_xor_sync(0xffffffffu, sum, 1);
                if (bb < B && n < N && !(col & 1)) {
                    uint16_t o = swiglu_bits(sum, other);
                    if (out_f16) o = __half_as_ushort(__float2half_rn(bf16_bits_to_f32(o)));
                    reinterpret_cast<uint16_t *>(y_)[(size_t)bb * (N >> 1) + (n >> 1)] = o;
                }
            } else if (bb < B && n < N) {
                if (EPI == EPI_F32) {
                    reinterpret_cast<float *>(y_)[(size_t)bb * N + n] = sum;
                } else {
                    if (residual) sum += bf16_bits_to_f32(residual[(size_t)bb * N + n]);
                    reinterpret_cast<uint16_t *>(y_)[(size_t)bb * N + n] = f32_to_bf16_bits(sum);
                }
            }
        }
        __syncthreads();
    }
}

int launch_gemv_generic(const GemvArgs &a) {
    const int blocks = (a.N / 8 + 31) / 32;
    const uint32_t *qw = reinterpret_cast<const uint32_t *>(a.qweight);
    const uint32_t *qz = reinterpret_cast<const uint32_t *>(a.qzeros);
    const int xf = a.x_format == ACT_F16, of = a.out_format == ACT_F16;
    switch (a.epilogue) {
        case EPI_BF16:
            gemv_generic_kernel<EPI_BF16><<<blocks, 256, 0, a.stream>>>(
                a.x, qw, qz, a.scales, a.residual, a.y, a.B, a.K, a.N, a.group_size, xf, of);
            break;
        case EPI_F32:
            gemv_generic_kernel<EPI_F32><<<blocks, 256, 0, a.stream>>>(
                a.x, qw, qz, a.scales, nullptr, a.y, a.B, a.K, a.N, a.group_size, xf, of);
            break;
        default:
            gemv_generic_kernel<EPI_SWIGLU><<<blocks, 256, 0, a.stream>>>(
                a.x, qw, qz, a.scales, nullptr, a.y, a.B, a.K, a.N, a.group_size, xf, of);
            break;
    }
    return check_cuda(cudaGetLastError(), "generic gemv launch");
}

// =====================================================================================
// Generic prefill GEMM: 64 x 64 block tile, 4 x 4 per thread, k-step 32, operands staged
// in shared memory as f32 (weights as the exact f32 product (q - z) * s).
// =====================================================================================
constexpr int GG_BM = 64, GG_BN = 64, GG_BK = 32;

__global__ void __launch_bounds__(256)
gemm_generic_kernel(const uint16_t *__restrict__ A, const uint32_t *__restrict__ qweight,
                    const uint32_t *__restrict__ qzeros, const uint16_t *__restrict__ scales,
                    uint16_t *__restrict__ C, int M, int K, int N, int group_size) {
    __shared__ float As[GG_BK][GG_BM + 4];
    __shared__ float Ws[GG_BK][GG_BN + 4];
    const int nb = N >> 3;
    const int m0 = blockIdx.y * GG_BM, n0 = blockIdx.x * GG_BN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // 16 x 16 threads
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) acc[i][jj] = 0.f;

    const int a_row = threadIdx.x >> 2, a_k8 = (threadIdx.x & 3) * 8;  // A: 64 rows x 4 chunks of 8 k
    const int w_row = threadIdx.x >> 3, w_cb = threadIdx.x & 7;        // W: 32 rows x 8 words
    for (int k0 = 0; k0 < K; k0 += GG_BK) {
        {
            uint32_t v[4] = {0u, 0u, 0u, 0u};
            if (m0 + a_row < M) {
                const uint4 t = *reinterpret_cast<const uint4 *>(A + (size_t)(m0 + a_row) * K + k0 + a_k8);
                v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                As[a_k8 + 2 * e][a_row] = bf16x2_lo(v[e]);
                As[a_k8 + 2 * e + 1][a_row] = bf16x2_hi(v[e]);
            }
        }
        {
            const int k = k0 + w_row, j = (n0 >> 3) + w_cb;
            float w[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (j < nb) {
                const int g = k / group_size;
                const uint32_t qw = __ldg(qweight + (size_t)k * nb + j);
                const uint32_t zw = __ldg(qzeros + (size_t)g * nb + j);
                const uint4 sv = *reinterpret_cast<const uint4 *>(scales + (size_t)g * N + 8 * j);
                const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const float s = (c & 1) ? bf16x2_hi(sw[c >> 1]) : bf16x2_lo(sw[c >> 1]);
                    w[c] = (float)((int)awq_nibble(qw, c) - (int)awq_nibble(zw, c)) * s;
                }
            }
#pragma unroll
            for (int c = 0; c < 8; ++c) Ws[w_row][w_cb * 8 + c] = w[c];
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GG_BK; ++kk) {
            float av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) wv[jj] = Ws[kk][tx * 4 + jj];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) acc[i][jj] = fmaf(av[i], wv[jj], acc[i][jj]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const int n = n0 + tx * 4 + jj;
            if (n < N) C[(size_t)m * N + n] = f32_to_bf16_bits(acc[i][jj]);
        }
    }
}

int launch_gemm_generic(const uint16_t *A, const int32_t *qweight, const int32_t *qzeros,
                        const uint16_t *scales, uint16_t *C, int M, int K, int N, int group_size,
                        cudaStream_t stream) {
    dim3 grid((N + GG_BN - 1) / GG_BN, (M + GG_BM - 1) / GG_BM);
    gemm_generic_kernel<<<grid, 256, 0, stream>>>(A, reinterpret_cast<const uint32_t *>(qweight),
                                                  reinterpret_cast<const uint32_t *>(qzeros), scales, C,
                                                  M, K, N, group_size);
    return check_cuda(cudaGetLastError(), "generic gemm launch");
}

// =====================================================================================
// RMSNorm (one block per row) and residual-add + RMSNorm.
// =====================================================================================
__device__ __forceinline__ float block_sum_256(float v, float *smem) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += smem[w];
    __syncthreads();
    return t;
}

// normed = bf16((x * rstd) * gamma), rstd = 1 / sqrt(mean(x^2) + eps) with the mean formed
// in f32 and the rsqrt in f64 as the numpy golden does (matvec_int4_swiglu_rms.py:496-500).
// One block per row; each thread keeps its (up to RN_PER_THREAD * 8) elements in registers
// between the two passes, 16 bytes per load.
constexpr int RN_THREADS = 256;
constexpr int RN_CHUNKS = 8;  // 16-byte chunks per thread held in registers: rows up to 16384 elements

__global__ void __launch_bounds__(RN_THREADS)
rmsnorm_kernel(const uint16_t *__restrict__ h, const float *__restrict__ partial,
               const uint16_t *__restrict__ gamma, float eps, uint16_t *__restrict__ h_out,
               uint16_t *__restrict__ normed, int K, int normed_f16) {
    __shared__ float red[8];
    pdl_launch_dependents();
    pdl_wait();
    const size_t row = (size_t)blockIdx.x * K;
    const int n_chunks = K >> 3;  // K % 8 == 0 is required by the launcher
    float v[RN_CHUNKS][8];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < RN_CHUNKS; ++c) {
        const int ch = threadIdx.x + c * RN_THREADS;
        if (ch < n_chunks) {
            const uint4 t = *reinterpret_cast<const uint4 *>(h + row + 8 * ch);
            const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                v[c][2 * e] = bf16x2_lo(w[e]);
                v[c][2 * e + 1] = bf16x2_hi(w[e]);
            }
            if (partial) {
                const float4 p0 = *reinterpret_cast<const float4 *>(partial + row + 8 * ch);
                const float4 p1 = *reinterpret_cast<const float4 *>(partial + row + 8 * ch + 4);
                const float pp[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
                uint32_t o[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    o[e] = pack_bf16x2(v[c][2 * e] + pp[2 * e], v[c][2 * e + 1] + pp[2 * e + 1]);
                    v[c][2 * e] = bf16x2_lo(o[e]);
                    v[c][2 * e + 1] = bf16x2_hi(o[e]);
                }
                if (h_out) *reinterpret_cast<uint4 *>(h_out + row + 8 * ch) = make_uint4(o[0], o[1], o[2], o[3]);
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) ss = fmaf(v[c][e], v[c][e], ss);
        }
    }
    if (!normed) return;
    const float total = block_sum_256(ss, red);
    const float rstd = (float)(1.0 / sqrt((double)(total / (float)K) + (double)eps));
#pragma unroll
    for (int c = 0; c < RN_CHUNKS; ++c) {
        const int ch = threadIdx.x + c * RN_THREADS;
        if (ch < n_chunks) {
            const uint4 gt = *reinterpret_cast<const uint4 *>(gamma + 8 * ch);
            const uint32_t gw[4] = {gt.x, gt.y, gt.z, gt.w};
            uint32_t o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                uint16_t lo = f32_to_bf16_bits((v[c][2 * e] * rstd) * bf16x2_lo(gw[e]));
                uint16_t hi = f32_to_bf16_bits((v[c][2 * e + 1] * rstd) * bf16x2_hi(gw[e]));
                if (normed_f16) {
                    lo = __half_as_ushort(__float2half_rn(bf16_bits_to_f32(lo)));
                    hi = __half_as_ushort(__float2half_rn(bf16_bits_to_f32(hi)));
                }
                o[e] = (uint32_t)lo | ((uint32_t)hi << 16);
            }
            *reinterpret_cast<uint4 *>(normed + row + 8 * ch) = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
}

// Tensor-parallel hand-over without a collective call: every rank's down projection has written its
// f32 partial [B, K] into its own send buffer and counted its finished sub-strips in flags[rank] on
// every rank (EPI_F32_PUSH).  One block per batch row waits for all ranks (bounded), then reads the
// partials with peer loads: h_out = bf16(h + sum over ranks in rank order) and, with gamma, its
// RMSNorm.  The last block to finish clears the counters for the slot's next use.
// flags: [0, 8) arrivals per rank, [8] blocks done.
__device__ __forceinline__ unsigned int ld_acquire_sys_u32(const unsigned int *p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(RN_THREADS)
tp_reduce_add_rmsnorm_kernel(const uint16_t *__restrict__ h, const PeerPartials parts, unsigned int *flags,
                             unsigned int expected, const uint16_t *__restrict__ gamma, float eps,
                             uint16_t *__restrict__ h_out, uint16_t *__restrict__ normed, int K, int normed_f16,
                             int *err_flag, long long wait_limit) {
    __shared__ float red[8];
    const int n_ranks = parts.n;
    pdl_launch_dependents();
    pdl_wait();
    int ok = 1;
    if ((int)threadIdx.x < n_ranks) {
        const long long t0 = clock64();
        while (ld_acquire_sys_u32(flags + threadIdx.x) < expected) {
            if (clock64() - t0 > wait_limit) {
                ok = 0;
                break;
            }
            __nanosleep(100);
        }
    }
    if (!__syncthreads_and(ok)) {
        if (threadIdx.x == 0) atomicExch(err_flag, 5);
        return;
    }
    const size_t row = (size_t)blockIdx.x * K;
    const int n_chunks = K >> 3;
    float v[RN_CHUNKS][8];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < RN_CHUNKS; ++c) {
        const int ch = threadIdx.x + c * RN_THREADS;
        if (ch < n_chunks) {
            float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int r = 0; r < TP_MAX_RANKS; ++r) {
                if (r >= n_ranks) break;
                const float *src = parts.partial[r] + row + 8 * ch;
                const float4 p0 = __ldcg(reinterpret_cast<const float4 *>(src));
                const float4 p1 = __ldcg(reinterpret_cast<const float4 *>(src + 4));
                sum[0] += p0.x; sum[1] += p0.y; sum[2] += p0.z; sum[3] += p0.w;
                sum[4] += p1.x; sum[5] += p1.y; sum[6] += p1.z; sum[7] += p1.w;
            }
            const uint4 t = *reinterpret_cast<const uint4 *>(h + row + 8 * ch);
            const uint32_t w[4] = {t.x, t.y, t.z, t.w};
            uint32_t o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                o[e] = pack_bf16x2(bf16x2_lo(w[e]) + sum[2 * e], bf16x2_hi(w[e]) + sum[2 * e + 1]);
                v[c][2 * e] = bf16x2_lo(o[e]);
                v[c][2 * e + 1] = bf16x2_hi(o[e]);
            }
            *reinterpret_cast<uint4 *>(h_out + row + 8 * ch) = make_uint4(o[0], o[1], o[2], o[3]);
#pragma unroll
            for (int e = 0; e < 8; ++e) ss = fmaf(v[c][e], v[c][e], ss);
        }
    }
    if (normed) {
        const float total = block_sum_256(ss, red);
        const float rstd = (float)(1.0 / sqrt((double)(total / (float)K) + (double)eps));
#pragma unroll
        for (int c = 0; c < RN_CHUNKS; ++c) {
            const int ch = threadIdx.x + c * RN_THREADS;
            if (ch < n_chunks) {
                const uint4 gt = *reinterpret_cast<const uint4 *>(gamma + 8 * ch);
                const uint32_t gw[4] = {gt.x, gt.y, gt.z, gt.w};
                uint32_t o[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    uint16_t lo = f32_to_bf16_bits((v[c][2 * e] * rstd) * bf16x2_lo(gw[e]));
                    uint16_t hi = f32_to_bf16_bits((v[c][2 * e + 1] * rstd) * bf16x2_hi(gw[e]));
                    if (normed_f16) {
                        lo = __half_as_ushort(__float2half_rn(bf16_bits_to_f32(lo)));
                        hi = __half_as_ushort(__float2half_rn(bf16_bits_to_f32(hi)));
                    }
                    o[e] = (uint32_t)lo | ((uint32_t)hi << 16);
                }
                *reinterpret_cast<uint4 *>(normed + row + 8 * ch) = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
    }
    // every block has passed its wait once all of them count here: the last one clears the slot
    __syncthreads();
    if (threadIdx.x == 0) {
        if (atomicAdd(flags + 8, 1u) == gridDim.x - 1) {
            for (int r = 0; r < 9; ++r) flags[r] = 0u;
            __threadfence_system();
        }
    }
}

// =====================================================================================
// Half-split RoPE (rope_halfsplit.cc; golden rms_qkv_int4_rope_multi.py:533-551): for every head of
// head_dim values, out[i] = x[i] cos[i] - x[i + half] sin[i], out[i + half] = x[i] sin[i] +
// x[i + half] cos[i], in f32 with one bf16 rounding; the LUT row of a token is [cos_0.. | sin_0..].
// One thread per pair of 8 + 8 values (16-byte loads).
// =====================================================================================
__global__ void rope_halfsplit_kernel(const uint16_t *__restrict__ x, size_t x_stride, const uint16_t *__restrict__ lut,
                                      uint16_t *__restrict__ out, size_t out_stride, int B, int n_heads, int head_dim) {
    const int half = head_dim >> 1, chunks = half >> 3;  // 16-byte chunks in a half head
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)B * n_heads * chunks;
    if (idx >= total) return;
    const int c = (int)(idx % chunks);
    const int head = (int)((idx / chunks) % n_heads);
    const int b = (int)(idx / ((size_t)chunks * n_heads));
    const uint16_t *xr = x + (size_t)b * x_stride + (size_t)head * head_dim + 8 * c;
    const uint16_t *lr = lut + (size_t)b * head_dim + 8 * c;
    const uint4 a4 = *reinterpret_cast<const uint4 *>(xr), b4 = *reinterpret_cast<const uint4 *>(xr + half);
    const uint4 c4 = *reinterpret_cast<const uint4 *>(lr), s4 = *reinterpret_cast<const uint4 *>(lr + half);
    const uint32_t x1[4] = {a4.x, a4.y, a4.z, a4.w}, x2[4] = {b4.x, b4.y, b4.z, b4.w};
    const uint32_t cs[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
    uint32_t o1[4], o2[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float a_lo = bf16x2_lo(x1[e]), a_hi = bf16x2_hi(x1[e]), b_lo = bf16x2_lo(x2[e]), b_hi = bf16x2_hi(x2[e]);
        const float c_lo = bf16x2_lo(cs[e]), c_hi = bf16x2_hi(cs[e]), s_lo = bf16x2_lo(sn[e]), s_hi = bf16x2_hi(sn[e]);
        // products and sums formed separately in f32, as numpy does (no fused multiply-add)
        o1[e] = pack_bf16x2(__fsub_rn(__fmul_rn(a_lo, c_lo), __fmul_rn(b_lo, s_lo)),
                            __fsub_rn(__fmul_rn(a_hi, c_hi), __fmul_rn(b_hi, s_hi)));
        o2[e] = pack_bf16x2(__fadd_rn(__fmul_rn(a_lo, s_lo), __fmul_rn(b_lo, c_lo)),
                            __fadd_rn(__fmul_rn(a_hi, s_hi), __fmul_rn(b_hi, c_hi)));
    }
    uint16_t *orow = out + (size_t)b * out_stride + (size_t)head * head_dim + 8 * c;
    *reinterpret_cast<uint4 *>(orow) = make_uint4(o1[0], o1[1], o1[2], o1[3]);
    *reinterpret_cast<uint4 *>(orow + half) = make_uint4(o2[0], o2[1], o2[2], o2[3]);
}

// =====================================================================================
// Layout converters (once per weight; clarity over speed).
// =====================================================================================
// [K, I] gate + [K, I] up -> [K, 2I] with column 2i = gate_i, 2i + 1 = up_i.
__global__ void interleave_words_kernel(const uint32_t *__restrict__ g, const uint32_t *__restrict__ u,
                                        uint32_t *__restrict__ out, int rows, int nb_out) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)rows * nb_out) return;
    const int j = (int)(idx % nb_out);
    const size_t r = idx / nb_out;
    const int nb_in = nb_out >> 1;
    const uint32_t gw = g[r * nb_in + (j >> 1)], uw = u[r * nb_in + (j >> 1)];
    uint32_t o = 0;
#pragma unroll
    for (int m = 0; m < 4; ++m) {
        const int src = 4 * (j & 1) + m;
        o |= awq_nibble(gw, src) << awq_shift_of_column(2 * m);
        o |= awq_nibble(uw, src) << awq_shift_of_column(2 * m + 1);
    }
    out[idx] = o;
}

__global__ void interleave_scales_kernel(const uint16_t *__restrict__ g, const uint16_t *__restrict__ u,
                                         uint16_t *__restrict__ out, int rows, int I) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)rows * I) return;
    const size_t r = idx / I;
    const int i = (int)(idx % I);
    out[r * 2 * I + 2 * i] = g[idx];
    out[r * 2 * I + 2 * i + 1] = u[idx];
}

// Layout B -> A words: word (k, j) gathers nibble k of rows 8j .. 8j+7 of A_q.
__global__ void repack_B_to_A_q_kernel(const uint8_t *__restrict__ A_q, uint32_t *__restrict__ qweight,
                                       int M, int K) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int nb = M >> 3;
    if (idx >= (size_t)K * nb) return;
    const int j = (int)(idx % nb);
    const int k = (int)(idx / nb);
    uint32_t o = 0;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const uint32_t byte = A_q[(size_t)(8 * j + c) * (K >> 1) + (k >> 1)];
        o |= ((byte >> (4 * (k & 1))) & 0xFu) << awq_shift_of_column(c);
    }
    qweight[idx] = o;
}

__global__ void repack_B_to_A_z_kernel(const uint8_t *__restrict__ A_z, uint32_t *__restrict__ qzeros,
                                       int M, int G) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int nb = M >> 3;
    if (idx >= (size_t)G * nb) return;
    const int j = (int)(idx % nb);
    const size_t g = idx / nb;
    uint32_t o = 0;
#pragma unroll
    for (int c = 0; c < 8; ++c) o |= ((uint32_t)A_z[g * M + 8 * j + c] & 0xFu) << awq_shift_of_column(c);
    qzeros[idx] = o;
}

__global__ void repack_A_to_B_q_kernel(const uint32_t *__restrict__ qweight, uint8_t *__restrict__ A_q,
                                       int M, int K) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int kh = K >> 1;
    if (idx >= (size_t)M * kh) return;
    const int k2 = (int)(idx % kh);
    const int n = (int)(idx / kh);
    const int nb = M >> 3;
    const uint32_t w0 = qweight[(size_t)(2 * k2) * nb + (n >> 3)];
    const uint32_t w1 = qweight[(size_t)(2 * k2 + 1) * nb + (n >> 3)];
    A_q[idx] = (uint8_t)(awq_nibble(w0, n & 7) | (awq_nibble(w1, n & 7) << 4));
}

__global__ void repack_A_to_B_z_kernel(const uint32_t *__restrict__ qzeros, uint8_t *__restrict__ A_z,
                                       int M, int G) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)G * M) return;
    const int n = (int)(idx % M);
    const size_t g = idx / M;
    A_z[idx] = (uint8_t)awq_nibble(qzeros[g * (M >> 3) + (n >> 3)], n & 7);
}

// =====================================================================================
// bf16 sibling path (un-quantised weights): y[M, N] = x[M, K] @ W[N, K]^T, one warp per output
// column, lanes stride over K with 16-byte loads, f32 accumulate, shuffle reduction.
// =====================================================================================
constexpr int LB_ROWS = 8;  // activation rows per pass

__global__ void __launch_bounds__(256)
linear_bf16_kernel(const uint16_t *__restrict__ x, const uint16_t *__restrict__ W, uint16_t *__restrict__ y,
                   int M, int K, int N) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + warp;
    const int m0 = blockIdx.y * LB_ROWS;
    if (n >= N) return;
    float acc[LB_ROWS];
#pragma unroll
    for (int r = 0; r < LB_ROWS; ++r) acc[r] = 0.f;
    for (int k = lane * 8; k < K; k += 256) {
        const uint4 wv = *reinterpret_cast<const uint4 *>(W + (size_t)n * K + k);
        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int r = 0; r < LB_ROWS; ++r) {
            if (m0 + r >= M) break;
            const uint4 xv = *reinterpret_cast<const uint4 *>(x + (size_t)(m0 + r) * K + k);
            const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                acc[r] = fmaf(bf16x2_lo(ww[e]), bf16x2_lo(xw[e]), acc[r]);
                acc[r] = fmaf(bf16x2_hi(ww[e]), bf16x2_hi(xw[e]), acc[r]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < LB_ROWS; ++r) {
        float v = acc[r];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0 && m0 + r < M) y[(size_t)(m0 + r) * N + n] = f32_to_bf16_bits(v);
    }
}

// The same product on the tensor cores, for more than a few rows (the GEMMs of the bf16 prefill FFN,
// ffn_swiglu/prefill/ffn_kernels.cc:55-83): y[M, N] = x[M, K] @ W[N, K]^T, both operands K-major, so
// x tiles are the A fragments and W tiles the B fragments of mma.sync.m16n8k16 as they lie.  64 x 64
// output tile per CTA, four warps of 32 x 32, K in steps of 32 through a two-stage cp.async ring; rows
// are padded to 80 bytes so that ldmatrix reads are free of bank conflicts.  A sibling path: it is
// not tuned beyond that.
constexpr int LT_BM = 64, LT_BN = 64, LT_BK = 32, LT_LD = LT_BK + 8;

__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void *src, bool valid) {
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}

__global__ void __launch_bounds__(128)
linear_bf16_tc_kernel(const uint16_t *__restrict__ x, const uint16_t *__restrict__ W, uint16_t *__restrict__ y, int M,
                      int K, int N) {
    __shared__ __align__(16) uint16_t As[2][LT_BM][LT_LD];
    __shared__ __align__(16) uint16_t Bs[2][LT_BN][LT_LD];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wm = warp >> 1, wn = warp & 1;
    const int m0 = blockIdx.y * LT_BM, n0 = blockIdx.x * LT_BN;
    const int n_kt = (K + LT_BK - 1) / LT_BK;

    auto issue = [&](int kt, int buf) {
        // 64 rows x four 16-byte chunks per matrix: two chunks of each per thread; rows and k beyond the
        // matrices are filled with zeros
#pragma unroll
        for (int c = threadIdx.x; c < LT_BM * 4; c += 128) {
            const int r = c >> 2, k = kt * LT_BK + (c & 3) * 8;
            const bool va = m0 + r < M && k < K, vb = n0 + r < N && k < K;
            cp_async16_zfill(smem_u32(&As[buf][r][(c & 3) * 8]), va ? x + (size_t)(m0 + r) * K + k : x, va);
            cp_async16_zfill(smem_u32(&Bs[buf][r][(c & 3) * 8]), vb ? W + (size_t)(n0 + r) * K + k : W, vb);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    float acc[2][4][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;

    issue(0, 0);
    for (int kt = 0; kt < n_kt; ++kt) {
        const int buf = kt & 1;
        if (kt + 1 < n_kt) {
            issue(kt + 1, buf ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < LT_BK; ks += 16) {
            uint32_t af[2][4], bfr[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i)
                ldmatrix_x4(af[i], smem_u32(&As[buf][wm * 32 + i * 16 + (lane & 15)][ks + (lane >> 4) * 8]));
#pragma unroll
            for (int j = 0; j < 2; ++j)  // two n-tiles of 8 per ldmatrix: {b0, b1} of tile 2j, then of tile 2j + 1
                ldmatrix_x4(bfr[j], smem_u32(&Bs[buf][wn * 32 + j * 16 + (lane & 7) + ((lane >> 4) << 3)][ks + ((lane >> 3) & 1) * 8]));
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    mma_bf16_16816(acc[i][j], af[i][0], af[i][1], af[i][2], af[i][3], bfr[j >> 1][(j & 1) * 2], bfr[j >> 1][(j & 1) * 2 + 1]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int m = m0 + wm * 32 + i * 16 + (lane >> 2) + 8 * h, n = n0 + wn * 32 + j * 8 + 2 * (lane & 3);
                if (m >= M) continue;
                if (n < N) y[(size_t)m * N + n] = f32_to_bf16_bits(acc[i][j][2 * h]);
                if (n + 1 < N) y[(size_t)m * N + n + 1] = f32_to_bf16_bits(acc[i][j][2 * h + 1]);
            }
}

// out = bf16(g * sigmoid(g) * u) in f32: the golden form of ffn_swiglu/decode/ffn_decode.py:309-311.
__global__ void silu_mul_bf16_kernel(const uint16_t *__restrict__ gate, const uint16_t *__restrict__ up,
                                     uint16_t *__restrict__ out, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float g = bf16_bits_to_f32(gate[i]), u = bf16_bits_to_f32(up[i]);
    out[i] = f32_to_bf16_bits(g * (1.0f / (1.0f + expf(-g))) * u);
}

// Per-tile packed buffer (the reference's NPU layout: matvec_int4_packed.py:57-103,
// matmul_int4_packed.py:57-86) -> logical layout B.  Tiles are ordered (row block, k chunk); a tile is
// [Q: m_tile x k_chunk/2 bytes | S: n_gpc x m_tile bf16 | Z: n_gpc x m_tile bytes], n_gpc = k_chunk / gs.
// One thread per output byte of A_q, then per (group, row) entry of A_s / A_z.
__global__ void repack_C_to_B_q_kernel(const uint8_t *__restrict__ packed, uint8_t *__restrict__ A_q, int M, int K,
                                       int m_tile, int k_chunk, int tile_bytes) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int kb = K / 2, cb = k_chunk / 2;
    if (idx >= (size_t)M * kb) return;
    const int m = (int)(idx / kb), j = (int)(idx % kb);
    const size_t tile = (size_t)(m / m_tile) * (K / k_chunk) + j / cb;
    A_q[idx] = packed[tile * tile_bytes + (size_t)(m % m_tile) * cb + j % cb];
}
__global__ void repack_C_to_B_sz_kernel(const uint8_t *__restrict__ packed, uint16_t *__restrict__ A_s,
                                        uint8_t *__restrict__ A_z, int M, int K, int gs, int m_tile, int k_chunk,
                                        int tile_bytes) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int G = K / gs, n_gpc = k_chunk / gs;
    if (idx >= (size_t)G * M) return;
    const int g = (int)(idx / M), m = (int)(idx % M);
    const size_t tile = (size_t)(m / m_tile) * (K / k_chunk) + g / n_gpc;
    const uint8_t *t = packed + tile * tile_bytes;
    const int q_bytes = m_tile * (k_chunk / 2), e = (g % n_gpc) * m_tile + m % m_tile;
    A_s[idx] = (uint16_t)t[q_bytes + 2 * e] | ((uint16_t)t[q_bytes + 2 * e + 1] << 8);
    A_z[idx] = t[q_bytes + 2 * n_gpc * m_tile + e];
}

static inline unsigned blocks_for(size_t n, int threads) { return (unsigned)((n + threads - 1) / threads); }

int launch_tp_reduce_add_rmsnorm(const uint16_t *h, const PeerPartials &parts, unsigned int *flags, int expected,
                                 const uint16_t *gamma, float eps, uint16_t *h_out, uint16_t *normed, int normed_f16, int B,
                                 int K, int *err_flag, cudaStream_t stream) {
    return check_cuda(launch_pdl(tp_reduce_add_rmsnorm_kernel, dim3(B), dim3(RN_THREADS), 0, stream, h, parts, flags,
                                 (unsigned int)expected, gamma, eps, h_out, normed, K, normed_f16, err_flag, wait_limit_cycles()),
                      "tp_reduce_add_rmsnorm launch");
}

}  // namespace awq

using namespace awq;

extern "C" int awq_b200_rmsnorm_act(const uint16_t *x, const uint16_t *gamma, float eps, void *out, int out_format,
                                    int B, int K, awq_stream_t stream) {
    AWQ_REQUIRE(B >= 0 && K > 0, "rmsnorm: bad size");
    AWQ_REQUIRE(K % 8 == 0 && K <= RN_THREADS * RN_CHUNKS * 8, "rmsnorm: K (%d) must be a multiple of 8, at most %d", K, RN_THREADS * RN_CHUNKS * 8);
    AWQ_REQUIRE(aligned16(x) && aligned16(gamma) && aligned16(out), "rmsnorm: pointers must be 16-byte aligned");
    AWQ_REQUIRE(out_format == ACT_BF16 || out_format == ACT_F16, "rmsnorm: unknown output format %d", out_format);
    if (B == 0) return AWQ_OK;
    AWQ_REQUIRE(x && gamma && out, "rmsnorm: null pointer");
    return check_cuda(launch_pdl(rmsnorm_kernel, dim3(B), dim3(256), 0, as_stream(stream), x, (const float *)nullptr,
                                 gamma, eps, (uint16_t *)nullptr, reinterpret_cast<uint16_t *>(out), K,
                                 out_format == ACT_F16 ? 1 : 0),
                      "rmsnorm launch");
}

extern "C" int awq_b200_rmsnorm_bf16(const uint16_t *x, const uint16_t *gamma, float eps, uint16_t *out,
                                     int B, int K, awq_stream_t stream) {
    return awq_b200_rmsnorm_act(x, gamma, eps, out, ACT_BF16, B, K, stream);
}

extern "C" int awq_b200_add_rmsnorm_bf16(const uint16_t *h, const float *partial_sum, const uint16_t *gamma,
                                         float eps, uint16_t *h_out, uint16_t *normed, int B, int K,
                                         awq_stream_t stream) {
    return awq_b200_add_rmsnorm_act(h, partial_sum, gamma, eps, h_out, normed, ACT_BF16, B, K, stream);
}

extern "C" int awq_b200_add_rmsnorm_act(const uint16_t *h, const float *partial_sum, const uint16_t *gamma,
                                        float eps, uint16_t *h_out, void *normed, int normed_format, int B, int K,
                                        awq_stream_t stream) {
    AWQ_REQUIRE(B >= 0 && K > 0, "add_rmsnorm: bad size");
    AWQ_REQUIRE(K % 8 == 0 && K <= RN_THREADS * RN_CHUNKS * 8, "add_rmsnorm: K (%d) must be a multiple of 8, at most %d", K, RN_THREADS * RN_CHUNKS * 8);
    AWQ_REQUIRE(aligned16(h) && aligned16(partial_sum) && aligned16(h_out) && aligned16(normed) && aligned16(gamma), "add_rmsnorm: pointers must be 16-byte aligned");
    AWQ_REQUIRE(normed_format == ACT_BF16 || normed_format == ACT_F16, "add_rmsnorm: unknown format %d", normed_format);
    if (B == 0) return AWQ_OK;
    AWQ_REQUIRE(h && partial_sum && h_out, "add_rmsnorm: null pointer");
    AWQ_REQUIRE((gamma == nullptr) == (normed == nullptr), "add_rmsnorm: gamma and normed go together");
    AWQ_REQUIRE(h_out != h, "add_rmsnorm: h_out must not alias h");
    return check_cuda(launch_pdl(rmsnorm_kernel, dim3(B), dim3(256), 0, as_stream(stream), h, partial_sum, gamma, eps,
                                 h_out, reinterpret_cast<uint16_t *>(normed), K, normed_format == ACT_F16 ? 1 : 0),
                      "add_rmsnorm launch");
}

extern "C" int awq_b200_tp_reduce_add_rmsnorm_act(const uint16_t *h, const void *const *peer_partials, uint32_t *flags, int n_ranks,
                                                  const uint16_t *gamma, float eps, uint16_t *h_out, void *normed,
                                                  int normed_format, int B, int K, void *workspace, awq_stream_t stream) {
    AWQ_REQUIRE(B >= 0 && B <= 8 && K > 0, "tp_reduce_add_rmsnorm: B must be 0..8");
    AWQ_REQUIRE(n_ranks >= 1 && n_ranks <= TP_MAX_RANKS, "tp_reduce_add_rmsnorm: 1..%d ranks", TP_MAX_RANKS);
    AWQ_REQUIRE(K % 8 == 0 && K <= RN_THREADS * RN_CHUNKS * 8, "tp_reduce_add_rmsnorm: K (%d) must be a multiple of 8, at most %d", K, RN_THREADS * RN_CHUNKS * 8);
    AWQ_REQUIRE(normed_format == ACT_BF16 || normed_format == ACT_F16, "tp_reduce_add_rmsnorm: unknown format %d", normed_format);
    if (B == 0) return AWQ_OK;
    AWQ_REQUIRE(h && peer_partials && flags && h_out && workspace, "tp_reduce_add_rmsnorm: null pointer");
    PeerPartials parts{};
    parts.n = n_ranks;
    for (int r = 0; r < n_ranks; ++r) {
        AWQ_REQUIRE(peer_partials[r] && aligned16(peer_partials[r]), "tp_reduce_add_rmsnorm: bad partial pointer of rank %d", r);
        parts.partial[r] = reinterpret_cast<const float *>(peer_partials[r]);
    }
    AWQ_REQUIRE((gamma == nullptr) == (normed == nullptr), "tp_reduce_add_rmsnorm: gamma and normed go together");
    AWQ_REQUIRE(aligned16(h) && aligned16(h_out) && aligned16(normed) && aligned16(gamma), "tp_reduce_add_rmsnorm: pointers must be 16-byte aligned");
    AWQ_REQUIRE(h_out != h, "tp_reduce_add_rmsnorm: h_out must not alias h");
    return launch_tp_reduce_add_rmsnorm(h, parts, flags, gemv_push_arrivals_per_rank(K), gamma, eps, h_out,
                                        reinterpret_cast<uint16_t *>(normed), normed_format == ACT_F16 ? 1 : 0, B, K,
                                        reinterpret_cast<int *>(workspace), as_stream(stream));
}

extern "C" int awq_b200_rope_halfsplit_bf16(const uint16_t *x, size_t x_stride, const uint16_t *lut, uint16_t *out,
                                            size_t out_stride, int B, int n_heads, int head_dim, awq_stream_t stream) {
    AWQ_REQUIRE(B >= 0 && n_heads >= 0 && head_dim > 0, "rope: bad size");
    AWQ_REQUIRE(head_dim % 16 == 0, "rope: head_dim (%d) must be a multiple of 16", head_dim);
    if (B == 0 || n_heads == 0) return AWQ_OK;
    AWQ_REQUIRE(x && lut && out, "rope: null pointer");
    AWQ_REQUIRE(x_stride >= (size_t)n_heads * head_dim && out_stride >= (size_t)n_heads * head_dim, "rope: row stride too small");
    AWQ_REQUIRE(aligned16(x) && aligned16(lut) && aligned16(out) && x_stride % 8 == 0 && out_stride % 8 == 0,
                "rope: pointers and row strides must be 16-byte aligned");
    const size_t total = (size_t)B * n_heads * (head_dim / 16);
    rope_halfsplit_kernel<<<blocks_for(total, 256), 256, 0, as_stream(stream)>>>(x, x_stride, lut, out, out_stride, B, n_heads,
                                                                                  head_dim);
    return check_cuda(cudaGetLastError(), "rope launch");
}

extern "C" int awq_b200_linear_bf16(const uint16_t *x, const uint16_t *W, uint16_t *y, int M, int K, int N,
                                    awq_stream_t stream) {
    AWQ_REQUIRE(M >= 0 && K > 0 && N >= 0, "linear_bf16: bad size");
    AWQ_REQUIRE(K % 8 == 0, "linear_bf16: K (%d) must be a multiple of 8", K);
    if (M == 0 || N == 0) return AWQ_OK;
    AWQ_REQUIRE(x && W && y, "linear_bf16: null pointer");
    AWQ_REQUIRE(aligned16(x) && aligned16(W), "linear_bf16: x and W must be 16-byte aligned");
    if (M >= 16) {  // a GEMM: tensor cores
        dim3 tgrid((N + LT_BN - 1) / LT_BN, (M + LT_BM - 1) / LT_BM);
        AWQ_REQUIRE(tgrid.y <= 65535u, "linear_bf16: M (%d) too large", M);
        linear_bf16_tc_kernel<<<tgrid, 128, 0, as_stream(stream)>>>(x, W, y, M, K, N);
        return check_cuda(cudaGetLastError(), "linear_bf16 launch");
    }
    dim3 grid((N + 7) / 8, (M + LB_ROWS - 1) / LB_ROWS);
    linear_bf16_kernel<<<grid, 256, 0, as_stream(stream)>>>(x, W, y, M, K, N);
    return check_cuda(cudaGetLastError(), "linear_bf16 launch");
}

extern "C" int awq_b200_silu_mul_bf16(const uint16_t *gate, const uint16_t *up, uint16_t *out, size_t n,
                                      awq_stream_t stream) {
    if (n == 0) return AWQ_OK;
    AWQ_REQUIRE(gate && up && out, "silu_mul_bf16: null pointer");
    silu_mul_bf16_kernel<<<blocks_for(n, 256), 256, 0, as_stream(stream)>>>(gate, up, out, n);
    return check_cuda(cudaGetLastError(), "silu_mul_bf16 launch");
}

extern "C" int awq_b200_interleave_gate_up(const int32_t *qw_gate, const int32_t *qz_gate,
                                           const uint16_t *s_gate, const int32_t *qw_up,
                                           const int32_t *qz_up, const uint16_t *s_up, int32_t *qweight,
                                           int32_t *qzeros, uint16_t *scales, int K, int I, int group_size,
                                           awq_stream_t stream) {
    AWQ_REQUIRE(K > 0 && I > 0 && group_size > 0 && K % group_size == 0, "interleave: bad size");
    AWQ_REQUIRE(I % 8 == 0, "interleave: I (%d) must be a multiple of 8", I);
    AWQ_REQUIRE(qw_gate && qz_gate && s_gate && qw_up && qz_up && s_up && qweight && qzeros && scales,
                "interleave: null pointer");
    const int G = K / group_size, nb_out = 2 * I / 8;
    cudaStream_t st = as_stream(stream);
    interleave_words_kernel<<<blocks_for((size_t)K * nb_out, 256), 256, 0, st>>>(
        (const uint32_t *)qw_gate, (const uint32_t *)qw_up, (uint32_t *)qweight, K, nb_out);
    interleave_words_kernel<<<blocks_for((size_t)G * nb_out, 256), 256, 0, st>>>(
        (const uint32_t *)qz_gate, (const uint32_t *)qz_up, (uint32_t *)qzeros, G, nb_out);
    interleave_scales_kernel<<<blocks_for((size_t)G * I, 256), 256, 0, st>>>(s_gate, s_up, scales, G, I);
    return check_cuda(cudaGetLastError(), "interleave launch");
}

extern "C" int awq_b200_repack_B_to_A(const uint8_t *A_q, const uint16_t *A_s, const uint8_t *A_z,
                                      int32_t *qweight, int32_t *qzeros, uint16_t *scales, int M, int K,
                                      int group_size, awq_stream_t stream) {
    AWQ_REQUIRE(M > 0 && K > 0 && group_size > 0, "repack_B_to_A: bad size");
    AWQ_REQUIRE(M % 8 == 0 && K % 2 == 0 && K % group_size == 0, "repack_B_to_A: M %% 8, K %% 2, K %% gs");
    AWQ_REQUIRE(A_q && A_s && A_z && qweight && qzeros && scales, "repack_B_to_A: null pointer");
    const int G = K / group_size;
    cudaStream_t st = as_stream(stream);
    repack_B_to_A_q_kernel<<<blocks_for((size_t)K * (M / 8), 256), 256, 0, st>>>(A_q, (uint32_t *)qweight, M, K);
    repack_B_to_A_z_kernel<<<blocks_for((size_t)G * (M / 8), 256), 256, 0, st>>>(A_z, (uint32_t *)qzeros, M, G);
    int rc = check_cuda(cudaMemcpyAsync(scales, A_s, (size_t)G * M * 2, cudaMemcpyDeviceToDevice, st),
                        "repack scales copy");
    if (rc) return rc;
    return check_cuda(cudaGetLastError(), "repack_B_to_A launch");
}

extern "C" int awq_b200_repack_A_to_B(const int32_t *qweight, const int32_t *qzeros, const uint16_t *scales,
                                      uint8_t *A_q, uint16_t *A_s, uint8_t *A_z, int M, int K, int group_size,
                                      awq_stream_t stream) {
    AWQ_REQUIRE(M > 0 && K > 0 && group_size > 0, "repack_A_to_B: bad size");
    AWQ_REQUIRE(M % 8 == 0 && K % 2 == 0 && K % group_size == 0, "repack_A_to_B: M %% 8, K %% 2, K %% gs");
    AWQ_REQUIRE(A_q && A_s && A_z && qweight && qzeros && scales, "repack_A_to_B: null pointer");
    const int G = K / group_size;
    cudaStream_t st = as_stream(stream);
    repack_A_to_B_q_kernel<<<blocks_for((size_t)M * (K / 2), 256), 256, 0, st>>>((const uint32_t *)qweight, A_q, M, K);
    repack_A_to_B_z_kernel<<<blocks_for((size_t)G * M, 256), 256, 0, st>>>((const uint32_t *)qzeros, A_z, M, G);
    int rc = check_cuda(cudaMemcpyAsync(A_s, scales, (size_t)G * M * 2, cudaMemcpyDeviceToDevice, st),
                        "repack scales copy");
    if (rc) return rc;
    return check_cuda(cudaGetLastError(), "repack_A_to_B launch");
}

extern "C" int awq_b200_repack_C_to_B(const uint8_t *packed, uint8_t *A_q, uint16_t *A_s, uint8_t *A_z, int M, int K,
                                      int group_size, int m_tile, int k_chunk, awq_stream_t stream) {
    AWQ_REQUIRE(M > 0 && K > 0 && group_size > 0 && m_tile > 0 && k_chunk > 0, "repack_C_to_B: bad size");
    AWQ_REQUIRE(M % m_tile == 0 && K % k_chunk == 0 && k_chunk % group_size == 0 && k_chunk % 2 == 0,
                "repack_C_to_B: M %% m_tile, K %% k_chunk, k_chunk %% group_size (M=%d K=%d m_tile=%d k_chunk=%d gs=%d)", M, K,
                m_tile, k_chunk, group_size);
    AWQ_REQUIRE(packed && A_q && A_s && A_z, "repack_C_to_B: null pointer");
    const int n_gpc = k_chunk / group_size, G = K / group_size;
    const int tile_bytes = m_tile * (k_chunk / 2) + 3 * n_gpc * m_tile;
    cudaStream_t st = as_stream(stream);
    repack_C_to_B_q_kernel<<<blocks_for((size_t)M * (K / 2), 256), 256, 0, st>>>(packed, A_q, M, K, m_tile, k_chunk, tile_bytes);
    repack_C_to_B_sz_kernel<<<blocks_for((size_t)G * M, 256), 256, 0, st>>>(packed, A_s, A_z, M, K, group_size, m_tile, k_chunk,
                                                                          tile_bytes);
    return check_cuda(cudaGetLastError(), "repack_C_to_B launch");
}
