// AWQ int4 -> bf16 dequant (layout A -> dense [K, N]) and the 1-D form of the dequant example.
//
// HBM-bound: 0.52 B read + 2 B written per weight.  One thread owns one packed word column
// (8 output columns) for DQ_ROWS consecutive k.  All of its weight words are requested before
// the first one is used (a 2048 x 2048 weight is a few microseconds of traffic, so what counts is
// how many bytes are in flight, not how few instructions run); the group's zero word and eight
// scales are loaded once per group, each k costs one coalesced 4-byte load and one 16-byte store.
#include "awq_common.cuh"

namespace awq {

constexpr int DQ_ROWS = 8;
constexpr int DQ_THREADS = 128;

// w = bf16_rne(float(q - z) * float(s)); the f32 product is exact, so this is the single
// rounding of awq_repacker.py:80-82.
__global__ void __launch_bounds__(DQ_THREADS)
dequant_kernel(const uint32_t *__restrict__ qweight, const uint32_t *__restrict__ qzeros,
               const uint16_t *__restrict__ scales, uint16_t *__restrict__ out, int K, int N,
               int group_size) {
    const int nb = N >> 3;
    const int j = blockIdx.x * DQ_THREADS + threadIdx.x;  // packed word column
    if (j >= nb) return;
    const int k_begin = blockIdx.y * DQ_ROWS;
    uint32_t qw[DQ_ROWS];
#pragma unroll
    for (int r = 0; r < DQ_ROWS; ++r) qw[r] = k_begin + r < K ? __ldg(qweight + (size_t)(k_begin + r) * nb + j) : 0u;
    int cur_group = -1;
    float s[8];
    int z[8];
#pragma unroll
    for (int r = 0; r < DQ_ROWS; ++r) {
        const int k = k_begin + r;
        if (k >= K) break;
        const int g = k / group_size;
        if (g != cur_group) {  // at most once per thread when DQ_ROWS divides the group size
            cur_group = g;
            const uint32_t zw = __ldg(qzeros + (size_t)g * nb + j);
            const uint4 sv = __ldg(reinterpret_cast<const uint4 *>(scales + (size_t)g * N + 8 * j));
            const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                z[c] = (int)awq_nibble(zw, c);
                s[c] = (c & 1) ? bf16x2_hi(sw[c >> 1]) : bf16x2_lo(sw[c >> 1]);
            }
        }
        uint32_t o[4];
#pragma unroll
        for (int c = 0; c < 8; c += 2) {
            const float w0 = (float)((int)awq_nibble(qw[r], c) - z[c]) * s[c];
            const float w1 = (float)((int)awq_nibble(qw[r], c + 1) - z[c + 1]) * s[c + 1];
            o[c >> 1] = pack_bf16x2(w0, w1);
        }
        *reinterpret_cast<uint4 *>(out + (size_t)k * N + 8 * j) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// out[i] = bf16((nib[i] - zeros[i / gs]) * scales[i / gs]); dequant_awq.py:391-396.
__global__ void dequant_1d_kernel(const uint8_t *__restrict__ packed_q,
                                  const uint16_t *__restrict__ scales,
                                  const uint8_t *__restrict__ zeros, uint16_t *__restrict__ out,
                                  int n, int group_size) {
    const int p = blockIdx.x * blockDim.x + threadIdx.x;  // byte index = nibble pair
    if (2 * p >= n) return;
    const uint32_t byte = packed_q[p];
    const int i0 = 2 * p, i1 = 2 * p + 1;
    const int g0 = i0 / group_size, g1 = i1 / group_size;
    const float w0 = ((float)(byte & 0xF) - (float)zeros[g0]) * bf16_bits_to_f32(scales[g0]);
    out[i0] = f32_to_bf16_bits(w0);
    if (i1 < n) {
        const float w1 = ((float)(byte >> 4) - (float)zeros[g1]) * bf16_bits_to_f32(scales[g1]);
        out[i1] = f32_to_bf16_bits(w1);
    }
}

}  // namespace awq

extern "C" int awq_b200_dequant_bf16(const int32_t *qweight, const int32_t *qzeros,
                                     const uint16_t *scales, uint16_t *out, int K, int N,
                                     int group_size, awq_stream_t stream) {
    using namespace awq;
    AWQ_REQUIRE(K >= 0 && N >= 0 && group_size > 0, "dequant: negative size or group_size <= 0");
    AWQ_REQUIRE(N % 8 == 0, "dequant: N (%d) must be a multiple of 8", N);
    AWQ_REQUIRE(K % group_size == 0, "dequant: K (%d) must be a multiple of group_size (%d)", K, group_size);
    if (K == 0 || N == 0) return AWQ_OK;
    AWQ_REQUIRE(qweight && qzeros && scales && out, "dequant: null pointer");
    AWQ_REQUIRE(aligned16(scales) && aligned16(out), "dequant: scales/out must be 16-byte aligned");
    dim3 grid((N / 8 + DQ_THREADS - 1) / DQ_THREADS, (K + DQ_ROWS - 1) / DQ_ROWS);
    AWQ_REQUIRE(grid.y <= 65535u, "dequant: K (%d) too large", K);
    dequant_kernel<<<grid, DQ_THREADS, 0, as_stream(stream)>>>(
        reinterpret_cast<const uint32_t *>(qweight), reinterpret_cast<const uint32_t *>(qzeros), scales,
        out, K, N, group_size);
    return check_cuda(cudaGetLastError(), "dequant launch");
}

extern "C" int awq_b200_dequant_1d_bf16(const uint8_t *packed_q, const uint16_t *scales,
                                        const uint8_t *zeros, uint16_t *out, int n, int group_size,
                                        awq_stream_t stream) {
    using namespace awq;
    AWQ_REQUIRE(n >= 0 && group_size > 0, "dequant_1d: bad size");
    AWQ_REQUIRE(n % 2 == 0, "dequant_1d: N must be even (2 int4 values per byte)");
    AWQ_REQUIRE(n % group_size == 0, "dequant_1d: N must be divisible by group_size");
    if (n == 0) return AWQ_OK;
    AWQ_REQUIRE(packed_q && scales && zeros && out, "dequant_1d: null pointer");
    const int threads = 256, pairs = n / 2;
    dequant_1d_kernel<<<(pairs + threads - 1) / threads, threads, 0, as_stream(stream)>>>(
        packed_q, scales, zeros, out, n, group_size);
    return check_cuda(cudaGetLastError(), "dequant_1d launch");
}
