// Pieces shared by the batched-decode GEMM kernels (awq_gemm_decode.cu: 16-bit operands; awq_gemm_decode_f8.cu: the
// packed nibbles and split token rows as fp8 operands): the stream-K walk over (tile, k-block) units, the slots the
// partial sums go through, and the second pass that adds them up.
#pragma once

#include <cudaTypedefs.h>
#include <stdint.h>

#include "awq_common.cuh"

namespace awq {

int encode_tensor_map_2d(CUtensorMap *map, int dtype, const void *base, uint64_t dim0, uint64_t dim1,
                         uint64_t stride1_bytes, uint32_t box0, uint32_t box1, int swizzle);
int encode_tensor_map_3d(CUtensorMap *map, int dtype, const void *base, uint64_t dim0, uint64_t dim1, uint64_t dim2,
                         uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0, uint32_t box1, uint32_t box2,
                         int swizzle);

constexpr int DG_BN = 256, DG_BK = 64, DG_GROUP = 128;
constexpr int DG_W_BYTES = DG_GROUP * (DG_BN / 8) * 4;  // 16 KB of packed words: a unit (128 k, one quantisation group)
constexpr int DG_S_BYTES = DG_BN * 2;
constexpr int DG_Z_BYTES = DG_BN / 8 * 4;
constexpr int DG_MAX_TILES = 4096;

// The walk over a CTA's units, the same for every warp role: unit u = tile * KB + kb (KB units of 128 k per tile),
// range [u0, u1).
struct UnitWalk {
    int KB, u, u1;
    __device__ __forceinline__ UnitWalk(int tiles, int kb_count) : KB(kb_count) {
        const long long U = (long long)tiles * kb_count, C = gridDim.x, c = blockIdx.x;
        u = (int)(c * U / C);
        u1 = (int)((c + 1) * U / C);
    }
    __device__ __forceinline__ bool valid() const { return u < u1; }
    __device__ __forceinline__ int tile() const { return u / KB; }
    __device__ __forceinline__ int kb() const { return u - tile() * KB; }
    // units of the current tile that this CTA still has, from u on
    __device__ __forceinline__ int left_in_tile() const {
        const int end = (tile() + 1) * KB;
        return (end < u1 ? end : u1) - u;
    }
};

// The first CTA whose range (UnitWalk) reaches into tile t.
__device__ __forceinline__ int dg_first_cta(int t, int KB, int tiles) {
    const long long U = (long long)tiles * KB, C = gridDim.x;
    return (int)((((long long)t * KB + 1) * C + U - 1) / U) - 1;
}
// Partial sums of a tile in the workspace: slot [contributor][token row m][column of the tile], so that the 32 lanes
// of a warp (columns) touch one 128-byte line.
template <int NB>
__device__ __forceinline__ float *dg_slot_word(float *slots, int slots_per_tile, int tile, int contributor, int m, int col) {
    return slots + (((size_t)tile * slots_per_tile + contributor) * NB + m) * DG_BN + col;
}

int dg_rows(int M);       // token rows the MMA sees: the batch rounded up to 16, 32 or 64
int dg_sm_count();
int dg_slots_per_tile(int tiles);
// The second pass over the slots of a main kernel of `main_ctas` CTAs: sums * sum_scale (* row_scale[m] if given), then the
// epilogue.
int launch_gemm_decode_fixup(int rows, uint16_t *C, const uint16_t *residual, int epilogue, int c_f16, float sum_scale,
                             const float *row_scale, int M, int N, int KB, int tiles, int main_ctas, const float *slots,
                             int slots_per_tile, cudaStream_t stream);

}  // namespace awq
