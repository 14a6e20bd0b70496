// Shared helpers for the int4-AWQ kernels: error plumbing, bf16 bit tricks, nibble unpack.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "awq_b200.h"

namespace awq {

// ---- host-side error plumbing -------------------------------------------------------
int set_error(int code, const char *fmt, ...);
int check_cuda(cudaError_t e, const char *what);
inline cudaStream_t as_stream(awq_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }
inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
int status_of_device_flag(int flag);  // error word of a kernel's scratch -> status + message
long long wait_limit_cycles();  // limit of every bounded device-side wait (awq_b200_set_wait_limit)
int device_sm_count();
bool device_is_sm100();

// Launch `kernel` so that it may overlap the tail of the previous kernel in `stream`
// (programmatic dependent launch); the kernel must call pdl_wait() before touching anything the
// previous kernel wrote or read.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

#define AWQ_REQUIRE(cond, ...)                                        \
    do {                                                              \
        if (!(cond)) return awq::set_error(AWQ_ERR_INVALID_ARGUMENT, __VA_ARGS__); \
    } while (0)

// ---- layout-A nibble order ------------------------------------------------------------
// Bits [4i+3:4i] of a packed word hold column ORDER[i] = {0,2,4,6,1,3,5,7}[i]; column c
// therefore sits at shift 4 * PERM[c], PERM = {0,4,1,5,2,6,3,7}.
__host__ __device__ __forceinline__ constexpr int awq_shift_of_column(int c) {
    return 4 * (((c & 1) << 2) | (c >> 1));
}
__host__ __device__ __forceinline__ uint32_t awq_nibble(uint32_t word, int c) {
    return (word >> awq_shift_of_column(c)) & 0xFu;
}

// ---- bf16 helpers ------------------------------------------------------------------------
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t lo16) { return __uint_as_float(lo16 << 16); }
__device__ __forceinline__ float bf16x2_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16x2_hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float f) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    return (uint32_t)f32_to_bf16_bits(lo) | ((uint32_t)f32_to_bf16_bits(hi) << 16);
}

// (v & 0x000f000f) | 0x43004300: two nibbles (bits 0-3 and 16-19) become the bf16 pair
// (128 + n_lo, 128 + n_hi): 0x4300 is 128.0 and its ulp is 1.
__device__ __forceinline__ uint32_t nib2_to_bf16x2_biased(uint32_t v) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(v), "r"(0x000F000Fu), "r"(0x43004300u));
    return r;
}

// silu(g) = g * 0.5 * (tanh(g / 2) + 1), the form of matvec_int4_swiglu_rms.py:515.
__device__ __forceinline__ float silu_tanh(float g) { return g * 0.5f * (tanhf(g * 0.5f) + 1.0f); }

// gate/up f32 sums -> bf16 -> silu * up -> bf16 bits (rounding points of
// matvec_int4_swiglu_rms.py:512-516).
__device__ __forceinline__ uint16_t swiglu_bits(float gate_sum, float up_sum) {
    float g = __bfloat162float(__float2bfloat16_rn(gate_sum));
    float u = __bfloat162float(__float2bfloat16_rn(up_sum));
    return f32_to_bf16_bits(silu_tanh(g) * u);
}

enum Epilogue : int {
    EPI_BF16 = 0,    // y bf16 [B, N] = bf16(sum (+ residual))
    EPI_F32 = 1,     // y f32  [B, N] = sum
    EPI_SWIGLU = 2,  // y bf16 [B, N/2] = swiglu(sum[2i], sum[2i+1])
    EPI_F32_PUSH = 3,  // EPI_F32 into this rank's send buffer, then every tensor-parallel rank is signalled
};

// Tensor-parallel hand-over through peer memory.  A rank writes its f32 partial [B, N] into its own
// send buffer and adds 1 per finished sub-strip to entry `rank` of every rank's arrival counters
// (flag[r]: uint32 words on rank r, mapped into this GPU's address space); the receivers read the
// partials with peer loads.
constexpr int TP_MAX_RANKS = 8;
struct PeerPush {
    unsigned int *flag[TP_MAX_RANKS];
    int n, rank;
};
struct PeerPartials {
    const float *partial[TP_MAX_RANKS];  // rank r's send buffer [B, K], mapped into this GPU's address space
    int n;
};

// 16-bit activation formats.  The stream-K kernel's fastest path wants fp16 activations (an fp16
// significand holds two nibbles, so one shift serves four nibbles); bf16 inputs are converted once.
enum ActFormat : int { ACT_BF16 = 0, ACT_F16 = 1 };

struct GemvArgs {
    const uint16_t *x;
    const int32_t *qweight;
    const int32_t *qzeros;
    const uint16_t *scales;
    const uint16_t *residual;  // EPI_BF16 only, may be null
    void *y;
    int B, K, N, group_size;
    int epilogue;
    void *workspace;
    size_t workspace_bytes;
    cudaStream_t stream;
    int x_format = ACT_BF16;    // format of x
    int out_format = ACT_BF16;  // EPI_SWIGLU only: format of the output
    bool native_bf16 = false;   // stream-K: multiply bf16 activations as they are (no fp16 conversion)
    bool deterministic = false; // stream-K: sum split-K partials in a fixed order (slower) instead of f32 atomics
    const PeerPush *push = nullptr;  // EPI_F32_PUSH only
};

// Generic CUDA-core kernel: any group size, any N % 8 == 0, B <= 64.
int launch_gemv_generic(const GemvArgs &a);
// TMA + mma.sync stream-K kernel: group 128, N % 32 == 0, K % 128 == 0, B <= 8.
bool gemv_streamk_supported(const GemvArgs &a);
int launch_gemv_streamk(const GemvArgs &a);
bool gemv_streamk_mb_supported(const GemvArgs &a, int B);  // multi-row pass (9..32 rows, awq_gemv_streamk_mb.cu)
int launch_gemv_streamk_mb(const GemvArgs &a, const uint16_t *x, const uint16_t *residual, void *y, int B);
size_t gemv_streamk_scratch_bytes(int N, bool deterministic);  // counters + split-K accumulators / partial slots
size_t gemv_streamk_workspace_bytes(int B, int K, int N);  // + room to convert B rows of x to fp16
size_t gemv_streamk_workspace_clear_bytes(int N);

int launch_gemm_generic(const uint16_t *A, const int32_t *qweight, const int32_t *qzeros,
                        const uint16_t *scales, uint16_t *C, int M, int K, int N, int group_size,
                        cudaStream_t stream);
bool gemm_tc_supported(int M, int K, int N, int group_size);
// Epilogues of the tensor-core GEMM: C bf16 [M, N] = bf16(sum (+ residual)), or SwiGLU over interleaved
// gate/up column pairs into C bf16 [M, N / 2].
enum GemmEpilogue : int { GEMM_EPI_BF16 = 0, GEMM_EPI_RESIDUAL = 1, GEMM_EPI_SWIGLU = 2, GEMM_EPI_F32 = 3 };  // F32: the f32 sums as they are (batched-decode GEMM only)
int launch_gemm_tc(const uint16_t *A, const int32_t *qweight, const int32_t *qzeros,
                   const uint16_t *scales, uint16_t *C, int M, int K, int N, int group_size,
                   cudaStream_t stream, int epilogue = GEMM_EPI_BF16, const uint16_t *residual = nullptr);

int gemm_tc_check(cudaStream_t stream);
// The same GEMM with the dequantised weights in tensor memory (operands swapped: weights are the MMA's M side).
bool gemm_tm_supported(int M, int K, int N, int group_size);
int launch_gemm_tm(const uint16_t *A, const int32_t *qweight, const int32_t *qzeros, const uint16_t *scales, uint16_t *C, int M, int K,
                   int N, cudaStream_t stream, int epilogue = GEMM_EPI_BF16, const uint16_t *residual = nullptr);
int gemm_tm_check(cudaStream_t stream);
// Batched-decode GEMM (M <= 128 token rows): stream-K over (column tile, k-block) units, split-K partials through `workspace`.
bool gemm_decode_supported(int M, int K, int N, int group_size);
size_t gemm_decode_workspace_bytes(int M, int N);
int launch_gemm_decode(const uint16_t *A, const int32_t *qweight, const int32_t *qzeros, const uint16_t *scales, uint16_t *C, int M,
                       int K, int N, cudaStream_t stream, int epilogue, const uint16_t *residual, void *workspace,
                       size_t workspace_bytes, int a_f16 = 0, int c_f16 = 0);  // fp16 token rows / fp16 output (not with a residual)
int gemm_decode_check(cudaStream_t stream);
// The same product for up to 32 token rows with the nibbles and the split token rows as fp8 operands (awq_gemm_decode_f8.cu);
// its workspace holds the split rows as well, hence K.
bool gemm_decode_f8_supported(int M, int K, int N, int group_size);
size_t gemm_decode_f8_workspace_bytes(int M, int K, int N);
int launch_gemm_decode_f8(const uint16_t *A, int a_f16, const int32_t *qweight, const int32_t *qzeros, const uint16_t *scales,
                          uint16_t *C, int M, int K, int N, cudaStream_t stream, int epilogue, const uint16_t *residual, int c_f16,
                          void *workspace, size_t workspace_bytes);
int gemm_decode_f8_check(cudaStream_t stream);
int gemv_push_arrivals_per_rank(int N);  // arrivals a rank signals per EPI_F32_PUSH launch of N columns
int launch_tp_reduce_add_rmsnorm(const uint16_t *h, const PeerPartials &parts, unsigned int *flags, int expected,
                                 const uint16_t *gamma, float eps, uint16_t *h_out, uint16_t *normed, int normed_f16, int B,
                                 int K, int *err_flag, cudaStream_t stream);

// Fused decode FFN stack (awq_ffn_fused.cu)
size_t ffn_fused_plan_bytes(int n_layers);
void ffn_fused_set_lookahead(int units);
void ffn_fused_set_split(int per_1024);
size_t ffn_fused_workspace_bytes(int n_layers);
size_t ffn_fused_tp_slot_bytes(int H, int n_ranks);
bool ffn_fused_supported(int B, int H, int I, int group_size);
int ffn_fused_plan(void *plan_dev, size_t plan_bytes, int n_layers, const int32_t *const *qw_gateup,
                   const int32_t *const *qz_gateup, const uint16_t *const *s_gateup, const int32_t *const *qw_down,
                   const int32_t *const *qz_down, const uint16_t *const *s_down, const uint16_t *const *gamma, int H, int I,
                   int group_size);
// Peer-mapped buffers of the tensor-parallel stack kernel: base[r] is rank r's buffer (two slots
// of `slot_stride` bytes: an f32 [8, H] partial, then at `flag_offset` 16 uint32 flag words).
struct FusedPeers {
    void *base[TP_MAX_RANKS];
    size_t slot_stride, flag_offset;
    int n, rank;
};
int launch_ffn_fused(const void *plan_dev, int n_layers, const uint16_t *x, uint16_t *out, uint16_t *inter, float eps, int B,
                     int H, int I, void *workspace, size_t workspace_bytes, cudaStream_t stream,
                     const FusedPeers *peers = nullptr);

}  // namespace awq
