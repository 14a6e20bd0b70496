// C ABI glue: argument checks, kernel selection, error strings, workspace helpers.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <atomic>

#include "awq_common.cuh"
#include "awq_ptx.cuh"

namespace awq {

static thread_local char g_error[512] = "";
static std::atomic<int> g_decode_mode{0};
static std::atomic<int> g_gemm_mode{0};
static std::atomic<int> g_deterministic{0};
static std::atomic<long long> g_wait_limit{WAIT_LIMIT_DEFAULT};

long long wait_limit_cycles() { return g_wait_limit.load(); }

int set_error(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

int check_cuda(cudaError_t e, const char *what) {
    if (e == cudaSuccess) return AWQ_OK;
    return set_error(AWQ_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

struct DevInfo {
    int sms = -1;
    int major = -1;
};
static DevInfo query_device() {
    static thread_local int cached_dev = -1;
    static thread_local DevInfo cached;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return DevInfo();
    if (dev != cached_dev) {
        DevInfo d;
        if (cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) d.sms = -1;
        if (cudaDeviceGetAttribute(&d.major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) d.major = -1;
        cached = d;
        cached_dev = dev;
    }
    return cached;
}
int device_sm_count() { return query_device().sms; }
bool device_is_sm100() { return query_device().major == 10; }

// The word a kernel leaves in its scratch when it could not finish.
int status_of_device_flag(int flag) {
    if (flag == 4)
        return set_error(AWQ_ERR_UNSUPPORTED,
                         "an activation exceeded the fp16 range (|x| > 65504) and became an infinity; select the bf16 "
                         "activation path with awq_b200_set_decode_kernel(3) and re-initialise the workspace");
    if (flag == 7)
        return set_error(AWQ_ERR_UNSUPPORTED,
                         "a split-K partial sum was NaN, infinite or beyond the range of the fixed-point hand-over "
                         "(|sum| < 8.38e6): the output is not valid; re-initialise the workspace");
    if (flag != 0)
        return set_error(AWQ_ERR_DEVICE_TIMEOUT,
                         "a device-side wait gave up (code %d: 1 = loader waiting for a free stage, 2 = consumer waiting "
                         "for data, 3 = loader waiting for the previous phase, 4 = normaliser waiting for data, 5 = waiting "
                         "for the other ranks' arrival flags, 6 = waiting for the other ranks' partial sums, 8 = waiting for "
                         "another contributor's split-K sums); re-initialise the workspace", flag);
    return AWQ_OK;
}

static int check_gemv_args(const char *who, const GemvArgs &a) {
    AWQ_REQUIRE(a.B >= 0 && a.K >= 0 && a.N >= 0 && a.group_size > 0, "%s: negative size or group_size <= 0", who);
    AWQ_REQUIRE(a.B <= 64, "%s: batch %d exceeds 64 (use the prefill GEMM)", who, a.B);
    AWQ_REQUIRE(a.N % 8 == 0, "%s: N (%d) must be a multiple of 8", who, a.N);
    AWQ_REQUIRE(a.K % a.group_size == 0, "%s: K (%d) must be a multiple of group_size (%d)", who, a.K, a.group_size);
    if (a.B == 0 || a.N == 0) return AWQ_OK;
    AWQ_REQUIRE(a.K > 0, "%s: K must be positive", who);
    AWQ_REQUIRE(a.x && a.qweight && a.qzeros && a.scales && a.y, "%s: null pointer", who);
    AWQ_REQUIRE(aligned16(a.scales), "%s: scales must be 16-byte aligned", who);
    // every kernel stores y (and loads the residual) in 16-byte pieces
    AWQ_REQUIRE(aligned16(a.y), "%s: the output must be 16-byte aligned", who);
    AWQ_REQUIRE(!a.residual || aligned16(a.residual), "%s: the residual must be 16-byte aligned", who);
    return AWQ_OK;
}

static int run_gemv(const char *who, GemvArgs a) {
    int rc = check_gemv_args(who, a);
    if (rc || a.B == 0 || a.N == 0) return rc;
    AWQ_REQUIRE(a.x_format == ACT_BF16 || a.x_format == ACT_F16, "%s: unknown activation format %d", who, a.x_format);
    AWQ_REQUIRE(a.out_format == ACT_BF16 || a.out_format == ACT_F16, "%s: unknown output format %d", who, a.out_format);
    const int mode = g_decode_mode.load();
    const bool fast_ok = gemv_streamk_supported(a);
    if (mode >= 2 && !fast_ok)
        return set_error(AWQ_ERR_UNSUPPORTED,
                         "%s: stream-K kernel needs group 128, K %% 128 == 0, N %% 32 == 0, 16-byte aligned "
                         "pointers and an sm_100 device (K=%d N=%d gs=%d)", who, a.K, a.N, a.group_size);
    if (mode != 1 && fast_ok) {
        // bf16 activations: converting them to fp16 first (a small kernel in front) buys a cheaper nibble decode, which
        // pays once a launch streams tens of megabytes; below that the extra launch costs more than it saves
        const bool small = (double)a.K * a.N * 0.52 < 48e6 && a.B <= 8;
        a.native_bf16 = mode == 3 || (mode == 0 && a.x_format == ACT_BF16 && small);
        a.deterministic = g_deterministic.load() != 0;
        return launch_gemv_streamk(a);
    }
    return launch_gemv_generic(a);
}

}  // namespace awq

using namespace awq;

extern "C" int awq_b200_version(void) { return 100; }
extern "C" const char *awq_b200_last_error(void) { return g_error; }

extern "C" int awq_b200_set_decode_kernel(int mode) {
    AWQ_REQUIRE(mode >= 0 && mode <= 3, "set_decode_kernel: mode must be 0, 1, 2 or 3");
    g_decode_mode.store(mode);
    return AWQ_OK;
}
extern "C" int awq_b200_set_deterministic(int on) {
    g_deterministic.store(on ? 1 : 0);
    return AWQ_OK;
}
extern "C" int awq_b200_set_wait_limit(long long cycles) {
    AWQ_REQUIRE(cycles >= 0, "set_wait_limit: negative limit");
    g_wait_limit.store(cycles == 0 ? WAIT_LIMIT_DEFAULT : cycles);
    return AWQ_OK;
}
extern "C" int awq_b200_set_gemm_kernel(int mode) {
    AWQ_REQUIRE(mode >= 0 && mode <= 3, "set_gemm_kernel: mode must be 0, 1, 2 or 3");
    g_gemm_mode.store(mode);
    return AWQ_OK;
}

extern "C" size_t awq_b200_workspace_bytes(int B, int K, int N) {
    if (K <= 0 || N <= 0) return 256;
    return gemv_streamk_workspace_bytes(B, K, N);
}

extern "C" int awq_b200_workspace_init(void *workspace, size_t workspace_bytes, awq_stream_t stream) {
    AWQ_REQUIRE(workspace && workspace_bytes >= 256, "workspace_init: null or tiny workspace");
    return check_cuda(cudaMemsetAsync(workspace, 0, workspace_bytes, as_stream(stream)), "workspace memset");
}

extern "C" int awq_b200_workspace_check(const void *workspace, awq_stream_t stream) {
    AWQ_REQUIRE(workspace, "workspace_check: null workspace");
    int flag = 0;
    int rc = check_cuda(cudaMemcpyAsync(&flag, workspace, sizeof(int), cudaMemcpyDeviceToHost, as_stream(stream)),
                        "workspace_check copy");
    if (rc) return rc;
    rc = check_cuda(cudaStreamSynchronize(as_stream(stream)), "workspace_check sync");
    if (rc) return rc;
    return status_of_device_flag(flag);
}

extern "C" int awq_b200_gemv_act(const void *x, int x_format, const int32_t *qweight, const int32_t *qzeros,
                                 const uint16_t *scales, const uint16_t *residual, void *y, int y_is_f32, int B,
                                 int K, int N, int group_size, void *workspace, size_t workspace_bytes,
                                 awq_stream_t stream) {
    AWQ_REQUIRE(!(y_is_f32 && residual), "gemv: the f32 partial output takes no residual");
    GemvArgs a{reinterpret_cast<const uint16_t *>(x), qweight, qzeros, scales, residual, y, B, K, N, group_size,
               y_is_f32 ? EPI_F32 : EPI_BF16, workspace, workspace_bytes, as_stream(stream)};
    a.x_format = x_format;
    return run_gemv(y_is_f32 ? "gemv_f32" : "gemv_bf16", a);
}

extern "C" int awq_b200_gemv_bf16(const uint16_t *x, const int32_t *qweight, const int32_t *qzeros,
                                  const uint16_t *scales, const uint16_t *residual, uint16_t *y, int B, int K,
                                  int N, int group_size, void *workspace, size_t workspace_bytes,
                                  awq_stream_t stream) {
    return awq_b200_gemv_act(x, ACT_BF16, qweight, qzeros, scales, residual, y, 0, B, K, N, group_size, workspace,
                             workspace_bytes, stream);
}

extern "C" int awq_b200_gemv_f32(const uint16_t *x, const int32_t *qweight, const int32_t *qzeros,
                                 const uint16_t *scales, float *y, int B, int K, int N, int group_size,
                                 void *workspace, size_t workspace_bytes, awq_stream_t stream) {
    return awq_b200_gemv_act(x, ACT_BF16, qweight, qzeros, scales, nullptr, y, 1, B, K, N, group_size, workspace,
                             workspace_bytes, stream);
}

extern "C" int awq_b200_gemv_f32_push(const void *x, int x_format, const int32_t *qweight, const int32_t *qzeros,
                                      const uint16_t *scales, float *y, int B, int K, int N, int group_size,
                                      void *const *peer_flags, int n_ranks, int rank, void *workspace,
                                      size_t workspace_bytes, awq_stream_t stream) {
    AWQ_REQUIRE(n_ranks >= 1 && n_ranks <= TP_MAX_RANKS && rank >= 0 && rank < n_ranks, "gemv_f32_push: rank %d of %d", rank,
                n_ranks);
    AWQ_REQUIRE(peer_flags, "gemv_f32_push: null peer array");
    AWQ_REQUIRE(B >= 1 && B <= 8, "gemv_f32_push: 1..8 batch rows");
    PeerPush push{};
    push.n = n_ranks;
    push.rank = rank;
    for (int r = 0; r < n_ranks; ++r) {
        AWQ_REQUIRE(peer_flags[r], "gemv_f32_push: null flag pointer for rank %d", r);
        push.flag[r] = reinterpret_cast<unsigned int *>(peer_flags[r]);
    }
    GemvArgs a{reinterpret_cast<const uint16_t *>(x), qweight, qzeros, scales, nullptr, y, B, K, N, group_size,
               EPI_F32_PUSH, workspace, workspace_bytes, as_stream(stream)};
    a.x_format = x_format;
    a.push = &push;
    int rc = check_gemv_args("gemv_f32_push", a);
    if (rc) return rc;
    AWQ_REQUIRE(x_format == ACT_BF16 || x_format == ACT_F16, "gemv_f32_push: unknown activation format %d", x_format);
    AWQ_REQUIRE(aligned16(y), "gemv_f32_push: y must be 16-byte aligned");
    if (!gemv_streamk_supported(a))
        return set_error(AWQ_ERR_UNSUPPORTED, "gemv_f32_push: needs group 128, K %% 128 == 0, N %% 32 == 0 (K=%d N=%d gs=%d)", K,
                         N, group_size);
    a.native_bf16 = g_decode_mode.load() == 3;
    a.deterministic = g_deterministic.load() != 0;
    return launch_gemv_streamk(a);
}

extern "C" int awq_b200_gateup_swiglu_act(const void *x, int x_format, const int32_t *qweight, const int32_t *qzeros,
                                          const uint16_t *scales, void *out, int out_format, int B, int K, int I,
                                          int group_size, void *workspace, size_t workspace_bytes,
                                          awq_stream_t stream) {
    AWQ_REQUIRE(I >= 0 && I % 4 == 0, "gateup_swiglu: I (%d) must be a multiple of 4", I);
    GemvArgs a{reinterpret_cast<const uint16_t *>(x), qweight, qzeros, scales, nullptr, out, B, K, 2 * I, group_size,
               EPI_SWIGLU, workspace, workspace_bytes, as_stream(stream)};
    a.x_format = x_format;
    a.out_format = out_format;
    return run_gemv("gateup_swiglu", a);
}

extern "C" int awq_b200_gateup_swiglu_bf16(const uint16_t *x, const int32_t *qweight, const int32_t *qzeros,
                                           const uint16_t *scales, uint16_t *out, int B, int K, int I,
                                           int group_size, void *workspace, size_t workspace_bytes,
                                           awq_stream_t stream) {
    return awq_b200_gateup_swiglu_act(x, ACT_BF16, qweight, qzeros, scales, out, ACT_BF16, B, K, I, group_size,
                                      workspace, workspace_bytes, stream);
}

extern "C" int awq_b200_ffn_decode_bf16(const uint16_t *x, const uint16_t *gamma, float eps,
                                        const int32_t *qw_gateup, const int32_t *qz_gateup,
                                        const uint16_t *s_gateup, const int32_t *qw_down, const int32_t *qz_down,
                                        const uint16_t *s_down, const uint16_t *residual, uint16_t *normed,
                                        uint16_t *inter, uint16_t *out, int B, int H, int I, int group_size,
                                        void *workspace, size_t workspace_bytes, awq_stream_t stream) {
    AWQ_REQUIRE(inter, "ffn_decode: inter buffer is required");
    AWQ_REQUIRE(!gamma || normed, "ffn_decode: normed buffer is required with gamma");
    // The intermediates travel between the three kernels as fp16 (exact for bf16-rounded values with
    // 2^-14 <= |x| <= 65504): that is the activation format the GEMV kernel multiplies fastest.
    // (With awq_b200_set_decode_kernel(3) they stay bf16, for activations beyond the fp16 range.)
    int rc;
    const int fmt = g_decode_mode.load() == 3 ? ACT_BF16 : ACT_F16;
    const void *xin = x;
    int xfmt = ACT_BF16;
    if (gamma) {
        if ((rc = awq_b200_rmsnorm_act(x, gamma, eps, normed, fmt, B, H, stream))) return rc;
        xin = normed;
        xfmt = fmt;
    }
    if ((rc = awq_b200_gateup_swiglu_act(xin, xfmt, qw_gateup, qz_gateup, s_gateup, inter, fmt, B, H, I, group_size,
                                         workspace, workspace_bytes, stream)))
        return rc;
    return awq_b200_gemv_act(inter, fmt, qw_down, qz_down, s_down, residual, out, 0, B, I, H, group_size, workspace,
                             workspace_bytes, stream);
}

extern "C" int awq_b200_set_ffn_stack_tuning(int lookahead_units, int split_per_1024) {
    if (lookahead_units >= 0) ffn_fused_set_lookahead(lookahead_units);
    if (split_per_1024 >= 0) ffn_fused_set_split(split_per_1024);
    return AWQ_OK;
}
extern "C" size_t awq_b200_ffn_stack_plan_bytes(int n_layers) { return ffn_fused_plan_bytes(n_layers); }
extern "C" size_t awq_b200_ffn_stack_workspace_bytes(int n_layers) { return ffn_fused_workspace_bytes(n_layers); }
extern "C" size_t awq_b200_ffn_stack_tp_slot_bytes(int H, int n_ranks) { return ffn_fused_tp_slot_bytes(H, n_ranks); }

extern "C" int awq_b200_ffn_stack_plan(void *plan, size_t plan_bytes, int n_layers, const int32_t *const *qw_gateup,
                                       const int32_t *const *qz_gateup, const uint16_t *const *s_gateup,
                                       const int32_t *const *qw_down, const int32_t *const *qz_down,
                                       const uint16_t *const *s_down, const uint16_t *const *gamma, int H, int I,
                                       int group_size) {
    AWQ_REQUIRE(qw_gateup && qz_gateup && s_gateup && qw_down && qz_down && s_down && gamma, "ffn_stack_plan: null array");
    return ffn_fused_plan(plan, plan_bytes, n_layers, qw_gateup, qz_gateup, s_gateup, qw_down, qz_down, s_down, gamma, H, I,
                          group_size);
}

extern "C" int awq_b200_ffn_stack_decode_bf16(const void *plan, int n_layers, const uint16_t *x, uint16_t *out,
                                              uint16_t *inter, float eps, int B, int H, int I, int group_size,
                                              void *workspace, size_t workspace_bytes, awq_stream_t stream) {
    AWQ_REQUIRE(n_layers >= 1 && B >= 0 && H > 0 && I > 0, "ffn_stack_decode: bad size");
    if (B == 0) return AWQ_OK;
    AWQ_REQUIRE(plan && x && out && inter, "ffn_stack_decode: null pointer");
    AWQ_REQUIRE(aligned16(x) && aligned16(out) && aligned16(inter), "ffn_stack_decode: pointers must be 16-byte aligned");
    if (!ffn_fused_supported(B, H, I, group_size))
        return set_error(AWQ_ERR_UNSUPPORTED,
                         "ffn_stack_decode: needs B <= 8, group 128, H and I multiples of 128 (B=%d H=%d I=%d gs=%d)", B, H, I,
                         group_size);
    return launch_ffn_fused(plan, n_layers, x, out, inter, eps, B, H, I, workspace, workspace_bytes, as_stream(stream));
}

extern "C" int awq_b200_ffn_stack_decode_tp_bf16(const void *plan, int n_layers, const uint16_t *x, uint16_t *out,
                                                 uint16_t *inter, float eps, int B, int H, int I_local, int group_size,
                                                 void *const *peer_base, size_t slot_stride, size_t flag_offset,
                                                 int n_ranks, int rank, void *workspace, size_t workspace_bytes,
                                                 awq_stream_t stream) {
    AWQ_REQUIRE(n_layers >= 1 && B >= 0 && H > 0 && I_local > 0, "ffn_stack_decode_tp: bad size");
    AWQ_REQUIRE(n_ranks >= 2 && n_ranks <= TP_MAX_RANKS && rank >= 0 && rank < n_ranks, "ffn_stack_decode_tp: rank %d of %d", rank,
                n_ranks);
    if (B == 0) return AWQ_OK;
    AWQ_REQUIRE(plan && x && out && inter && peer_base, "ffn_stack_decode_tp: null pointer");
    AWQ_REQUIRE(aligned16(x) && aligned16(out) && aligned16(inter), "ffn_stack_decode_tp: pointers must be 16-byte aligned");
    AWQ_REQUIRE(flag_offset >= ffn_fused_tp_slot_bytes(H, n_ranks) && slot_stride >= flag_offset + 64 && slot_stride % 16 == 0 &&
                    flag_offset % 16 == 0,
                "ffn_stack_decode_tp: a slot holds awq_b200_ffn_stack_tp_slot_bytes(H, n_ranks) = %zu bytes and 16 flag words "
                "behind them", ffn_fused_tp_slot_bytes(H, n_ranks));
    if (!ffn_fused_supported(B, H, I_local, group_size))
        return set_error(AWQ_ERR_UNSUPPORTED,
                         "ffn_stack_decode_tp: needs B <= 8, group 128, H and I multiples of 128 (B=%d H=%d I=%d gs=%d)", B, H,
                         I_local, group_size);
    FusedPeers peers{};
    peers.n = n_ranks;
    peers.rank = rank;
    peers.slot_stride = slot_stride;
    peers.flag_offset = flag_offset;
    for (int r = 0; r < n_ranks; ++r) {
        AWQ_REQUIRE(peer_base[r] && aligned16(peer_base[r]), "ffn_stack_decode_tp: bad buffer pointer of rank %d", r);
        peers.base[r] = peer_base[r];
    }
    return launch_ffn_fused(plan, n_layers, x, out, inter, eps, B, H, I_local, workspace, workspace_bytes, as_stream(stream),
                            &peers);
}

extern "C" int awq_b200_gemm_bf16(const uint16_t *A, const int32_t *qweight, const int32_t *qzeros,
                                  const uint16_t *scales, uint16_t *C, int M, int K, int N, int group_size,
                                  awq_stream_t stream) {
    AWQ_REQUIRE(M >= 0 && K >= 0 && N >= 0 && group_size > 0, "gemm: negative size or group_size <= 0");
    AWQ_REQUIRE(N % 8 == 0, "gemm: N (%d) must be a multiple of 8", N);
    AWQ_REQUIRE(K % group_size == 0, "gemm: K (%d) must be a multiple of group_size (%d)", K, group_size);
    AWQ_REQUIRE(group_size % 32 == 0, "gemm: group_size must be a multiple of 32 (kernel inner vector width)");
    if (M == 0 || N == 0) return AWQ_OK;
    AWQ_REQUIRE(K > 0, "gemm: K must be positive");
    AWQ_REQUIRE(A && qweight && qzeros && scales && C, "gemm: null pointer");
    AWQ_REQUIRE(aligned16(A) && aligned16(scales), "gemm: A and scales must be 16-byte aligned");
    const int mode = g_gemm_mode.load();
    const bool tc_ok = gemm_tc_supported(M, K, N, group_size) && aligned16(qweight) && aligned16(qzeros) && aligned16(C);
    if (mode == 2 && !tc_ok)
        return set_error(AWQ_ERR_UNSUPPORTED, "gemm: tensor-core kernel does not cover M=%d K=%d N=%d gs=%d", M, K, N,
                         group_size);
    // automatic: from 1024 rows on the kernel that keeps the dequantised weights in tensor memory measured faster
    // (194 against 212 us on 2048 x 4096 x 14336), below that the tile with the weights in shared memory
    if ((mode == 3 || (mode == 0 && M >= 1024)) && tc_ok) return launch_gemm_tm(A, qweight, qzeros, scales, C, M, K, N, as_stream(stream));
    if (mode != 1 && tc_ok) return launch_gemm_tc(A, qweight, qzeros, scales, C, M, K, N, group_size, as_stream(stream));
    return launch_gemm_generic(A, qweight, qzeros, scales, C, M, K, N, group_size, as_stream(stream));
}

extern "C" int awq_b200_gemm_fused_bf16(const uint16_t *A, const int32_t *qweight, const int32_t *qzeros,
                                        const uint16_t *scales, const uint16_t *residual, uint16_t *C, int swiglu, int M,
                                        int K, int N, int group_size, awq_stream_t stream) {
    AWQ_REQUIRE(M >= 0 && K > 0 && N > 0 && group_size > 0, "gemm_fused: bad size");
    AWQ_REQUIRE(!(swiglu && residual), "gemm_fused: SwiGLU and residual do not combine");
    if (M == 0) return AWQ_OK;
    AWQ_REQUIRE(A && qweight && qzeros && scales && C, "gemm_fused: null pointer");
    AWQ_REQUIRE(aligned16(A) && aligned16(scales) && aligned16(qweight) && aligned16(qzeros) && aligned16(C) &&
                    aligned16(residual), "gemm_fused: pointers must be 16-byte aligned");
    if (!gemm_tc_supported(M, K, N, group_size) || g_gemm_mode.load() == 1)
        return set_error(AWQ_ERR_UNSUPPORTED, "gemm_fused: needs the tensor-core kernel (group 128, K %% 128 == 0, N %% 32 == 0; "
                         "M=%d K=%d N=%d gs=%d)", M, K, N, group_size);
    const int epi = swiglu ? GEMM_EPI_SWIGLU : (residual ? GEMM_EPI_RESIDUAL : GEMM_EPI_BF16);
    if (g_gemm_mode.load() == 3 || (g_gemm_mode.load() == 0 && M >= 1024)) return launch_gemm_tm(A, qweight, qzeros, scales, C, M, K, N, as_stream(stream), epi, residual);
    return launch_gemm_tc(A, qweight, qzeros, scales, C, M, K, N, group_size, as_stream(stream), epi, residual);
}

extern "C" int awq_b200_gemm_check(awq_stream_t stream) {
    const int rc = gemm_tc_check(as_stream(stream));
    const int rc2 = gemm_decode_check(as_stream(stream));
    const int rc3 = gemm_tm_check(as_stream(stream));
    const int rc4 = gemm_decode_f8_check(as_stream(stream));
    return rc ? rc : (rc2 ? rc2 : (rc3 ? rc3 : rc4));
}

extern "C" size_t awq_b200_gemm_decode_workspace_bytes(int M, int N) { return gemm_decode_workspace_bytes(M, N); }

extern "C" int awq_b200_gemm_decode_f32(const uint16_t *A, const int32_t *qweight, const int32_t *qzeros, const uint16_t *scales,
                                        float *C, int M, int K, int N, int group_size, void *workspace, size_t workspace_bytes,
                                        awq_stream_t stream) {
    AWQ_REQUIRE(M >= 0 && K > 0 && N > 0 && group_size > 0, "gemm_decode_f32: bad size");
    if (M == 0) return AWQ_OK;
    AWQ_REQUIRE(A && qweight && qzeros && scales && C, "gemm_decode_f32: null pointer");
    AWQ_REQUIRE(aligned16(A) && aligned16(scales) && aligned16(qweight) && aligned16(qzeros) && aligned16(C) && aligned16(workspace),
                "gemm_decode_f32: pointers must be 16-byte aligned");
    if (!gemm_decode_supported(M, K, N, group_size))
        return set_error(AWQ_ERR_UNSUPPORTED, "gemm_decode_f32: needs M <= 64, group 128, K %% 128 == 0, N %% 32 == 0 "
                         "(M=%d K=%d N=%d gs=%d)", M, K, N, group_size);
    return launch_gemm_decode(A, qweight, qzeros, scales, reinterpret_cast<uint16_t *>(C), M, K, N, as_stream(stream), GEMM_EPI_F32,
                              nullptr, workspace, workspace_bytes);
}

extern "C" int awq_b200_gemm_decode_act(const void *A, int a_format, const int32_t *qweight, const int32_t *qzeros,
                                        const uint16_t *scales, const uint16_t *residual, void *C, int c_format, int swiglu, int M,
                                        int K, int N, int group_size, void *workspace, size_t workspace_bytes,
                                        awq_stream_t stream) {
    AWQ_REQUIRE(M >= 0 && K > 0 && N > 0 && group_size > 0, "gemm_decode_act: bad size");
    AWQ_REQUIRE(a_format == AWQ_ACT_BF16 || a_format == AWQ_ACT_F16, "gemm_decode_act: a_format must be AWQ_ACT_BF16 or AWQ_ACT_F16");
    AWQ_REQUIRE(c_format == AWQ_ACT_BF16 || c_format == AWQ_ACT_F16 || c_format == AWQ_OUT_F32,
                "gemm_decode_act: c_format must be AWQ_ACT_BF16, AWQ_ACT_F16 or AWQ_OUT_F32");
    AWQ_REQUIRE(!(swiglu && residual), "gemm_decode_act: SwiGLU and residual do not combine");
    AWQ_REQUIRE(!(c_format != AWQ_ACT_BF16 && residual), "gemm_decode_act: the residual add goes with a bf16 output");
    AWQ_REQUIRE(!(c_format == AWQ_OUT_F32 && swiglu), "gemm_decode_act: the f32 output carries plain sums, not SwiGLU");
    if (M == 0) return AWQ_OK;
    AWQ_REQUIRE(A && qweight && qzeros && scales && C, "gemm_decode_act: null pointer");
    AWQ_REQUIRE(aligned16(A) && aligned16(scales) && aligned16(qweight) && aligned16(qzeros) && aligned16(C) &&
                    aligned16(residual) && aligned16(workspace), "gemm_decode_act: pointers must be 16-byte aligned");
    if (!gemm_decode_supported(M, K, N, group_size))
        return set_error(AWQ_ERR_UNSUPPORTED, "gemm_decode_act: needs M <= 64, group 128, K %% 128 == 0, N %% 32 == 0 "
                         "(M=%d K=%d N=%d gs=%d)", M, K, N, group_size);
    const int epi = c_format == AWQ_OUT_F32 ? GEMM_EPI_F32 : (swiglu ? GEMM_EPI_SWIGLU : (residual ? GEMM_EPI_RESIDUAL : GEMM_EPI_BF16));
    return launch_gemm_decode(reinterpret_cast<const uint16_t *>(A), qweight, qzeros, scales, reinterpret_cast<uint16_t *>(C), M, K, N,
                              as_stream(stream), epi, residual, workspace, workspace_bytes, a_format == AWQ_ACT_F16,
                              c_format == AWQ_ACT_F16);
}

extern "C" size_t awq_b200_gemm_decode_f8_workspace_bytes(int M, int K, int N) { return gemm_decode_f8_workspace_bytes(M, K, N); }

extern "C" int awq_b200_gemm_decode_f8(const void *A, int a_format, const int32_t *qweight, const int32_t *qzeros,
                                       const uint16_t *scales, const uint16_t *residual, void *C, int c_format, int swiglu, int M,
                                       int K, int N, int group_size, void *workspace, size_t workspace_bytes,
                                       awq_stream_t stream) {
    AWQ_REQUIRE(M >= 0 && K > 0 && N > 0 && group_size > 0, "gemm_decode_f8: bad size");
    AWQ_REQUIRE(a_format == AWQ_ACT_BF16 || a_format == AWQ_ACT_F16, "gemm_decode_f8: a_format must be AWQ_ACT_BF16 or AWQ_ACT_F16");
    AWQ_REQUIRE(c_format == AWQ_ACT_BF16 || c_format == AWQ_ACT_F16 || c_format == AWQ_OUT_F32,
                "gemm_decode_f8: c_format must be AWQ_ACT_BF16, AWQ_ACT_F16 or AWQ_OUT_F32");
    AWQ_REQUIRE(!(swiglu && residual), "gemm_decode_f8: SwiGLU and residual do not combine");
    AWQ_REQUIRE(!(c_format != AWQ_ACT_BF16 && residual), "gemm_decode_f8: the residual add goes with a bf16 output");
    AWQ_REQUIRE(!(c_format == AWQ_OUT_F32 && swiglu), "gemm_decode_f8: the f32 output carries plain sums, not SwiGLU");
    if (M == 0) return AWQ_OK;
    AWQ_REQUIRE(A && qweight && qzeros && scales && C, "gemm_decode_f8: null pointer");
    AWQ_REQUIRE(aligned16(A) && aligned16(scales) && aligned16(qweight) && aligned16(qzeros) && aligned16(C) &&
                    aligned16(residual) && aligned16(workspace), "gemm_decode_f8: pointers must be 16-byte aligned");
    if (!gemm_decode_f8_supported(M, K, N, group_size))
        return set_error(AWQ_ERR_UNSUPPORTED, "gemm_decode_f8: needs M <= 32, group 128, K %% 128 == 0, N %% 32 == 0 "
                         "(M=%d K=%d N=%d gs=%d)", M, K, N, group_size);
    const int epi = c_format == AWQ_OUT_F32 ? GEMM_EPI_F32 : (swiglu ? GEMM_EPI_SWIGLU : (residual ? GEMM_EPI_RESIDUAL : GEMM_EPI_BF16));
    return launch_gemm_decode_f8(reinterpret_cast<const uint16_t *>(A), a_format == AWQ_ACT_F16, qweight, qzeros, scales,
                                 reinterpret_cast<uint16_t *>(C), M, K, N, as_stream(stream), epi, residual, c_format == AWQ_ACT_F16,
                                 workspace, workspace_bytes);
}

extern "C" int awq_b200_gemm_decode_bf16(const uint16_t *A, const int32_t *qweight, const int32_t *qzeros,
                                         const uint16_t *scales, const uint16_t *residual, uint16_t *C, int swiglu, int M,
                                         int K, int N, int group_size, void *workspace, size_t workspace_bytes,
                                         awq_stream_t stream) {
    AWQ_REQUIRE(M >= 0 && K > 0 && N > 0 && group_size > 0, "gemm_decode: bad size");
    AWQ_REQUIRE(!(swiglu && residual), "gemm_decode: SwiGLU and residual do not combine");
    if (M == 0) return AWQ_OK;
    AWQ_REQUIRE(A && qweight && qzeros && scales && C, "gemm_decode: null pointer");
    AWQ_REQUIRE(aligned16(A) && aligned16(scales) && aligned16(qweight) && aligned16(qzeros) && aligned16(C) &&
                    aligned16(residual) && aligned16(workspace), "gemm_decode: pointers must be 16-byte aligned");
    if (!gemm_decode_supported(M, K, N, group_size))
        return set_error(AWQ_ERR_UNSUPPORTED, "gemm_decode: needs M <= 64, group 128, K %% 128 == 0, N %% 32 == 0 "
                         "(M=%d K=%d N=%d gs=%d)", M, K, N, group_size);
    return launch_gemm_decode(A, qweight, qzeros, scales, C, M, K, N, as_stream(stream),
                              swiglu ? GEMM_EPI_SWIGLU : (residual ? GEMM_EPI_RESIDUAL : GEMM_EPI_BF16), residual, workspace,
                              workspace_bytes);
}
