/*
 * awq_b200.h -- C ABI of libawq_b200.so: mlir-air's int4-AWQ LLM hot path as
 * hand-written sm_100a CUDA kernels.
 *
 * Every entry point
 *   - is extern "C", takes plain pointers and sizes, and returns an int status
 *     (AWQ_OK == 0, negative on error; awq_b200_last_error() gives the text);
 *   - works on DEVICE pointers the caller owns (16-byte aligned), on the CUDA
 *     stream passed as `stream` (a cudaStream_t cast to void*; NULL = default
 *     stream), and is asynchronous with respect to the host;
 *   - never allocates device memory: kernels that need scratch take a caller-owned
 *     `workspace` (size from awq_b200_workspace_bytes, zeroed once with
 *     awq_b200_workspace_init).  One workspace must not be shared by calls that
 *     can overlap on the GPU.
 *
 * Weight layout ("layout A", HF AutoAWQ gemm format, the layout handled by
 * programming_examples/llms/llama32_1b_int4/awq_repacker.py:33-54):
 *   qweight int32 [K, N/8]   nibble at bits [4i+3:4i] of word (k, j) is the
 *                            uint4 of output column 8j + {0,2,4,6,1,3,5,7}[i]
 *   qzeros  int32 [K/gs, N/8] same packing
 *   scales  bf16  [K/gs, N]
 *   W[k, n] = (q[k, n] - z[k / gs, n]) * s[k / gs, n]
 * bf16 values cross the ABI as uint16_t bit patterns (the reference passes
 * ml_dtypes.bfloat16 viewed as int16, python/air/backend/xrt.py:757-758).
 */
#ifndef AWQ_B200_H_
#define AWQ_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AWQ_OK 0
#define AWQ_ERR_INVALID_ARGUMENT (-1) /* bad shape / null / misaligned pointer       */
#define AWQ_ERR_WORKSPACE (-2)        /* workspace missing or too small              */
#define AWQ_ERR_CUDA (-3)             /* a CUDA runtime / driver call failed         */
#define AWQ_ERR_DEVICE_TIMEOUT (-4)   /* a bounded device-side wait gave up          */
#define AWQ_ERR_UNSUPPORTED (-5)      /* not an sm_100 device, or shape not covered  */

typedef void *awq_stream_t;

/* Library version (major * 10000 + minor * 100 + patch). */
int awq_b200_version(void);

/* Text of the calling thread's most recent error ("" if none).  Replaces the
 * Python exceptions of the reference backend (python/air/backend/abc.py:52-61,
 * python/air/backend/xrt.py:204-218). */
const char *awq_b200_last_error(void);

/* 16-bit activation formats of the *_act entry points.  Public inputs and outputs are bf16; fp16
 * is the format activations take between the kernels of one FFN, because the GEMV kernel
 * multiplies fp16 activations fastest.  A bf16 value converts to fp16 without loss when
 * 2^-14 <= |x| <= 65504; smaller values land in fp16 subnormals (they keep 2^-24 absolute
 * resolution and reach zero below 2^-25), larger ones become infinities, which surface as an
 * AWQ_ERR_UNSUPPORTED from the next *_check call (use awq_b200_set_decode_kernel(3) then). */
#define AWQ_ACT_BF16 0
#define AWQ_ACT_F16 1
/* f32 sums as the output of awq_b200_gemm_decode_act (beside the two 16-bit formats). */
#define AWQ_OUT_F32 2

/* Choose the decode kernel: 0 = automatic (TMA + tensor-core stream-K kernel when the
 * shape allows it, else the generic kernel), 1 = force generic, 2 = force stream-K
 * (returns AWQ_ERR_UNSUPPORTED where it cannot run), 3 = stream-K multiplying bf16
 * activations as they are (no fp16 conversion; for activations beyond the fp16 range).
 * Process-wide; for tests. */
int awq_b200_set_decode_kernel(int mode);

/* Every wait a kernel of this library makes on the device (for a shared-memory stage, for another
 * CTA's phase counter, for another rank's partial sums or flags) gives up after `cycles` SM clock
 * cycles, sets the error word of its workspace and lets the kernel drain and return; the next
 * *_check call reports AWQ_ERR_DEVICE_TIMEOUT.  Default 2^31 (about a second); 0 restores the
 * default.  Process-wide, read when a kernel is launched (a captured graph keeps the value it was
 * captured with).  The bounded counterpart of the reference waiting on run.wait() and checking
 * ERT_CMD_STATE_COMPLETED (python/air/backend/xrt.py:204-218). */
int awq_b200_set_wait_limit(long long cycles);

/* Kept for compatibility: split-K partial sums are handed over as fixed-point integers (2^-20
 * resolution, |partial sum| < 8.38e6, beyond which the next *_check call reports
 * AWQ_ERR_UNSUPPORTED), and integer addition does not depend on the order of the adds, so results
 * are bit-reproducible whatever this is set to. */
int awq_b200_set_deterministic(int on);

/* ---- AWQ dequant --------------------------------------------------------------
 * out bf16 [K, N] = bf16_rne((q - z) * s).  Bit-exact with dequant_to_bf16
 * (programming_examples/llms/llama32_1b_int4/awq_repacker.py:57-82),
 * awq_dequant_layer (.../awq_pack.py:84-104) and the device kernel
 * dequant_int4_bf16 (programming_examples/dequant_awq/dequant.cc:42-85). */
int awq_b200_dequant_bf16(const int32_t *qweight, const int32_t *qzeros, const uint16_t *scales,
                          uint16_t *out, int K, int N, int group_size, awq_stream_t stream);

/* 1-D form of programming_examples/dequant_awq/dequant_awq.py:382-396: n nibbles packed
 * two per byte (low nibble = even index), one bf16 scale and one uint8 zero per group. */
int awq_b200_dequant_1d_bf16(const uint8_t *packed_q, const uint16_t *scales, const uint8_t *zeros,
                             uint16_t *out, int n, int group_size, awq_stream_t stream);

/* ---- workspace ---------------------------------------------------------------- */
/* Bytes of scratch the decode kernels need for a [B, K] x [K, N] product (counters, split-K
 * partials, and room to convert B rows of bf16 activations to fp16). */
size_t awq_b200_workspace_bytes(int B, int K, int N);
/* Zero the workspace (once after allocation, and again after any call that
 * returned AWQ_ERR_DEVICE_TIMEOUT). */
int awq_b200_workspace_init(void *workspace, size_t workspace_bytes, awq_stream_t stream);
/* Synchronise `stream` and report whether any kernel using this workspace gave up on a
 * bounded device-side wait (AWQ_ERR_DEVICE_TIMEOUT).  The counterpart of the reference's
 * check that a run reached ERT_CMD_STATE_COMPLETED (python/air/backend/xrt.py:204-218). */
int awq_b200_workspace_check(const void *workspace, awq_stream_t stream);

/* ---- decode GEMV ----------------------------------------------------------------
 * y bf16 [B, N] = bf16(x[B, K] @ W (+ residual[B, N])), f32 accumulate, one rounding.
 * Replaces matvec_int4_bf16_packed / zero_vectorized_bf16 / partial_plus_r_bf16
 * (programming_examples/matrix_vector_multiplication/int4_awq/mv_int4_bf16.cc:65-150,
 * 391-436) and follows the goldens matvec_int4_packed.py:272-287 and
 * matvec_int4_packed_add.py:302-319.  residual may be NULL.  1 <= B <= 64. */
int awq_b200_gemv_bf16(const uint16_t *x, const int32_t *qweight, const int32_t *qzeros,
                       const uint16_t *scales, const uint16_t *residual, uint16_t *y, int B, int K,
                       int N, int group_size, void *workspace, size_t workspace_bytes,
                       awq_stream_t stream);

/* The same product as awq_b200_gemv_bf16 for callers that cannot allocate device memory
 * (a plugin interface that carries only inputs and outputs, a serving process that bans
 * cudaMalloc after start-up, plain C hosts without an allocator).  It has no counterpart in
 * the reference.  The kernel's scratch is a fixed array inside the library image, about
 * 2 MB on every GPU that loads the library, held until the process exits; nothing is
 * allocated or freed by this call.  Limits: N <= 32768, group size 128, K % 128 == 0,
 * N % 32 == 0, 1 <= B <= 64; anything else returns an error rather than falling back.
 * The first call on each device looks up the array's device address, so make that first
 * call outside any stream capture.  All calls on a device share the one array: calls that
 * may run at the same time on the GPU (different streams) race and give wrong results. */
int awq_b200_gemv_bf16_static(const uint16_t *x, const int32_t *qweight, const int32_t *qzeros,
                              const uint16_t *scales, const uint16_t *residual, uint16_t *y, int B,
                              int K, int N, int group_size, awq_stream_t stream);

/* Synchronise `stream` and report whether a kernel launched by awq_b200_gemv_bf16_static on the
 * current device gave up on a bounded wait (AWQ_ERR_DEVICE_TIMEOUT) or clamped an activation.  The
 * error word lives in the built-in array and the next static call clears it, so ask before that
 * next call.  Allocates nothing.  No counterpart in the reference beyond its run-state check
 * (python/air/backend/xrt.py:204-218). */
int awq_b200_static_check(awq_stream_t stream);

/* General form: x in `x_format` (AWQ_ACT_*), y bf16 (y_is_f32 = 0, optional residual) or f32. */
int awq_b200_gemv_act(const void *x, int x_format, const int32_t *qweight, const int32_t *qzeros,
                      const uint16_t *scales, const uint16_t *residual, void *y, int y_is_f32, int B,
                      int K, int N, int group_size, void *workspace, size_t workspace_bytes,
                      awq_stream_t stream);

/* Same product, f32 output without rounding or residual: the per-rank partial of a
 * K-split (row-parallel) down projection, summed across ranks by the caller. */
int awq_b200_gemv_f32(const uint16_t *x, const int32_t *qweight, const int32_t *qzeros,
                      const uint16_t *scales, float *y, int B, int K, int N, int group_size,
                      void *workspace, size_t workspace_bytes, awq_stream_t stream);

/* ---- RMSNorm ---------------------------------------------------------------------
 * out bf16 [B, K] = bf16(x * rsqrt(mean(x^2) + eps) * gamma); the inline RMSNorm of
 * programming_examples/decode_ffn_swiglu/matvec_int4_swiglu_rms.py:228-358, golden :496-500. */
int awq_b200_rmsnorm_bf16(const uint16_t *x, const uint16_t *gamma, float eps, uint16_t *out, int B,
                          int K, awq_stream_t stream);

int awq_b200_rmsnorm_act(const uint16_t *x, const uint16_t *gamma, float eps, void *out, int out_format,
                         int B, int K, awq_stream_t stream);

/* h_out bf16 [B, K] = bf16(h + partial_sum) and normed = rmsnorm(h_out, gamma): the residual
 * add that follows the allreduce of a K-split down projection, fused with the next layer's norm.
 * gamma/normed may be NULL (no norm). */
int awq_b200_add_rmsnorm_bf16(const uint16_t *h, const float *partial_sum, const uint16_t *gamma,
                              float eps, uint16_t *h_out, uint16_t *normed, int B, int K,
                              awq_stream_t stream);

int awq_b200_add_rmsnorm_act(const uint16_t *h, const float *partial_sum, const uint16_t *gamma,
                             float eps, uint16_t *h_out, void *normed, int normed_format, int B, int K,
                             awq_stream_t stream);

/* ---- fused gate/up GEMV + SwiGLU ---------------------------------------------------
 * One AWQ matrix [K, 2I] whose columns are gate/up interleaved (column 2i = gate_i,
 * 2i+1 = up_i; the row interleave of llama32_1b_int4_weights.py:173-205 seen from
 * layout A).  out bf16 [B, I] = bf16(silu(bf16(g)) * bf16(u)), silu(g) = g/2 (tanh(g/2)+1).
 * Replaces the GEMV loop + SwiGLU of matvec_int4_swiglu_rms.py:374-459, golden :511-516. */
int awq_b200_gateup_swiglu_bf16(const uint16_t *x, const int32_t *qweight, const int32_t *qzeros,
                                const uint16_t *scales, uint16_t *out, int B, int K, int I,
                                int group_size, void *workspace, size_t workspace_bytes,
                                awq_stream_t stream);

int awq_b200_gateup_swiglu_act(const void *x, int x_format, const int32_t *qweight,
                               const int32_t *qzeros, const uint16_t *scales, void *out, int out_format,
                               int B, int K, int I, int group_size, void *workspace,
                               size_t workspace_bytes, awq_stream_t stream);

/* Interleave two [K, I] AWQ matrices (separate gate and up projections, as stored in an
 * HF checkpoint) into the [K, 2I] form above.  Done once per weight. */
int awq_b200_interleave_gate_up(const int32_t *qw_gate, const int32_t *qz_gate,
                                const uint16_t *s_gate, const int32_t *qw_up, const int32_t *qz_up,
                                const uint16_t *s_up, int32_t *qweight, int32_t *qzeros,
                                uint16_t *scales, int K, int I, int group_size, awq_stream_t stream);

/* ---- decode FFN ----------------------------------------------------------------------
 * out bf16 [B, H] = bf16(down(swiglu(gateup . norm(x))) + residual) with
 * norm = RMSNorm(gamma, eps) when gamma != NULL.  The LGU -> LD chain of
 * llms/llama32_1b_int4/multi_launch_builder/o_gemv_ffn_int4_multi.py:9-12 and the four
 * launches of ffn_swiglu/decode/ffn_decode.py:48-250.  `inter` (16-bit [B, I]) and `normed`
 * (16-bit [B, H], only with gamma) are caller-provided scratch for the intermediates, as they
 * are function arguments in the reference (ffn_decode.py:300-303); their contents are in the
 * library's internal activation format (fp16).  residual may be NULL. */
int awq_b200_ffn_decode_bf16(const uint16_t *x, const uint16_t *gamma, float eps,
                             const int32_t *qw_gateup, const int32_t *qz_gateup,
                             const uint16_t *s_gateup, const int32_t *qw_down,
                             const int32_t *qz_down, const uint16_t *s_down,
                             const uint16_t *residual, uint16_t *normed, uint16_t *inter,
                             uint16_t *out, int B, int H, int I, int group_size, void *workspace,
                             size_t workspace_bytes, awq_stream_t stream);

/* ---- tensor-parallel hand-over over peer memory (no collective call) ----------------------
 * The reference has no multi-GPU form of this path; its only inter-GPU mechanism is a
 * symmetric heap with peer loads/stores and flag words (runtime_lib/airgpu/symmetric_heap.cpp:172-312,
 * test/gpu/multi_gpu/handwritten/allgather.mlir:19-41), which is the model for this pair.
 *
 * awq_b200_gemv_f32_push: this rank's down projection, y f32 [B, N] = x[B, K] @ W_shard, B <= 8,
 * written to y, which must be memory the other ranks have mapped (this rank's send buffer).  When
 * the launch's last sub-strip is stored the kernel issues one system-scope fence and adds 1 to
 * peer_flags[r][rank] on every rank r (uint32 [16] per rank: [0, 8) arrivals per sender, [8] used
 * by the receiver).  peer_flags is a HOST array of n_ranks device pointers valid on this GPU
 * (peer mappings; entry `rank` is this rank's own flag block).
 *
 * awq_b200_tp_reduce_add_rmsnorm_act: waits (bounded, about a second; a timeout is reported by
 * awq_b200_workspace_check on `workspace`) until every rank has signalled its
 * [B, K] partial in `flags` (this rank's flag block), then reads the partials with peer loads
 * (peer_partials: HOST array of n_ranks device pointers to the ranks' send buffers):
 * h_out = bf16(h + sum_r partial_r) in rank order and, when gamma != NULL, normed =
 * RMSNorm(h_out); the last block clears the 9 flag words.  A send buffer + flag block may be
 * reused once the reduce that followed it has itself been followed by this rank's next push (two
 * of them used alternately are enough for a layer loop).  The kernels of different GPUs wait for
 * one another: every rank must enqueue the same sequence. */
int awq_b200_gemv_f32_push(const void *x, int x_format, const int32_t *qweight,
                           const int32_t *qzeros, const uint16_t *scales, float *y, int B, int K,
                           int N, int group_size, void *const *peer_flags, int n_ranks, int rank,
                           void *workspace, size_t workspace_bytes, awq_stream_t stream);
int awq_b200_tp_reduce_add_rmsnorm_act(const uint16_t *h, const void *const *peer_partials,
                                       uint32_t *flags, int n_ranks, const uint16_t *gamma,
                                       float eps, uint16_t *h_out, void *normed,
                                       int normed_format, int B, int K, void *workspace,
                                       awq_stream_t stream);

/* ---- whole decode FFN stack in one launch ---------------------------------------------------
 * For l in 0 .. n_layers-1:  h <- bf16(h + down_l(swiglu(gateup_l . RMSNorm(h, gamma_l, eps)))),
 * h starting as x and ending in out; batch B <= 8.  The single-launch form of the decode
 * block's FFN (llms/llama32_1b_int4/multi_launch_builder/o_gemv_ffn_int4_fused.py:4-30: RMS,
 * gate/up + SwiGLU, down + residual in ONE launch, intermediates staying on chip) applied to
 * the layer loop of llms/llama32_1b_int4/llama32_1b_int4_inference.py:445-455, with the same
 * rounding points as awq_b200_ffn_decode_bf16 called once per layer.
 *
 * The weights are described once by a plan: tensor maps written to `plan` (device memory,
 * 128-byte aligned, awq_b200_ffn_stack_plan_bytes(n_layers) bytes).  The pointer arguments of
 * awq_b200_ffn_stack_plan are HOST arrays of n_layers DEVICE pointers (layout A, gate/up
 * interleaved, gamma bf16 [H]); it copies synchronously, so call it outside stream capture.
 * The plan stays valid as long as the weights do not move.
 *
 * decode: `inter` is 16-bit [B, I] scratch; `workspace` holds at least
 * awq_b200_ffn_stack_workspace_bytes(n_layers) bytes prepared by awq_b200_workspace_init.
 * x may alias out.  All CTAs of the launch wait for one another on counters in the workspace,
 * so the stream must be the only user of that workspace, and the launch takes one CTA per SM
 * with all of its shared memory (a cooperative launch: it fails at once, instead of timing out,
 * where the CTAs cannot all be resident because something else holds SMs).
 * Split-K sums are added as integers: results are bit-reproducible.  Needs group 128, H % 128 == 0, I % 128 == 0; AWQ_ERR_UNSUPPORTED otherwise.
 * Device-side waits are bounded; awq_b200_workspace_check reports a timeout. */
/* Tuning of the stack kernel; a negative value leaves a setting as it is.
 * lookahead_units: 36 KB units per half-CTA requested into L2 ahead of the shared-memory ring
 *   (default 0 = off, at most 64).
 * split_per_1024: 0 = every down unit waits until the whole gate/up phase of its layer is finished;
 *   any other value (default) = it starts as soon as the four 32-output sub-strips that produce its 128
 *   inputs are finished (same results). */
int awq_b200_set_ffn_stack_tuning(int lookahead_units, int split_per_1024);
size_t awq_b200_ffn_stack_plan_bytes(int n_layers);
size_t awq_b200_ffn_stack_workspace_bytes(int n_layers);
int awq_b200_ffn_stack_plan(void *plan, size_t plan_bytes, int n_layers,
                            const int32_t *const *qw_gateup, const int32_t *const *qz_gateup,
                            const uint16_t *const *s_gateup, const int32_t *const *qw_down,
                            const int32_t *const *qz_down, const uint16_t *const *s_down,
                            const uint16_t *const *gamma, int H, int I, int group_size);
int awq_b200_ffn_stack_decode_bf16(const void *plan, int n_layers, const uint16_t *x,
                                   uint16_t *out, uint16_t *inter, float eps, int B, int H, int I,
                                   int group_size, void *workspace, size_t workspace_bytes,
                                   awq_stream_t stream);

/* The same launch for tensor-parallel ranks (one process per GPU): the plan describes this rank's
 * shards (gate/up columns [H, 2 I_local], down rows [I_local, H], cut as in the per-layer path),
 * and after each layer's down projection the ranks exchange their f32 partials inside the kernel:
 * the warp that finishes a 64-column piece of the partial stores it into the receive area of
 * every rank as 8-byte words that carry the value and the exchange's number together (no fence, no
 * flag), and on every rank one warp per piece polls the words of all ranks, adds them in rank
 * order and writes the new hidden state.  peer_base: HOST array of n_ranks device pointers to the
 * ranks' buffers mapped into this GPU's address space (entry `rank` is this rank's own); a buffer
 * holds two slots of slot_stride bytes, each a receive area of at least
 * awq_b200_ffn_stack_tp_slot_bytes(H, n_ranks) bytes followed at flag_offset by 16 uint32 words,
 * all zero when first used and owned by this entry point afterwards (nothing is ever reset; the
 * last word behind slot 0 counts launches).  Every call on these buffers must have the same n_layers.
 * Every rank must make the same sequence of calls, and the
 * kernels of the ranks wait for one another (bounded; awq_b200_workspace_check reports a timeout).
 * No counterpart in the reference, whose only inter-GPU mechanism is its symmetric heap
 * (runtime_lib/airgpu/symmetric_heap.cpp:172-312). */
/* The messages of the exchange are numbered by the launches that finished on a rank (a word behind the
 * rank's first slot) times the layer count: a set of receive slots belongs to one plan, and after a launch
 * that failed on any rank (AWQ_ERR_DEVICE_TIMEOUT from awq_b200_workspace_check, an argument error on one
 * rank only) all ranks must zero their slots and flag blocks together before the next launch. */
size_t awq_b200_ffn_stack_tp_slot_bytes(int H, int n_ranks);
int awq_b200_ffn_stack_decode_tp_bf16(const void *plan, int n_layers, const uint16_t *x,
                                      uint16_t *out, uint16_t *inter, float eps, int B, int H,
                                      int I_local, int group_size, void *const *peer_base,
                                      size_t slot_stride, size_t flag_offset, int n_ranks, int rank,
                                      void *workspace, size_t workspace_bytes, awq_stream_t stream);

/* ---- prefill GEMM ----------------------------------------------------------------------
 * C bf16 [M, N] = bf16(A[M, K] @ W), f32 accumulate.  Replaces
 * matmul_int4_bf16_packed_f32 / zero_vectorized_f32_mn / f32_to_bf16_mn
 * (mv_int4_bf16.cc:181-389), golden matrix_multiplication/int4_awq/matmul_int4_packed.py:89-105. */
int awq_b200_gemm_bf16(const uint16_t *A, const int32_t *qweight, const int32_t *qzeros,
                       const uint16_t *scales, uint16_t *C, int M, int K, int N, int group_size,
                       awq_stream_t stream);

/* The same GEMM with the decode block's epilogues, for token batches too large for the GEMV kernel
 * (M = batch, the batched-decode golden of matmul_int4_packed.py:97-105):
 *   swiglu != 0: W is gate/up column-interleaved [K, N]; C bf16 [M, N/2] = swiglu(bf16(sum_2i), bf16(sum_2i+1))
 *                with the rounding points of matvec_int4_swiglu_rms.py:511-516;
 *   residual != NULL: C bf16 [M, N] = bf16(sum + residual), residual bf16 [M, N] joining the f32 sum
 *                before the one rounding (matvec_int4_packed_add.py:313-319).
 * Tensor-core kernel only (AWQ_ERR_UNSUPPORTED where it does not apply). */
int awq_b200_gemm_fused_bf16(const uint16_t *A, const int32_t *qweight, const int32_t *qzeros,
                             const uint16_t *scales, const uint16_t *residual, uint16_t *C, int swiglu,
                             int M, int K, int N, int group_size, awq_stream_t stream);

/* The same three products for a decode batch of 9 <= M <= 64 token rows (the batched-decode golden of
 * matmul_int4_packed.py:97-105 with M = batch; the reference's decode kernels take one row at a time,
 * mv_int4_bf16.cc:403-436).  Bound by streaming the weights like the GEMV, so the work is cut into
 * (256-column tile, 128-row k-block) units dealt evenly to the SMs; the f32 sums of each SM's share of a
 * tile go through `workspace` (awq_b200_gemm_decode_workspace_bytes(M, N) bytes; no initialisation
 * needed; calls sharing it must not overlap) and a second small launch adds them in a fixed order and
 * applies the epilogue, so results do not depend on the order of arrival.  Two kernel launches per call.
 * group_size 128, K % 128 == 0, N % 32 == 0 (AWQ_ERR_UNSUPPORTED otherwise). */
size_t awq_b200_gemm_decode_workspace_bytes(int M, int N);
int awq_b200_gemm_decode_bf16(const uint16_t *A, const int32_t *qweight, const int32_t *qzeros,
                              const uint16_t *scales, const uint16_t *residual, uint16_t *C, int swiglu,
                              int M, int K, int N, int group_size, void *workspace,
                              size_t workspace_bytes, awq_stream_t stream);

/* The same product with the f32 sums as output, C f32 [M, N]: a tensor-parallel rank's partial of the down
 * projection, to be added up across the ranks (no counterpart in the reference, which has no multi-GPU
 * form of this path). */
int awq_b200_gemm_decode_f32(const uint16_t *A, const int32_t *qweight, const int32_t *qzeros,
                             const uint16_t *scales, float *C, int M, int K, int N, int group_size,
                             void *workspace, size_t workspace_bytes, awq_stream_t stream);

/* General form of the two above.  A in `a_format` (AWQ_ACT_*): with fp16 token rows the weights are
 * dequantised to fp16 as well ((q - z) exact, one rounding of the product with the scale to 11
 * significant bits, where the bf16 form keeps 8), which is what a decode stack of several layers wants
 * between its kernels.  C in `c_format`: AWQ_ACT_BF16 (any epilogue), AWQ_ACT_F16 (plain or SwiGLU; the
 * SwiGLU value is rounded to bf16 as the reference does, then stored as fp16) or AWQ_OUT_F32 (plain sums,
 * C f32 [M, N]).  Scales below 2^-14 lose precision as fp16 (see AWQ_ACT_*). */
int awq_b200_gemm_decode_act(const void *A, int a_format, const int32_t *qweight, const int32_t *qzeros,
                             const uint16_t *scales, const uint16_t *residual, void *C, int c_format,
                             int swiglu, int M, int K, int N, int group_size, void *workspace,
                             size_t workspace_bytes, awq_stream_t stream);

/* The same product for M <= 32 token rows with the packed nibbles themselves as the tensor core's operand
 * (a nibble q in a byte is the e4m3 number q * 2^-9) and the token rows split into two e4m3 pieces per
 * element (exact for a value of 8 significant bits, i.e. any bf16 value or an fp16 copy of one, within
 * 2^-14 of its row's largest magnitude; a genuine fp16 value is rounded to 8 significant bits, as a bf16
 * conversion would); zero point and scale are
 * applied to the per-group sums in f32, as the reference's golden does, so no weight is rounded.  Three
 * launches: the split of the token rows, the product, the addition of the partial sums.  Arguments as
 * awq_b200_gemm_decode_act; the workspace also holds the split rows, hence K in its size. */
size_t awq_b200_gemm_decode_f8_workspace_bytes(int M, int K, int N);
int awq_b200_gemm_decode_f8(const void *A, int a_format, const int32_t *qweight, const int32_t *qzeros,
                            const uint16_t *scales, const uint16_t *residual, void *C, int c_format,
                            int swiglu, int M, int K, int N, int group_size, void *workspace,
                            size_t workspace_bytes, awq_stream_t stream);

/* Synchronise `stream` and report whether a tensor-core GEMM (prefill or batched decode) gave up on a
 * bounded device-side wait since the last check (AWQ_ERR_DEVICE_TIMEOUT); the counterpart of
 * xrt.py:204-218. */
int awq_b200_gemm_check(awq_stream_t stream);

/* Choose the prefill kernel: 0 = automatic, 1 = generic CUDA-core kernel, 2 = tcgen05 kernel with the
 * dequantised weights as a shared-memory tile, 3 = tcgen05 kernel with the dequantised weights in tensor
 * memory (2 and 3: AWQ_ERR_UNSUPPORTED where they cannot run; automatic takes 3 from 1024 rows on). */
int awq_b200_set_gemm_kernel(int mode);

/* ---- bf16 sibling path (un-quantised weights) ----------------------------------------------
 * y bf16 [M, N] = bf16(x[M, K] @ W[N, K]^T): the GEMV/GEMM of ffn_swiglu/decode/ffn_kernels.cc:52-117
 * (matvec_vectorized_bf16_bf16) and ffn_swiglu/prefill/ffn_kernels.cc:55-83 (matmul_bf16).
 * out = bf16(g * sigmoid(g) * u): swiglu_bf16 (ffn_kernels.cc:123-151), golden ffn_decode.py:309-311. */
int awq_b200_linear_bf16(const uint16_t *x, const uint16_t *W, uint16_t *y, int M, int K, int N,
                         awq_stream_t stream);
int awq_b200_silu_mul_bf16(const uint16_t *gate, const uint16_t *up, uint16_t *out, size_t n,
                           awq_stream_t stream);

/* ---- half-split rotary embedding -----------------------------------------------------------
 * out[b, h, i] = x[i] cos[i] - x[i + d/2] sin[i]; out[b, h, i + d/2] = x[i] sin[i] + x[i + d/2] cos[i]
 * for every head h of d = head_dim values, f32 arithmetic, one bf16 rounding: rope_halfsplit.cc as
 * linked by llms/llama32_1b_int4/multi_launch_builder/rms_qkv_int4_rope_multi.py:237-333, golden
 * _rope_ref (:533-551).  x and out are [B, n_heads * head_dim] with row strides in elements (so Q
 * and K can be rotated in place inside one [B, Nq + 2 Nkv] projection output); lut is bf16
 * [B, head_dim], one row [cos_0 .. cos_{d/2-1} | sin_0 .. sin_{d/2-1}] per token
 * (llama32_1b/llama32_1b_weights.py:395-440).  out may alias x. */
int awq_b200_rope_halfsplit_bf16(const uint16_t *x, size_t x_stride, const uint16_t *lut,
                                 uint16_t *out, size_t out_stride, int B, int n_heads,
                                 int head_dim, awq_stream_t stream);

/* ---- layout converters (once per weight) ------------------------------------------------
 * Layout B is mlir-air's logical form (matvec_int4_packed.py:346-350):
 *   A_q uint8 [M, K/2] (low nibble = even k), A_s bf16 [K/gs, M], A_z uint8 [K/gs, M], M = N.
 * B -> A inverts repack_hf_awq_linear (awq_repacker.py:85-109); A -> B restates it. */
int awq_b200_repack_B_to_A(const uint8_t *A_q, const uint16_t *A_s, const uint8_t *A_z,
                           int32_t *qweight, int32_t *qzeros, uint16_t *scales, int M, int K,
                           int group_size, awq_stream_t stream);
int awq_b200_repack_A_to_B(const int32_t *qweight, const int32_t *qzeros, const uint16_t *scales,
                           uint8_t *A_q, uint16_t *A_s, uint8_t *A_z, int M, int K, int group_size,
                           awq_stream_t stream);

/* Layout C, the per-tile packed buffer the reference hands its NPU kernels, back to layout B:
 * `packed` holds M / m_tile x K / k_chunk tiles in (row block, k chunk) order, each
 * [Q: m_tile x k_chunk/2 bytes | S: (k_chunk/gs) x m_tile bf16 | Z: (k_chunk/gs) x m_tile bytes]
 * (tile_bytes = m_tile k_chunk / 2 + 3 (k_chunk / gs) m_tile; 8576 at the GEMV defaults 8 / 2048 / 128).
 * Inverts pack_inputs of matrix_vector_multiplication/int4_awq/matvec_int4_packed.py:57-103
 * (any N_CORES / M_PER_LAUNCH: launches, cores and outer steps enumerate consecutive row blocks) and
 * of matrix_multiplication/int4_awq/matmul_int4_packed.py:57-86 (M = N, m_tile = N_TILE), and so
 * what awq_pack_for_npu (llms/llama32_1b_int4/awq_pack.py:112-146) produced.  Follow with
 * awq_b200_repack_B_to_A to get the layout the kernels read. */
int awq_b200_repack_C_to_B(const uint8_t *packed, uint8_t *A_q, uint16_t *A_s, uint8_t *A_z, int M,
                           int K, int group_size, int m_tile, int k_chunk, awq_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* AWQ_B200_H_ */
