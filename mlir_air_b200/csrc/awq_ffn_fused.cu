// Decode FFN layer stack in ONE persistent launch:
//
//   for each layer:  h <- h + down( swiglu( gateup . rmsnorm(h, gamma) ) )        (batch <= 8)
//
// the LGU -> LD chain the reference fuses per layer into one multi-launch ELF
// (llms/llama32_1b_int4/multi_launch_builder/o_gemv_ffn_int4_multi.py:9-12), here for all layers of
// the stack, so the weight stream from HBM never stops at a kernel boundary.
//
// Same units, shared-memory ring, nibble decode and split-K reduction as the single-product
// stream-K kernel (awq_gemv_streamk.cu); what is new is how the phases chain inside the launch:
//
//  * An SM's units of a phase are one contiguous range of the phase's strip-major unit list, and
//    the CTA's two halves share it dynamically: half 0 takes units from the front of the range,
//    half 1 from the back, each claiming its next unit from a shared-memory counter when its ring
//    has room, until the two meet.  Neither waits for the other and the faster half simply takes
//    more units, so both reach the end of the phase within about a unit of each other.  (With the
//    range cut in the middle the two halves of an SM finished a gate/up phase up to 7 us apart: the
//    hardware does not share issue slots evenly between two sets of warps, and which set it
//    prefers varies from SM to SM.)  The loader of a half writes a descriptor of the claimed unit
//    into shared memory next to the stage, and an end-of-phase marker takes one ring turn.
//  * The loader keeps the ring full across phase changes: the weights of the next phase's first
//    units are requested before the phase's activations exist.
//  * A phase's activations exist when every 64-column sub-strip of the previous phase has been
//    finalised; finalising warps count up `done_gu` / `done_d` in global memory (release), the
//    loaders wait for the count (acquire, bounded).  All CTAs of the launch are resident
//    (one per SM), so the wait cannot starve anybody.
//  * RMSNorm has no phase of its own.  The warp that finalises a down sub-strip adds the squares
//    of its new hidden values to the layer's per-row sum; a gate/up unit's stage receives the raw
//    8 x 128 hidden values and the 128 norm weights of its k range by TMA with the weights, and
//    the normaliser warp turns them into activations in place (bf16 rounding, then the fp16 form
//    the MMA multiplies) as soon as they land.
//  * The loader also prefetches into L2, a few units ahead of the ring and across phase and
//    layer boundaries (weights depend on nothing), so HBM keeps streaming while a phase change
//    waits for the slowest CTA; the ring then refills from L2.
//  * Tensor-parallel ranks run the same launch on their shards.  The warp that finishes a down
//    sub-strip then stores its f32 partial sums straight into the receive area of every rank
//    (its own included) as 8-byte words, value and the exchange's tag together, so a word is
//    either absent or complete and needs no fence and no flag of its own.  On every rank one
//    normaliser warp per sub-strip polls the words of all ranks, adds them in rank order (every
//    rank gets the same bits), and ends the sub-strip exactly as a single GPU does: residual,
//    bf16 hidden state, squares for the next RMSNorm, the phase counter.  Kernels of different
//    GPUs wait for one another here, never two launches on one GPU.
//  * Rounding points are those of the separate kernels: bf16 normed activations, bf16 gate and
//    up sums before SwiGLU, bf16 SwiGLU output, bf16 hidden state.
#include <cudaTypedefs.h>
#include <cuda_fp16.h>

#include <mutex>
#include <vector>

#include "awq_common.cuh"
#include "awq_ptx.cuh"
#include "awq_streamk.cuh"

namespace awq {

int encode_tensor_map_2d(CUtensorMap *map, int dtype, const void *base, uint64_t dim0, uint64_t dim1,
                         uint64_t stride1_bytes, uint32_t box0, uint32_t box1, int swizzle);
int encode_tensor_map_3d(CUtensorMap *map, int dtype, const void *base, uint64_t dim0, uint64_t dim1, uint64_t dim2,
                         uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0, uint32_t box1, uint32_t box2,
                         int swizzle);

// One layer's tensor maps, device resident (TMA reads the descriptor from global memory).
struct alignas(128) FusedLayer {
    CUtensorMap w_gu, s_gu, z_gu;  // gate/up interleaved [H, 2I]
    CUtensorMap w_d, s_d, z_d;     // down [I, H]
    const uint16_t *gamma;         // bf16 [H]
};
static_assert(sizeof(FusedLayer) % 128 == 0, "tensor maps must stay 64-byte aligned in the array");

constexpr int FF_MAX_LAYERS = 1024;  // 2 claim words per layer in shared memory
// State of one launch in the workspace, zeroed by the launcher: two phase counters; per k-group of the down
// projection (128 SwiGLU outputs) how many of the four 32-output sub-strips that feed it have been finished so far
// (it grows by four per layer), and per k-group of the gate/up projection (128 hidden values) how many of its two
// 64-column sub-strips (two per layer); then one f32 sum of squares per (layer boundary, batch row).
constexpr size_t FF_STATE_OFF = SK_WS_END;
constexpr size_t FF_STATE_HEADER = 64;
constexpr int FF_READY_WORDS = 1024;  // >= SK_MAX_GROUPS, per direction
constexpr size_t FF_READY_BYTES = 2 * FF_READY_WORDS * sizeof(int);
__host__ __device__ constexpr size_t ff_state_bytes(int n_layers) {
    return FF_STATE_HEADER + FF_READY_BYTES + (size_t)(n_layers + 1) * 8 * sizeof(float);
}

__device__ __forceinline__ int ld_acquire_gpu(const int *p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Wait until *ctr >= target; gives up after `limit` cycles.
__device__ __forceinline__ bool wait_count(const int *ctr, int target, long long limit) {
    if (ld_acquire_gpu(ctr) >= target) return true;
    const long long t0 = clock64();
    while (ld_acquire_gpu(ctr) < target) {
        if (clock64() - t0 > limit) return false;
        __nanosleep(64);
    }
    return true;
}

// One CTA per SM, made of two independent halves.  A half is what a CTA of the single-product
// kernel is: 8 consumer warps and its own 3-stage ring, plus a loader warp (one thread drives
// TMA) and a normaliser warp.  The SM's units of a phase are one contiguous range that the two
// halves take from both ends.
constexpr int FF_HALVES = 2;
constexpr int FF_CONSUMER_WARPS = FF_HALVES * SK_CONSUMER_WARPS;
constexpr int FF_WARPS = FF_CONSUMER_WARPS + 2 * FF_HALVES;
constexpr int FF_THREADS = FF_WARPS * 32;
constexpr int FF_OFF_GAMMA = SK_OFF_Z + SK_Z_BYTES;  // 128 bf16 norm weights of the unit's k range
constexpr int FF_GAMMA_BYTES = SK_GROUP * 2;
constexpr int FF_RING_BYTES = SK_STAGES * SK_STAGE_BYTES;
constexpr int FF_BARS_PER_HALF = 3 * SK_STAGES;
constexpr int FF_BAR_BYTES = FF_HALVES * FF_BARS_PER_HALF * 8;
constexpr int FF_DESC_BYTES = FF_HALVES * SK_STAGES * 16;  // per stage: layer, phase (| FF_END), strip, group
constexpr int FF_CLAIM_WORDS = 2 * FF_MAX_LAYERS;          // units of this SM taken so far, one word per phase
constexpr int FF_END = 2;                                  // descriptor flag: the half has no more units in this phase
constexpr int FF_SMEM_BYTES = FF_HALVES * FF_RING_BYTES + FF_BAR_BYTES + FF_DESC_BYTES + FF_CLAIM_WORDS * 4 + 16 + 1024;
static_assert(FF_OFF_GAMMA + FF_GAMMA_BYTES <= SK_STAGE_BYTES, "stage too small");
static_assert(FF_SMEM_BYTES + 1024 + 128 <= 228 * 1024, "shared memory budget");

__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap *map, int x, int y) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];" ::"l"(map), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_prefetch_l2_3d(const CUtensorMap *map, int x, int y, int z, uint64_t policy) {
    asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.L2::cache_hint [%0, {%1, %2, %3}], %4;" ::"l"(map), "r"(x), "r"(y),
                 "r"(z), "l"(policy)
                 : "memory");
}
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

struct FusedArgs {
    const FusedLayer *layers;
    int n_layers;
    const uint16_t *x;  // bf16 [B, H] input hidden state
    uint16_t *out;      // bf16 [B, H] hidden state after every layer (updated in place from layer 1 on)
    uint16_t *inter;    // fp16 [B, I] SwiGLU output of the current layer
    float eps;
    int B, H, I;
    int lookahead;  // units the L2 prefetch runs ahead of the shared-memory ring
    unsigned long long *accum;  // split-K accumulator words (zero between uses): gate/up strips, then down strips
    int *err_flag;
    int *state;     // done_gu, done_d, ..., then sumsq[(n_layers + 1) * 8]
    // Tensor parallelism (tp_n > 1): this rank holds a shard of every layer (gate/up columns, down
    // rows).  Receive area of rank r, slot s: for every source rank and every 64-column sub-strip of
    // the hidden state 16 x 32 words of (tag << 32 | f32 bits), laid out so that a warp's store and
    // load instructions touch 256 consecutive bytes.  Successive exchanges alternate between the slots.
    int tp_n, tp_rank;
    unsigned long long *ll_recv[2][TP_MAX_RANKS];  // every rank's receive slots, mapped into this GPU's address space
    unsigned int *epoch;                           // launches so far on this rank (base of the tags), in peer memory
    long long wait_limit;                          // cycles after which a device-side wait gives up
    int w3d_gu, w3d_d;  // the weight tensor map of a phase is 3-D: one copy fetches both 256-column boxes of a unit
    int per_group;      // a down unit starts when the sub-strips that feed its k-group are finished, not when all of gate/up is
};
constexpr int FF_LL_WORDS = 16 * 32;  // words of one sub-strip from one rank

__device__ __forceinline__ void st_relaxed_sys_u64(unsigned long long *p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys_u64(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// The unit range [lo, hi) of this SM in a phase of U units.
__device__ __forceinline__ void ff_sm_range(long long U, int &lo, int &hi) {
    const long long S = gridDim.x, s = blockIdx.x;
    lo = (int)(s * U / S);
    hi = (int)((s + 1) * U / S);
}

// Take one more unit of a phase (n units in this SM's range) if any is left: one shared-memory atomic on
// the phase's own word, which starts at zero.
__device__ __forceinline__ bool ff_claim(unsigned int *word, int n) { return atomicAdd(word, 1u) < (unsigned int)n; }

// End of a down sub-strip: lane's 2 x 8 finished sums of batch row b at columns n + 32 h + i.
// hidden state = bf16(sum + residual), its squares go to the next layer's RMSNorm sums.  `res0`,
// `res1`: the residual values, loaded by the caller (before it waited for the sums).
__device__ __forceinline__ void ff_down_epilogue(const float (&own)[2][8], const uint4 (&rres)[2], uint16_t *out, float *sumsq_next,
                                                 int B, int N, int n, int b, int lane) {
    float ss = 0.f;
    if (b < B) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int nh = n + 32 * h;
            if (nh >= N) continue;
            const uint32_t rw[4] = {rres[h].x, rres[h].y, rres[h].z, rres[h].w};
            uint32_t o[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                o[i] = pack_bf16x2(own[h][2 * i] + bf16x2_lo(rw[i]), own[h][2 * i + 1] + bf16x2_hi(rw[i]));
                const float lo = bf16x2_lo(o[i]), hi = bf16x2_hi(o[i]);
                ss = fmaf(lo, lo, ss);
                ss = fmaf(hi, hi, ss);
            }
            *reinterpret_cast<uint4 *>(out + (size_t)b * N + nh) = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
    // lanes with the same batch row differ in bits 3 and 4
    ss += __shfl_xor_sync(0xffffffffu, ss, 8);
    ss += __shfl_xor_sync(0xffffffffu, ss, 16);
    if (lane < 8 && b < B) atomicAdd(sumsq_next + b, ss);
}
__device__ __forceinline__ void ff_load_residual(uint4 (&rres)[2], const uint16_t *residual, int B, int N, int n, int b) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        rres[h] = make_uint4(0u, 0u, 0u, 0u);
        if (b < B && n + 32 * h < N) rres[h] = __ldcg(reinterpret_cast<const uint4 *>(residual + (size_t)b * N + n + 32 * h));
    }
}

__global__ void __launch_bounds__(FF_THREADS, 1)
ffn_fused_kernel(const __grid_constant__ CUtensorMap tmXi, const __grid_constant__ CUtensorMap tmH0,
                 const __grid_constant__ CUtensorMap tmH, const FusedArgs a) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ float red[FF_WARPS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // role and half of this warp: consumers 0-7 / 8-15, loaders 16 / 17, normalisers 18 / 19
    const int role = warp < FF_CONSUMER_WARPS ? 0 : (warp < FF_CONSUMER_WARPS + FF_HALVES ? 1 : 2);
    const int half = role == 0 ? warp / SK_CONSUMER_WARPS : (warp - FF_CONSUMER_WARPS) % FF_HALVES;
    const uint32_t smem_base = ((smem_u32(smem_raw) + 1023u) & ~1023u) + half * FF_RING_BYTES;
    const uint32_t bar_base =
        ((smem_u32(smem_raw) + 1023u) & ~1023u) + FF_HALVES * FF_RING_BYTES + half * FF_BARS_PER_HALF * 8;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };                      // TMA landed
    auto empty_bar = [&](int s) { return bar_base + 8u * (SK_STAGES + s); };       // consumers and normaliser done
    auto xready_bar = [&](int s) { return bar_base + 8u * (2 * SK_STAGES + s); };  // activations normalised
    const uint32_t aux_base = ((smem_u32(smem_raw) + 1023u) & ~1023u) + FF_HALVES * FF_RING_BYTES + FF_BAR_BYTES;
    auto desc_addr = [&](int s) { return aux_base + (uint32_t)(half * SK_STAGES + s) * 16u; };
    unsigned int *claim_words = reinterpret_cast<unsigned int *>(smem_raw + (aux_base - smem_u32(smem_raw)) + FF_DESC_BYTES);

    const int B = a.B, H = a.H, I = a.I;
    // phase 0: gate/up, K = H, N = 2I; phase 1: down, K = I, N = H
    const int G0 = H / SK_GROUP, V0 = (2 * I + SK_STRIP - 1) / SK_STRIP;
    const int G1 = I / SK_GROUP, V1 = (H + SK_STRIP - 1) / SK_STRIP;
    int *done_gu = a.state, *done_d = a.state + 1;
    const bool tp = a.tp_n > 1;
    // tensor parallel: exchanges so far on these buffers (all launches run the same number of layers); every
    // warp reads the count before anything of this launch can end
    const unsigned int exch0 = tp ? *a.epoch * (unsigned int)a.n_layers : 0u;
    int *ready_gu = a.state + FF_STATE_HEADER / sizeof(int), *ready_d = ready_gu + FF_READY_WORDS;
    float *sumsq = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(a.state) + FF_STATE_HEADER + FF_READY_BYTES);
    // Per-group readiness: a down unit needs only its own 128 SwiGLU outputs, so it starts as soon as the
    // four sub-strips that produce them are finished; an SM that is done with its gate/up units does not wait for the
    // slowest one.  In the other direction a gate/up unit's 128 raw hidden values are requested as soon as the two
    // down sub-strips that produce them are finished, but the normaliser warp turns them into activations only when the
    // whole down phase is over: the RMSNorm factor belongs to the whole row.  (Applying the factor to the finished sums
    // instead would lift that too and measured another 3 % faster, but it rounds h * gamma instead of h * rstd * gamma
    // to bf16, which is not the reference's rounding point: the distance to the oracle doubled, 1.2e-2 after four
    // layers.)
    const bool fg = a.per_group != 0;  // tensor parallel too: gate/up and down shards of a rank depend on each other only inside the rank

    if (role == 1 && lane == 0) {  // each loader sets up its half's barriers
        for (int s = 0; s < SK_STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), SK_CONSUMER_WARPS + 1);
            mbar_init(xready_bar(s), 1);
        }
        mbar_fence_init();
    }
    for (int i = threadIdx.x; i < 2 * a.n_layers; i += FF_THREADS) claim_words[i] = 0u;
    // sum of squares of the input rows (layer 0's RMSNorm): rows b, b + gridDim.x, ... per CTA
    for (int row_i = blockIdx.x; row_i < B; row_i += gridDim.x) {
        const uint16_t *row = a.x + (size_t)row_i * H;
        float ss = 0.f;
        for (int ch = threadIdx.x; ch < (H >> 3); ch += FF_THREADS) {
            const uint4 t = *reinterpret_cast<const uint4 *>(row + 8 * ch);
            const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float lo = bf16x2_lo(w[e]), hi = bf16x2_hi(w[e]);
                ss = fmaf(lo, lo, ss);
                ss = fmaf(hi, hi, ss);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        if (threadIdx.x == 0) {
            float total = 0.f;
            for (int w = 0; w < FF_WARPS; ++w) total += red[w];
            sumsq[row_i] = total;
            __threadfence();
            atomicAdd(done_d, 1);
        }
        __syncthreads();
    }
    __syncthreads();

    // this SM's unit range of a gate/up phase and of a down phase (the same in every layer), and how far into it
    // (from its own end) a half prefetches: a little past the middle
    int lo0, hi0, lo1, hi1;
    ff_sm_range((long long)V0 * G0, lo0, hi0);
    ff_sm_range((long long)V1 * G1, lo1, hi1);
    const int lim0 = (hi0 - lo0) / 2 + 2 < hi0 - lo0 ? (hi0 - lo0) / 2 + 2 : hi0 - lo0;
    const int lim1 = (hi1 - lo1) / 2 + 2 < hi1 - lo1 ? (hi1 - lo1) / 2 + 2 : hi1 - lo1;
    auto maps = [&](int l, int p, const CUtensorMap *&tmW, const CUtensorMap *&tmS, const CUtensorMap *&tmZ) {
        const FusedLayer *Ly = a.layers + l;
        tmW = p ? &Ly->w_d : &Ly->w_gu;
        tmS = p ? &Ly->s_d : &Ly->s_gu;
        tmZ = p ? &Ly->z_d : &Ly->z_gu;
    };
    // this half's c-th unit of a range [lo, hi): half 0 walks up from lo, half 1 down from hi - 1
    auto unit_of = [&](int lo, int hi, int c) { return half ? hi - 1 - c : lo + c; };
    // Request this half's c-th unit of phase (l, p) into L2.  Weights depend on nothing, so HBM keeps streaming
    // while a phase waits.  Issued by the normaliser warp: the loader thread has no time to spare.
    auto prefetch_unit = [&](int l, int p, int c) {
        const int G = p ? G1 : G0;
        const int u = p ? unit_of(lo1, hi1, c) : unit_of(lo0, hi0, c), v = u / G, g = u - v * G;
        const CUtensorMap *tmW, *tmS, *tmZ;
        maps(l, p, tmW, tmS, tmZ);
        if (p ? a.w3d_d : a.w3d_gu) {
            tma_prefetch_l2_3d(tmW, 0, g * SK_GROUP, v * (SK_STRIP / SK_BOX_COLS), l2_policy_evict_first());
        } else {
#pragma unroll
            for (int bx = 0; bx < SK_STRIP / SK_BOX_COLS; ++bx)
                tma_prefetch_l2_2d(tmW, (v * SK_STRIP + bx * SK_BOX_COLS) / 8, g * SK_GROUP);
        }
    };

    if (role == 1) {
        // ------------------------------ loader (one thread) ------------------------------
        if (lane != 0) return;
        const uint64_t stream_policy = l2_policy_evict_first();
        int issued = 0;  // ring turns so far (units and end-of-phase markers)
        auto acquire_slot = [&](int &slot) -> bool {  // slot of ring turn `issued`, once its previous turn was released
            slot = issued % SK_STAGES;
            const int round = issued / SK_STAGES;
            if (round > 0 && !mbar_wait_bounded(empty_bar(slot), (round - 1) & 1, a.wait_limit)) {
                atomicExch(a.err_flag, 1);
                return false;
            }
            return true;
        };
        auto put_desc = [&](int slot, int l, int p, int v, int g) {
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(desc_addr(slot)), "r"(l), "r"(p), "r"(v), "r"(g) : "memory");
        };
        auto load_weights = [&](int slot, int l, int p, int v, int g) {
            const CUtensorMap *tmW, *tmS, *tmZ;
            maps(l, p, tmW, tmS, tmZ);
            const uint32_t st = smem_base + slot * SK_STAGE_BYTES;
            const uint32_t bar = full_bar(slot);
            put_desc(slot, l, p, v, g);  // before the arrive below, whose release makes it visible with the data
            mbar_expect_tx(bar, p ? SK_TX_BYTES : SK_TX_BYTES + FF_GAMMA_BYTES);
            if (p ? a.w3d_d : a.w3d_gu) {
                tma_load_3d_hint(st, tmW, 0, g * SK_GROUP, v * (SK_STRIP / SK_BOX_COLS), bar, stream_policy);
            } else {
#pragma unroll
                for (int bx = 0; bx < SK_STRIP / SK_BOX_COLS; ++bx)
                    tma_load_2d_hint(st + bx * SK_WBOX_BYTES, tmW, (v * SK_STRIP + bx * SK_BOX_COLS) / 8, g * SK_GROUP, bar,
                                     stream_policy);
            }
            tma_load_2d(st + SK_OFF_S, tmS, v * (SK_STRIP / 2), g, bar);  // the scales as 32-bit pairs: 512 in one box
            tma_load_2d(st + SK_OFF_Z, tmZ, v * (SK_STRIP / 8), g, bar);
        };
        auto load_activations = [&](int slot, int l, int p, int g) {
            const uint32_t st = smem_base + slot * SK_STAGE_BYTES;
            const uint32_t bar = full_bar(slot);
            // down: the SwiGLU output as it is; gate/up: the raw hidden state and the norm weights
            // of the unit's k range, which the normaliser warp turns into activations in place
            const CUtensorMap *tmX = p ? &tmXi : (l == 0 ? &tmH0 : &tmH);
            tma_load_3d(st + SK_OFF_X, tmX, 0, 0, g * (SK_GROUP / 64), bar);  // both [8 x 64] boxes of the group
            if (!p) bulk_load_1d(st + FF_OFF_GAMMA, a.layers[l].gamma + (size_t)g * SK_GROUP, FF_GAMMA_BYTES, bar);
        };
        for (int l = 0; l < a.n_layers; ++l) {
            for (int p = 0; p < 2; ++p) {
                const int G = p ? G1 : G0;
                const int lo = p ? lo1 : lo0, hi = p ? hi1 : hi0;
                unsigned int *word = claim_words + 2 * l + p;
                int mine = 0;  // units this half has taken in this phase
                bool more = true;
                // a phase begins: the weights of its first units do not depend on the previous phase
                int slots[SK_STAGES], gs[SK_STAGES], n_first = 0;
                while (n_first < SK_STAGES && (more = ff_claim(word, hi - lo))) {
                    const int u = unit_of(lo, hi, mine), v = u / G, g = u - v * G;
                    if (!acquire_slot(slots[n_first])) return;
                    load_weights(slots[n_first], l, p, v, g);
                    gs[n_first++] = g;
                    ++issued;
                    ++mine;
                }
                // the phase's activations exist once every sub-strip of the previous phase is finalised
                // (tensor parallel: a down sub-strip is finalised by the warp that added up all ranks' sums);
                // with per-group readiness a unit's activations exist once the sub-strips that cover its k-group are
                const int target = p ? (l + 1) * V0 * SK_CONSUMER_WARPS : B + l * V1 * SK_CONSUMER_WARPS;
                bool phase_open = false;
                auto unit_ready = [&](int g) -> bool {
                    if (phase_open) return true;
                    if (!fg || (!p && tp)) {  // tensor parallel: the hidden state comes out of the exchange, which counts only the phase
                        if (!wait_count(p ? done_gu : done_d, target, a.wait_limit)) return false;
                        phase_open = true;
                    } else if (ld_acquire_gpu(p ? done_gu : done_d) >= target) {
                        phase_open = true;
                    } else if (p) {
                        if (!wait_count(ready_gu + g, 4 * (l + 1), a.wait_limit)) return false;
                    } else if (l > 0) {
                        if (!wait_count(ready_d + g, 2 * l, a.wait_limit)) return false;
                    }  // layer 0 reads the caller's input
                    fence_proxy_async_all();  // generic-proxy writes of the previous phase before the tensor copies read them
                    return true;
                };
                for (int i = 0; i < n_first; ++i) {
                    if (!unit_ready(gs[i])) {
                        atomicExch(a.err_flag, 3);
                        return;
                    }
                    load_activations(slots[i], l, p, gs[i]);
                }
                while (more && (more = ff_claim(word, hi - lo))) {
                    const int u = unit_of(lo, hi, mine), v = u / G, g = u - v * G;
                    int slot;
                    if (!acquire_slot(slot)) return;
                    load_weights(slot, l, p, v, g);
                    if (!unit_ready(g)) {
                        atomicExch(a.err_flag, 3);
                        return;
                    }
                    load_activations(slot, l, p, g);
                    ++issued;
                    ++mine;
                }
                // the range is used up: one ring turn tells this half's warps that the phase is over for them
                int slot;
                if (!acquire_slot(slot)) return;
                put_desc(slot, l, p | FF_END, 0, 0);
                mbar_arrive(full_bar(slot));
                ++issued;
            }
        }
        return;
    }

    auto read_desc = [&](int slot, int &l, int &p, int &v, int &g) {
        const uint4 d = lds128(desc_addr(slot));
        l = (int)d.x;
        p = (int)d.y;
        v = (int)d.z;
        g = (int)d.w;
    };

    if (role == 2) {
        // ------------------------------ normaliser warp ------------------------------
        // Follows the half's ring turn by turn.  RMSNorm of a gate/up unit's 8 x 128 hidden values, in place in
        // the stage: lane (r, q4) takes 16-byte chunks q4, q4 + 4, q4 + 8, q4 + 12 of batch row r where the
        // tensor copy of the 128B-swizzled [8 x 64] box pair put them; bf16 rounding, then the fp16 form
        const int r = lane >> 2, q4 = lane & 3;
        int rstd_layer = -1;
        float rstd = 0.f;
        for (int turn = 0;; ++turn) {
            const int slot = turn % SK_STAGES;
            if (!mbar_wait_bounded(full_bar(slot), (turn / SK_STAGES) & 1, a.wait_limit)) {
                if (lane == 0) atomicExch(a.err_flag, 4);
                return;
            }
            int l, p, v, g;
            read_desc(slot, l, p, v, g);
            if (lane == 0 && a.lookahead > 0) {
                // keep L2 `lookahead` units ahead of what this half is loading: its own direction inside the
                // phase, and at the end of a phase its first units of the next one
                if (p & FF_END) {
                    const int nl = (p & 1) ? l + 1 : l, np = (p & 1) ^ 1;
                    if (nl < a.n_layers)
                        for (int c = 0; c < a.lookahead && c < (np ? lim1 : lim0); ++c) prefetch_unit(nl, np, c);
                } else {
                    const int u = v * (p ? G1 : G0) + g;
                    const int c = (p ? (half ? hi1 - 1 - u : u - lo1) : (half ? hi0 - 1 - u : u - lo0)) + SK_STAGES - 1 + a.lookahead;
                    if (c < (p ? lim1 : lim0)) prefetch_unit(l, p, c);
                }
            }
            if (p == 0) {
                if (rstd_layer != l) {
                    // the row sums are complete when the whole down phase before this layer is (with per-group readiness
                    // the loader may have requested h before that)
                    if (fg && !tp) {
                        int ok = 0;
                        if (lane == 0) ok = wait_count(done_d, B + l * V1 * SK_CONSUMER_WARPS, a.wait_limit) ? 1 : 0;
                        if (!__shfl_sync(0xffffffffu, ok, 0)) {
                            if (lane == 0) atomicExch(a.err_flag, 3);
                            return;
                        }
                    }
                    rstd_layer = l;
                    if (r < B) {
                        const float total = __ldcg(sumsq + (size_t)l * 8 + r);
                        rstd = (float)(1.0 / sqrt((double)(total / (float)H) + (double)a.eps));
                    }
                }
                const uint32_t st = smem_base + slot * SK_STAGE_BYTES;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int ch = q4 + 4 * j;
                    const uint32_t addr = st + SK_OFF_X + (ch >> 3) * 1024 + r * 128 + (((ch & 7) ^ r) << 4);
                    const uint4 hv = lds128(addr), gv = lds128(st + FF_OFF_GAMMA + ch * 16);
                    const uint32_t hw[4] = {hv.x, hv.y, hv.z, hv.w}, gw[4] = {gv.x, gv.y, gv.z, gv.w};
                    uint32_t o[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float lo = bf16_bits_to_f32(f32_to_bf16_bits((bf16x2_lo(hw[e]) * rstd) * bf16x2_lo(gw[e])));
                        const float hi = bf16_bits_to_f32(f32_to_bf16_bits((bf16x2_hi(hw[e]) * rstd) * bf16x2_hi(gw[e])));
                        o[e] = (uint32_t)bf16_value_to_f16_bits(lo) | ((uint32_t)bf16_value_to_f16_bits(hi) << 16);
                    }
                    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(o[0]), "r"(o[1]), "r"(o[2]),
                                 "r"(o[3])
                                 : "memory");
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(xready_bar(slot));
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar(slot));  // the descriptor has been read: the turn may be reused
            if (!(p & FF_END)) continue;
            p &= 1;
            if (tp && p) {
                // ---- this layer's exchange: sub-strips gw, gw + W, ... of the hidden state are ended here ----
                const unsigned int tag = exch0 + (unsigned int)l + 1u;
                const int sl = (int)((exch0 + (unsigned int)l) & 1u);
                const int n_sub = V1 * SK_CONSUMER_WARPS;
                const uint16_t *hres = l == 0 ? a.x : a.out;
                const int W = 2 * (int)gridDim.x, gw = 2 * (int)blockIdx.x + half;
                for (int sub = gw; sub < n_sub; sub += W) {
                    const SkLane sg(sub % SK_CONSUMER_WARPS, lane);
                    const int sb = 2 * sg.t4 + sg.odd, n = (sub / SK_CONSUMER_WARPS) * SK_STRIP + sg.colw;
                    uint4 rres[2];
                    ff_load_residual(rres, hres, B, H, n, sb);
                    float own[2][8];
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int i = 0; i < 8; ++i) own[h][i] = 0.f;
                    bool good = true;
                    const long long t0 = clock64();
                    for (int rk = 0; rk < a.tp_n && good; ++rk) {
                        const unsigned long long *src =
                            a.ll_recv[sl][a.tp_rank] + ((size_t)rk * n_sub + sub) * FF_LL_WORDS + lane;
                        unsigned long long w[16];
                        bool all;
                        do {
#pragma unroll
                            for (int i = 0; i < 16; ++i) w[i] = ld_relaxed_sys_u64(src + i * 32);
                            all = true;
#pragma unroll
                            for (int i = 0; i < 16; ++i) all = all && (unsigned int)(w[i] >> 32) == tag;
                            all = __all_sync(0xffffffffu, all);
                            // the lanes must leave together: one lane's clock decides for the warp
                            const bool late = __shfl_sync(0xffffffffu, clock64() - t0 > a.wait_limit ? 1 : 0, 0) != 0;
                            if (!all && late) good = false;
                        } while (!all && good);
                        if (good) {
#pragma unroll
                            for (int i = 0; i < 16; ++i) own[i >> 3][i & 7] += __uint_as_float((unsigned int)w[i]);
                        }
                    }
                    if (!good) {
                        if (lane == 0) atomicExch(a.err_flag, 6);
                        return;
                    }
                    ff_down_epilogue(own, rres, a.out, sumsq + (size_t)(l + 1) * 8, B, H, n, sb, lane);
                    __threadfence();
                    __syncwarp();
                    if (lane == 0) atomicAdd(done_d, 1);
                }
            }
            if (p && l == a.n_layers - 1) break;
        }
        if (tp && blockIdx.x == 0 && half == 0 && lane == 0) *a.epoch = exch0 / (unsigned int)a.n_layers + 1u;
        return;
    }

    // ------------------------------ consumers ------------------------------
    const int cw = warp % SK_CONSUMER_WARPS;  // this warp's 64 columns of every strip
    const SkLane geo(cw, lane);
    const int t4 = geo.t4, odd = geo.odd, colw = geo.colw;
    const int b = 2 * t4 + odd;  // batch row of this lane after the lane exchange
    bool failed = false;
    uint32_t xr_parity = 0;  // bit s: parity of the next completion of xready_bar(s) (only gate/up units use it)
    float res[4][4];
    int cur_l = 0, cur_p = 0, cur_v = -1, seg_groups = 0;  // strip being accumulated, k groups of it added so far

    // Hand over what this warp accumulated for strip cur_v of phase (cur_l, cur_p).
    auto flush = [&]() {
        const int l = cur_l, p = cur_p, v = cur_v;
        const int G = p ? G1 : G0, N = p ? H : 2 * I;
        float own[2][8];
        sk_lane_exchange(res, odd, own);
        const int n = v * SK_STRIP + colw;
        // a strip shared with other halves: value and progress travel in one 64-bit atomic per sum; the warp
        // whose add completes the count has the total (gate/up and down strips use separate accumulators)
        if (seg_groups != G &&
            !sk_handover(a.accum + ((size_t)((p ? V0 : 0) + v) * SK_CONSUMER_WARPS + cw) * SK_ACC_WORDS, own, seg_groups, G, lane,
                         a.wait_limit, a.err_flag))
            return;
        if (failed) return;
        if (!p) {
            sk_epilogue<EPI_SWIGLU>(own, nullptr, a.inter, B, N, n, b, 1);
        } else if (tp) {
            // this rank's sums of the sub-strip go to every rank, value and tag in one 8-byte word; the
            // warp that collects the sub-strip on each rank ends it
            const unsigned long long tag = (unsigned long long)(exch0 + (unsigned int)l + 1u) << 32;
            const int sl = (int)((exch0 + (unsigned int)l) & 1u);
            const size_t w0 = ((size_t)a.tp_rank * (V1 * SK_CONSUMER_WARPS) + v * SK_CONSUMER_WARPS + cw) * FF_LL_WORDS + lane;
            for (int rk = 0; rk < a.tp_n; ++rk) {
                unsigned long long *dst = a.ll_recv[sl][(a.tp_rank + rk) % a.tp_n] + w0;  // own rank first, then round the ring
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    st_relaxed_sys_u64(dst + i * 32, tag | (unsigned long long)__float_as_uint(own[i >> 3][i & 7]));
            }
            return;
        } else {
            // hidden state: bf16(sum + residual), and its squares for the next layer's RMSNorm
            uint4 rres[2];
            ff_load_residual(rres, l == 0 ? a.x : a.out, B, N, n, b);
            ff_down_epilogue(own, rres, a.out, sumsq + (size_t)(l + 1) * 8, B, N, n, b, lane);
        }
        __threadfence();
        __syncwarp();
        if (lane == 0) {
            // this sub-strip's 32 SwiGLU outputs are a quarter of down k-group 2 v + cw / 4; its 64 hidden values are half
            // of gate/up k-group 4 v + cw / 2
            if (fg) atomicAdd(p ? ready_d + 4 * v + cw / 2 : ready_gu + 2 * v + cw / 4, 1);
            atomicAdd(p ? done_d : done_gu, 1);
        }
    };

    for (int turn = 0;; ++turn) {
        const int slot = turn % SK_STAGES;
        int l = 0, p = 0, v = 0, g = 0;
        if (!failed && !mbar_wait_bounded(full_bar(slot), (turn / SK_STAGES) & 1, a.wait_limit)) {
            failed = true;
            if (lane == 0) atomicExch(a.err_flag, 2);
        }
        if (failed) break;  // nothing more can be trusted: leave (the other warps' waits run out too)
        read_desc(slot, l, p, v, g);
        if (p & FF_END) {
            // the half's last unit of this phase has been consumed
            if (cur_v >= 0) flush();
            cur_v = -1;
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar(slot));
            if ((p & 1) && l == a.n_layers - 1) break;
            continue;
        }
        if (cur_v >= 0 && v != cur_v) {  // units of one phase come strip by strip
            flush();
            cur_v = -1;
        }
        if (cur_v < 0) {
            cur_l = l;
            cur_p = p;
            cur_v = v;
            seg_groups = 0;
#pragma unroll
            for (int e = 0; e < 4; ++e)
#pragma unroll
                for (int q = 0; q < 4; ++q) res[e][q] = 0.f;
        }
        ++seg_groups;
        if (!p) {
            if (!mbar_wait_bounded(xready_bar(slot), (xr_parity >> slot) & 1u, a.wait_limit)) {
                failed = true;
                if (lane == 0) atomicExch(a.err_flag, 2);
                break;
            }
            xr_parity ^= 1u << slot;
        }
        sk_consume_unit<true>(smem_base + slot * SK_STAGE_BYTES, geo, res, empty_bar(slot), lane);
    }
}

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
static int g_ffn_lookahead = 0;  // measured: with the halves sharing an SM's units dynamically the L2 look-ahead no longer pays
void ffn_fused_set_lookahead(int units) { g_ffn_lookahead = units < 0 ? 0 : (units > 64 ? 64 : units); }
static int g_ffn_per_group = 1;
void ffn_fused_set_split(int per_group) { g_ffn_per_group = per_group != 0; }  // second tuning knob: 0 = a launch-wide barrier between phases

size_t ffn_fused_plan_bytes(int n_layers) { return (size_t)(n_layers > 0 ? n_layers : 0) * sizeof(FusedLayer); }

size_t ffn_fused_workspace_bytes(int n_layers) { return FF_STATE_OFF + ff_state_bytes(n_layers); }

// Receive area of one slot: for each rank and each 64-column sub-strip of the hidden state 16 x 32 words.
size_t ffn_fused_tp_slot_bytes(int H, int n_ranks) {
    return (size_t)(n_ranks > 0 ? n_ranks : 0) * ((H + SK_STRIP - 1) / SK_STRIP) * SK_CONSUMER_WARPS * FF_LL_WORDS * 8;
}

bool ffn_fused_supported(int B, int H, int I, int group_size) {
    return group_size == SK_GROUP && B >= 1 && B <= 8 && H > 0 && I > 0 && H % SK_GROUP == 0 && I % SK_GROUP == 0 &&
           (2 * I + SK_STRIP - 1) / SK_STRIP + (H + SK_STRIP - 1) / SK_STRIP <= SK_MAX_STRIPS && H / SK_GROUP <= SK_MAX_GROUPS &&
           I / SK_GROUP <= SK_MAX_GROUPS && device_is_sm100();
}

int ffn_fused_plan(void *plan_dev, size_t plan_bytes, int n_layers, const int32_t *const *qw_gateup,
                   const int32_t *const *qz_gateup, const uint16_t *const *s_gateup, const int32_t *const *qw_down,
                   const int32_t *const *qz_down, const uint16_t *const *s_down, const uint16_t *const *gamma, int H, int I,
                   int group_size) {
    AWQ_REQUIRE(n_layers >= 1 && n_layers <= FF_MAX_LAYERS, "ffn_stack_plan: 1..%d layers", FF_MAX_LAYERS);
    AWQ_REQUIRE(ffn_fused_supported(1, H, I, group_size),
                "ffn_stack_plan: needs group 128, hidden and intermediate sizes that are multiples of 128 (H=%d I=%d gs=%d)", H,
                I, group_size);
    AWQ_REQUIRE(plan_dev && plan_bytes >= ffn_fused_plan_bytes(n_layers), "ffn_stack_plan: plan buffer of %zu bytes needed",
                ffn_fused_plan_bytes(n_layers));
    AWQ_REQUIRE((reinterpret_cast<uintptr_t>(plan_dev) & 127u) == 0, "ffn_stack_plan: plan buffer must be 128-byte aligned");
    std::vector<FusedLayer> host((size_t)n_layers);
    const int N0 = 2 * I, nb0 = N0 / 8, G0 = H / SK_GROUP;
    const int N1 = H, nb1 = N1 / 8, G1 = I / SK_GROUP;
    for (int l = 0; l < n_layers; ++l) {
        AWQ_REQUIRE(qw_gateup[l] && qz_gateup[l] && s_gateup[l] && qw_down[l] && qz_down[l] && s_down[l] && gamma[l],
                    "ffn_stack_plan: null pointer in layer %d", l);
        AWQ_REQUIRE(aligned16(qw_gateup[l]) && aligned16(qz_gateup[l]) && aligned16(s_gateup[l]) && aligned16(qw_down[l]) &&
                        aligned16(qz_down[l]) && aligned16(s_down[l]) && aligned16(gamma[l]),
                    "ffn_stack_plan: pointers of layer %d must be 16-byte aligned", l);
        FusedLayer &L = host[(size_t)l];
        int rc;
        // weights: where the columns are whole 256-column boxes, a 3-D view (32 words, k rows, boxes) lets one copy
        // fetch both boxes of a unit; scales as 32-bit pairs, so that a strip's 512 fit one box of 256 elements
        auto weight_map = [&](CUtensorMap *m, const int32_t *qw, int nb, int K) {
            if (nb % 32 == 0)
                return encode_tensor_map_3d(m, CU_TENSOR_MAP_DATA_TYPE_INT32, qw, 32, K, nb / 32, (uint64_t)nb * 4, 128, 32,
                                            SK_GROUP, SK_STRIP / SK_BOX_COLS, CU_TENSOR_MAP_SWIZZLE_128B);
            return encode_tensor_map_2d(m, CU_TENSOR_MAP_DATA_TYPE_INT32, qw, nb, K, (uint64_t)nb * 4, 32, SK_GROUP,
                                        CU_TENSOR_MAP_SWIZZLE_128B);
        };
        if ((rc = weight_map(&L.w_gu, qw_gateup[l], nb0, H))) return rc;
        if ((rc = encode_tensor_map_2d(&L.s_gu, CU_TENSOR_MAP_DATA_TYPE_UINT32, s_gateup[l], N0 / 2, G0, (uint64_t)N0 * 2,
                                       SK_STRIP / 2, 1, CU_TENSOR_MAP_SWIZZLE_NONE)))
            return rc;
        if ((rc = encode_tensor_map_2d(&L.z_gu, CU_TENSOR_MAP_DATA_TYPE_INT32, qz_gateup[l], nb0, G0, (uint64_t)nb0 * 4,
                                       SK_STRIP / 8, 1, CU_TENSOR_MAP_SWIZZLE_NONE)))
            return rc;
        if ((rc = weight_map(&L.w_d, qw_down[l], nb1, I))) return rc;
        if ((rc = encode_tensor_map_2d(&L.s_d, CU_TENSOR_MAP_DATA_TYPE_UINT32, s_down[l], N1 / 2, G1, (uint64_t)N1 * 2,
                                       SK_STRIP / 2, 1, CU_TENSOR_MAP_SWIZZLE_NONE)))
            return rc;
        if ((rc = encode_tensor_map_2d(&L.z_d, CU_TENSOR_MAP_DATA_TYPE_INT32, qz_down[l], nb1, G1, (uint64_t)nb1 * 4,
                                       SK_STRIP / 8, 1, CU_TENSOR_MAP_SWIZZLE_NONE)))
            return rc;
        L.gamma = gamma[l];
    }
    return check_cuda(cudaMemcpy(plan_dev, host.data(), host.size() * sizeof(FusedLayer), cudaMemcpyHostToDevice),
                      "ffn_stack_plan: copy of the tensor maps");
}

int launch_ffn_fused(const void *plan_dev, int n_layers, const uint16_t *x, uint16_t *out, uint16_t *inter, float eps, int B,
                     int H, int I, void *workspace, size_t workspace_bytes, cudaStream_t stream, const FusedPeers *peers) {
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(ffn_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FF_SMEM_BYTES);
    });
    if (attr_err != cudaSuccess) return check_cuda(attr_err, "fused ffn: shared memory attribute");
    const size_t need = ffn_fused_workspace_bytes(n_layers);
    if (!workspace || workspace_bytes < need)
        return set_error(AWQ_ERR_WORKSPACE, "ffn_stack_decode: workspace of %zu bytes needed, %zu given", need, workspace_bytes);

    CUtensorMap tmXi, tmH0, tmH;
    int rc;
    // activations [B, K] as (64 k, rows, K / 64 blocks): one copy fetches both [8 x 64] boxes of a group
    auto act_map = [&](CUtensorMap *m, int dtype, const void *base, int K) {
        return encode_tensor_map_3d(m, dtype, base, 64, (uint64_t)B, (uint64_t)K / 64, (uint64_t)K * 2, 128, 64, 8, 2,
                                    CU_TENSOR_MAP_SWIZZLE_128B);
    };
    if ((rc = act_map(&tmXi, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, inter, I))) return rc;
    if ((rc = act_map(&tmH0, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, x, H))) return rc;
    if ((rc = act_map(&tmH, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, out, H))) return rc;
    const int G0 = H / SK_GROUP, V0 = (2 * I + SK_STRIP - 1) / SK_STRIP;
    const int G1 = I / SK_GROUP, V1 = (H + SK_STRIP - 1) / SK_STRIP;
    const long long U0 = (long long)V0 * G0, U1 = (long long)V1 * G1;
    int ctas = device_sm_count();  // one per SM: all CTAs must be resident, they wait for one another
    if (ctas <= 0) ctas = 148;
    if ((long long)ctas > U0) ctas = (int)U0;
    if ((long long)ctas > U1) ctas = (int)U1;

    uint8_t *ws = reinterpret_cast<uint8_t *>(workspace);
    FusedArgs a;
    a.layers = reinterpret_cast<const FusedLayer *>(plan_dev);
    a.n_layers = n_layers;
    a.x = x;
    a.out = out;
    a.inter = inter;
    a.eps = eps;
    a.B = B;
    a.H = H;
    a.I = I;
    a.lookahead = g_ffn_lookahead;
    a.wait_limit = wait_limit_cycles();
    a.w3d_gu = (2 * I / 8) % 32 == 0 ? 1 : 0;
    a.w3d_d = (H / 8) % 32 == 0 ? 1 : 0;
    a.per_group = g_ffn_per_group;
    a.tp_n = 1;
    a.tp_rank = 0;
    a.epoch = nullptr;
    for (int sl = 0; sl < 2; ++sl)
        for (int r = 0; r < TP_MAX_RANKS; ++r) a.ll_recv[sl][r] = nullptr;
    if (peers && peers->n > 1) {
        if (peers->flag_offset < ffn_fused_tp_slot_bytes(H, peers->n))
            return set_error(AWQ_ERR_INVALID_ARGUMENT, "ffn_stack_decode_tp: a slot must hold %zu bytes for %d ranks and H = %d",
                             ffn_fused_tp_slot_bytes(H, peers->n), peers->n, H);
        a.tp_n = peers->n;
        a.tp_rank = peers->rank;
        for (int sl = 0; sl < 2; ++sl)
            for (int r = 0; r < peers->n; ++r)
                a.ll_recv[sl][r] = reinterpret_cast<unsigned long long *>(reinterpret_cast<uint8_t *>(peers->base[r]) +
                                                                          (size_t)sl * peers->slot_stride);
        // the last word of the flag block behind this rank's slot 0
        a.epoch = reinterpret_cast<unsigned int *>(reinterpret_cast<uint8_t *>(peers->base[peers->rank]) + peers->flag_offset) + 15;
    }
    a.accum = reinterpret_cast<unsigned long long *>(ws + SK_WS_ACCUM);
    a.err_flag = reinterpret_cast<int *>(ws);
    a.state = reinterpret_cast<int *>(ws + FF_STATE_OFF);
    if ((rc = check_cuda(cudaMemsetAsync(ws + FF_STATE_OFF, 0, ff_state_bytes(n_layers), stream), "fused ffn: state reset")))
        return rc;
    // Cooperative: the CTAs wait for one another, so they must all be resident.  With this attribute a launch
    // that cannot place them all (another kernel holding SMs) fails at once instead of running into its waits.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(FF_THREADS);
    cfg.dynamicSmemBytes = FF_SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return check_cuda(cudaLaunchKernelEx(&cfg, ffn_fused_kernel, tmXi, tmH0, tmH, a), "fused ffn launch");
}

}  // namespace awq
