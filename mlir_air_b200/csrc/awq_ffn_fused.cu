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
//  * Every CTA walks a static list: its gate/up unit range of layer 0, its down range of layer 0,
//    its gate/up range of layer 1, ...  The loader keeps the ring full across phase
//    changes: the weights of the next phase's first units are requested before the phase's
//    activations exist.
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

// One layer's tensor maps, device resident (TMA reads the descriptor from global memory).
struct alignas(128) FusedLayer {
    CUtensorMap w_gu, s_gu, z_gu;  // gate/up interleaved [H, 2I]
    CUtensorMap w_d, s_d, z_d;     // down [I, H]
    const uint16_t *gamma;         // bf16 [H]
};
static_assert(sizeof(FusedLayer) % 128 == 0, "tensor maps must stay 64-byte aligned in the array");

constexpr int FF_MAX_LAYERS = 1024;
// State of one launch in the workspace, zeroed by the launcher: two phase counters, then one
// f32 sum of squares per (layer boundary, batch row).
constexpr size_t FF_STATE_OFF = SK_WS_END;
constexpr size_t FF_STATE_HEADER = 64;
__host__ __device__ constexpr size_t ff_state_bytes(int n_layers) {
    return FF_STATE_HEADER + (size_t)(n_layers + 1) * 8 * sizeof(float);
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
// TMA) and a normaliser warp.  The SM's units of a phase are one contiguous range, cut between
// the halves at `split` / 1024 of its length: the hardware does not share issue slots evenly
// between two sets of warps, and the set it prefers gets the larger part so that both finish
// together.
constexpr int FF_HALVES = 2;
constexpr int FF_CONSUMER_WARPS = FF_HALVES * SK_CONSUMER_WARPS;
constexpr int FF_WARPS = FF_CONSUMER_WARPS + 2 * FF_HALVES;
constexpr int FF_THREADS = FF_WARPS * 32;
constexpr int FF_OFF_GAMMA = SK_OFF_Z + SK_Z_BYTES;  // 128 bf16 norm weights of the unit's k range
constexpr int FF_GAMMA_BYTES = SK_GROUP * 2;
constexpr int FF_RING_BYTES = SK_STAGES * SK_STAGE_BYTES;
constexpr int FF_BARS_PER_HALF = 3 * SK_STAGES;
constexpr int FF_SMEM_BYTES = FF_HALVES * FF_RING_BYTES + FF_HALVES * FF_BARS_PER_HALF * 8 + 16 + 1024;
static_assert(FF_OFF_GAMMA + FF_GAMMA_BYTES <= SK_STAGE_BYTES, "stage too small");
static_assert(FF_SMEM_BYTES + 1024 + 128 <= 228 * 1024, "shared memory budget");

__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap *map, int x, int y) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];" ::"l"(map), "r"(x), "r"(y) : "memory");
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
    int split;      // share of an SM's units that half 0 takes, in 1/1024
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

// The unit range [u0, u1) of one half in one phase: the SM's range [s U / S, (s + 1) U / S), cut.
__device__ __forceinline__ void ff_range(long long U, int half, int split, long long &u0, long long &u1) {
    const long long S = gridDim.x, s = blockIdx.x;
    const long long lo = s * U / S, hi = (s + 1) * U / S;
    const long long mid = lo + ((hi - lo) * split + 512) / 1024;
    u0 = half ? mid : lo;
    u1 = half ? hi : mid;
}

// One half's walk over its units: for every layer its gate/up range, then its down range.
struct UnitCursor {
    int l, p, v, g, left;  // layer, phase (0 gate/up, 1 down), strip, group, units left in the phase
    int G0, V0, G1, V1, n_layers, half, split;
    __device__ __forceinline__ UnitCursor(int g0, int v0, int g1, int v1, int layers, int half_, int split_)
        : G0(g0), V0(v0), G1(g1), V1(v1), n_layers(layers), half(half_), split(split_) {
        l = 0;
        p = 0;
        enter();
    }
    __device__ __forceinline__ int groups() const { return p ? G1 : G0; }
    // position on the first unit of phase (l, p), skipping phases in which this half has no unit
    __device__ __forceinline__ void enter() {
        while (l < n_layers) {
            const int G = groups();
            long long u0, u1;
            ff_range((long long)(p ? V1 : V0) * G, half, split, u0, u1);
            if (u1 > u0) {
                v = (int)(u0 / G);
                g = (int)(u0 % G);
                left = (int)(u1 - u0);
                return;
            }
            if (++p == 2) { p = 0; ++l; }
        }
    }
    __device__ __forceinline__ bool valid() const { return l < n_layers; }
    __device__ __forceinline__ void next() {
        if (--left > 0) {
            if (++g == groups()) { g = 0; ++v; }
            return;
        }
        if (++p == 2) { p = 0; ++l; }
        enter();
    }
};

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
    auto empty_bar = [&](int s) { return bar_base + 8u * (SK_STAGES + s); };       // consumers done
    auto xready_bar = [&](int s) { return bar_base + 8u * (2 * SK_STAGES + s); };  // activations normalised

    const int B = a.B, H = a.H, I = a.I;
    // phase 0: gate/up, K = H, N = 2I; phase 1: down, K = I, N = H
    const int G0 = H / SK_GROUP, V0 = (2 * I + SK_STRIP - 1) / SK_STRIP;
    const int G1 = I / SK_GROUP, V1 = (H + SK_STRIP - 1) / SK_STRIP;
    int *done_gu = a.state, *done_d = a.state + 1;
    const bool tp = a.tp_n > 1;
    // tensor parallel: exchanges so far on these buffers (all launches run the same number of layers); every
    // warp reads the count before anything of this launch can end
    const unsigned int exch0 = tp ? *a.epoch * (unsigned int)a.n_layers : 0u;
    float *sumsq = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(a.state) + FF_STATE_HEADER);

    if (role == 1 && lane == 0) {  // each loader sets up its half's barriers
        for (int s = 0; s < SK_STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), SK_CONSUMER_WARPS);
            mbar_init(xready_bar(s), 1);
        }
        mbar_fence_init();
    }
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

    if (role == 1) {
        // ------------------------------ loader (one thread) ------------------------------
        if (lane != 0) return;
        const uint64_t stream_policy = l2_policy_evict_first();
        UnitCursor cur(G0, V0, G1, V1, a.n_layers, half, a.split), pf = cur;
        int issued = 0, prefetched = 0;
        auto maps = [&](int l, int p, const CUtensorMap *&tmW, const CUtensorMap *&tmS, const CUtensorMap *&tmZ) {
            const FusedLayer *Ly = a.layers + l;
            tmW = p ? &Ly->w_d : &Ly->w_gu;
            tmS = p ? &Ly->s_d : &Ly->s_gu;
            tmZ = p ? &Ly->z_d : &Ly->z_gu;
        };
        // keep HBM streaming into L2 `lookahead` units ahead of the ring, across phase and layer
        // boundaries: weights depend on nothing, so the stream does not stop while a phase waits
        auto run_prefetch = [&]() {
            while (pf.valid() && prefetched < issued + a.lookahead) {
                const CUtensorMap *tmW, *tmS, *tmZ;
                maps(pf.l, pf.p, tmW, tmS, tmZ);
#pragma unroll
                for (int bx = 0; bx < SK_STRIP / SK_BOX_COLS; ++bx)
                    tma_prefetch_l2_2d(tmW, (pf.v * SK_STRIP + bx * SK_BOX_COLS) / 8, pf.g * SK_GROUP);
                pf.next();
                ++prefetched;
            }
        };
        auto acquire_slot = [&](int &slot) -> bool {  // slot of unit number `issued`, once the consumers released it
            slot = issued % SK_STAGES;
            const int round = issued / SK_STAGES;
            if (round > 0 && !mbar_wait_bounded(empty_bar(slot), (round - 1) & 1, a.wait_limit)) {
                atomicExch(a.err_flag, 1);
                return false;
            }
            return true;
        };
        auto load_weights = [&](int slot, const UnitCursor &u) {
            const CUtensorMap *tmW, *tmS, *tmZ;
            maps(u.l, u.p, tmW, tmS, tmZ);
            const uint32_t st = smem_base + slot * SK_STAGE_BYTES;
            const uint32_t bar = full_bar(slot);
            mbar_expect_tx(bar, u.p ? SK_TX_BYTES : SK_TX_BYTES + FF_GAMMA_BYTES);
#pragma unroll
            for (int bx = 0; bx < SK_STRIP / SK_BOX_COLS; ++bx)
                tma_load_2d_hint(st + bx * SK_WBOX_BYTES, tmW, (u.v * SK_STRIP + bx * SK_BOX_COLS) / 8, u.g * SK_GROUP, bar,
                                 stream_policy);
#pragma unroll
            for (int bx = 0; bx < SK_STRIP / SK_BOX_COLS; ++bx)
                tma_load_2d(st + SK_OFF_S + bx * SK_BOX_COLS * 2, tmS, u.v * SK_STRIP + bx * SK_BOX_COLS, u.g, bar);
            tma_load_2d(st + SK_OFF_Z, tmZ, u.v * (SK_STRIP / 8), u.g, bar);
        };
        auto load_activations = [&](int slot, const UnitCursor &u) {
            const uint32_t st = smem_base + slot * SK_STAGE_BYTES;
            const uint32_t bar = full_bar(slot);
            // down: the SwiGLU output as it is; gate/up: the raw hidden state and the norm weights
            // of the unit's k range, which the normaliser warp turns into activations in place
            const CUtensorMap *tmX = u.p ? &tmXi : (u.l == 0 ? &tmH0 : &tmH);
            tma_load_2d(st + SK_OFF_X, tmX, u.g * SK_GROUP, 0, bar);
            tma_load_2d(st + SK_OFF_X + 1024, tmX, u.g * SK_GROUP + 64, 0, bar);
            if (!u.p) bulk_load_1d(st + FF_OFF_GAMMA, a.layers[u.l].gamma + (size_t)u.g * SK_GROUP, FF_GAMMA_BYTES, bar);
        };
        while (cur.valid()) {
            // a phase begins: the weights of its first units do not depend on the previous phase
            const int l = cur.l, p = cur.p;
            const int n_units = cur.left;
            const int n_first = n_units < SK_STAGES ? n_units : SK_STAGES;
            int slots[SK_STAGES];
            UnitCursor first = cur;
            for (int i = 0; i < n_first; ++i) {
                run_prefetch();
                if (!acquire_slot(slots[i])) return;
                load_weights(slots[i], cur);
                ++issued;
                cur.next();
            }
            // the phase's activations exist once every sub-strip of the previous phase is finalised
            // (tensor parallel: a down sub-strip is finalised by the warp that added up all ranks' sums)
            const int target = p ? (l + 1) * V0 * SK_CONSUMER_WARPS : B + l * V1 * SK_CONSUMER_WARPS;
            if (!wait_count(p ? done_gu : done_d, target, a.wait_limit)) {
                atomicExch(a.err_flag, 3);
                return;
            }
            fence_proxy_async_all();  // generic-proxy writes of the previous phase before the tensor copies read them
            for (int i = 0; i < n_first; ++i) {
                load_activations(slots[i], first);
                first.next();
            }
            for (int i = n_first; i < n_units; ++i) {
                run_prefetch();
                int slot;
                if (!acquire_slot(slot)) return;
                load_weights(slot, cur);
                load_activations(slot, cur);
                ++issued;
                cur.next();
            }
        }
        return;
    }

    if (role == 2) {
        // ------------------------------ normaliser warp ------------------------------
        // RMSNorm of a gate/up unit's 8 x 128 hidden values, in place in the stage: lane (r, q4)
        // takes 16-byte chunks q4, q4 + 4, q4 + 8, q4 + 12 of batch row r where the tensor copy of
        // the 128B-swizzled [8 x 64] box pair put them; bf16 rounding, then the fp16 form
        const int r = lane >> 2, q4 = lane & 3;
        int slot = 0, round = 0;
        for (int l = 0; l < a.n_layers; ++l) {
            for (int p = 0; p < 2; ++p) {
                long long u0, u1;
                ff_range((long long)(p ? V1 : V0) * (p ? G1 : G0), half, a.split, u0, u1);
                const int n_units = (int)(u1 - u0);
                float rstd = 0.f;
                for (int i = 0; i < n_units; ++i) {
                    // every unit's barrier is waited for, also those of down units that need no work
                    // here: a parity wait is only meaningful one completion ahead
                    if (!mbar_wait_bounded(full_bar(slot), round & 1, a.wait_limit)) {
                        if (lane == 0) atomicExch(a.err_flag, 4);
                        return;
                    }
                    if (!p) {
                        if (i == 0 && r < B) {  // complete: the loader passed the phase barrier before it requested h
                            const float total = __ldcg(sumsq + (size_t)l * 8 + r);
                            rstd = (float)(1.0 / sqrt((double)(total / (float)H) + (double)a.eps));
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
                    if (++slot == SK_STAGES) { slot = 0; ++round; }
                }
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
            }
        }
        if (tp && blockIdx.x == 0 && half == 0 && lane == 0) *a.epoch = exch0 / (unsigned int)a.n_layers + 1u;
        return;
    }

    // ------------------------------ consumers ------------------------------
    const int cw = warp % SK_CONSUMER_WARPS;  // this warp's 64 columns of every strip
    const SkLane geo(cw, lane);
    const int g8 = geo.g8, t4 = geo.t4, odd = geo.odd, colw = geo.colw;
    const int b = 2 * t4 + odd;  // batch row of this lane after the lane exchange
    bool failed = false;
    int slot = 0, round = 0;
    uint32_t xr_parity = 0;  // bit s: parity of the next completion of xready_bar(s) (only gate/up units use it)

    for (int l = 0; l < a.n_layers; ++l) {
        for (int p = 0; p < 2; ++p) {
            const int G = p ? G1 : G0, N = p ? H : 2 * I;
            long long u0, u1;
            ff_range((long long)(p ? V1 : V0) * G, half, a.split, u0, u1);
            const int n_units = (int)(u1 - u0);
            const uint16_t *residual = l == 0 ? a.x : a.out;
            float res[4][4];
            int cur_v = -1, seg_groups = 0;  // strip being accumulated, k groups of it added so far

            // Finish the strip segment this warp has been accumulating (strip cur_v).
            auto flush = [&]() {
                const int v = cur_v;
                float own[2][8];
                sk_lane_exchange(res, odd, own);
                const int n = v * SK_STRIP + colw;
                // a strip shared with other halves: value and progress travel in one 64-bit atomic per sum; the warp
                // whose add completes the count has the total (gate/up and down strips use separate accumulators)
                if (seg_groups != G &&
                    !sk_handover(a.accum + ((size_t)((p ? V0 : 0) + v) * SK_CONSUMER_WARPS + cw) * SK_ACC_WORDS, own, seg_groups, G,
                                 lane, a.wait_limit, a.err_flag))
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
                    ff_load_residual(rres, residual, B, N, n, b);
                    ff_down_epilogue(own, rres, a.out, sumsq + (size_t)(l + 1) * 8, B, N, n, b, lane);
                }
                __threadfence();
                __syncwarp();
                if (lane == 0) atomicAdd(p ? done_d : done_gu, 1);
            };

            int v = n_units > 0 ? (int)(u0 / G) : 0, g = n_units > 0 ? (int)(u0 % G) : 0;
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
                if (!failed) {
                    bool ok = mbar_wait_bounded(full_bar(slot), round & 1, a.wait_limit);
                    if (ok && !p) ok = mbar_wait_bounded(xready_bar(slot), (xr_parity >> slot) & 1u, a.wait_limit);
                    if (!ok) {
                        failed = true;
                        if (lane == 0) atomicExch(a.err_flag, 2);
                    }
                }
                if (!p) xr_parity ^= 1u << slot;
                if (!failed) sk_consume_unit<true>(smem_base + slot * SK_STAGE_BYTES, geo, res, empty_bar(slot), lane);
                if (++g == G) { g = 0; ++v; }
                if (++slot == SK_STAGES) { slot = 0; ++round; }
            }
            if (cur_v >= 0) flush();
        }
    }
}

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
static int g_ffn_lookahead = 2;
static int g_ffn_split = 512;
void ffn_fused_set_lookahead(int units) { g_ffn_lookahead = units < 0 ? 0 : (units > 64 ? 64 : units); }
void ffn_fused_set_split(int per_1024) { g_ffn_split = per_1024 < 0 ? 0 : (per_1024 > 1024 ? 1024 : per_1024); }

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
        if ((rc = encode_tensor_map_2d(&L.w_gu, CU_TENSOR_MAP_DATA_TYPE_INT32, qw_gateup[l], nb0, H, (uint64_t)nb0 * 4, 32,
                                       SK_GROUP, CU_TENSOR_MAP_SWIZZLE_128B)))
            return rc;
        if ((rc = encode_tensor_map_2d(&L.s_gu, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, s_gateup[l], N0, G0, (uint64_t)N0 * 2,
                                       SK_BOX_COLS, 1, CU_TENSOR_MAP_SWIZZLE_NONE)))
            return rc;
        if ((rc = encode_tensor_map_2d(&L.z_gu, CU_TENSOR_MAP_DATA_TYPE_INT32, qz_gateup[l], nb0, G0, (uint64_t)nb0 * 4,
                                       SK_STRIP / 8, 1, CU_TENSOR_MAP_SWIZZLE_NONE)))
            return rc;
        if ((rc = encode_tensor_map_2d(&L.w_d, CU_TENSOR_MAP_DATA_TYPE_INT32, qw_down[l], nb1, I, (uint64_t)nb1 * 4, 32,
                                       SK_GROUP, CU_TENSOR_MAP_SWIZZLE_128B)))
            return rc;
        if ((rc = encode_tensor_map_2d(&L.s_d, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, s_down[l], N1, G1, (uint64_t)N1 * 2,
                                       SK_BOX_COLS, 1, CU_TENSOR_MAP_SWIZZLE_NONE)))
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
    if ((rc = encode_tensor_map_2d(&tmXi, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, inter, I, B, (uint64_t)I * 2, 64, 8,
                                   CU_TENSOR_MAP_SWIZZLE_128B)))
        return rc;
    if ((rc = encode_tensor_map_2d(&tmH0, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, x, H, B, (uint64_t)H * 2, 64, 8,
                                   CU_TENSOR_MAP_SWIZZLE_128B)))
        return rc;
    if ((rc = encode_tensor_map_2d(&tmH, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, out, H, B, (uint64_t)H * 2, 64, 8,
                                   CU_TENSOR_MAP_SWIZZLE_128B)))
        return rc;
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
    a.split = g_ffn_split;
    a.wait_limit = wait_limit_cycles();
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
    ffn_fused_kernel<<<ctas, FF_THREADS, FF_SMEM_BYTES, stream>>>(tmXi, tmH0, tmH, a);
    return check_cuda(cudaGetLastError(), "fused ffn launch");
}

}  // namespace awq
