// Decode GEMV for callers that cannot allocate device memory.
//
// Some hosts of this library have no way to hand it a scratch buffer: a plugin slot whose
// interface carries only the reference's inputs and outputs, a runtime that forbids
// cudaMalloc once serving has started, or C code that links the .so without any allocator of
// its own.  For them the scratch of the stream-K decode kernel (the split-K
// accumulators) lives in a fixed array inside the library image instead of a caller-owned
// workspace.  Every GPU that loads the library holds that array (about 2 MB) until the
// process exits.
#include <mutex>

#include "awq_common.cuh"

namespace awq {

// Room for 64 strips of 512 columns (N <= 32768): a 16 KB header, then 32 KB of 64-bit accumulator
// words per strip.
constexpr int STATIC_MAX_N = 32768;
constexpr size_t STATIC_SCRATCH_BYTES = 16384 + (size_t)64 * 32768;

static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];

// In host code `g_static_scratch` is only a handle for the symbol, not a device address; the
// address each device gave the array is looked up once per device (with that device current)
// and kept here.
constexpr int STATIC_MAX_DEVICES = 64;
static void *g_scratch_addr[STATIC_MAX_DEVICES];
static std::mutex g_scratch_mutex;

static int static_scratch_for_current_device(void **out) {
    int dev = -1;
    int rc = check_cuda(cudaGetDevice(&dev), "gemv_static: cudaGetDevice");
    if (rc) return rc;
    if (dev < 0 || dev >= STATIC_MAX_DEVICES)
        return set_error(AWQ_ERR_UNSUPPORTED, "gemv_static: device ordinal %d is beyond %d", dev, STATIC_MAX_DEVICES - 1);
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_addr[dev]) {
        void *ptr = nullptr;
        rc = check_cuda(cudaGetSymbolAddress(&ptr, g_static_scratch), "gemv_static: cudaGetSymbolAddress");
        if (rc) return rc;
        if (!ptr) return set_error(AWQ_ERR_CUDA, "gemv_static: the scratch symbol has no address on device %d", dev);
        g_scratch_addr[dev] = ptr;
    }
    *out = g_scratch_addr[dev];
    return AWQ_OK;
}

}  // namespace awq

using namespace awq;

extern "C" int awq_b200_gemv_bf16_static(const uint16_t *x, const int32_t *qweight, const int32_t *qzeros,
                                         const uint16_t *scales, const uint16_t *residual, uint16_t *y, int B,
                                         int K, int N, int group_size, awq_stream_t stream) {
    AWQ_REQUIRE(B >= 1 && B <= 64, "gemv_static: batch %d outside 1..64", B);
    AWQ_REQUIRE(K > 0 && N > 0, "gemv_static: K and N must be positive");
    AWQ_REQUIRE(N <= STATIC_MAX_N, "gemv_static: N = %d exceeds the built-in scratch (at most %d columns); "
                "use awq_b200_gemv_bf16 with a caller-owned workspace", N, STATIC_MAX_N);
    AWQ_REQUIRE(x && qweight && qzeros && scales && y, "gemv_static: null pointer");
    AWQ_REQUIRE(aligned16(y) && (!residual || aligned16(residual)),
                "gemv_static: the output and the residual must be 16-byte aligned");
    void *scratch = nullptr;
    int rc = static_scratch_for_current_device(&scratch);
    if (rc) return rc;
    GemvArgs a{x, qweight, qzeros, scales, residual, y, B, K, N, group_size, EPI_BF16,
               scratch, STATIC_SCRATCH_BYTES, as_stream(stream)};
    a.native_bf16 = true;  // multiply the bf16 activations as they are: no conversion buffer needed
    if (!gemv_streamk_supported(a))
        return set_error(AWQ_ERR_UNSUPPORTED,
                         "gemv_static: needs group size 128, K %% 128 == 0, N %% 32 == 0, 16-byte aligned pointers "
                         "and an sm_100 device (K=%d N=%d group=%d)", K, N, group_size);
    if (gemv_streamk_scratch_bytes(N, false) > STATIC_SCRATCH_BYTES)
        return set_error(AWQ_ERR_UNSUPPORTED, "gemv_static: %zu bytes of scratch are needed for N = %d, the built-in "
                         "array has %zu", gemv_streamk_scratch_bytes(N, false), N, STATIC_SCRATCH_BYTES);
    // The array keeps whatever the previous call left.  The error flag and the strips' accumulators
    // must read zero when the kernel starts, so clear them on the caller's stream first.
    rc = check_cuda(cudaMemsetAsync(scratch, 0, gemv_streamk_workspace_clear_bytes(N), as_stream(stream)),
                    "gemv_static: clearing the accumulators");
    if (rc) return rc;
    return launch_gemv_streamk(a);
}

// The kernel reports a wait that gave up in word 0 of the built-in array, and the next static call
// clears that word again: ask before making that next call.
extern "C" int awq_b200_static_check(awq_stream_t stream) {
    void *scratch = nullptr;
    int rc = static_scratch_for_current_device(&scratch);
    if (rc) return rc;
    int flag = 0;
    rc = check_cuda(cudaMemcpyAsync(&flag, scratch, sizeof(int), cudaMemcpyDeviceToHost, as_stream(stream)),
                    "static_check copy");
    if (rc) return rc;
    rc = check_cuda(cudaStreamSynchronize(as_stream(stream)), "static_check sync");
    if (rc) return rc;
    return status_of_device_flag(flag);
}
