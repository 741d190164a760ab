// fm_w4a8_linear_static: a W4A8 decode linear layer for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need a
// layer evaluated: code running inside someone else's stream capture (an allocation is
// not a capturable operation), plugins of an inference server whose contract hands them
// device buffers and forbids further allocations so that the server's memory plan stays
// fixed, and real-time loops that must not take the allocator's locks.  The regular
// path (quant_act followed by gemv_w4a8) needs a place for the quantised activations
// between its two kernels, and normally the caller allocates that with fm_alloc.  This
// entry point keeps that intermediate in a fixed array that is part of the library's
// device image instead, so it needs nothing but the caller's input and output buffers.
//
// Limits and rules:
//   * M (tokens) 1..4, K a multiple of 128 and at most 16384; larger shapes are refused
//     with FM_EREJECT (-4) and a message in fm_last_error().
//   * The array is 73 728 bytes and every GPU that loads the library carries it until
//     the process exits.
//   * All calls on one GPU share the array.  Each call rewrites every byte it later
//     reads, so nothing has to be cleared, but two calls whose kernels overlap on the GPU
//     (different streams, or different host threads on different streams) race on it.
//     Calls on one stream are ordered and safe.
//   * The first call on each device looks up the array's device address
//     (cudaGetSymbolAddress) and the SM count and caches them; make that first call
//     outside of any stream capture.
//   * No cudaMalloc / cudaFree / allocating library call is made, and the engine
//     (fm_init, fm_alloc, the engine stream) is not involved.
#include <mutex>

#include "../../include/fm_engine.h"
#include "fm_internal.h"

namespace {

constexpr int kMaxTokens = 4;
constexpr int kMaxK = 16384;
constexpr size_t kCodesBytes = (size_t)kMaxTokens * (kMaxK / 2);          // one int8 stream, all tokens
constexpr size_t kScaleBytes = (size_t)kMaxTokens * (kMaxK / 128) * 4;    // f32 scales or int32 sums
constexpr size_t kScratchBytes = 2 * kCodesBytes + 2 * 4096;              // 65536 + 8192 = 73728
static_assert(kScaleBytes <= 4096, "scale region");

// Quantised activations between quant_act and gemv_w4a8:
//   [0, 32768) even-k int8 codes, [32768, 65536) odd-k codes, then 4096 bytes of f32
//   group scales and 4096 bytes of int32 group sums.
// In host code this name is only a handle for cudaGetSymbolAddress, not an address.
static __device__ __align__(256) unsigned char g_w4a8_act_scratch[kScratchBytes];

struct PerDevice {
    bool ready = false;
    unsigned char* scratch = nullptr;    // device address of g_w4a8_act_scratch on this GPU
    int sm_count = 0;
};
PerDevice g_dev[64];
std::mutex g_mu;

}  // namespace

extern "C" int fm_w4a8_linear_static(const void* wq, const void* ws_f16, const float* x, float* y,
                                     int M, int N, int K, void* stream, int wait) {
    const char* kn = "fm_w4a8_linear_static";
    if (M < 1 || M > kMaxTokens)
        return fm::reject(kn, "M=%d is outside 1..%d", M, kMaxTokens);
    if (K < 128 || K % 128 != 0 || K > kMaxK)
        return fm::reject(kn, "K=%d must be a multiple of 128 and at most %d (size of the built-in scratch)", K, kMaxK);
    if (N < 1) return fm::reject(kn, "N=%d must be positive", N);
    if (!wq || !ws_f16 || !x || !y) return fm::reject(kn, "null pointer");
    if (!fm::aligned(wq, 16) || !fm::aligned(x, 16) || !fm::aligned(ws_f16, 2) || !fm::aligned(y, 4))
        return fm::reject(kn, "misaligned pointer (wq and x need 16 bytes, ws 2, y 4)");

    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fm::cuda_fail(kn, e);
    if (dev < 0 || dev >= 64) return fm::reject(kn, "device ordinal %d is not supported", dev);
    PerDevice* d = &g_dev[dev];
    {
        std::lock_guard<std::mutex> lock(g_mu);
        if (!d->ready) {                      // set-up, once per device, with that device current
            unsigned char* p = nullptr;
            e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_w4a8_act_scratch);
            if (e != cudaSuccess || p == nullptr) return fm::cuda_fail(kn, e);
            int sms = 0;
            e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            if (e != cudaSuccess) return fm::cuda_fail(kn, e);
            d->scratch = p;
            d->sm_count = sms;
            d->ready = true;
        }
    }
    int8_t* ae = reinterpret_cast<int8_t*>(d->scratch);
    int8_t* ao = reinterpret_cast<int8_t*>(d->scratch + kCodesBytes);
    float* asc = reinterpret_cast<float*>(d->scratch + 2 * kCodesBytes);
    int* asu = reinterpret_cast<int*>(d->scratch + 2 * kCodesBytes + 4096);
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    e = fm::quant_act_raw(x, ae, ao, asc, asu, K, M, s);
    if (e != cudaSuccess) return fm::cuda_fail(kn, e);
    e = fm::gemv_w4a8_raw(static_cast<const uint32_t*>(wq), ws_f16, ae, ao, asc, asu, y, M, N, K, d->sm_count, s);
    if (e != cudaSuccess) return fm::cuda_fail(kn, e);
    if (wait) {
        e = cudaStreamSynchronize(s);
        if (e != cudaSuccess) return fm::cuda_fail(kn, e);
    }
    return fm::FM_OK;
}
