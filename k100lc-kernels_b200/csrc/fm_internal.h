// Internal interfaces between the engine (fm_engine.cu) and the kernel files.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace fm {

enum : int { FM_OK = 0, FM_ENOKERNEL = -1, FM_ENARGS = -2, FM_EDYN = -3, FM_EREJECT = -4, FM_ECUDA = -5 };

// What a launcher receives: the caller's geometry (in the reference's units:
// work-groups and threads per work-group), the engine stream and the device facts.
struct LaunchCtx {
    uint32_t gx, gy, wx, wy;
    cudaStream_t stream;
    int sm_count;
};

typedef int (*LaunchFn)(const LaunchCtx& ctx, const uint64_t* argv);

struct KernelEntry {
    const char* name;     // lookup string, e.g. "gemv_w4a8<1,false,1>"
    int nargs;            // explicit arguments
    LaunchFn fn;
    const char* sig;      // one letter per argument: p = pointer, i = 32-bit int, f = f32
};

// Provided by the engine -------------------------------------------------
// true when [p, p+bytes) lies inside one live fm_alloc allocation (or checks are off)
bool range_ok(const void* p, size_t bytes);
int reject(const char* kernel, const char* fmt, ...);   // records the message, returns FM_EREJECT
int cuda_fail(const char* kernel, cudaError_t e);       // records the message, returns FM_ECUDA
int after_launch(const char* kernel);                   // cudaGetLastError -> FM_OK / FM_ECUDA
bool pdl_enabled();                                     // programmatic dependent launch on?
// engine-owned device workspace of at least `bytes` (contents undefined); nullptr when it would
// have to grow inside a stream capture or the allocation fails
void* engine_scratch(size_t bytes);
// true when `table` was filled by fm_stream_table with exactly these shapes and has not been
// overwritten since (or checks are off): every pointer inside it was range-checked then; with
// npeers > 0 the offset array must come from fm_stream_peers and cover every y of the table
// (`whole_y`: the kernel writes below row_base too — the multi-token layout — so the peer window must reach
// down to the lowest y pointer of the table)
// (`ws_bytes`: a kernel whose scale rows are longer than rows*(K/128)*2 bytes — NVFP4 — asks for that many
// bytes behind every ws pointer of the table; `need_x`: the kernel reads the x entries, none may be null)
bool stream_table_ok(const void* table, int nlayers, int rows, int K, int row_base, const void* peer_delta,
                     int npeers, bool whole_y = false, size_t ws_bytes = 0, bool need_x = false);

// true when `table` / `shapes` were filled by fm_stream_table_var for at least `nlayers` layers and are still valid (or
// checks are off); reports the smallest and largest row count of the layers and the device array of TMA maps for the
// layers that are chunks of longer rows (two maps of 128 bytes per layer: weights, scales; nullptr when the driver
// refused one).  With npeers > 0 the peer offsets must cover every y of the table.
bool stream_var_ok(const void* table, const void* shapes, int nlayers, const void* peer_delta, int npeers, int* min_rows,
                   int* max_rows, const void** chunk_maps);
bool encode_chunk_maps(void* wmap128, void* smap128, const void* wbase, const void* sbase, uint64_t rows, uint64_t wpitch,
                       uint64_t spitch);

// Device array of `nlayers` TMA tensor maps (128 bytes each) over the wq entries of a validated layer table, each
// layer's packed codes seen as [rows][K/2] bytes with a box of 128 bytes x 128 rows and the 128-byte swizzle.  Built by
// fm_stream_table (or when first asked for) and kept with the table's record; nullptr when the table has no record
// with these shapes, the driver refuses the encoding, or the array would have to be allocated inside a stream capture.
const void* stream_table_maps(const void* table, int nlayers, int rows, int K);
// one such map (gemm_w4.cu holds the encoder): false when the driver refuses it
bool encode_bytes_rows_map(void* map128, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_bytes);

// true when [ptr, ptr+bytes) lies inside the local window that fm_stream_peers validated for the offset array
// `peer_delta` (so every receiver has the same bytes at the same offset), or checks are off
bool peer_window_ok(const void* peer_delta, int npeers, const void* ptr, size_t bytes);

// Registries of the kernel files -------------------------------------------
const KernelEntry* quant_kernels(int* n);
const KernelEntry* gemv_w4_kernels(int* n);
const KernelEntry* gemv_nvfp4_kernels(int* n);
const KernelEntry* int4_dot_kernels(int* n);
const KernelEntry* gemm_w4_kernels(int* n);
const KernelEntry* stream_kernels(int* n);
const KernelEntry* norm_act_kernels(int* n);
const KernelEntry* nvfp4_gemm_kernels(int* n);
const KernelEntry* moe_kernels(int* n);

// Launchers without the engine (no allocation registry, no engine stream): the caller
// owns every buffer and names the stream.  Same kernels as the by-name entries.
cudaError_t quant_act_raw(const float* x, int8_t* ae, int8_t* ao, float* asc, int* asu, int K, int tokens,
                          cudaStream_t stream);
cudaError_t gemv_w4a8_raw(const uint32_t* wq, const void* ws_f16, const int8_t* ae, const int8_t* ao,
                          const float* asc, const int* asu, float* y, int M, int N, int K, int sm_count,
                          cudaStream_t stream);

// Single-layer launch of the ring kernel (decode_stream.cu) behind gemv_w4a8<2..4,..>: K = 5120 and every operand
// 16-byte aligned; the caller has range-checked the pointers.  `iacc` != nullptr also stores the integer
// accumulators [M][rows][K/128].
int stream_gemv_w4a8(const LaunchCtx& c, const char* kn, const void* wq, const void* ws, const void* ae, const void* ao,
                     const void* asc, const void* asu, float* y, int M, int ystride, int rows, int* iacc);
// The same behind gemv_w4a4<2..4> and its r2 names (aq [M][K/2], asc [M][K/32]; iacc [M][rows][K/32]).
int stream_gemv_w4a4(const LaunchCtx& c, const char* kn, const void* wq, const void* ws, const void* aq, const void* asc,
                     float* y, int M, int ystride, int rows, int* iacc);
namespace stream { struct StreamParams; }
// nvfp4_decode_stream on the tcgen05 path (nvfp4_tc_stream.cu).  FM_OK after enqueueing, negative after a rejection,
// 1 when this path cannot take the launch and the caller should use another consumer.
int nvfp4_tc_stream(const char* kn, const LaunchCtx& c, const stream::StreamParams& sp, float gscale, bool dump);
int stream_read_status(cudaStream_t stream);   // 0, or the code of the first bounded wait that ran out in such a launch

int gemm_read_status(cudaStream_t stream);   // 0, or the code of the first bounded wait that ran out

// argv decoding ------------------------------------------------------------
template <typename T> static inline T* arg_ptr(uint64_t v) { return reinterpret_cast<T*>(static_cast<uintptr_t>(v)); }
static inline int arg_i32(uint64_t v) { return static_cast<int>(static_cast<uint32_t>(v)); }
static inline uint32_t arg_u32(uint64_t v) { return static_cast<uint32_t>(v); }
static inline float arg_f32(uint64_t v) {
    uint32_t b = static_cast<uint32_t>(v);
    float f;
    __builtin_memcpy(&f, &b, 4);
    return f;
}
static inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

#define FM_REQUIRE(cond, kernel, ...) \
    do { if (!(cond)) return ::fm::reject(kernel, __VA_ARGS__); } while (0)
#define FM_RANGE(ptr, bytes, kernel, what) \
    do { if (!::fm::range_ok((ptr), (bytes))) \
        return ::fm::reject(kernel, "%s: %zu bytes at %p are not inside a live fm_alloc allocation", what, (size_t)(bytes), (const void*)(ptr)); } while (0)

// Launch helper: plain launch or, when enabled, with the programmatic-stream-
// serialization attribute so the kernel may start while its predecessor drains
// (the kernel itself calls pdl_wait() before touching anything the predecessor wrote).
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                        cudaStream_t stream, bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

}  // namespace fm
