/* fm_engine.h — C ABI of libfm_engine.so for NVIDIA B200 (sm_100a).
 *
 * The first 14 entry points are a drop-in for the reference engine
 * (Hong-agent/K100LC-kernels, runtime/fm_engine.h:10-28 and
 * runtime/fm_engine.cpp:70-139): same names, argument meaning and return
 * codes, so that the reference's ctypes binding
 * (python/k100lc_kernels/runtime.py:129-163) and C++ users
 * (examples/cpp_alloc.cpp) work unchanged.  Kernels are selected by the
 * reference's lookup strings ("quant_act", "gemv_w4a8<1,false,1>", ...).
 *
 * Everything after the "extensions" banner has no counterpart in the
 * reference (which is single-device and has no timers or collectives).
 *
 * Return codes of the launch family:
 *    0  launched (asynchronously, on the engine's single in-order stream)
 *   -1  unknown kernel name                     (reference fm_engine.cpp:83-86)
 *   -2  explicit-argument count mismatch        (reference fm_engine.cpp:87-91)
 *   -3  fm_launch_dyn: kernarg_size > 1024      (reference fm_engine.cpp:108)
 *   -4  rejected before launch: a pointer argument does not lie inside a live
 *       fm_alloc allocation for the footprint the kernel would touch, a
 *       pointer is misaligned, or the geometry/shape is one the kernel cannot
 *       run (the reference would read or write out of bounds instead)
 *   -5  CUDA error; text via fm_last_error()
 */
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- reference ABI ---------------------------------------------------- */

/* runtime/fm_engine.h:10, fm_engine.cpp:38-41.  `hsaco` named the kernel
 * image in the reference; here the kernels are linked into the library and
 * the argument is only recorded.  Idempotent.  Device = $FM_DEVICE, else
 * $LOCAL_RANK, else 0 (unless fm_set_device was called first). */
int   fm_init(const char* hsaco);
/* fm_engine.h:11-12, fm_engine.cpp:43-49.  NULL when out of memory. */
void* fm_alloc(size_t n);
void  fm_free(void* p);
/* fm_engine.h:13-16, fm_engine.cpp:51-65.  Ordered on the engine stream;
 * upload/download return after the copy has completed. */
int   fm_upload(void* dev, const void* host, size_t n);
int   fm_download(void* host, const void* dev, size_t n);
int   fm_copy(void* dst, const void* src, size_t n);
int   fm_memset(void* dev, int v, size_t n);
/* fm_engine.h:17, fm_engine.cpp:67. */
int   fm_sync(void);
/* fm_engine.h:19-22, fm_engine.cpp:75-101.  grid / workgroup count work-groups
 * and threads per group as on the reference; argv[i] is the i-th explicit
 * argument (pointers as device addresses, scalars in the low bytes, f32 as bit
 * pattern). */
int   fm_launch(const char* kernel, uint32_t grid, uint32_t workgroup,
                const uint64_t* argv, int nargs);
int   fm_launch2d(const char* kernel, uint32_t gx, uint32_t gy,
                  uint32_t wx, uint32_t wy, const uint64_t* argv, int nargs);
/* fm_engine.h:23-28, fm_engine.cpp:103-132.  `layout` is nargs x (off,size,kind);
 * only its kind==0 count and kernarg_size are validated here. */
int   fm_launch_dyn(const char* kernel, uint32_t gx, uint32_t gy,
                    uint32_t wx, uint32_t wy,
                    const uint32_t* layout, uint32_t nargs,
                    uint32_t group_size, uint32_t private_size,
                    uint32_t kernarg_size, const uint64_t* argv, int nargv);
/* fm_engine.cpp:70-73, 134-139.  A plan is a flat uint64 array of records
 * [kernel_id, grid, workgroup, nargs, argv...]; returns the number of records
 * enqueued.  A plan is replayed as a CUDA graph (re-captured when its contents
 * change). */
int   fm_has_kernel(const char* kernel);
int   fm_kernel_id(const char* kernel);
int   fm_launch_batch(const uint64_t* plan, int nrec);

/* ---- extensions (no counterpart in the reference) ---------------------- */

const char* fm_last_error(void);
int   fm_device_count(void);
int   fm_set_device(int dev);          /* before fm_init */
int   fm_device_attr(int what);        /* 0 SM count, 1 L2 bytes, 2 device ordinal,
                                          3 total memory MiB, 4 SM clock kHz */
int   fm_kernel_count(void);
const char* fm_kernel_name(int id);
int   fm_kernel_nargs(int id);
const char* fm_kernel_sig(int id);    /* one letter per argument: p pointer, i int32, f float32 */
unsigned long long fm_launch_count(void);   /* kernels launched so far */

/* pinned host memory and asynchronous copies on the engine stream */
void* fm_host_alloc(size_t n);
void  fm_host_free(void* p);
int   fm_upload_async(void* dev, const void* pinned_host, size_t n);
int   fm_download_async(void* pinned_host, const void* dev, size_t n);

/* Upload on a second queue, for double-buffered inputs.  The copy starts when everything enqueued on the engine
 * stream before the call has finished and runs beside what is enqueued after it; fm_upload_join makes the
 * engine stream wait for it.  Per step t:  fm_upload_beside(x[(t+1)%2]); launch step t (reads x[t%2]);
 * fm_upload_join().  Not available inside a graph capture.  fm_sync also waits for the second queue. */
int   fm_upload_beside(void* dev, const void* pinned_host, size_t n);
int   fm_upload_join(void);
/* Device-to-device copy on the second queue, behind what that queue already holds; dst may be a peer's allocation
 * opened with fm_ipc_import (copy engines, no SM needed: it runs beside the kernels of the engine stream). */
int   fm_copy_beside(void* dst, const void* src, size_t n);
/* Download on a third queue, for double-buffered outputs: `height` rows of `width` bytes, `dpitch` / `hpitch` bytes
 * between the starts of rows on the device / the host (height 1: a plain copy of `width` bytes).  The copy starts
 * when everything enqueued on the engine stream before the call has finished and runs beside what is enqueued after
 * it.  fm_download_join(lag) makes the engine stream wait for the download issued `lag` calls before the latest
 * (0..3).  Per step t:  fm_download_join(1); launch step t (writes y[t%2]); fm_download_beside(host, .., y[t%2], ..).
 * Not available inside a graph capture.  fm_sync also waits for the third queue. */
int   fm_download_beside(void* pinned_host, size_t hpitch, const void* dev, size_t dpitch, size_t width, size_t height);
int   fm_download_join(int lag);

/* Layer table of the fused decode stream ("w4a8_decode_stream"): host_layers holds
 * nlayers x {wq, ws, x, y} device addresses.  Every address is checked against the live
 * allocations for the footprint that (rows, K, row_base) implies — wq rows*K/2 bytes,
 * ws rows*(K/128)*2, x K*4, y (row_base+rows)*4 — then the table is copied to dev_table
 * (nlayers*32 bytes) and remembered as validated until something overwrites it.
 * For "w4a8_decode_stream_m" (M tokens per layer, y token-major with `ystride` floats between tokens)
 * pass row_base + (M-1)*ystride as row_base here: the checked footprint of y then covers every token.
 * 0 ok, -4 a pointer fails the check, -1 other errors. */
int   fm_stream_table(void* dev_table, const uint64_t* host_layers, int nlayers, int rows, int K, int row_base);
/* Layer table of "w4a8_layers_stream": layers of different shapes in one launch.  A layer here is 5120 k of a set of
 * weight rows; a weight matrix with longer rows (K = 6144, 17408, ...) is ceil(K/5120) consecutive layers over the same
 * rows and the same y, the second and later ones with accumulate = 1.  host_layers holds nlayers x 16 values:
 *   wq, ws      first byte of this chunk in the first row (wq + chunk*2560, ws + chunk*80)
 *   0, y        (no x), output of the weight matrix
 *   ae, ao, asc, asu   the token's quantised activations of this chunk (quant_act outputs at k = chunk*5120: 2560 + 2560
 *               bytes of codes, 40 scales, 40 sums); behind the matrix's K they must be zero (pad the arrays to a
 *               multiple of 5120 k and clear them once)
 *   rows, wpitch, spitch    weight rows, bytes between rows of wq (K/2) and of ws (K/128*2)
 *   wbytes, sbytes          valid bytes of a row in this chunk: 2560 / 80, less in the last chunk of a longer row
 *   accumulate, row_base, chunk    chunk = which 5120 k of the row (0, 1, ...)
 * Every range is checked against the live allocations; dev_table receives nlayers*32 bytes, dev_shapes nlayers*64.
 * 0 ok, -4 a pointer or a shape fails the check, -1 other errors. */
int   fm_stream_table_var(void* dev_table, void* dev_shapes, const uint64_t* host_layers, int nlayers);
/* Which rows [*r0, *r1) of a layer of `rows` rows CTA `cta` of a grid of `grid` CTAs computes in the stream kernels that
 * deal out whole 16-row stages ("w4a8_layers_stream", and the uniform streams when a CTA has three or more stages per
 * layer): `first` is the table index of the layer — of the first chunk of its weight matrix in a table of
 * fm_stream_table_var.  The same function the kernels call; needs no device.  0 ok, -1 arguments out of range. */
int   fm_stream_rows(int rows, int first, int grid, int cta, int* r0, int* r1);

/* Peer memory for the row-sharded stream (one process per GPU).  fm_ipc_export gives the
 * 64-byte CUDA IPC handle of the fm_alloc allocation that contains `dev`, the offset of
 * `dev` in it and its size; another rank opens it with fm_ipc_import (peer access is
 * enabled on the way) and releases it with fm_free.  fm_stream_peers checks that
 * [peer_bases[q], +span) lies inside an imported allocation — or inside a pinned host buffer from
 * fm_host_alloc, which makes the kernel deliver y to the host while it runs instead of a
 * device-to-host copy afterwards — for every q (npeers 1..8) and that [local_base, +span) is a
 * local allocation, then writes the npeers byte offsets (copy - local) to dev_deltas for
 * w4a8_decode_stream / w4a4_decode_stream. */
int   fm_ipc_export(const void* dev, void* out_handle64, unsigned long long* out_offset,
                    unsigned long long* out_size);
void* fm_ipc_import(const void* handle64, unsigned long long size);
int   fm_stream_peers(void* dev_deltas, const uint64_t* peer_bases, int npeers, const void* local_base,
                      unsigned long long span);

/* Drains the stream and returns (then clears) the status word of the tcgen05 GEMM kernels:
 * 0, or the code of the first bounded wait that ran out (the results are then invalid). */
int   fm_gemm_status(void);

/* Drains the stream and returns (then clears) the status word of the decode GEMV entries that run on the bulk-copy
 * ring (gemv_w4a8<2..4,..> at K = 5120): 0, or the code of the first bounded wait that ran
 * out (the results are then invalid).  The multi-layer stream entries take a status word as an argument instead. */
int   fm_stream_status(void);

/* device timers on the engine stream */
int   fm_event_create(void);
int   fm_event_record(int ev);
float fm_event_elapsed_ms(int ev_start, int ev_stop);   /* <0 on error */

/* explicit CUDA-graph capture of everything enqueued between begin and end */
int   fm_graph_begin(void);
int   fm_graph_end(void);              /* graph id >= 0, or <0 */
int   fm_graph_launch(int graph);
int   fm_graph_free(int graph);

/* one process per GPU: NCCL communicator over NVLink/NVSwitch */
int   fm_comm_unique_id(void* out128);
int   fm_comm_init(const void* id128, int nranks, int rank);
int   fm_comm_rank(void);
int   fm_comm_size(void);
int   fm_allgather(void* recv, const void* send, size_t bytes_per_rank);
int   fm_comm_destroy(void);

/* No counterpart in the reference.  A whole W4A8 decode layer, y[M][N] = W . x, for callers
 * that are not allowed to allocate device memory where they call it (code inside another
 * component's stream capture, server plugins with a fixed memory plan, real-time loops):
 * quant_act followed by gemv_w4a8, with the quantised activations kept in a 73 728-byte
 * array inside the library's device image instead of a caller-allocated buffer.
 *   wq [N][K/2] bytes (two's-complement nibbles), ws_f16 [N][K/128], x [M][K] f32, y [M][N] f32
 *   are the caller's device buffers; `stream` is a cudaStream_t (NULL = default stream);
 *   wait != 0 blocks until the result is ready.
 * Limits: M 1..4; K a multiple of 128, at most 16384 — beyond that -4 with a message.
 * The first call on a device resolves the array's address; make it outside stream capture.
 * All calls on a GPU share the array: calls on one stream are safe, calls whose kernels
 * overlap on the GPU race.  Does not use the engine (no fm_init needed) and makes no
 * allocating call. */
int   fm_w4a8_linear_static(const void* wq, const void* ws_f16, const float* x, float* y,
                            int M, int N, int K, void* stream, int wait);

#ifdef __cplusplus
}
#endif
