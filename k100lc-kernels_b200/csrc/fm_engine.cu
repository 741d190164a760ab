// libfm_engine.so: the C ABI of the reference engine (runtime/fm_engine.{h,cpp},
// by-name launch with a uint64 argv) re-implemented over the CUDA runtime for B200,
// plus the extensions declared in include/fm_engine.h (timers, pinned copies,
// explicit graphs, an NCCL communicator).
//
// Observable semantics kept from the reference runtime (runtime/hsa_rt.cpp):
//   * one process-global engine, one in-order queue (here: one CUDA stream);
//   * launches return immediately, fm_sync drains, copies are ordered on the queue
//     and upload/download return when done (hsa_rt.cpp:732-761);
//   * fm_alloc returns NULL when out of memory (hsa_rt.cpp:698-708);
//   * fm_init is idempotent and ignores a second image name (hsa_rt.cpp:383-396);
//   * argv is consumed before the call returns (runtime.py:169-175 relies on it).
// Differences: errors come back as negative codes instead of ending the process, and
// every pointer argument is checked against the live allocations before a launch.
#include "../../include/fm_engine.h"

#include <cuda_runtime.h>
#include <dlfcn.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <iterator>
#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "stage_split.h"
#include "fm_internal.h"

namespace fm {
namespace {

struct Graph {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    unsigned long long kernels = 0;      // kernel launches recorded in it
};

struct Engine {
    std::recursive_mutex mu;
    bool ready = false;
    int device = -1;            // -1: choose at init
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    cudaStream_t copy_stream = nullptr;       // second queue for uploads that run beside the kernels (fm_upload_beside)
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    cudaStream_t down_stream = nullptr;       // third queue for downloads that run beside the kernels (fm_download_beside)
    cudaEvent_t ev_dfork = nullptr, ev_down[4] = {nullptr, nullptr, nullptr, nullptr};
    unsigned long long downloads = 0;         // fm_download_beside calls so far (ev_down is a ring over them)
    bool copy_pending = false;
    std::string image;
    bool check_bounds = true;
    bool pdl = false;
    bool capturing = false;
    unsigned long long launches = 0;          // kernels enqueued for execution so far
    unsigned long long launches_at_capture = 0;
    std::vector<KernelEntry> kernels;
    std::unordered_map<std::string, int> by_name;
    std::map<uintptr_t, size_t> allocs;          // base -> bytes
    // A validated record names every allocation (device, imported or pinned) that its pointers lie in:
    // freeing one of them drops the record, so a launch that still names it is rejected (-4) until
    // fm_stream_table / fm_stream_peers is called again.
    struct Table { size_t bytes; int nlayers, rows, K, row_base; uintptr_t y_lo, y_hi, y_ptr_lo; size_t ws_avail; bool x_all;
                   std::vector<uintptr_t> deps;
                   unsigned long long serial = 0;        // distinguishes this record from an earlier one at the same address
                   std::vector<uintptr_t> wq;            // the wq entry of every layer (for the TMA tensor maps)
                   uintptr_t shapes = 0;                 // fm_stream_table_var: device array of per-layer shapes (64 bytes each)
                   int min_rows = 0, max_rows = 0; };
    struct MapSet { void* dev; unsigned long long serial; };
    std::map<uintptr_t, MapSet> table_maps;      // table address -> device array of tensor maps built for record `serial`
    unsigned long long table_serial = 0;
    std::map<uintptr_t, Table> tables;           // validated stream layer tables
    struct Peers { int npeers; uintptr_t lo, hi; std::vector<uintptr_t> deps; };
    std::map<uintptr_t, Peers> peers;            // validated peer-offset arrays (device address -> window)
    unsigned long long epoch = 0;                // bumped whenever an allocation is freed or a validated record is dropped
    std::map<uintptr_t, size_t> imported;        // peer allocations opened through CUDA IPC
    std::map<uintptr_t, size_t> pinned;          // fm_host_alloc buffers (device-addressable host memory)
    void* scratch = nullptr;                     // kernel-internal workspace (grows on demand)
    size_t scratch_bytes = 0;
    std::vector<void*> retired_scratch;          // outgrown workspaces, still referenced by captured graphs
    std::vector<cudaEvent_t> events;
    std::vector<Graph> graphs;
    struct PlanGraph { int gid; unsigned long long epoch; std::vector<uint64_t> words; };
    std::unordered_map<uint64_t, PlanGraph> plan_graphs;   // plan hash -> captured graph, the epoch it was checked in, its words
    // NCCL (resolved with dlopen when a communicator is first asked for)
    void* nccl_lib = nullptr;
    void* comm = nullptr;
    int comm_rank = 0, comm_size = 1;
};

Engine& E() {
    static Engine e;
    return e;
}

// The text of the last failure is kept per host thread: entry points that do not take the engine
// lock (fm_w4a8_linear_static) may fail concurrently with engine calls on other threads, and a
// caller reads the message on the thread that saw the error code.
std::string& last_error() {
    static thread_local std::string s;
    return s;
}

void set_error(const char* fmt, va_list ap) {
    char buf[512];
    vsnprintf(buf, sizeof buf, fmt, ap);
    last_error() = buf;
    if (getenv("FM_DEBUG")) fprintf(stderr, "fm_engine: %s\n", buf);
}

void set_errorf(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    set_error(fmt, ap);
    va_end(ap);
}

void add_kernels(const KernelEntry* k, int n) {
    Engine& e = E();
    for (int i = 0; i < n; i++) {
        e.by_name[k[i].name] = (int)e.kernels.size();
        e.kernels.push_back(k[i]);
    }
}

int find_kernel(const char* name) {
    Engine& e = E();
    auto it = e.by_name.find(name ? name : "");
    return it == e.by_name.end() ? -1 : it->second;
}

int env_int(const char* k, int dflt) {
    const char* v = getenv(k);
    return (v && *v) ? atoi(v) : dflt;
}

int ensure_init() {
    Engine& e = E();
    if (e.ready) return 0;
    int dev = e.device;
    if (dev < 0) dev = env_int("FM_DEVICE", env_int("LOCAL_RANK", 0));
    int count = 0;
    cudaError_t err = cudaGetDeviceCount(&count);
    if (err != cudaSuccess || count == 0) {
        set_errorf("no CUDA device: %s", err == cudaSuccess ? "device count is 0" : cudaGetErrorString(err));
        return FM_ECUDA;
    }
    if (dev >= count) dev = dev % count;
    if ((err = cudaSetDevice(dev)) != cudaSuccess) {
        set_errorf("cudaSetDevice(%d): %s", dev, cudaGetErrorString(err));
        return FM_ECUDA;
    }
    cudaDeviceProp prop;
    if ((err = cudaGetDeviceProperties(&prop, dev)) != cudaSuccess) {
        set_errorf("cudaGetDeviceProperties: %s", cudaGetErrorString(err));
        return FM_ECUDA;
    }
    if (prop.major != 10) {
        set_errorf("device %d is sm_%d%d; this library carries sm_100a code only", dev, prop.major, prop.minor);
        return FM_ECUDA;
    }
    if ((err = cudaStreamCreateWithFlags(&e.stream, cudaStreamNonBlocking)) != cudaSuccess) {
        set_errorf("cudaStreamCreate: %s", cudaGetErrorString(err));
        return FM_ECUDA;
    }
    e.device = dev;
    e.sm_count = prop.multiProcessorCount;
    e.check_bounds = env_int("FM_CHECK_BOUNDS", 1) != 0;
    e.pdl = env_int("FM_PDL", 0) != 0;
    {   // workspace for kernel-internal intermediates, reserved up front so that a first use inside a
        // stream capture finds it ($FM_SCRATCH_MB, default 64: int4 activations of M x K <= 64 Mi widened)
        const size_t mb = (size_t)env_int("FM_SCRATCH_MB", 64);
        if (mb > 0 && cudaMalloc(&e.scratch, mb << 20) == cudaSuccess) e.scratch_bytes = mb << 20;
        else { cudaGetLastError(); e.scratch = nullptr; e.scratch_bytes = 0; }
    }
    if (e.kernels.empty()) {
        int n = 0;
        const KernelEntry* k;
        k = quant_kernels(&n); add_kernels(k, n);
        k = gemv_w4_kernels(&n); add_kernels(k, n);
        k = gemv_nvfp4_kernels(&n); add_kernels(k, n);
        k = int4_dot_kernels(&n); add_kernels(k, n);
        k = gemm_w4_kernels(&n); add_kernels(k, n);
        k = stream_kernels(&n); add_kernels(k, n);
        k = norm_act_kernels(&n); add_kernels(k, n);
        k = nvfp4_gemm_kernels(&n); add_kernels(k, n);
        k = moe_kernels(&n); add_kernels(k, n);
    }
    e.ready = true;
    return 0;
}

// the kernel table is also needed without a device (fm_has_kernel, catalog generation)
void ensure_table() {
    Engine& e = E();
    if (!e.kernels.empty()) return;
    int n = 0;
    const KernelEntry* k;
    k = quant_kernels(&n); add_kernels(k, n);
    k = gemv_w4_kernels(&n); add_kernels(k, n);
    k = gemv_nvfp4_kernels(&n); add_kernels(k, n);
    k = int4_dot_kernels(&n); add_kernels(k, n);
    k = gemm_w4_kernels(&n); add_kernels(k, n);
    k = stream_kernels(&n); add_kernels(k, n);
    k = norm_act_kernels(&n); add_kernels(k, n);
    k = nvfp4_gemm_kernels(&n); add_kernels(k, n);
    k = moe_kernels(&n); add_kernels(k, n);
}

// The tensor maps of a layer table whose record is dropped: captured graphs may still hold kernel nodes that point at
// them, so while any graph is alive (or a capture is running) they are only retired, and freed with the last graph.
void drop_table_maps(uintptr_t table) {
    Engine& e = E();
    auto im = e.table_maps.find(table);
    if (im == e.table_maps.end()) return;
    bool graphs_alive = e.capturing;
    for (const Graph& g : e.graphs) graphs_alive = graphs_alive || g.exec != nullptr;
    if (graphs_alive) {
        e.retired_scratch.push_back(im->second.dev);
    } else {
        cudaStreamSynchronize(e.stream);
        cudaFree(im->second.dev);
    }
    e.table_maps.erase(im);
}

// a write into [p, p+n) makes any validated layer table it touches unvalidated
void touch(const void* p, size_t n) {
    Engine& e = E();
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    for (auto it = e.tables.begin(); it != e.tables.end();) {
        const Engine::Table& t = it->second;
        const bool hit = (a < it->first + t.bytes && it->first < a + n) ||
                         (t.shapes && a < t.shapes + (size_t)t.nlayers * 64 && t.shapes < a + n);
        if (hit) { drop_table_maps(it->first); it = e.tables.erase(it); e.epoch++; }
        else ++it;
    }
    for (auto it = e.peers.begin(); it != e.peers.end();) {
        if (a < it->first + (size_t)it->second.npeers * 8 && it->first < a + n) { it = e.peers.erase(it); e.epoch++; }
        else ++it;
    }
}

// base address of the device, imported or pinned allocation that contains `a` (0 when none does)
uintptr_t owner_of(uintptr_t a) {
    Engine& e = E();
    for (const auto* m : {&e.allocs, &e.pinned}) {
        auto it = m->upper_bound(a);
        if (it == m->begin()) continue;
        --it;
        if (a >= it->first && a < it->first + it->second) return it->first;
    }
    return 0;
}

void add_dep(std::vector<uintptr_t>& deps, uintptr_t a) {
    const uintptr_t b = owner_of(a);
    if (b == 0) return;
    for (uintptr_t d : deps) if (d == b) return;
    deps.push_back(b);
}

// The allocation at `base` is going away: every validated table or peer-offset array that points
// into it (or lives in it) is dropped, and the epoch moves on so that cached plan graphs, which may
// hold kernel nodes with pointers into it, are captured afresh through the checks.
void release_dependents(uintptr_t base) {
    Engine& e = E();
    e.epoch++;
    auto uses = [&](const std::vector<uintptr_t>& deps) {
        for (uintptr_t d : deps) if (d == base) return true;
        return false;
    };
    for (auto it = e.tables.begin(); it != e.tables.end();) {
        if (uses(it->second.deps)) { drop_table_maps(it->first); it = e.tables.erase(it); }
        else ++it;
    }
    for (auto it = e.peers.begin(); it != e.peers.end();) it = uses(it->second.deps) ? e.peers.erase(it) : std::next(it);
}

int do_launch(int kid, uint32_t gx, uint32_t gy, uint32_t wx, uint32_t wy, const uint64_t* argv, int nargs) {
    Engine& e = E();
    const KernelEntry& k = e.kernels[kid];
    if (k.nargs != nargs) {
        set_errorf("%s takes %d explicit arguments, %d given", k.name, k.nargs, nargs);
        return FM_ENARGS;
    }
    LaunchCtx ctx{gx, gy, wx, wy, e.stream, e.sm_count};
    return k.fn(ctx, argv);
}

uint64_t fnv1a(const uint64_t* p, size_t n) {
    uint64_t h = 1469598103934665603ull;
    for (size_t i = 0; i < n; i++) {
        h ^= p[i];
        h *= 1099511628211ull;
    }
    return h;
}

// walks a plan, launching each record; returns records enqueued
int run_plan(const uint64_t* plan, int nrec) {
    Engine& e = E();
    size_t i = 0;
    int done = 0;
    for (; done < nrec; done++) {
        const int kid = (int)plan[i];
        const uint32_t grid = (uint32_t)plan[i + 1], wg = (uint32_t)plan[i + 2];
        const int nargs = (int)plan[i + 3];
        if (kid < 0 || kid >= (int)e.kernels.size()) {
            set_errorf("plan record %d: bad kernel id %d", done, kid);
            break;
        }
        if (do_launch(kid, grid, 1, wg, 1, plan + i + 4, nargs) != FM_OK) break;
        i += 4 + (size_t)nargs;
    }
    return done;
}

size_t plan_words(const uint64_t* plan, int nrec) {
    size_t i = 0;
    for (int r = 0; r < nrec; r++) i += 4 + (size_t)plan[i + 3];
    return i;
}

// ---- NCCL through dlopen: the library loads and runs without NCCL present ----
typedef struct { char internal[128]; } NcclUniqueId;
typedef int (*nccl_get_uid_t)(NcclUniqueId*);
typedef int (*nccl_init_rank_t)(void**, int, NcclUniqueId, int);
typedef int (*nccl_allgather_t)(const void*, void*, size_t, int, void*, cudaStream_t);
typedef int (*nccl_destroy_t)(void*);
typedef const char* (*nccl_errstr_t)(int);

void* nccl_sym(const char* name) {
    Engine& e = E();
    if (!e.nccl_lib) {
        const char* names[] = {getenv("FM_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
        for (const char* n : names) {
            if (n && *n && (e.nccl_lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL))) break;
        }
        if (!e.nccl_lib) {
            set_errorf("cannot load NCCL (set FM_NCCL_LIB): %s", dlerror());
            return nullptr;
        }
    }
    void* s = dlsym(e.nccl_lib, name);
    if (!s) set_errorf("NCCL symbol %s missing", name);
    return s;
}

}  // namespace

// ---- services for the kernel files -----------------------------------------
bool range_ok(const void* p, size_t bytes) {
    Engine& e = E();
    if (!e.check_bounds) return true;
    if (bytes == 0) return true;
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    auto it = e.allocs.upper_bound(a);
    if (it == e.allocs.begin()) return false;
    --it;
    return a >= it->first && a + bytes <= it->first + it->second;
}

int reject(const char* kernel, const char* fmt, ...) {
    char msg[400];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(msg, sizeof msg, fmt, ap);
    va_end(ap);
    set_errorf("%s rejected: %s", kernel, msg);
    return FM_EREJECT;
}

int cuda_fail(const char* kernel, cudaError_t err) {
    set_errorf("%s: CUDA error %d (%s)", kernel, (int)err, cudaGetErrorString(err));
    return FM_ECUDA;
}

int after_launch(const char* kernel) {
    E().launches++;
    if (E().capturing) return FM_OK;          // errors surface when the capture ends
    cudaError_t err = cudaPeekAtLastError();
    return err == cudaSuccess ? FM_OK : cuda_fail(kernel, cudaGetLastError());
}

bool pdl_enabled() { return E().pdl; }

// Device workspace owned by the engine for intermediates that the reference ABI has no argument
// for.  It only grows, and growing means a synchronising free + allocation, which a stream
// capture forbids: inside a capture a request beyond the current size returns nullptr.
void* engine_scratch(size_t bytes) {
    Engine& e = E();
    if (bytes <= e.scratch_bytes) return e.scratch;
    if (e.capturing) return nullptr;
    // graphs captured earlier may hold kernel nodes that point into the old buffer: while any graph is
    // alive it is only retired (and freed with the last graph); without graphs it is freed at once
    if (e.scratch) {
        bool graphs_alive = false;
        for (const Graph& g : e.graphs) graphs_alive = graphs_alive || g.exec != nullptr;
        if (graphs_alive) {
            e.retired_scratch.push_back(e.scratch);
        } else {
            cudaStreamSynchronize(e.stream);
            cudaFree(e.scratch);
        }
    }
    e.scratch = nullptr;
    e.scratch_bytes = 0;
    const size_t want = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
    if (cudaMalloc(&e.scratch, want) != cudaSuccess) {
        cudaGetLastError();
        e.scratch = nullptr;
        return nullptr;
    }
    e.scratch_bytes = want;
    return e.scratch;
}

bool stream_table_ok(const void* table, int nlayers, int rows, int K, int row_base, const void* peer_delta,
                     int npeers, bool whole_y, size_t ws_bytes, bool need_x) {
    Engine& e = E();
    if (!e.check_bounds) return true;
    auto it = e.tables.find(reinterpret_cast<uintptr_t>(table));
    if (it == e.tables.end()) return false;
    const Engine::Table& t = it->second;
    if (!(t.nlayers >= nlayers && t.rows == rows && t.K == K && t.row_base == row_base)) return false;
    if (ws_bytes > t.ws_avail) return false;
    if (need_x && !t.x_all) return false;
    if (npeers == 0) return true;
    // every y of the table must lie inside the window the peer offsets were validated for
    auto ip = e.peers.find(reinterpret_cast<uintptr_t>(peer_delta));
    if (ip == e.peers.end() || ip->second.npeers != npeers) return false;
    return (whole_y ? t.y_ptr_lo : t.y_lo) >= ip->second.lo && t.y_hi <= ip->second.hi;
}

bool stream_var_ok(const void* table, const void* shapes, int nlayers, const void* peer_delta, int npeers, int* min_rows,
                   int* max_rows, const void** chunk_maps) {
    Engine& e = E();
    auto it = e.tables.find(reinterpret_cast<uintptr_t>(table));
    if (it == e.tables.end()) return false;                 // (the shapes are needed even when the checks are off)
    const Engine::Table& t = it->second;
    if (!t.shapes || t.shapes != reinterpret_cast<uintptr_t>(shapes) || t.nlayers < nlayers) return false;
    *min_rows = t.min_rows;
    *max_rows = t.max_rows;
    auto im = e.table_maps.find(it->first);
    *chunk_maps = (im != e.table_maps.end() && im->second.serial == t.serial) ? im->second.dev : nullptr;
    if (npeers == 0 || !e.check_bounds) return true;
    auto ip = e.peers.find(reinterpret_cast<uintptr_t>(peer_delta));
    if (ip == e.peers.end() || ip->second.npeers != npeers) return false;
    return t.y_lo >= ip->second.lo && t.y_hi <= ip->second.hi;
}

const void* stream_table_maps(const void* table, int nlayers, int rows, int K) {
    Engine& e = E();
    const uintptr_t key = reinterpret_cast<uintptr_t>(table);
    auto it = e.tables.find(key);
    if (it == e.tables.end()) return nullptr;
    const Engine::Table& t = it->second;
    if (t.nlayers < nlayers || t.rows != rows || t.K != K || (int)t.wq.size() < nlayers) return nullptr;
    auto im = e.table_maps.find(key);
    if (im != e.table_maps.end() && im->second.serial == t.serial) return im->second.dev;
    if (e.capturing) return nullptr;                        // building needs an allocation and a synchronous copy
    std::vector<unsigned char> host((size_t)t.nlayers * 128);
    for (int l = 0; l < t.nlayers; l++)
        if (!encode_bytes_rows_map(host.data() + (size_t)l * 128, reinterpret_cast<const void*>(t.wq[l]), (uint64_t)rows,
                                   (uint64_t)K / 2, 128))
            return nullptr;
    if (im != e.table_maps.end()) drop_table_maps(key);      // maps of an older record at this address
    void* dev = nullptr;
    if (cudaMalloc(&dev, host.size()) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    if (cudaMemcpy(dev, host.data(), host.size(), cudaMemcpyHostToDevice) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(dev);
        return nullptr;
    }
    e.table_maps[key] = Engine::MapSet{dev, t.serial};
    return dev;
}

bool peer_window_ok(const void* peer_delta, int npeers, const void* ptr, size_t bytes) {
    Engine& e = E();
    if (!e.check_bounds) return true;
    auto ip = e.peers.find(reinterpret_cast<uintptr_t>(peer_delta));
    if (ip == e.peers.end() || ip->second.npeers != npeers) return false;
    const uintptr_t a = reinterpret_cast<uintptr_t>(ptr);
    return a >= ip->second.lo && a + bytes <= ip->second.hi;
}

}  // namespace fm

using namespace fm;
#define LOCK std::lock_guard<std::recursive_mutex> lock_(E().mu)
#define NEED_INIT(fail) do { if (ensure_init() != 0) return fail; } while (0)

extern "C" {

int fm_init(const char* image) {
    LOCK;
    if (E().ready) return 0;
    if (image) E().image = image;
    return ensure_init() == 0 ? 0 : -1;
}

void* fm_alloc(size_t n) {
    LOCK;
    NEED_INIT(nullptr);
    void* p = nullptr;
    if (n == 0) n = 1;
    if (cudaMalloc(&p, n) != cudaSuccess) {
        cudaGetLastError();
        set_errorf("fm_alloc(%zu): out of device memory", n);
        return nullptr;
    }
    E().allocs[reinterpret_cast<uintptr_t>(p)] = n;
    return p;
}

void fm_free(void* p) {
    LOCK;
    if (!p || !E().ready) return;
    cudaStreamSynchronize(E().stream);        // nothing in flight may still use it
    if (E().copy_stream) cudaStreamSynchronize(E().copy_stream);
    if (E().down_stream) cudaStreamSynchronize(E().down_stream);
    auto it = E().allocs.find(reinterpret_cast<uintptr_t>(p));
    if (it != E().allocs.end()) {
        touch(p, it->second);
        release_dependents(it->first);
        E().allocs.erase(it);
    }
    auto im = E().imported.find(reinterpret_cast<uintptr_t>(p));
    if (im != E().imported.end()) {              // a peer's allocation: unmap, do not free
        E().imported.erase(im);
        cudaIpcCloseMemHandle(p);
        return;
    }
    cudaFree(p);
}

static int copy_sync(void* dst, const void* src, size_t n, cudaMemcpyKind kind, const char* what) {
    Engine& e = E();
    if (n == 0) return 0;
    cudaError_t err = cudaMemcpyAsync(dst, src, n, kind, e.stream);
    if (err == cudaSuccess) err = cudaStreamSynchronize(e.stream);
    if (err != cudaSuccess) {
        cuda_fail(what, err);
        return -1;
    }
    return 0;
}

int fm_upload(void* dev, const void* host, size_t n) {
    LOCK;
    NEED_INIT(-1);
    if (!range_ok(dev, n)) { set_errorf("fm_upload: %zu bytes at %p exceed the allocation", n, dev); return -1; }
    touch(dev, n);
    return copy_sync(dev, host, n, cudaMemcpyHostToDevice, "fm_upload");
}

int fm_download(void* host, const void* dev, size_t n) {
    LOCK;
    NEED_INIT(-1);
    if (!range_ok(dev, n)) { set_errorf("fm_download: %zu bytes at %p exceed the allocation", n, dev); return -1; }
    return copy_sync(host, dev, n, cudaMemcpyDeviceToHost, "fm_download");
}

int fm_copy(void* dst, const void* src, size_t n) {
    LOCK;
    NEED_INIT(-1);
    if (!range_ok(dst, n) || !range_ok(src, n)) { set_errorf("fm_copy: range exceeds an allocation"); return -1; }
    if (n == 0) return 0;
    touch(dst, n);
    cudaError_t err = cudaMemcpyAsync(dst, src, n, cudaMemcpyDeviceToDevice, E().stream);
    if (err != cudaSuccess) { cuda_fail("fm_copy", err); return -1; }
    return 0;
}

int fm_memset(void* dev, int v, size_t n) {
    LOCK;
    NEED_INIT(-1);
    if (!range_ok(dev, n)) { set_errorf("fm_memset: range exceeds the allocation"); return -1; }
    if (n == 0) return 0;
    touch(dev, n);
    cudaError_t err = cudaMemsetAsync(dev, v, n, E().stream);
    if (err != cudaSuccess) { cuda_fail("fm_memset", err); return -1; }
    return 0;
}

int fm_sync(void) {
    LOCK;
    NEED_INIT(-1);
    cudaError_t err = cudaStreamSynchronize(E().stream);
    if (err == cudaSuccess && E().copy_stream) err = cudaStreamSynchronize(E().copy_stream);
    if (err == cudaSuccess && E().down_stream) err = cudaStreamSynchronize(E().down_stream);
    if (err != cudaSuccess) { cuda_fail("fm_sync", err); return -1; }
    return 0;
}

int fm_launch2d(const char* kernel, uint32_t gx, uint32_t gy, uint32_t wx, uint32_t wy,
                const uint64_t* argv, int nargs) {
    LOCK;
    NEED_INIT(FM_ECUDA);
    const int kid = find_kernel(kernel);
    if (kid < 0) {
        set_errorf("no kernel named %s", kernel ? kernel : "(null)");
        return FM_ENOKERNEL;
    }
    return do_launch(kid, gx, gy, wx, wy, argv, nargs);
}

int fm_launch(const char* kernel, uint32_t grid, uint32_t workgroup, const uint64_t* argv, int nargs) {
    return fm_launch2d(kernel, grid, 1, workgroup, 1, argv, nargs);
}

int fm_launch_dyn(const char* kernel, uint32_t gx, uint32_t gy, uint32_t wx, uint32_t wy,
                  const uint32_t* layout, uint32_t nargs, uint32_t group_size, uint32_t private_size,
                  uint32_t kernarg_size, const uint64_t* argv, int nargv) {
    (void)group_size;
    (void)private_size;
    if (kernarg_size > 1024) return FM_EDYN;
    int explicit_n = 0;
    for (uint32_t i = 0; i < nargs; i++)
        if (layout[3 * i + 2] == 0) explicit_n++;
    if (explicit_n != nargv) return FM_ENARGS;
    return fm_launch2d(kernel, gx, gy, wx, wy, argv, nargv);
}

int fm_has_kernel(const char* kernel) {
    LOCK;
    ensure_table();
    return find_kernel(kernel) >= 0 ? 1 : 0;
}

int fm_kernel_id(const char* kernel) {
    LOCK;
    ensure_table();
    return find_kernel(kernel);
}

int fm_launch_batch(const uint64_t* plan, int nrec) {
    LOCK;
    NEED_INIT(0);
    Engine& e = E();
    if (nrec <= 0) return 0;
    if (e.capturing || getenv("FM_NO_GRAPH")) return run_plan(plan, nrec);
    const size_t words = plan_words(plan, nrec);
    const uint64_t h = fnv1a(plan, words) ^ ((uint64_t)nrec << 48);
    auto it = e.plan_graphs.find(h);
    // A cached graph is replayed only while nothing it was checked against has changed: same words
    // (a hash collision must not replay another plan), and no allocation freed or validated table
    // dropped since the capture (the epoch).  Otherwise it is captured afresh, which runs every
    // record through the launchers' range and table checks again.
    if (it != e.plan_graphs.end() &&
        (it->second.epoch != e.epoch || it->second.words.size() != words ||
         memcmp(it->second.words.data(), plan, words * 8) != 0)) {
        fm_graph_free(it->second.gid);
        e.plan_graphs.erase(it);
        it = e.plan_graphs.end();
    }
    if (it == e.plan_graphs.end()) {
        // first sight of this exact plan: capture it (a patched plan hashes differently
        // and is captured afresh, so LaunchPlan.set_arg/set_grid are honoured)
        if (e.plan_graphs.size() >= 64) {          // bound the cache
            for (auto& kv : e.plan_graphs) fm_graph_free(kv.second.gid);
            e.plan_graphs.clear();
        }
        if (fm_graph_begin() != 0) return run_plan(plan, nrec);
        const int done = run_plan(plan, nrec);
        const int gid = fm_graph_end();
        if (done != nrec || gid < 0) {
            if (gid >= 0) fm_graph_free(gid);
            // nothing of the capture has run: enqueue the records in front of the rejected one for
            // real, so that the count returned is the count enqueued (as with the reference's batch)
            return run_plan(plan, done);
        }
        it = e.plan_graphs.emplace(h, Engine::PlanGraph{gid, e.epoch, std::vector<uint64_t>(plan, plan + words)}).first;
    }
    return fm_graph_launch(it->second.gid) == 0 ? nrec : 0;
}

// ---- extensions -----------------------------------------------------------

const char* fm_last_error(void) { return last_error().c_str(); }

int fm_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}

int fm_set_device(int dev) {
    LOCK;
    if (E().ready) return E().device == dev ? 0 : -1;
    E().device = dev;
    return 0;
}

int fm_device_attr(int what) {
    LOCK;
    NEED_INIT(-1);
    int v = 0;
    switch (what) {
        case 0: return E().sm_count;
        case 1: cudaDeviceGetAttribute(&v, cudaDevAttrL2CacheSize, E().device); return v;
        case 2: return E().device;
        case 3: { size_t fr = 0, tot = 0; cudaMemGetInfo(&fr, &tot); return (int)(tot >> 20); }
        case 4: cudaDeviceGetAttribute(&v, cudaDevAttrClockRate, E().device); return v;
        default: return -1;
    }
}

int fm_kernel_count(void) { LOCK; ensure_table(); return (int)E().kernels.size(); }
const char* fm_kernel_name(int id) {
    LOCK; ensure_table();
    return (id >= 0 && id < (int)E().kernels.size()) ? E().kernels[id].name : nullptr;
}
int fm_kernel_nargs(int id) {
    LOCK; ensure_table();
    return (id >= 0 && id < (int)E().kernels.size()) ? E().kernels[id].nargs : -1;
}
const char* fm_kernel_sig(int id) {
    LOCK; ensure_table();
    return (id >= 0 && id < (int)E().kernels.size()) ? E().kernels[id].sig : nullptr;
}
unsigned long long fm_launch_count(void) { return E().launches; }

void* fm_host_alloc(size_t n) {
    LOCK;
    NEED_INIT(nullptr);
    void* p = nullptr;
    if (cudaHostAlloc(&p, n ? n : 1, cudaHostAllocPortable | cudaHostAllocMapped) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    E().pinned[reinterpret_cast<uintptr_t>(p)] = n ? n : 1;
    return p;
}
void fm_host_free(void* p) {
    if (!p) return;
    {
        LOCK;
        if (E().ready) cudaStreamSynchronize(E().stream);      // a kernel in flight may still be storing into it
        if (E().pinned.count(reinterpret_cast<uintptr_t>(p))) release_dependents(reinterpret_cast<uintptr_t>(p));
        E().pinned.erase(reinterpret_cast<uintptr_t>(p));
    }
    cudaFreeHost(p);
}

int fm_upload_async(void* dev, const void* host, size_t n) {
    LOCK;
    NEED_INIT(-1);
    if (!range_ok(dev, n)) { set_errorf("fm_upload_async: range exceeds the allocation"); return -1; }
    touch(dev, n);
    cudaError_t err = cudaMemcpyAsync(dev, host, n, cudaMemcpyHostToDevice, E().stream);
    if (err != cudaSuccess) { cuda_fail("fm_upload_async", err); return -1; }
    return 0;
}
// Upload on a second queue.  The copy starts once everything enqueued on the engine stream BEFORE this call has
// finished (so it may overwrite a buffer whose last reader is already enqueued), and runs beside whatever is
// enqueued AFTER it; fm_upload_join makes the engine stream wait for it.  Pattern for double-buffered inputs:
//   fm_upload_beside(x[(t+1)%2], ...); fm_graph_launch(step t, reading x[t%2]); fm_upload_join();
int fm_upload_beside(void* dev, const void* host, size_t n) {
    LOCK;
    NEED_INIT(-1);
    Engine& e = E();
    if (e.capturing) { set_errorf("fm_upload_beside: not inside a graph capture"); return -1; }
    if (!range_ok(dev, n)) { set_errorf("fm_upload_beside: range exceeds the allocation"); return -1; }
    if (!e.copy_stream) {
        if (cudaStreamCreateWithFlags(&e.copy_stream, cudaStreamNonBlocking) != cudaSuccess ||
            cudaEventCreateWithFlags(&e.ev_fork, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&e.ev_join, cudaEventDisableTiming) != cudaSuccess) {
            cuda_fail("fm_upload_beside", cudaGetLastError());
            return -1;
        }
    }
    touch(dev, n);
    cudaError_t err = cudaEventRecord(e.ev_fork, e.stream);
    if (err == cudaSuccess) err = cudaStreamWaitEvent(e.copy_stream, e.ev_fork, 0);
    if (err == cudaSuccess) err = cudaMemcpyAsync(dev, host, n, cudaMemcpyHostToDevice, e.copy_stream);
    if (err == cudaSuccess) err = cudaEventRecord(e.ev_join, e.copy_stream);
    if (err != cudaSuccess) { cuda_fail("fm_upload_beside", err); return -1; }
    e.copy_pending = true;
    return 0;
}
// Device-to-device copy on the second queue, behind whatever that queue already holds (an fm_upload_beside, say):
// `dst` may lie in a peer's allocation opened with fm_ipc_import, which makes this the copy-engine way to hand a
// freshly uploaded slice to the other GPUs while the kernels of the engine stream keep running.
int fm_copy_beside(void* dst, const void* src, size_t n) {
    LOCK;
    NEED_INIT(-1);
    Engine& e = E();
    if (e.capturing) { set_errorf("fm_copy_beside: not inside a graph capture"); return -1; }
    if (!range_ok(dst, n) || !range_ok(src, n)) { set_errorf("fm_copy_beside: range exceeds an allocation"); return -1; }
    if (!e.copy_stream) { set_errorf("fm_copy_beside: call fm_upload_beside first (it opens the second queue)"); return -1; }
    if (n == 0) return 0;
    touch(dst, n);
    cudaError_t err = cudaMemcpyAsync(dst, src, n, cudaMemcpyDeviceToDevice, e.copy_stream);
    if (err == cudaSuccess) err = cudaEventRecord(e.ev_join, e.copy_stream);
    if (err != cudaSuccess) { cuda_fail("fm_copy_beside", err); return -1; }
    e.copy_pending = true;
    return 0;
}
int fm_upload_join(void) {
    LOCK;
    NEED_INIT(-1);
    Engine& e = E();
    if (!e.copy_pending) return 0;
    cudaError_t err = cudaStreamWaitEvent(e.stream, e.ev_join, 0);
    if (err != cudaSuccess) { cuda_fail("fm_upload_join", err); return -1; }
    e.copy_pending = false;
    return 0;
}

// Download on a third queue: `height` rows of `width` bytes, `dpitch` / `hpitch` bytes between the starts of rows on
// the device / the host (height 1: a plain copy).  The copy starts once everything enqueued on the engine stream BEFORE
// this call has finished and runs beside whatever is enqueued after it.  fm_download_join(lag) makes the engine stream
// wait for the download issued `lag` calls before the latest (0..3).  Pattern for double-buffered outputs:
//   fm_download_join(1); fm_graph_launch(step t, writing y[t%2]); fm_download_beside(host, ..., y[t%2], ...);
int fm_download_beside(void* host, size_t hpitch, const void* dev, size_t dpitch, size_t width, size_t height) {
    LOCK;
    NEED_INIT(-1);
    Engine& e = E();
    if (e.capturing) { set_errorf("fm_download_beside: not inside a graph capture"); return -1; }
    if (width == 0 || height == 0) return 0;
    if (height > 1 && (dpitch < width || hpitch < width)) { set_errorf("fm_download_beside: a pitch is smaller than the width"); return -1; }
    if (!range_ok(dev, (height - 1) * dpitch + width)) { set_errorf("fm_download_beside: range exceeds the allocation"); return -1; }
    if (!e.down_stream) {
        bool ok = cudaStreamCreateWithFlags(&e.down_stream, cudaStreamNonBlocking) == cudaSuccess &&
                  cudaEventCreateWithFlags(&e.ev_dfork, cudaEventDisableTiming) == cudaSuccess;
        for (int i = 0; ok && i < 4; i++) ok = cudaEventCreateWithFlags(&e.ev_down[i], cudaEventDisableTiming) == cudaSuccess;
        if (!ok) { cuda_fail("fm_download_beside", cudaGetLastError()); return -1; }
    }
    cudaError_t err = cudaEventRecord(e.ev_dfork, e.stream);
    if (err == cudaSuccess) err = cudaStreamWaitEvent(e.down_stream, e.ev_dfork, 0);
    if (err == cudaSuccess)
        err = height == 1 ? cudaMemcpyAsync(host, dev, width, cudaMemcpyDeviceToHost, e.down_stream)
                          : cudaMemcpy2DAsync(host, hpitch, dev, dpitch, width, height, cudaMemcpyDeviceToHost, e.down_stream);
    if (err == cudaSuccess) err = cudaEventRecord(e.ev_down[e.downloads % 4], e.down_stream);
    if (err != cudaSuccess) { cuda_fail("fm_download_beside", err); return -1; }
    e.downloads++;
    return 0;
}
int fm_download_join(int lag) {
    LOCK;
    NEED_INIT(-1);
    Engine& e = E();
    if (lag < 0 || lag > 3) { set_errorf("fm_download_join: lag=%d must be 0..3", lag); return -1; }
    if (e.downloads <= (unsigned long long)lag) return 0;       // nothing that old has been issued
    cudaError_t err = cudaStreamWaitEvent(e.stream, e.ev_down[(e.downloads - 1 - lag) % 4], 0);
    if (err != cudaSuccess) { cuda_fail("fm_download_join", err); return -1; }
    return 0;
}

int fm_download_async(void* host, const void* dev, size_t n) {
    LOCK;
    NEED_INIT(-1);
    if (!range_ok(dev, n)) { set_errorf("fm_download_async: range exceeds the allocation"); return -1; }
    cudaError_t err = cudaMemcpyAsync(host, dev, n, cudaMemcpyDeviceToHost, E().stream);
    if (err != cudaSuccess) { cuda_fail("fm_download_async", err); return -1; }
    return 0;
}

int fm_stream_table(void* dev_table, const uint64_t* host_layers, int nlayers, int rows, int K, int row_base) {
    LOCK;
    NEED_INIT(-1);
    Engine& e = E();
    if (nlayers <= 0 || rows <= 0 || K <= 0 || K % 128 || row_base < 0) {
        set_errorf("fm_stream_table: bad nlayers/rows/K/row_base");
        return -1;
    }
    const size_t bytes = (size_t)nlayers * 32;
    if (!range_ok(dev_table, bytes)) { set_errorf("fm_stream_table: the table does not fit its allocation"); return -1; }
    const size_t need[4] = {(size_t)rows * (K / 2), (size_t)rows * (K / 128) * 2, (size_t)K * 4,
                            ((size_t)row_base + rows) * 4};
    uintptr_t y_lo = ~(uintptr_t)0, y_hi = 0, y_ptr_lo = ~(uintptr_t)0;
    std::vector<uintptr_t> deps;                   // allocations the table points into (and the one it lives in)
    std::vector<uintptr_t> wqs((size_t)nlayers);
    for (int l = 0; l < nlayers; l++) wqs[l] = static_cast<uintptr_t>(host_layers[4 * l]);
    add_dep(deps, reinterpret_cast<uintptr_t>(dev_table));
    size_t ws_avail = ~(size_t)0;                  // fewest bytes between a ws pointer and the end of its allocation
    bool x_all = true;                             // every layer has a (validated) x
    const size_t align[4] = {16, 16, 16, 4};
    const char* what[4] = {"wq", "ws", "x", "y"};
    for (int l = 0; l < nlayers; l++)
        for (int j = 0; j < 4; j++) {
            const void* ptr = reinterpret_cast<const void*>(static_cast<uintptr_t>(host_layers[4 * l + j]));
            if (j == 2 && ptr == nullptr) { x_all = false; continue; }   // x is optional: most kernels read the codes
            if (!range_ok(ptr, need[j]) || !aligned(ptr, align[j])) {
                set_errorf("fm_stream_table: layer %d: %s (%zu bytes at %p) is misaligned or outside its allocation",
                           l, what[j], need[j], ptr);
                return FM_EREJECT;
            }
            add_dep(deps, static_cast<uintptr_t>(host_layers[4 * l + j]));
            if (j == 1) {
                const uintptr_t w = static_cast<uintptr_t>(host_layers[4 * l + j]);
                auto ia = e.allocs.upper_bound(w);
                if (ia != e.allocs.begin()) {
                    --ia;
                    const size_t avail = w < ia->first + ia->second ? ia->first + ia->second - w : 0;
                    if (avail < ws_avail) ws_avail = avail;
                } else {
                    ws_avail = 0;
                }
            }
            if (j == 3) {
                const uintptr_t y = static_cast<uintptr_t>(host_layers[4 * l + j]);
                if (y + (size_t)row_base * 4 < y_lo) y_lo = y + (size_t)row_base * 4;
                if (y + need[3] > y_hi) y_hi = y + need[3];
                if (y < y_ptr_lo) y_ptr_lo = y;
            }
        }
    if (copy_sync(dev_table, host_layers, bytes, cudaMemcpyHostToDevice, "fm_stream_table") != 0) return -1;
    touch(dev_table, bytes);
    e.tables[reinterpret_cast<uintptr_t>(dev_table)] =
        Engine::Table{bytes, nlayers, rows, K, row_base, y_lo, y_hi, y_ptr_lo, ws_avail, x_all, deps, ++e.table_serial, wqs};
    // The TMA tensor maps over the wq entries are built now, while allocating is allowed (a launch inside a graph
    // capture could not).  Best effort: a table the driver refuses to encode simply has none.
    if (K % 256 == 0) stream_table_maps(dev_table, nlayers, rows, K);
    return 0;
}

int fm_stream_table_var(void* dev_table, void* dev_shapes, const uint64_t* host_layers, int nlayers) {
    LOCK;
    NEED_INIT(-1);
    Engine& e = E();
    if (nlayers <= 0) { set_errorf("fm_stream_table_var: nlayers must be positive"); return -1; }
    const size_t tbytes = (size_t)nlayers * 32, sbytes_all = (size_t)nlayers * 64;
    if (!range_ok(dev_table, tbytes) || !range_ok(dev_shapes, sbytes_all) || !aligned(dev_table, 8) || !aligned(dev_shapes, 16)) {
        set_errorf("fm_stream_table_var: the table or the shape array does not fit its allocation (or is misaligned)");
        return -1;
    }
    struct Shape { uint64_t ae, ao, asc, asu; int rows, wpitch, spitch, wbytes, sbytes, accumulate, row_base, chunk; };
    static_assert(sizeof(Shape) == 64, "shape entry");
    std::vector<uint64_t> tab((size_t)nlayers * 4);
    std::vector<Shape> shp((size_t)nlayers);
    std::vector<uintptr_t> deps;
    add_dep(deps, reinterpret_cast<uintptr_t>(dev_table));
    add_dep(deps, reinterpret_cast<uintptr_t>(dev_shapes));
    uintptr_t y_lo = ~(uintptr_t)0, y_hi = 0;
    int min_rows = 1 << 30, max_rows = 0;
    for (int l = 0; l < nlayers; l++) {
        const uint64_t* h = host_layers + (size_t)l * 16;
        Shape& sh = shp[l];
        sh = Shape{h[4], h[5], h[6], h[7], (int)h[8], (int)h[9], (int)h[10], (int)h[11], (int)h[12], (int)h[13], (int)h[14], (int)h[15]};
        const bool shape_ok = sh.rows > 0 && sh.wbytes > 0 && sh.wbytes <= 2560 && sh.wbytes % 16 == 0 && sh.wpitch >= sh.wbytes &&
                              sh.wpitch % 16 == 0 && sh.sbytes > 0 && sh.sbytes <= 80 && sh.sbytes % 16 == 0 &&
                              sh.spitch >= sh.sbytes && sh.spitch % 16 == 0 && sh.sbytes * 32 == sh.wbytes &&
                              (sh.accumulate == 0 || sh.accumulate == 1) && sh.row_base >= 0 && sh.chunk >= 0 &&
                              (long long)sh.chunk * 2560 + sh.wbytes <= sh.wpitch && (long long)sh.chunk * 80 + sh.sbytes <= sh.spitch;
        if (!shape_ok) {
            set_errorf("fm_stream_table_var: layer %d: rows=%d wpitch=%d wbytes=%d spitch=%d sbytes=%d accumulate=%d row_base=%d is "
                       "not a shape this kernel takes (chunks of at most 5120 k, 16-byte granules, sbytes = wbytes / 32)", l, sh.rows,
                       sh.wpitch, sh.wbytes, sh.spitch, sh.sbytes, sh.accumulate, sh.row_base);
            return FM_EREJECT;
        }
        if (sh.accumulate) {                             // a later chunk continues the entry in front of it
            const Shape* pv = l ? &shp[l - 1] : nullptr;
            if (!pv || host_layers[(size_t)(l - 1) * 16 + 3] != h[3] || pv->rows != sh.rows || pv->row_base != sh.row_base ||
                pv->chunk + 1 != sh.chunk) {
                set_errorf("fm_stream_table_var: layer %d adds to y but the entry in front of it is not the chunk before it of the "
                           "same rows and the same y", l);
                return FM_EREJECT;
            }
        }
        const void* ptrs[7] = {(const void*)(uintptr_t)h[0], (const void*)(uintptr_t)h[1], (const void*)(uintptr_t)h[3],
                               (const void*)(uintptr_t)h[4], (const void*)(uintptr_t)h[5], (const void*)(uintptr_t)h[6],
                               (const void*)(uintptr_t)h[7]};
        const size_t need[7] = {(size_t)(sh.rows - 1) * sh.wpitch + sh.wbytes, (size_t)(sh.rows - 1) * sh.spitch + sh.sbytes,
                                ((size_t)sh.row_base + sh.rows) * 4, 2560, 2560, 160, 160};
        const size_t algn[7] = {16, 16, 4, 16, 16, 16, 16};
        const char* what[7] = {"wq", "ws", "y", "ae", "ao", "asc", "asu"};
        for (int j = 0; j < 7; j++) {
            if (!range_ok(ptrs[j], need[j]) || !aligned(ptrs[j], algn[j])) {
                set_errorf("fm_stream_table_var: layer %d: %s (%zu bytes at %p) is misaligned or outside its allocation", l, what[j],
                           need[j], ptrs[j]);
                return FM_EREJECT;
            }
            add_dep(deps, reinterpret_cast<uintptr_t>(ptrs[j]));
        }
        tab[4 * l] = h[0]; tab[4 * l + 1] = h[1]; tab[4 * l + 2] = 0; tab[4 * l + 3] = h[3];
        const uintptr_t y = (uintptr_t)h[3];
        if (y + (size_t)sh.row_base * 4 < y_lo) y_lo = y + (size_t)sh.row_base * 4;
        if (y + need[2] > y_hi) y_hi = y + need[2];
        if (sh.rows < min_rows) min_rows = sh.rows;
        if (sh.rows > max_rows) max_rows = sh.rows;
    }
    if (copy_sync(dev_table, tab.data(), tbytes, cudaMemcpyHostToDevice, "fm_stream_table_var") != 0) return -1;
    if (copy_sync(dev_shapes, shp.data(), sbytes_all, cudaMemcpyHostToDevice, "fm_stream_table_var") != 0) return -1;
    touch(dev_table, tbytes);
    touch(dev_shapes, sbytes_all);
    Engine::Table t{tbytes, nlayers, max_rows, 5120, 0, y_lo, y_hi, y_lo, 0, false, deps, ++e.table_serial, {}};
    t.shapes = reinterpret_cast<uintptr_t>(dev_shapes);
    t.min_rows = min_rows;
    t.max_rows = max_rows;
    e.tables[reinterpret_cast<uintptr_t>(dev_table)] = t;
    // TMA maps for the layers that are chunks of longer rows (a box copy per 16 rows instead of a bulk copy per row);
    // best effort: without them the kernel copies row by row
    bool any = false, ok = true;
    std::vector<unsigned char> maps((size_t)nlayers * 256, 0);
    for (int l = 0; l < nlayers && ok; l++) {
        const Shape& sh = shp[l];
        if (sh.wpitch == 2560 && sh.spitch == 80) continue;
        any = true;
        ok = sh.wpitch % 512 == 0 &&
             encode_chunk_maps(maps.data() + (size_t)l * 256, maps.data() + (size_t)l * 256 + 128,
                               reinterpret_cast<const void*>((uintptr_t)tab[4 * l] - (size_t)sh.chunk * 2560),
                               reinterpret_cast<const void*>((uintptr_t)tab[4 * l + 1] - (size_t)sh.chunk * 80), (uint64_t)sh.rows,
                               (uint64_t)sh.wpitch, (uint64_t)sh.spitch);
    }
    if (any && ok && !e.capturing) {
        void* dev = nullptr;
        if (cudaMalloc(&dev, maps.size()) == cudaSuccess &&
            cudaMemcpy(dev, maps.data(), maps.size(), cudaMemcpyHostToDevice) == cudaSuccess) {
            e.table_maps[reinterpret_cast<uintptr_t>(dev_table)] = Engine::MapSet{dev, t.serial};
        } else {
            cudaGetLastError();
            if (dev) cudaFree(dev);
        }
    }
    return 0;
}

int fm_stream_rows(int rows, int first, int grid, int cta, int* r0, int* r1) {
    if (rows <= 0 || first < 0 || grid <= 0 || cta < 0 || cta >= grid || !r0 || !r1) {
        set_errorf("fm_stream_rows: rows=%d first=%d grid=%d cta=%d out of range", rows, first, grid, cta);
        return -1;
    }
    fm::stage_split(rows, first, grid, cta, 16, r0, r1);
    return 0;
}

int fm_ipc_export(const void* dev, void* out_handle64, unsigned long long* out_offset, unsigned long long* out_size) {
    LOCK;
    NEED_INIT(-1);
    Engine& e = E();
    const uintptr_t a = reinterpret_cast<uintptr_t>(dev);
    auto it = e.allocs.upper_bound(a);
    if (it == e.allocs.begin()) { set_errorf("fm_ipc_export: %p is not inside an fm_alloc allocation", dev); return -1; }
    --it;
    if (a >= it->first + it->second || e.imported.count(it->first)) {
        set_errorf("fm_ipc_export: %p is not inside a local fm_alloc allocation", dev);
        return -1;
    }
    cudaIpcMemHandle_t h;
    cudaError_t err = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(it->first));
    if (err != cudaSuccess) { cuda_fail("fm_ipc_export", err); return -1; }
    static_assert(sizeof(h) == 64, "IPC handle size");
    memcpy(out_handle64, &h, 64);
    *out_offset = a - it->first;
    *out_size = it->second;
    return 0;
}

void* fm_ipc_import(const void* handle64, unsigned long long size) {
    LOCK;
    NEED_INIT(nullptr);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void* p = nullptr;
    cudaError_t err = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (err != cudaSuccess) { cuda_fail("fm_ipc_import", err); return nullptr; }
    E().allocs[reinterpret_cast<uintptr_t>(p)] = (size_t)size;
    E().imported[reinterpret_cast<uintptr_t>(p)] = (size_t)size;
    return p;
}

int fm_stream_peers(void* dev_deltas, const uint64_t* peer_bases, int npeers, const void* local_base,
                    unsigned long long span) {
    LOCK;
    NEED_INIT(-1);
    Engine& e = E();
    if (npeers < 1 || npeers > 8) { set_errorf("fm_stream_peers: npeers must be 1..8"); return -1; }
    if (!range_ok(dev_deltas, (size_t)npeers * 8) || !range_ok(local_base, span)) {
        set_errorf("fm_stream_peers: the offset array or the local window is outside its allocation");
        return FM_EREJECT;
    }
    long long delta[8];
    std::vector<uintptr_t> deps;
    add_dep(deps, reinterpret_cast<uintptr_t>(dev_deltas));
    add_dep(deps, reinterpret_cast<uintptr_t>(local_base));
    for (int q = 0; q < npeers; q++) {
        const uintptr_t pb = static_cast<uintptr_t>(peer_bases[q]);
        add_dep(deps, pb);
        bool ok = false;                             // a peer GPU's imported allocation, or a pinned host buffer
        for (const auto* m : {&e.imported, &e.pinned}) {
            auto it = m->upper_bound(pb);
            if (it == m->begin()) continue;
            --it;
            ok = ok || (pb >= it->first && pb + span <= it->first + it->second);
        }
        if (!ok) {
            set_errorf("fm_stream_peers: window %d (%llu bytes at %p) is neither inside an imported allocation nor "
                       "inside an fm_host_alloc buffer", q, span, reinterpret_cast<void*>(pb));
            return FM_EREJECT;
        }
        delta[q] = (long long)pb - (long long)reinterpret_cast<uintptr_t>(local_base);
    }
    if (copy_sync(dev_deltas, delta, (size_t)npeers * 8, cudaMemcpyHostToDevice, "fm_stream_peers") != 0) return -1;
    touch(dev_deltas, (size_t)npeers * 8);
    const uintptr_t lo = reinterpret_cast<uintptr_t>(local_base);
    e.peers[reinterpret_cast<uintptr_t>(dev_deltas)] = Engine::Peers{npeers, lo, lo + (uintptr_t)span, deps};
    return 0;
}

int fm_gemm_status(void) {
    LOCK;
    NEED_INIT(-1);
    return gemm_read_status(E().stream);
}

int fm_stream_status(void) {
    LOCK;
    NEED_INIT(-1);
    return stream_read_status(E().stream);
}

int fm_event_create(void) {
    LOCK;
    NEED_INIT(-1);
    cudaEvent_t ev;
    if (cudaEventCreate(&ev) != cudaSuccess) { cudaGetLastError(); return -1; }
    E().events.push_back(ev);
    return (int)E().events.size() - 1;
}
int fm_event_record(int ev) {
    LOCK;
    if (ev < 0 || ev >= (int)E().events.size()) return -1;
    return cudaEventRecord(E().events[ev], E().stream) == cudaSuccess ? 0 : -1;
}
float fm_event_elapsed_ms(int a, int b) {
    LOCK;
    Engine& e = E();
    if (a < 0 || b < 0 || a >= (int)e.events.size() || b >= (int)e.events.size()) return -1.f;
    if (cudaEventSynchronize(e.events[b]) != cudaSuccess) return -1.f;
    float ms = -1.f;
    if (cudaEventElapsedTime(&ms, e.events[a], e.events[b]) != cudaSuccess) { cudaGetLastError(); return -1.f; }
    return ms;
}

int fm_graph_begin(void) {
    LOCK;
    NEED_INIT(-1);
    Engine& e = E();
    if (e.capturing) { set_errorf("fm_graph_begin: a capture is already open"); return -1; }
    cudaError_t err = cudaStreamBeginCapture(e.stream, cudaStreamCaptureModeThreadLocal);
    if (err != cudaSuccess) { cuda_fail("fm_graph_begin", err); return -1; }
    e.capturing = true;
    e.launches_at_capture = e.launches;
    return 0;
}
int fm_graph_end(void) {
    LOCK;
    Engine& e = E();
    if (!e.capturing) { set_errorf("fm_graph_end: no capture is open"); return -1; }
    e.capturing = false;
    Graph g;
    g.kernels = e.launches - e.launches_at_capture;   // recorded, not executed yet
    e.launches = e.launches_at_capture;
    cudaError_t err = cudaStreamEndCapture(e.stream, &g.graph);
    if (err != cudaSuccess || !g.graph) { cuda_fail("fm_graph_end", err); cudaGetLastError(); return -1; }
    err = cudaGraphInstantiate(&g.exec, g.graph, 0);
    if (err != cudaSuccess) { cudaGraphDestroy(g.graph); cuda_fail("cudaGraphInstantiate", err); return -1; }
    for (size_t i = 0; i < e.graphs.size(); i++)
        if (!e.graphs[i].exec) { e.graphs[i] = g; return (int)i; }
    e.graphs.push_back(g);
    return (int)e.graphs.size() - 1;
}
int fm_graph_launch(int id) {
    LOCK;
    Engine& e = E();
    if (id < 0 || id >= (int)e.graphs.size() || !e.graphs[id].exec) { set_errorf("bad graph id %d", id); return -1; }
    cudaError_t err = cudaGraphLaunch(e.graphs[id].exec, e.stream);
    if (err != cudaSuccess) { cuda_fail("fm_graph_launch", err); return -1; }
    e.launches += e.graphs[id].kernels;
    return 0;
}
int fm_graph_free(int id) {
    LOCK;
    Engine& e = E();
    if (id < 0 || id >= (int)e.graphs.size() || !e.graphs[id].exec) return -1;
    cudaStreamSynchronize(e.stream);
    cudaGraphExecDestroy(e.graphs[id].exec);
    cudaGraphDestroy(e.graphs[id].graph);
    e.graphs[id] = Graph();
    bool graphs_alive = false;
    for (const Graph& g : e.graphs) graphs_alive = graphs_alive || g.exec != nullptr;
    if (!graphs_alive) {                       // no graph can point into an outgrown workspace any more
        for (void* q : e.retired_scratch) cudaFree(q);
        e.retired_scratch.clear();
    }
    return 0;
}

int fm_comm_unique_id(void* out128) {
    LOCK;
    auto f = (nccl_get_uid_t)nccl_sym("ncclGetUniqueId");
    if (!f) return -1;
    NcclUniqueId id;
    const int rc = f(&id);
    if (rc != 0) { set_errorf("ncclGetUniqueId failed (%d)", rc); return -1; }
    memcpy(out128, &id, 128);
    return 0;
}
int fm_comm_init(const void* id128, int nranks, int rank) {
    LOCK;
    NEED_INIT(-1);
    Engine& e = E();
    if (e.comm) { set_errorf("communicator already initialised"); return -1; }
    auto f = (nccl_init_rank_t)nccl_sym("ncclCommInitRank");
    if (!f) return -1;
    NcclUniqueId id;
    memcpy(&id, id128, 128);
    const int rc = f(&e.comm, nranks, id, rank);
    if (rc != 0) {
        auto es = (nccl_errstr_t)nccl_sym("ncclGetErrorString");
        set_errorf("ncclCommInitRank failed: %s", es ? es(rc) : "?");
        e.comm = nullptr;
        return -1;
    }
    e.comm_rank = rank;
    e.comm_size = nranks;
    return 0;
}
int fm_comm_rank(void) { return E().comm_rank; }
int fm_comm_size(void) { return E().comm_size; }
int fm_allgather(void* recv, const void* send, size_t bytes) {
    LOCK;
    Engine& e = E();
    if (!e.comm) { set_errorf("fm_allgather: no communicator"); return -1; }
    if (!range_ok(recv, bytes * e.comm_size) || !range_ok(send, bytes)) {
        set_errorf("fm_allgather: range exceeds an allocation");
        return -1;
    }
    auto f = (nccl_allgather_t)nccl_sym("ncclAllGather");
    if (!f) return -1;
    const int rc = f(send, recv, bytes, /*ncclInt8*/ 0, e.comm, e.stream);
    if (rc != 0) {
        auto es = (nccl_errstr_t)nccl_sym("ncclGetErrorString");
        set_errorf("ncclAllGather failed: %s", es ? es(rc) : "?");
        return -1;
    }
    return 0;
}
int fm_comm_destroy(void) {
    LOCK;
    Engine& e = E();
    if (!e.comm) return 0;
    cudaStreamSynchronize(e.stream);
    // captured graphs may hold collectives of this communicator; NCCL waits for them to be
    // released before it lets the communicator go, so every graph is destroyed first
    for (size_t i = 0; i < e.graphs.size(); i++)
        if (e.graphs[i].exec) {
            cudaGraphExecDestroy(e.graphs[i].exec);
            cudaGraphDestroy(e.graphs[i].graph);
            e.graphs[i] = Graph();
        }
    e.plan_graphs.clear();
    auto f = (nccl_destroy_t)nccl_sym("ncclCommDestroy");
    if (f) f(e.comm);
    e.comm = nullptr;
    e.comm_size = 1;
    e.comm_rank = 0;
    return 0;
}

}  // extern "C"
