// Device, memory, stream and event entry points of the C ABI, plus the NCCL communicator.
//
// Replaces the host-only allocation of the reference's Storage (include/Storage.h:77, 88-93,
// 175-181: `new char[]` + memcpy) with a stream-ordered device pool and pinned host staging.
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <cstring>
#include <mutex>
#include <thread>
#include <vector>

#include "common.cuh"

namespace ctk {

static thread_local std::string t_last_error;
std::atomic<uint64_t> g_launches{0};

ctk_status fail(ctk_status code, const std::string& msg) {
    t_last_error = msg;
    return code;
}

static std::mutex g_mu;
static int g_sm_count[64] = {0};
static bool g_pool_ready[64] = {false};

int sm_count() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (g_sm_count[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        g_sm_count[dev] = n;
    }
    return g_sm_count[dev];
}

struct Scratch {
    void* p = nullptr;
    size_t bytes = 0;
};
static Scratch g_scratch[64][2];

ctk_status device_scratch(int slot, size_t bytes, void** out) {
    int dev = 0;
    CTK_CUDA(cudaGetDevice(&dev));
    CTK_REQUIRE(dev >= 0 && dev < 64 && slot >= 0 && slot < 2, "device_scratch: bad device or slot");
    std::lock_guard<std::mutex> lock(g_mu);
    Scratch& s = g_scratch[dev][slot];
    if (s.bytes < bytes) {
        if (s.p) {
            CTK_CUDA(cudaDeviceSynchronize());  // earlier kernels may still use the old block
            CTK_CUDA(cudaFree(s.p));
            s.p = nullptr;
            s.bytes = 0;
        }
        size_t want = bytes < (1u << 20) ? (1u << 20) : bytes;
        CTK_CUDA(cudaMalloc(&s.p, want));
        CTK_CUDA(cudaMemset(s.p, 0, want));
        s.bytes = want;
    }
    *out = s.p;
    return CTK_OK;
}

// The default memory pool keeps freed blocks instead of returning them to the driver, so the
// per-op allocate/free pattern of value-semantic tensors costs no cudaMalloc after warm-up.
static ctk_status ensure_pool() {
    int dev = 0;
    CTK_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(CTK_ERR_INVALID, "device ordinal out of range");
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_pool_ready[dev]) {
        cudaMemPool_t pool;
        CTK_CUDA(cudaDeviceGetDefaultMemPool(&pool, dev));
        uint64_t threshold = UINT64_MAX;
        CTK_CUDA(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &threshold));
        g_pool_ready[dev] = true;
    }
    return CTK_OK;
}

}  // namespace ctk

using namespace ctk;

extern "C" {

const char* ctk_last_error(void) { return t_last_error.c_str(); }
int ctk_version(void) { return 100; }
uint64_t ctk_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

ctk_status ctk_device_count(int* count) {
    CTK_REQUIRE(count, "ctk_device_count: null");
    CTK_CUDA(cudaGetDeviceCount(count));
    return CTK_OK;
}
ctk_status ctk_set_device(int ordinal) {
    CTK_CUDA(cudaSetDevice(ordinal));
    return CTK_OK;
}
ctk_status ctk_get_device(int* ordinal) {
    CTK_REQUIRE(ordinal, "ctk_get_device: null");
    CTK_CUDA(cudaGetDevice(ordinal));
    return CTK_OK;
}
ctk_status ctk_device_sync(void) {
    CTK_CUDA(cudaDeviceSynchronize());
    return CTK_OK;
}
ctk_status ctk_device_info(int* sms, size_t* total_bytes, size_t* free_bytes) {
    size_t f = 0, t = 0;
    CTK_CUDA(cudaMemGetInfo(&f, &t));
    if (sms) *sms = sm_count();
    if (total_bytes) *total_bytes = t;
    if (free_bytes) *free_bytes = f;
    return CTK_OK;
}

ctk_status ctk_malloc(void** p, size_t bytes) {
    CTK_REQUIRE(p, "ctk_malloc: null out pointer");
    *p = nullptr;
    if (bytes == 0) return CTK_OK;
    ctk_status st = ensure_pool();
    if (st) return st;
    // Ordered on the legacy default stream: it synchronises with every blocking stream, so a
    // block freed here is never handed out while a kernel on another blocking stream still uses it.
    CTK_CUDA(cudaMallocAsync(p, bytes, static_cast<cudaStream_t>(0)));
    return CTK_OK;
}
ctk_status ctk_free(void* p) {
    if (!p) return CTK_OK;
    CTK_CUDA(cudaFreeAsync(p, static_cast<cudaStream_t>(0)));
    return CTK_OK;
}
// Grows the pool to at least `bytes` of backing memory now (one allocation, freed at once; the pool
// keeps what it maps), so the first steps of a loop do not stop for the driver to map memory piece
// by piece.  Synchronises the device.
ctk_status ctk_pool_reserve(size_t bytes) {
    if (bytes == 0) return CTK_OK;
    ctk_status st = ensure_pool();
    if (st) return st;
    int dev = 0;
    CTK_CUDA(cudaGetDevice(&dev));
    cudaMemPool_t pool;
    CTK_CUDA(cudaDeviceGetDefaultMemPool(&pool, dev));
    uint64_t have = 0;
    CTK_CUDA(cudaMemPoolGetAttribute(pool, cudaMemPoolAttrReservedMemCurrent, &have));
    if (have >= bytes) return CTK_OK;
    void* p = nullptr;
    CTK_CUDA(cudaMallocAsync(&p, bytes - have, static_cast<cudaStream_t>(0)));
    CTK_CUDA(cudaFreeAsync(p, static_cast<cudaStream_t>(0)));
    CTK_CUDA(cudaDeviceSynchronize());
    return CTK_OK;
}
// Long-lived buffers (caches that a caller manages itself): plain cudaMalloc / cudaFree, outside the
// stream-ordered pool, so they neither fragment it nor pin its high-water mark.  Both synchronise.
ctk_status ctk_malloc_longlived(void** p, size_t bytes) {
    CTK_REQUIRE(p, "ctk_malloc_longlived: null out pointer");
    *p = nullptr;
    if (bytes == 0) return CTK_OK;
    CTK_CUDA(cudaMalloc(p, bytes));
    return CTK_OK;
}
ctk_status ctk_free_longlived(void* p) {
    if (!p) return CTK_OK;
    CTK_CUDA(cudaFree(p));
    return CTK_OK;
}
ctk_status ctk_malloc_host(void** p, size_t bytes) {
    CTK_REQUIRE(p, "ctk_malloc_host: null out pointer");
    *p = nullptr;
    if (bytes == 0) return CTK_OK;
    CTK_CUDA(cudaMallocHost(p, bytes));
    return CTK_OK;
}
ctk_status ctk_free_host(void* p) {
    if (!p) return CTK_OK;
    CTK_CUDA(cudaFreeHost(p));
    return CTK_OK;
}
ctk_status ctk_host_is_pinned(const void* p, int* is_pinned) {
    CTK_REQUIRE(p && is_pinned, "ctk_host_is_pinned: null");
    cudaPointerAttributes attr;
    cudaError_t e = cudaPointerGetAttributes(&attr, p);
    if (e != cudaSuccess) {
        cudaGetLastError();  // plain pageable memory on old drivers: not an error for the caller
        *is_pinned = 0;
        return CTK_OK;
    }
    *is_pinned = (attr.type == cudaMemoryTypeHost) ? 1 : 0;
    return CTK_OK;
}
ctk_status ctk_memcpy_h2d(void* dst, const void* src, size_t bytes, void* stream) {
    if (bytes == 0) return CTK_OK;
    CTK_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, as_stream(stream)));
    return CTK_OK;
}
ctk_status ctk_memcpy_d2h(void* dst, const void* src, size_t bytes, void* stream) {
    if (bytes == 0) return CTK_OK;
    CTK_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, as_stream(stream)));
    return CTK_OK;
}
ctk_status ctk_memcpy_d2d(void* dst, const void* src, size_t bytes, void* stream) {
    if (bytes == 0) return CTK_OK;
    CTK_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, as_stream(stream)));
    return CTK_OK;
}
ctk_status ctk_memset(void* p, int v, size_t bytes, void* stream) {
    if (bytes == 0) return CTK_OK;
    CTK_CUDA(cudaMemsetAsync(p, v, bytes, as_stream(stream)));
    return CTK_OK;
}

ctk_status ctk_stream_create(void** s) {
    CTK_REQUIRE(s, "ctk_stream_create: null");
    cudaStream_t st;
    CTK_CUDA(cudaStreamCreate(&st));  // blocking stream: ordered against the legacy default stream
    *s = st;
    return CTK_OK;
}
ctk_status ctk_stream_create_ex(void** s, int non_blocking) {
    CTK_REQUIRE(s, "ctk_stream_create_ex: null");
    cudaStream_t st;
    CTK_CUDA(cudaStreamCreateWithFlags(&st, non_blocking ? cudaStreamNonBlocking : cudaStreamDefault));
    *s = st;
    return CTK_OK;
}
ctk_status ctk_stream_create_priority(void** s, int non_blocking, int high_priority) {
    CTK_REQUIRE(s, "ctk_stream_create_priority: null");
    int least = 0, greatest = 0;
    CTK_CUDA(cudaDeviceGetStreamPriorityRange(&least, &greatest));
    cudaStream_t st;
    CTK_CUDA(cudaStreamCreateWithPriority(&st, non_blocking ? cudaStreamNonBlocking : cudaStreamDefault, high_priority ? greatest : least));
    *s = st;
    return CTK_OK;
}
ctk_status ctk_stream_destroy(void* s) {
    if (s) CTK_CUDA(cudaStreamDestroy(as_stream(s)));
    return CTK_OK;
}
ctk_status ctk_stream_sync(void* s) {
    CTK_CUDA(cudaStreamSynchronize(as_stream(s)));
    return CTK_OK;
}
// ---- stream capture into an executable graph ----
// begin: starts capturing the work issued to `stream` (not the legacy default stream) by this thread.
// end: ends the capture and instantiates the graph; *graph_exec is NULL and an error is returned if
// the capture was invalidated.  launch / destroy: the executable graph.
ctk_status ctk_stream_begin_capture(void* stream) {
    CTK_REQUIRE(stream, "ctk_stream_begin_capture: a stream of its own is needed (the default stream cannot be captured)");
    CTK_CUDA(cudaStreamBeginCapture(static_cast<cudaStream_t>(stream), cudaStreamCaptureModeThreadLocal));
    return CTK_OK;
}
ctk_status ctk_stream_end_capture(void* stream, void** graph_exec) {
    CTK_REQUIRE(stream && graph_exec, "ctk_stream_end_capture: null");
    *graph_exec = nullptr;
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(static_cast<cudaStream_t>(stream), &graph);
    if (e != cudaSuccess || !graph) {
        cudaGetLastError();
        return fail(CTK_ERR_CUDA, std::string("stream capture failed: ") + cudaGetErrorString(e));
    }
    cudaGraphExec_t exec = nullptr;
    e = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(CTK_ERR_CUDA, std::string("graph instantiation failed: ") + cudaGetErrorString(e));
    }
    *graph_exec = exec;
    return CTK_OK;
}
ctk_status ctk_graph_launch(void* graph_exec, void* stream, int kernels_in_graph) {
    CTK_REQUIRE(graph_exec && stream, "ctk_graph_launch: null");
    CTK_CUDA(cudaGraphLaunch(static_cast<cudaGraphExec_t>(graph_exec), static_cast<cudaStream_t>(stream)));
    if (kernels_in_graph > 0) g_launches.fetch_add(static_cast<uint64_t>(kernels_in_graph), std::memory_order_relaxed);
    return CTK_OK;
}
ctk_status ctk_graph_destroy(void* graph_exec) {
    if (graph_exec) CTK_CUDA(cudaGraphExecDestroy(static_cast<cudaGraphExec_t>(graph_exec)));
    return CTK_OK;
}

ctk_status ctk_event_create(void** e) {
    CTK_REQUIRE(e, "ctk_event_create: null");
    cudaEvent_t ev;
    CTK_CUDA(cudaEventCreate(&ev));
    *e = ev;
    return CTK_OK;
}
ctk_status ctk_event_destroy(void* e) {
    if (e) CTK_CUDA(cudaEventDestroy(reinterpret_cast<cudaEvent_t>(e)));
    return CTK_OK;
}
ctk_status ctk_event_record(void* e, void* s) {
    CTK_CUDA(cudaEventRecord(reinterpret_cast<cudaEvent_t>(e), as_stream(s)));
    return CTK_OK;
}
ctk_status ctk_event_sync(void* e) {
    CTK_CUDA(cudaEventSynchronize(reinterpret_cast<cudaEvent_t>(e)));
    return CTK_OK;
}
ctk_status ctk_event_elapsed_ms(void* e0, void* e1, float* ms) {
    CTK_REQUIRE(ms, "ctk_event_elapsed_ms: null");
    CTK_CUDA(cudaEventElapsedTime(ms, reinterpret_cast<cudaEvent_t>(e0), reinterpret_cast<cudaEvent_t>(e1)));
    return CTK_OK;
}
ctk_status ctk_stream_wait_event(void* s, void* e) {
    CTK_CUDA(cudaStreamWaitEvent(as_stream(s), reinterpret_cast<cudaEvent_t>(e), 0));
    return CTK_OK;
}

}  // extern "C"

// ---- bounded host-side wait -----------------------------------------------------------------------
// The loop every blocking wait of the data-parallel path runs instead of an unbounded stream
// synchronisation: poll "is the work done", poll "is the communicator healthy", give up at a deadline.
// The three callbacks make the same loop testable without a GPU (ranks over gloo where one never
// contributes): query returns 1 when done, 0 when pending, < 0 on an error of its own; health returns
// 0 while fine; abort is called once before an error is returned.
extern "C" ctk_status ctk_watchdog_wait(ctk_watch_fn query, ctk_watch_fn health, ctk_watch_fn abort_fn, void* user, int timeout_ms, int poll_us) {
    CTK_REQUIRE(query && timeout_ms >= 0, "ctk_watchdog_wait: a query callback and a non-negative timeout are needed");
    const auto t0 = std::chrono::steady_clock::now();
    const auto limit = std::chrono::milliseconds(timeout_ms);
    const auto nap = std::chrono::microseconds(poll_us > 0 ? poll_us : 50);
    const auto spin_for = std::chrono::milliseconds(20);  // a step normally ends within this: poll hot, like a plain synchronisation
    auto last_check = t0;
    for (;;) {
        const int q = query(user);
        if (q > 0) return CTK_OK;
        const auto now = std::chrono::steady_clock::now();
        std::string why;
        if (q < 0) {
            why = "the awaited work reported an error (" + std::to_string(q) + ")";
        } else if (now - last_check >= std::chrono::microseconds(500) || now - t0 > limit) {
            // health and deadline twice a millisecond: the health call may take a lock inside the library
            last_check = now;
            if (health) {
                const int h = health(user);
                if (h != 0) why = "the communicator reported an asynchronous error (" + std::to_string(h) + ")";
            }
            if (why.empty() && now - t0 > limit) why = "no completion within " + std::to_string(timeout_ms) + " ms: a peer did not take part";
        }
        if (!why.empty()) {
            if (abort_fn) abort_fn(user);
            return fail(CTK_ERR_NCCL, "data-parallel wait gave up: " + why);
        }
        if (now - t0 < spin_for) std::this_thread::yield();
        else std::this_thread::sleep_for(nap);
    }
}

// ---- NCCL: loaded at first use so the library itself has no link-time NCCL dependency ----
namespace {
struct Nccl {
    void* h = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*ReduceScatter)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*MemAlloc)(void**, size_t) = nullptr;
    ncclResult_t (*MemFree)(void*) = nullptr;
    ncclResult_t (*CommRegister)(const ncclComm_t, void*, size_t, void**) = nullptr;
    ncclResult_t (*CommDeregister)(const ncclComm_t, void*) = nullptr;
    ncclResult_t (*CommWindowRegister)(ncclComm_t, void*, size_t, ncclWindow_t*, int) = nullptr;  // optional (NCCL >= 2.27)
    ncclResult_t (*CommWindowDeregister)(ncclComm_t, ncclWindow_t) = nullptr;
    ncclResult_t (*GetVersion)(int*) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};
Nccl g_nccl;

ctk_status load_nccl() {
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_nccl.h) return CTK_OK;
    // An already loaded libnccl (e.g. the one a host framework brought) is reused by soname.
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    void* h = nullptr;
    for (const char* n : names) {
        h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (h) break;
    }
    if (!h) return fail(CTK_ERR_NCCL, std::string("dlopen libnccl.so.2: ") + dlerror());
#define CTK_SYM(field, name)                                                  \
    g_nccl.field = reinterpret_cast<decltype(g_nccl.field)>(dlsym(h, name)); \
    if (!g_nccl.field) return fail(CTK_ERR_NCCL, std::string("dlsym ") + name)
#define CTK_SYM_OPT(field, name) g_nccl.field = reinterpret_cast<decltype(g_nccl.field)>(dlsym(h, name))
    CTK_SYM(GetUniqueId, "ncclGetUniqueId");
    CTK_SYM(CommInitRank, "ncclCommInitRank");
    CTK_SYM(CommInitRankConfig, "ncclCommInitRankConfig");
    CTK_SYM(CommDestroy, "ncclCommDestroy");
    CTK_SYM(CommAbort, "ncclCommAbort");
    CTK_SYM(CommGetAsyncError, "ncclCommGetAsyncError");
    CTK_SYM(AllReduce, "ncclAllReduce");
    CTK_SYM(ReduceScatter, "ncclReduceScatter");
    CTK_SYM(AllGather, "ncclAllGather");
    CTK_SYM(GetErrorString, "ncclGetErrorString");
    CTK_SYM_OPT(MemAlloc, "ncclMemAlloc");
    CTK_SYM_OPT(MemFree, "ncclMemFree");
    CTK_SYM_OPT(CommRegister, "ncclCommRegister");
    CTK_SYM_OPT(CommDeregister, "ncclCommDeregister");
    CTK_SYM_OPT(CommWindowRegister, "ncclCommWindowRegister");
    CTK_SYM_OPT(CommWindowDeregister, "ncclCommWindowDeregister");
    CTK_SYM_OPT(GetVersion, "ncclGetVersion");
#undef CTK_SYM
#undef CTK_SYM_OPT
    g_nccl.h = h;
    return CTK_OK;
}

// What a `void* comm` of the C ABI points to.
struct Comm {
    ncclComm_t c = nullptr;
    int world = 1, rank = 0;
    bool aborted = false;
    struct Buffer {
        void* p = nullptr;
        size_t bytes = 0;
        void* handle = nullptr;       // ncclCommRegister
        ncclWindow_t win = nullptr;   // ncclCommWindowRegister
    };
    std::vector<Buffer> buffers;
};
Comm* as_comm(void* h) { return static_cast<Comm*>(h); }
}  // namespace

#define CTK_NCCL(call)                                                                                   \
    do {                                                                                                 \
        ncclResult_t _r = (call);                                                                        \
        if (_r != ncclSuccess) return fail(CTK_ERR_NCCL, std::string(#call) + ": " + g_nccl.GetErrorString(_r)); \
    } while (0)

extern "C" {

ctk_status ctk_comm_unique_id(void* id_out) {
    CTK_REQUIRE(id_out, "ctk_comm_unique_id: null");
    static_assert(sizeof(ncclUniqueId) == CTK_COMM_ID_BYTES, "ncclUniqueId size");
    ctk_status st = load_nccl();
    if (st) return st;
    CTK_NCCL(g_nccl.GetUniqueId(reinterpret_cast<ncclUniqueId*>(id_out)));
    return CTK_OK;
}
// max_ctas / nvls_ctas: upper bound on the CTAs one collective may occupy, and the CTAs of its
// in-switch (NVLS) part; 0 leaves NCCL's own choice.  The collectives share the SMs with the persistent
// MatMul kernels, so a communicator for gradient exchange under backward wants few of them.
ctk_status ctk_comm_init_rank_config(void** comm, const void* id, int world, int rank, int max_ctas, int nvls_ctas) {
    CTK_REQUIRE(comm && id && world > 0 && rank >= 0 && rank < world && max_ctas >= 0 && nvls_ctas >= 0, "ctk_comm_init_rank: bad arguments");
    ctk_status st = load_nccl();
    if (st) return st;
    ncclUniqueId uid;
    memcpy(&uid, id, sizeof(uid));
    ncclComm_t c;
    if (max_ctas == 0 && nvls_ctas == 0) {
        CTK_NCCL(g_nccl.CommInitRank(&c, world, uid, rank));
    } else {
        ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
        if (max_ctas > 0) cfg.maxCTAs = max_ctas;
        if (nvls_ctas > 0) cfg.nvlsCTAs = nvls_ctas;
        CTK_NCCL(g_nccl.CommInitRankConfig(&c, world, uid, rank, &cfg));
    }
    Comm* w = new Comm();
    w->c = c;
    w->world = world;
    w->rank = rank;
    *comm = w;
    return CTK_OK;
}
ctk_status ctk_comm_init_rank(void** comm, const void* id, int world, int rank) { return ctk_comm_init_rank_config(comm, id, world, rank, 0, 0); }

ctk_status ctk_comm_info(void* comm, int* world, int* rank, int* nccl_version) {
    CTK_REQUIRE(comm, "ctk_comm_info: null communicator");
    if (world) *world = as_comm(comm)->world;
    if (rank) *rank = as_comm(comm)->rank;
    if (nccl_version) {
        *nccl_version = 0;
        if (g_nccl.GetVersion) g_nccl.GetVersion(nccl_version);
    }
    return CTK_OK;
}

// Device memory the communicator knows: allocated by NCCL's allocator and registered with the
// communicator (symmetric != 0: as a symmetric window, every rank registering the same size in the same
// order -- a collective call), so that collectives on it can reduce in the switch straight out of
// user memory with a handful of CTAs instead of staging through NCCL's own buffers.  Falls back to
// unregistered memory where the loaded NCCL lacks the calls.  Collective: every rank calls it.
ctk_status ctk_comm_alloc(void* comm, size_t bytes, int symmetric, void** ptr) {
    CTK_REQUIRE(comm && ptr && bytes > 0, "ctk_comm_alloc: bad arguments");
    Comm* w = as_comm(comm);
    Comm::Buffer b;
    b.bytes = bytes;
    if (g_nccl.MemAlloc && g_nccl.MemFree) {
        CTK_NCCL(g_nccl.MemAlloc(&b.p, bytes));
        if (symmetric && g_nccl.CommWindowRegister && g_nccl.CommWindowDeregister) {
            CTK_NCCL(g_nccl.CommWindowRegister(w->c, b.p, bytes, &b.win, NCCL_WIN_COLL_SYMMETRIC));
        } else if (g_nccl.CommRegister && g_nccl.CommDeregister) {
            CTK_NCCL(g_nccl.CommRegister(w->c, b.p, bytes, &b.handle));
        }
    } else {
        CTK_CUDA(cudaMalloc(&b.p, bytes));
    }
    w->buffers.push_back(b);
    *ptr = b.p;
    return CTK_OK;
}
static ctk_status release_buffer(Comm* w, Comm::Buffer& b) {
    if (!w->aborted) {
        if (b.win) CTK_NCCL(g_nccl.CommWindowDeregister(w->c, b.win));
        if (b.handle) CTK_NCCL(g_nccl.CommDeregister(w->c, b.handle));
    }
    if (g_nccl.MemAlloc && g_nccl.MemFree) CTK_NCCL(g_nccl.MemFree(b.p));
    else CTK_CUDA(cudaFree(b.p));
    return CTK_OK;
}
ctk_status ctk_comm_free(void* comm, void* ptr) {
    CTK_REQUIRE(comm, "ctk_comm_free: null communicator");
    if (!ptr) return CTK_OK;
    Comm* w = as_comm(comm);
    for (size_t i = 0; i < w->buffers.size(); ++i)
        if (w->buffers[i].p == ptr) {
            Comm::Buffer b = w->buffers[i];
            w->buffers.erase(w->buffers.begin() + static_cast<long>(i));
            return release_buffer(w, b);
        }
    return fail(CTK_ERR_INVALID, "ctk_comm_free: not a buffer of this communicator");
}

// Stops the communicator where it stands (ncclCommAbort): its kernels in flight end, later calls on
// it fail.  What a rank does after ctk_comm_wait reported that a peer is gone.
ctk_status ctk_comm_abort(void* comm) {
    CTK_REQUIRE(comm, "ctk_comm_abort: null communicator");
    Comm* w = as_comm(comm);
    if (w->aborted) return CTK_OK;
    w->aborted = true;
    CTK_NCCL(g_nccl.CommAbort(w->c));
    return CTK_OK;
}
ctk_status ctk_comm_destroy(void* comm) {
    if (!comm) return CTK_OK;
    Comm* w = as_comm(comm);
    ctk_status rc = CTK_OK;
    for (auto& b : w->buffers) {
        ctk_status r = release_buffer(w, b);
        if (r && !rc) rc = r;
    }
    w->buffers.clear();
    if (!w->aborted) {
        ncclResult_t r = g_nccl.CommDestroy(w->c);
        if (r != ncclSuccess && !rc) rc = fail(CTK_ERR_NCCL, std::string("ncclCommDestroy: ") + g_nccl.GetErrorString(r));
    }
    delete w;
    return rc;
}

// Waits, on the host, until `event` (recorded behind the step's last collective or kernel) has
// completed -- but never longer than timeout_ms, and not past an asynchronous NCCL error: a peer that
// died or never joined leaves a collective spinning on the GPU for ever, and an unbounded stream
// synchronisation with it.  On giving up the communicator is aborted, which ends its kernels, and
// CTK_ERR_NCCL is returned; the CUDA context stays usable.
namespace {
struct CommWait {
    Comm* w;
    cudaEvent_t ev;
    int cuda_error;
};
int comm_wait_query(void* u) {
    CommWait* x = static_cast<CommWait*>(u);
    const cudaError_t e = cudaEventQuery(x->ev);
    if (e == cudaSuccess) return 1;
    if (e == cudaErrorNotReady) return 0;
    x->cuda_error = static_cast<int>(e);
    return -static_cast<int>(e);
}
int comm_wait_health(void* u) {
    CommWait* x = static_cast<CommWait*>(u);
    ncclResult_t async = ncclSuccess;
    const ncclResult_t r = g_nccl.CommGetAsyncError(x->w->c, &async);
    if (r != ncclSuccess) return static_cast<int>(r);
    return (async == ncclSuccess || async == ncclInProgress) ? 0 : static_cast<int>(async);
}
int comm_wait_abort(void* u) {
    CommWait* x = static_cast<CommWait*>(u);
    if (!x->w->aborted) {
        x->w->aborted = true;
        g_nccl.CommAbort(x->w->c);
    }
    return 0;
}
}  // namespace
ctk_status ctk_comm_wait(void* comm, void* event, int timeout_ms) {
    CTK_REQUIRE(comm && event, "ctk_comm_wait: null argument");
    Comm* w = as_comm(comm);
    if (w->aborted) return fail(CTK_ERR_NCCL, "ctk_comm_wait: the communicator was aborted");
    CommWait x{w, reinterpret_cast<cudaEvent_t>(event), 0};
    return ctk_watchdog_wait(comm_wait_query, comm_wait_health, comm_wait_abort, &x, timeout_ms, 50);
}

#define CTK_COMM_LIVE(name)                                                                   \
    Comm* w = as_comm(comm);                                                                  \
    if (w->aborted) return fail(CTK_ERR_NCCL, std::string(name) + ": the communicator was aborted")

ctk_status ctk_allreduce_sum_f32(void* comm, float* buf, int64_t n, void* stream) {
    CTK_RANGE("ctk_allreduce_sum_f32");
    CTK_REQUIRE(comm && buf && n >= 0, "ctk_allreduce_sum_f32: bad arguments");
    if (n == 0) return CTK_OK;
    CTK_COMM_LIVE("ctk_allreduce_sum_f32");
    CTK_NCCL(g_nccl.AllReduce(buf, buf, static_cast<size_t>(n), ncclFloat, ncclSum, w->c, as_stream(stream)));
    return CTK_OK;
}
// recv[0, count) of this rank = sum over ranks of send[rank * count, (rank + 1) * count); send holds
// world * count floats.  recv may point into send at rank * count (in place).
ctk_status ctk_reduce_scatter_sum_f32(void* comm, const float* send, float* recv, int64_t count, void* stream) {
    CTK_RANGE("ctk_reduce_scatter_sum_f32");
    CTK_REQUIRE(comm && send && recv && count >= 0, "ctk_reduce_scatter_sum_f32: bad arguments");
    if (count == 0) return CTK_OK;
    CTK_COMM_LIVE("ctk_reduce_scatter_sum_f32");
    CTK_NCCL(g_nccl.ReduceScatter(send, recv, static_cast<size_t>(count), ncclFloat, ncclSum, w->c, as_stream(stream)));
    return CTK_OK;
}
// recv[r * count, (r + 1) * count) = rank r's send[0, count) for every r; send may point into recv at
// rank * count (in place).
ctk_status ctk_allgather_f32(void* comm, const float* send, float* recv, int64_t count, void* stream) {
    CTK_RANGE("ctk_allgather_f32");
    CTK_REQUIRE(comm && send && recv && count >= 0, "ctk_allgather_f32: bad arguments");
    if (count == 0) return CTK_OK;
    CTK_COMM_LIVE("ctk_allgather_f32");
    CTK_NCCL(g_nccl.AllGather(send, recv, static_cast<size_t>(count), ncclFloat, w->c, as_stream(stream)));
    return CTK_OK;
}

}  // extern "C"
