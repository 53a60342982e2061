// Device, memory, stream and event entry points of the C ABI, plus the NCCL communicator.
//
// Replaces the host-only allocation of the reference's Storage (include/Storage.h:77, 88-93,
// 175-181: `new char[]` + memcpy) with a stream-ordered device pool and pinned host staging.
#include <dlfcn.h>
#include <nccl.h>

#include <mutex>
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

// ---- NCCL: loaded at first use so the library itself has no link-time NCCL dependency ----
namespace {
struct Nccl {
    void* h = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};
Nccl g_nccl;

ctk_status load_nccl() {
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_nccl.h) return CTK_OK;
    // An already loaded libnccl (e.g. the one a host framework brought) is reused by soname.
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
        g_nccl.h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (g_nccl.h) break;
    }
    if (!g_nccl.h) return fail(CTK_ERR_NCCL, std::string("dlopen libnccl.so.2: ") + dlerror());
#define CTK_SYM(field, name)                                                         \
    g_nccl.field = reinterpret_cast<decltype(g_nccl.field)>(dlsym(g_nccl.h, name)); \
    if (!g_nccl.field) return fail(CTK_ERR_NCCL, std::string("dlsym ") + name)
    CTK_SYM(GetUniqueId, "ncclGetUniqueId");
    CTK_SYM(CommInitRank, "ncclCommInitRank");
    CTK_SYM(CommDestroy, "ncclCommDestroy");
    CTK_SYM(AllReduce, "ncclAllReduce");
    CTK_SYM(GetErrorString, "ncclGetErrorString");
#undef CTK_SYM
    return CTK_OK;
}
}  // namespace

#define CTK_NCCL(call)                                                                                   \
    do {                                                                                                 \
        ncclResult_t _r = (call);                                                                        \
        if (_r != ncclSuccess) return fail(CTK_ERR_NCCL, std::string(#call) + ": " + g_nccl.GetErrorString(_r)); \
    } while (0)

ctk_status ctk_comm_unique_id(void* id_out) {
    CTK_REQUIRE(id_out, "ctk_comm_unique_id: null");
    static_assert(sizeof(ncclUniqueId) == CTK_COMM_ID_BYTES, "ncclUniqueId size");
    ctk_status st = load_nccl();
    if (st) return st;
    CTK_NCCL(g_nccl.GetUniqueId(reinterpret_cast<ncclUniqueId*>(id_out)));
    return CTK_OK;
}
ctk_status ctk_comm_init_rank(void** comm, const void* id, int world, int rank) {
    CTK_REQUIRE(comm && id && world > 0 && rank >= 0 && rank < world, "ctk_comm_init_rank: bad arguments");
    ctk_status st = load_nccl();
    if (st) return st;
    ncclUniqueId uid;
    memcpy(&uid, id, sizeof(uid));
    ncclComm_t c;
    CTK_NCCL(g_nccl.CommInitRank(&c, world, uid, rank));
    *comm = c;
    return CTK_OK;
}
ctk_status ctk_comm_destroy(void* comm) {
    if (!comm) return CTK_OK;
    CTK_NCCL(g_nccl.CommDestroy(reinterpret_cast<ncclComm_t>(comm)));
    return CTK_OK;
}
ctk_status ctk_allreduce_sum_f32(void* comm, float* buf, int64_t n, void* stream) {
    CTK_REQUIRE(comm && buf && n >= 0, "ctk_allreduce_sum_f32: bad arguments");
    if (n == 0) return CTK_OK;
    CTK_NCCL(g_nccl.AllReduce(buf, buf, static_cast<size_t>(n), ncclFloat, ncclSum,
                              reinterpret_cast<ncclComm_t>(comm), as_stream(stream)));
    return CTK_OK;
}

}  // extern "C"
