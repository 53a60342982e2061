// Shared host/device helpers of the sm_100a kernel library.
#pragma once
#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>
#include <stdint.h>
#include <atomic>
#include <string>

#include "ctorch_b200.h"

namespace ctk {

// Thread-local message of the last failure; returns `code` so launchers can `return fail(...)`.
ctk_status fail(ctk_status code, const std::string& msg);
extern std::atomic<uint64_t> g_launches;
inline void count_launch(int n = 1) { g_launches.fetch_add(static_cast<uint64_t>(n), std::memory_order_relaxed); }

// Number of SMs of the current device (cached per device ordinal).
int sm_count();
// Library-owned per-device scratch, grown on demand (never shrinks).  slot 0: reductions,
// slot 1: matmul workspace.
ctk_status device_scratch(int slot, size_t bytes, void** out);

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

// NVTX range around the host side of an entry point (header-only NVTX: a no-op costing a few
// nanoseconds unless a profiler has injected itself), so a timeline shows which C-ABI call issued
// which kernels.
struct Range {
    explicit Range(const char* name) { nvtxRangePushA(name); }
    ~Range() { nvtxRangePop(); }
    Range(const Range&) = delete;
    Range& operator=(const Range&) = delete;
};

// One-time set-up that belongs to a (kernel, device) pair -- cudaFuncSetAttribute, occupancy queries --
// is guarded by one of these per kernel instantiation: first() is true once per device ordinal, for
// the device that is current at the call (a process may drive several GPUs through ctk_set_device).
struct PerDeviceOnce {
    bool done[64] = {false};
    bool first() {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return true;  // unknown device: redo the set-up, it is idempotent
        if (done[dev]) return false;
        done[dev] = true;
        return true;
    }
};

}  // namespace ctk

// (A failed call also leaves its code as the thread's "last error"; it is taken back here, or the
// next kernel launch check -- which reads that state -- would report this failure as its own.)
#define CTK_CUDA(call)                                                                          \
    do {                                                                                        \
        cudaError_t _e = (call);                                                                \
        if (_e != cudaSuccess) {                                                                \
            (void)cudaGetLastError();                                                           \
            return ctk::fail(CTK_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(_e)); \
        }                                                                                       \
    } while (0)

#define CTK_LAUNCH_CHECK(name)                                                                    \
    do {                                                                                          \
        cudaError_t _e = cudaGetLastError();                                                      \
        if (_e != cudaSuccess)                                                                    \
            return ctk::fail(CTK_ERR_CUDA, std::string(name) + " launch: " + cudaGetErrorString(_e)); \
        ctk::count_launch();                                                                      \
    } while (0)

#define CTK_RANGE(name) ctk::Range _ctk_nvtx_range(name)

#define CTK_REQUIRE(cond, msg)                                    \
    do {                                                          \
        if (!(cond)) return ctk::fail(CTK_ERR_INVALID, (msg));    \
    } while (0)

// Grid size for a grid-stride streaming kernel: a whole number of waves of the SM count.
static inline int ctk_stream_grid(int64_t work_items, int threads, int ctas_per_sm) {
    int64_t need = (work_items + threads - 1) / threads;
    int64_t cap = static_cast<int64_t>(ctk::sm_count()) * ctas_per_sm;
    if (need < 1) need = 1;
    return static_cast<int>(need < cap ? need : cap);
}
