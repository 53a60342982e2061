// Reductions to a scalar (Sum, Dot, MSE, MAE) and the elementwise backward of the two mean
// losses.  HBM-bound: 128-bit streaming loads, four independent fp32 accumulators per thread,
// shuffle reduction per warp, fp64 across warps and CTAs, one launch (the last CTA to finish adds
// the per-CTA partials in a fixed order).  Compiled with -fmad=false.
//
// The reference adds sequentially in fp32 (src/Tensor.cpp:638-666, MSE/MAE/Dot_BASIC_kernel.cpp);
// the tree used here is at least as accurate, which is how parity of these sums is judged.
#include <math.h>

#include <atomic>

#include "ew_skeleton.cuh"
#include "reduce_common.cuh"

namespace ctk {

static std::atomic<bool> g_library_scratch_dirty{false};
void mark_reduce_scratch_dirty() { g_library_scratch_dirty.store(true); }

ctk_status reduce_scratch(void* user, cudaStream_t st, ReduceScratch** out) {
    void* p = user;
    if (!p) {
        ctk_status s = device_scratch(0, sizeof(ReduceScratch), &p);
        if (s) return s;
    }
    CTK_REQUIRE((reinterpret_cast<uintptr_t>(p) & 7u) == 0, "reduction scratch must be 8-byte aligned");
    *out = static_cast<ReduceScratch*>(p);
    // The ticket must start at zero.  The library's own block is zeroed when it is allocated and every
    // kernel rewinds the ticket it used, so only a caller-supplied block (not trusted to be clean) or
    // a kernel that gave up on a bounded wait (reported through the status word) costs a memset.
    if (user || g_library_scratch_dirty.exchange(false)) CTK_CUDA(cudaMemsetAsync(&(*out)->ticket, 0, sizeof(unsigned int), st));
    return CTK_OK;
}

}  // namespace ctk

namespace {
using namespace ctk;

constexpr int kThreads = 256;
constexpr int kCtasPerSm = 4;

enum { R_SUM = 0, R_DOT = 1, R_MSE = 2, R_MAE = 3, R_MATCH = 4 };

template <int KIND>
__device__ __forceinline__ float term(float x, float y) {
    if (KIND == R_SUM) return x;
    if (KIND == R_DOT) return x * y;
    if (KIND == R_MATCH) return static_cast<int>(x) == static_cast<int>(y) ? 1.0f : 0.0f;
    float d = x - y;
    if (KIND == R_MSE) return d * d;
    return fabsf(d);
}

template <int KIND>
__global__ void __launch_bounds__(kThreads) reduce_kernel(const float* __restrict__ a, const float* __restrict__ b, int64_t n,
                                                          bool vec_ok, float post_div, ReduceScratch* scratch, float* out) {
    __shared__ double smem[33];
    const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
    float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
    if (vec_ok) {
        const int64_t n4 = n >> 2;
#pragma unroll 4
        for (int64_t i = tid; i < n4; i += nthreads) {
            float4 x = __ldcs(reinterpret_cast<const float4*>(a) + i);
            float4 y = (KIND == R_SUM) ? x : __ldcs(reinterpret_cast<const float4*>(b) + i);
            acc0 += term<KIND>(x.x, y.x);
            acc1 += term<KIND>(x.y, y.y);
            acc2 += term<KIND>(x.z, y.z);
            acc3 += term<KIND>(x.w, y.w);
        }
        for (int64_t j = (n4 << 2) + tid; j < n; j += nthreads) acc0 += term<KIND>(a[j], KIND == R_SUM ? 0.f : b[j]);
    } else {
        for (int64_t j = tid; j < n; j += nthreads) acc0 += term<KIND>(a[j], KIND == R_SUM ? 0.f : b[j]);
    }
    double v = (static_cast<double>(acc0) + static_cast<double>(acc1)) + (static_cast<double>(acc2) + static_cast<double>(acc3));
    v = block_sum(v, smem);
    grid_finish(v, scratch, out, post_div, false, smem);
}

// src/AutoDiff.cpp:1491-1516: (((p - t) * 2) / n) * g ;  :1602-1642: (sign(p - t) / n) * g
// x[0] = p, x[1] = t, x[2] = upstream scalar.
template <bool MSE>
struct MeanLossBwdF {
    float fn;
    bool use_g;
    __device__ __forceinline__ void operator()(const float* x, float* y) const {
        float d = x[0] - x[1];
        float c;
        if (MSE) {
            float d2 = d * 2.0f;
            c = d2 / fn;
        } else {
            float s = d > 0.0f ? 1.0f : (d < 0.0f ? -1.0f : 0.0f);
            c = s / fn;
        }
        y[0] = c * (use_g ? x[2] : 1.0f);
    }
};

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <int KIND>
ctk_status launch_reduce(const char* name, const float* a, const float* b, int64_t n, float post_div, float* out, void* scratch, void* stream) {
    CTK_REQUIRE(n >= 0 && out, "reduction: bad arguments");
    CTK_REQUIRE(n == 0 || (a && (KIND == R_SUM || b)), "reduction: null input");
    cudaStream_t st = as_stream(stream);
    ReduceScratch* s = nullptr;
    ctk_status rc = reduce_scratch(scratch, st, &s);
    if (rc) return rc;
    int grid = ctk_stream_grid((n + 3) / 4, kThreads * 4, kCtasPerSm);
    if (grid > kMaxReduceBlocks) grid = kMaxReduceBlocks;
    bool vec_ok = aligned16(a) && (KIND == R_SUM || aligned16(b));
    reduce_kernel<KIND><<<grid, kThreads, 0, st>>>(a, b, n, vec_ok, post_div, s, out);
    CTK_LAUNCH_CHECK(name);
    return CTK_OK;
}

}  // namespace

extern "C" {

size_t ctk_reduce_scratch_bytes(void) { return sizeof(ctk::ReduceScratch); }

ctk_status ctk_sum_f32(const float* a, int64_t n, float* out, void* scratch, void* stream) {
    return launch_reduce<R_SUM>("sum", a, nullptr, n, 0.0f, out, scratch, stream);
}
ctk_status ctk_dot_f32(const float* a, const float* b, int64_t n, float* out, void* scratch, void* stream) {
    return launch_reduce<R_DOT>("dot", a, b, n, 0.0f, out, scratch, stream);
}
ctk_status ctk_mse_f32(const float* a, const float* b, int64_t n, float* out, void* scratch, void* stream) {
    CTK_REQUIRE(n > 0, "ctk_mse_f32: empty input");
    return launch_reduce<R_MSE>("mse", a, b, n, static_cast<float>(n), out, scratch, stream);
}
ctk_status ctk_mae_f32(const float* a, const float* b, int64_t n, float* out, void* scratch, void* stream) {
    CTK_REQUIRE(n > 0, "ctk_mae_f32: empty input");
    return launch_reduce<R_MAE>("mae", a, b, n, static_cast<float>(n), out, scratch, stream);
}

ctk_status ctk_count_matches_f32(const float* a, const float* b, int64_t n, float* out, void* scratch, void* stream) {
    return launch_reduce<R_MATCH>("count_matches", a, b, n, 0.0f, out, scratch, stream);
}

static ctk_status mean_loss_backward(bool mse, const float* p, const float* t, const float* g, float* dp, int64_t n, void* stream) {
    CTK_REQUIRE(n >= 0, "mean loss backward: negative size");
    if (n == 0) return CTK_OK;
    CTK_REQUIRE(p && t && dp, "mean loss backward: null pointer");
    // Without an upstream scalar the third input is the prediction again, read as a broadcast
    // scalar and ignored by the functor (use_g == false multiplies by exactly 1).
    ctk::EwArgs<3, 1> A{};
    A.n = n; A.inner = 1; A.out_limit[0] = n;
    A.in[0] = p; A.in[1] = t; A.in[2] = g ? g : p;
    A.mode[0] = A.mode[1] = ctk::EW_STREAM; A.mode[2] = ctk::EW_SCALAR;
    A.out[0] = dp;
    const bool use_g = g != nullptr;
    if (mse) return ctk::ew_launch("mse_backward", A, MeanLossBwdF<true>{static_cast<float>(n), use_g}, ctk::as_stream(stream));
    return ctk::ew_launch("mae_backward", A, MeanLossBwdF<false>{static_cast<float>(n), use_g}, ctk::as_stream(stream));
}

ctk_status ctk_mse_backward_f32(const float* p, const float* t, const float* g, float* dp, int64_t n, void* stream) {
    return mean_loss_backward(true, p, t, g, dp, n, stream);
}
ctk_status ctk_mae_backward_f32(const float* p, const float* t, const float* g, float* dp, int64_t n, void* stream) {
    return mean_loss_backward(false, p, t, g, dp, n, stream);
}

}  // extern "C"
