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

// One flag per device ordinal: the library's scratch block is per device, and a kernel that gave up is
// reported through a status word that does not say where it ran, so every device's block is marked.
static std::atomic<bool> g_library_scratch_dirty[64];
void mark_reduce_scratch_dirty() {
    for (auto& f : g_library_scratch_dirty) f.store(true);
}

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
    int dev = 0;
    CTK_CUDA(cudaGetDevice(&dev));
    const bool dirty = dev >= 0 && dev < 64 && g_library_scratch_dirty[dev].exchange(false);
    if (user || dirty) CTK_CUDA(cudaMemsetAsync(&(*out)->ticket, 0, sizeof(unsigned int), st));
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

// ---- column sums: out[j] = sum over rows of x[r, j] -------------------------------------------------------
// Pass 1: a CTA owns 256 rows x 128 columns; warp w adds rows w, w + 8, ... (one 128-bit load per lane
// and row, 512 contiguous bytes per warp), the eight warps add up through shared memory in fixed order,
// and the CTA writes one row of partial sums.  Pass 2 adds the partial rows in order.  No atomics: the
// result is the same from call to call.
constexpr int kColRows = 256, kColWarps = 8;
__global__ void __launch_bounds__(kColWarps * 32) colsum_partial_kernel(const float* __restrict__ x, int64_t rows, int64_t cols, float* __restrict__ part) {
    __shared__ float4 acc_sm[kColWarps][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t col = (static_cast<int64_t>(blockIdx.x) * 32 + lane) * 4;
    const int64_t r0 = static_cast<int64_t>(blockIdx.y) * kColRows;
    const int64_t r1 = r0 + kColRows < rows ? r0 + kColRows : rows;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (col < cols) {
        if (col + 4 <= cols && (cols & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0) {
#pragma unroll 4
            for (int64_t r = r0 + warp; r < r1; r += kColWarps) {
                const float4 v = __ldcs(reinterpret_cast<const float4*>(x + r * cols + col));
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
        } else {
            for (int64_t r = r0 + warp; r < r1; r += kColWarps) {
                const float* p = x + r * cols + col;
                acc.x += p[0];
                if (col + 1 < cols) acc.y += p[1];
                if (col + 2 < cols) acc.z += p[2];
                if (col + 3 < cols) acc.w += p[3];
            }
        }
    }
    acc_sm[warp][lane] = acc;
    __syncthreads();
    if (warp == 0 && col < cols) {
        float4 t = acc_sm[0][lane];
        for (int w = 1; w < kColWarps; ++w) { const float4 v = acc_sm[w][lane]; t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w; }
        float* o = part + static_cast<int64_t>(blockIdx.y) * cols + col;
        o[0] = t.x;
        if (col + 1 < cols) o[1] = t.y;
        if (col + 2 < cols) o[2] = t.z;
        if (col + 3 < cols) o[3] = t.w;
    }
}
__global__ void __launch_bounds__(256) colsum_final_kernel(const float* __restrict__ part, int64_t chunks, int64_t cols, float* __restrict__ out) {
    const int64_t j = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (j >= cols) return;
    float t = 0.f;
    for (int64_t c = 0; c < chunks; ++c) t += part[c * cols + j];
    out[j] = t;
}

}  // namespace

extern "C" {

size_t ctk_reduce_scratch_bytes(void) { return sizeof(ctk::ReduceScratch); }

ctk_status ctk_sum_f32(const float* a, int64_t n, float* out, void* scratch, void* stream) {
    CTK_RANGE("ctk_sum_f32");
    return launch_reduce<R_SUM>("sum", a, nullptr, n, 0.0f, out, scratch, stream);
}
ctk_status ctk_dot_f32(const float* a, const float* b, int64_t n, float* out, void* scratch, void* stream) {
    CTK_RANGE("ctk_dot_f32");
    return launch_reduce<R_DOT>("dot", a, b, n, 0.0f, out, scratch, stream);
}
ctk_status ctk_mse_f32(const float* a, const float* b, int64_t n, float* out, void* scratch, void* stream) {
    CTK_RANGE("ctk_mse_f32");
    CTK_REQUIRE(n > 0, "ctk_mse_f32: empty input");
    return launch_reduce<R_MSE>("mse", a, b, n, static_cast<float>(n), out, scratch, stream);
}
ctk_status ctk_mae_f32(const float* a, const float* b, int64_t n, float* out, void* scratch, void* stream) {
    CTK_RANGE("ctk_mae_f32");
    CTK_REQUIRE(n > 0, "ctk_mae_f32: empty input");
    return launch_reduce<R_MAE>("mae", a, b, n, static_cast<float>(n), out, scratch, stream);
}

ctk_status ctk_colsum_f32(const float* x, int64_t rows, int64_t cols, float* out, void* stream) {
    CTK_RANGE("ctk_colsum_f32");
    CTK_REQUIRE(rows >= 0 && cols >= 0, "ctk_colsum_f32: negative shape");
    if (cols == 0) return CTK_OK;
    CTK_REQUIRE(out && (x || rows == 0), "ctk_colsum_f32: null pointer");
    cudaStream_t st = ctk::as_stream(stream);
    const int64_t chunks = (rows + kColRows - 1) / kColRows;
    if (chunks == 0) {
        CTK_CUDA(cudaMemsetAsync(out, 0, static_cast<size_t>(cols) * sizeof(float), st));
        return CTK_OK;
    }
    CTK_REQUIRE(chunks <= 65535, "ctk_colsum_f32: more than 65535 x 256 rows");
    float* part = nullptr;
    CTK_CUDA(cudaMallocAsync(reinterpret_cast<void**>(&part), static_cast<size_t>(chunks * cols) * sizeof(float), st));
    colsum_partial_kernel<<<dim3(static_cast<unsigned>((cols + 127) / 128), static_cast<unsigned>(chunks)), kColWarps * 32, 0, st>>>(x, rows, cols, part);
    CTK_LAUNCH_CHECK("colsum_partial_kernel");
    colsum_final_kernel<<<static_cast<unsigned>((cols + 255) / 256), 256, 0, st>>>(part, chunks, cols, out);
    CTK_LAUNCH_CHECK("colsum_final_kernel");
    CTK_CUDA(cudaFreeAsync(part, st));
    return CTK_OK;
}

ctk_status ctk_count_matches_f32(const float* a, const float* b, int64_t n, float* out, void* scratch, void* stream) {
    CTK_RANGE("ctk_count_matches_f32");
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
    CTK_RANGE("ctk_mse_backward_f32");
    return mean_loss_backward(true, p, t, g, dp, n, stream);
}
ctk_status ctk_mae_backward_f32(const float* p, const float* t, const float* g, float* dp, int64_t n, void* stream) {
    CTK_RANGE("ctk_mae_backward_f32");
    return mean_loss_backward(false, p, t, g, dp, n, stream);
}

}  // extern "C"
