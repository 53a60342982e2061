// Row-wise Softmax and Softmax+CrossEntropy, forward and backward, for [rows, cols] fp32.
//
// HBM-bound.  Each row is read from HBM once and kept on chip while its max, exp-sum and outputs
// are computed:
//   cols <= 1024 : a group of G <= 32 lanes owns a row, values live in registers, reductions are
//                  warp shuffles (G = 8/16/32 so several short rows share a warp);
//   cols <= 48K  : a CTA owns a row staged in shared memory (one 128-bit coalesced pass in),
//                  reductions by shuffle + one shared-memory hop;
//   larger       : a CTA owns a row and re-reads it from L2/HBM.
// Per-row losses are added in fp64 and finished in one launch (see reduce_common.cuh).
// Compiled with -fmad=false; the one fused multiply-add of the reference loop is explicit.
//
// Reference semantics: Softmax_BASIC_kernel.cpp:70-91 (max, e = exp(x-max), sum, e/sum),
// CrossEntropy_BASIC_kernel.cpp:41-66 and :88-120 (loss -= t*log(max(p,1e-10)), SUMMED over rows),
// src/AutoDiff.cpp:1417-1490 (softmax backward from the saved output) and :1517-1601
// ((softmax - target) * upstream scalar).
#include <math.h>

#include <type_traits>

#include "reduce_common.cuh"

namespace {
using namespace ctk;

constexpr int kRegThreads = 256;   // register-row kernels: 8 warps per CTA
constexpr int kRowThreads = 512;   // CTA-per-row kernels
constexpr int kSmemRowMaxCols = 48 * 1024;

enum { ALG_SOFTMAX = 0, ALG_SOFTMAX_BWD = 1, ALG_CE_ONEHOT = 2, ALG_CE_INDEX = 3, ALG_CE_BWD = 4, ALG_CE_FUSED = 5 };

struct RowArgs {
    const float* x;    // logits / softmax input / saved softmax output y (backward)
    const float* t;    // one-hot targets / upstream gradient g (softmax backward) / labels (index forms)
    float* out;        // y / dx / dlogits
    const float* gdev; // upstream scalar (CE backward), may be null
    int* bad;          // out-of-range label flag, may be null
    int64_t rows, cols;
};

// ---- group reductions over G lanes of a warp -------------------------------------------------
template <int G>
__device__ __forceinline__ float group_max(float v) {
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
template <int G>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---- row holders -----------------------------------------------------------------------------
// The three holders expose the same interface: load(row), rmax(), rsum(partial), and
// each(f) / update(f) over the elements this thread owns.
template <int G, int ITEMS>
struct RegRow {
    float v[ITEMS];
    int lane;
    int64_t cols;
    __device__ __forceinline__ void load(const float* __restrict__ row) {
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) {
            int64_t j = lane + it * G;
            v[it] = j < cols ? __ldcs(row + j) : -INFINITY;
        }
    }
    template <class F> __device__ __forceinline__ void each(F f) const {
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) {
            int64_t j = lane + it * G;
            if (j < cols) f(j, v[it]);
        }
    }
    template <class F> __device__ __forceinline__ void update(F f) {
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) {
            int64_t j = lane + it * G;
            if (j < cols) v[it] = f(j, v[it]);
        }
    }
    __device__ __forceinline__ float rmax() const {
        float m = -INFINITY;
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) m = fmaxf(m, v[it]);
        return group_max<G>(m);
    }
    __device__ __forceinline__ float rsum(float partial) const { return group_sum<G>(partial); }
    __device__ __forceinline__ bool leader() const { return lane == 0; }
};

struct SmemRow {
    float* buf;       // cols floats of dynamic shared memory
    float* red_f;     // 33 floats
    double* red_d;    // 33 doubles
    int64_t cols;
    __device__ __forceinline__ void load(const float* __restrict__ row) {
        __syncthreads();  // previous row's readers are done with buf
        if ((reinterpret_cast<uintptr_t>(row) & 15u) == 0) {
            const int64_t c4 = cols >> 2;
            for (int64_t i = threadIdx.x; i < c4; i += blockDim.x)
                reinterpret_cast<float4*>(buf)[i] = __ldcs(reinterpret_cast<const float4*>(row) + i);
            for (int64_t j = (c4 << 2) + threadIdx.x; j < cols; j += blockDim.x) buf[j] = __ldcs(row + j);
        } else {
            for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) buf[j] = __ldcs(row + j);
        }
        __syncthreads();
    }
    template <class F> __device__ __forceinline__ void each(F f) const {
        for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) f(j, buf[j]);
    }
    template <class F> __device__ __forceinline__ void update(F f) {
        for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) buf[j] = f(j, buf[j]);
    }
    __device__ __forceinline__ float rmax() const {
        float m = -INFINITY;
        for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) m = fmaxf(m, buf[j]);
        return block_max(m, red_f);
    }
    __device__ __forceinline__ float rsum(float partial) const { return static_cast<float>(block_sum(static_cast<double>(partial), red_d)); }
    __device__ __forceinline__ bool leader() const { return threadIdx.x == 0; }
};

// Row too long for shared memory: every pass re-reads it (L2 absorbs most of the re-reads).
struct GlobalRow {
    const float* row;
    float* red_f;
    double* red_d;
    int64_t cols;
    __device__ __forceinline__ void load(const float* __restrict__ r) { row = r; }
    template <class F> __device__ __forceinline__ void each(F f) const {
        for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) f(j, __ldg(row + j));
    }
    __device__ __forceinline__ float rmax() const {
        float m = -INFINITY;
        for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) m = fmaxf(m, __ldg(row + j));
        return block_max(m, red_f);
    }
    __device__ __forceinline__ float rsum(float partial) const { return static_cast<float>(block_sum(static_cast<double>(partial), red_d)); }
    __device__ __forceinline__ bool leader() const { return threadIdx.x == 0; }
};

// ---- the row algorithms, written once over a holder --------------------------------------------
// Returns this row's loss contribution (valid in the leader) for the CE forms, 0 otherwise.
template <int ALG, class Row>
__device__ __forceinline__ float process_row(Row& r, const RowArgs& A, int64_t row, bool& poison) {
    const int64_t cols = A.cols;
    const float* xrow = A.x + row * cols;
    float* orow = A.out ? A.out + row * cols : nullptr;
    r.load(xrow);
    if (ALG == ALG_SOFTMAX_BWD) {
        // holder caches y; g is streamed twice (second pass hits L1/L2)
        const float* grow = A.t + row * cols;
        float part = 0.0f;
        r.each([&](int64_t j, float y) { part += __ldg(grow + j) * y; });
        const float dot = r.rsum(part);
        r.each([&](int64_t j, float y) { __stcs(orow + j, y * (__ldg(grow + j) - dot)); });
        return 0.0f;
    }
    const float m = r.rmax();
    float part = 0.0f;
    r.each([&](int64_t, float v) { part += expf(v - m); });
    const float s = r.rsum(part);
    if (ALG == ALG_SOFTMAX) {
        r.each([&](int64_t j, float v) {
            float e = expf(v - m);
            __stcs(orow + j, s > 0.0f ? e / s : e);
        });
        return 0.0f;
    }
    if (ALG == ALG_CE_ONEHOT) {
        const float* trow = A.t + row * cols;
        float loss = 0.0f;
        r.each([&](int64_t j, float v) {
            float t = __ldcs(trow + j);
            if (t != 0.0f) {  // a zero target adds exactly zero: log(max(p,1e-10)) is finite
                float p = fmaxf(expf(v - m) / s, 1e-10f);
                loss = fmaf(-t, logf(p), loss);
            }
        });
        return r.rsum(loss);
    }
    if (ALG == ALG_CE_BWD) {
        const float* trow = A.t + row * cols;
        const float g = A.gdev ? __ldg(A.gdev) : 1.0f;
        r.each([&](int64_t j, float v) {
            float p = expf(v - m) / s;
            float d = p - __ldcs(trow + j);
            __stcs(orow + j, d * g);
        });
        return 0.0f;
    }
    // index-label forms
    const int c = static_cast<int>(__ldg(A.t + row));
    const bool ok = (c >= 0 && c < static_cast<int>(cols));
    if (!ok) poison = true;
    float loss = 0.0f;
    if (r.leader() && ok) {
        float p = fmaxf(expf(__ldg(xrow + c) - m) / s, 1e-10f);
        loss = -logf(p);
    }
    if (ALG == ALG_CE_FUSED) {
        r.each([&](int64_t j, float v) {
            float p = expf(v - m) / s;
            __stcs(orow + j, p - (static_cast<int>(j) == c ? 1.0f : 0.0f));
        });
    }
    return loss;
}

template <int ALG> __host__ __device__ constexpr bool alg_has_loss() { return ALG == ALG_CE_ONEHOT || ALG == ALG_CE_INDEX || ALG == ALG_CE_FUSED; }

template <int ALG, int G, int ITEMS>
__global__ void __launch_bounds__(kRegThreads) reg_rows_kernel(RowArgs A, ReduceScratch* scratch, float* loss_out) {
    __shared__ double smem[33];
    constexpr int kGroupsPerCta = kRegThreads / G;
    RegRow<G, ITEMS> r;
    r.lane = threadIdx.x % G;
    r.cols = A.cols;
    const int64_t group = static_cast<int64_t>(blockIdx.x) * kGroupsPerCta + threadIdx.x / G;
    const int64_t ngroups = static_cast<int64_t>(gridDim.x) * kGroupsPerCta;
    double acc = 0.0;
    bool poison = false;
    // Every group of a warp runs the same trip count so the shuffles stay converged; a group with
    // no row left owns zero elements (loads, stores and sums nothing) and its result is dropped.
    const int64_t trips = (A.rows + ngroups - 1) / ngroups;
    for (int64_t it = 0; it < trips; ++it) {
        const int64_t row = group + it * ngroups;
        const bool live = row < A.rows;
        r.cols = live ? A.cols : 0;
        bool p = false;
        const float l = process_row<ALG>(r, A, live ? row : A.rows - 1, p);
        if (live) {
            poison |= p;
            if (alg_has_loss<ALG>() && r.leader()) acc += static_cast<double>(l);
        }
    }
    if (alg_has_loss<ALG>()) {
        if (poison && A.bad) *A.bad = 1;
        int any_poison = __syncthreads_or(poison ? 1 : 0);
        double total = block_sum(acc, smem);
        // A poisoned CTA contributes NaN so the final value is NaN whichever CTA finishes last.
        grid_finish(any_poison ? NAN : total, scratch, loss_out, 0.0f, false, smem);
    }
}

template <int ALG, class Row>
__global__ void __launch_bounds__(kRowThreads) cta_rows_kernel(RowArgs A, ReduceScratch* scratch, float* loss_out) {
    extern __shared__ __align__(16) float dyn_smem[];
    __shared__ double red_d[33];
    __shared__ float red_f[33];
    Row r;
    r.cols = A.cols;
    r.red_f = red_f;
    r.red_d = red_d;
    if constexpr (std::is_same<Row, SmemRow>::value) r.buf = dyn_smem;
    double acc = 0.0;
    bool poison = false;
    for (int64_t row = blockIdx.x; row < A.rows; row += gridDim.x) {
        float l = process_row<ALG>(r, A, row, poison);
        if (alg_has_loss<ALG>() && r.leader()) acc += static_cast<double>(l);
    }
    if (alg_has_loss<ALG>()) {
        if (poison && A.bad && threadIdx.x == 0) *A.bad = 1;
        int any_poison = __syncthreads_or(poison ? 1 : 0);
        double total = block_sum(acc, red_d);
        grid_finish(any_poison ? NAN : total, scratch, loss_out, 0.0f, false, red_d);
    }
}

template <int ALG, int G, int ITEMS>
void launch_reg(const RowArgs& A, ReduceScratch* s, float* loss_out, cudaStream_t st) {
    constexpr int kGroupsPerCta = kRegThreads / G;
    int64_t need = (A.rows + kGroupsPerCta - 1) / kGroupsPerCta;
    int64_t cap = static_cast<int64_t>(ctk::sm_count()) * 8;
    int grid = static_cast<int>(need < cap ? need : cap);
    if (grid < 1) grid = 1;
    if (grid > kMaxReduceBlocks) grid = kMaxReduceBlocks;
    reg_rows_kernel<ALG, G, ITEMS><<<grid, kRegThreads, 0, st>>>(A, s, loss_out);
}

template <int ALG>
ctk_status launch_rows(const char* name, const RowArgs& A, float* loss_out, void* scratch, void* stream) {
    CTK_REQUIRE(A.rows >= 0 && A.cols >= 0, "row kernel: negative shape");
    cudaStream_t st = as_stream(stream);
    ReduceScratch* s = nullptr;
    if (alg_has_loss<ALG>()) {
        CTK_REQUIRE(loss_out, "row kernel: null loss output");
        ctk_status rc = reduce_scratch(scratch, st, &s);
        if (rc) return rc;
    }
    if (A.rows == 0 || A.cols == 0) {
        if (alg_has_loss<ALG>()) CTK_CUDA(cudaMemsetAsync(loss_out, 0, sizeof(float), st));
        return CTK_OK;
    }
    CTK_REQUIRE(A.x && A.cols < (int64_t(1) << 31), "row kernel: null input or cols >= 2^31");
    const int64_t c = A.cols;
    if (c <= 8) launch_reg<ALG, 8, 1>(A, s, loss_out, st);
    else if (c <= 16) launch_reg<ALG, 16, 1>(A, s, loss_out, st);
    else if (c <= 32) launch_reg<ALG, 32, 1>(A, s, loss_out, st);
    else if (c <= 64) launch_reg<ALG, 32, 2>(A, s, loss_out, st);
    else if (c <= 128) launch_reg<ALG, 32, 4>(A, s, loss_out, st);
    else if (c <= 256) launch_reg<ALG, 32, 8>(A, s, loss_out, st);
    else if (c <= 512) launch_reg<ALG, 32, 16>(A, s, loss_out, st);
    else if (c <= 1024) launch_reg<ALG, 32, 32>(A, s, loss_out, st);
    else {
        int64_t cap = static_cast<int64_t>(ctk::sm_count()) * (c <= 12 * 1024 ? 4 : 1);
        int grid = static_cast<int>(A.rows < cap ? A.rows : cap);
        if (grid > kMaxReduceBlocks) grid = kMaxReduceBlocks;
        if (c <= kSmemRowMaxCols) {
            size_t bytes = static_cast<size_t>(c) * sizeof(float);
            static bool attr_set = false;  // raises the opt-in limit once per process, per instantiation
            if (!attr_set) {
                CTK_CUDA(cudaFuncSetAttribute(cta_rows_kernel<ALG, SmemRow>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              kSmemRowMaxCols * static_cast<int>(sizeof(float))));
                attr_set = true;
            }
            cta_rows_kernel<ALG, SmemRow><<<grid, kRowThreads, bytes, st>>>(A, s, loss_out);
        } else {
            cta_rows_kernel<ALG, GlobalRow><<<grid, kRowThreads, 0, st>>>(A, s, loss_out);
        }
    }
    CTK_LAUNCH_CHECK(name);
    return CTK_OK;
}

}  // namespace

extern "C" {

ctk_status ctk_softmax_rows_f32(const float* x, float* y, int64_t rows, int64_t cols, void* stream) {
    CTK_REQUIRE((x && y) || rows == 0 || cols == 0, "ctk_softmax_rows_f32: null pointer");
    RowArgs A{x, nullptr, y, nullptr, nullptr, rows, cols};
    return launch_rows<ALG_SOFTMAX>("softmax_rows", A, nullptr, nullptr, stream);
}

ctk_status ctk_softmax_backward_rows_f32(const float* y, const float* g, float* dx, int64_t rows, int64_t cols, void* stream) {
    CTK_REQUIRE((y && g && dx) || rows == 0 || cols == 0, "ctk_softmax_backward_rows_f32: null pointer");
    RowArgs A{y, g, dx, nullptr, nullptr, rows, cols};
    return launch_rows<ALG_SOFTMAX_BWD>("softmax_backward_rows", A, nullptr, nullptr, stream);
}

ctk_status ctk_ce_onehot_f32(const float* logits, const float* onehot, int64_t rows, int64_t cols, float* out,
                             void* scratch, void* stream) {
    CTK_REQUIRE((logits && onehot) || rows == 0 || cols == 0, "ctk_ce_onehot_f32: null pointer");
    RowArgs A{logits, onehot, nullptr, nullptr, nullptr, rows, cols};
    return launch_rows<ALG_CE_ONEHOT>("ce_onehot", A, out, scratch, stream);
}

ctk_status ctk_ce_index_f32(const float* logits, const float* labels, int64_t rows, int64_t cols, float* out,
                            int* bad_label_flag, void* scratch, void* stream) {
    CTK_REQUIRE((logits && labels) || rows == 0 || cols == 0, "ctk_ce_index_f32: null pointer");
    RowArgs A{logits, labels, nullptr, nullptr, bad_label_flag, rows, cols};
    return launch_rows<ALG_CE_INDEX>("ce_index", A, out, scratch, stream);
}

ctk_status ctk_ce_backward_f32(const float* logits, const float* onehot, const float* g_device, float* dlogits,
                               int64_t rows, int64_t cols, void* stream) {
    CTK_REQUIRE((logits && onehot && dlogits) || rows == 0 || cols == 0, "ctk_ce_backward_f32: null pointer");
    RowArgs A{logits, onehot, dlogits, g_device, nullptr, rows, cols};
    return launch_rows<ALG_CE_BWD>("ce_backward", A, nullptr, nullptr, stream);
}

ctk_status ctk_ce_fused_index_f32(const float* logits, const float* labels, int64_t rows, int64_t cols, float* out,
                                  float* dlogits, int* bad_label_flag, void* scratch, void* stream) {
    CTK_REQUIRE((logits && labels && dlogits) || rows == 0 || cols == 0, "ctk_ce_fused_index_f32: null pointer");
    RowArgs A{logits, labels, dlogits, nullptr, bad_label_flag, rows, cols};
    return launch_rows<ALG_CE_FUSED>("ce_fused_index", A, out, scratch, stream);
}

}  // extern "C"
