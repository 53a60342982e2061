// Row-wise Softmax and Softmax+CrossEntropy, forward and backward, for [rows, cols] fp32.
//
// HBM-bound.  Each row is read from HBM once and kept on chip while its max, exp-sum and outputs
// are computed:
//   cols <= 128  : a group of G <= 32 lanes owns a row, values live in registers, reductions are
//                  warp shuffles (G = 8/16/32 so several short rows share a warp);
//   cols <= 4096 : a CTA of 128/256 threads owns a row in registers (128-bit loads), reductions by
//                  shuffle + one shared-memory hop, many CTAs per SM;
//   cols <= 32K  : a CTA of 512 threads owns a row in registers while the NEXT row is already being
//                  fetched into shared memory by a bulk asynchronous copy (cp.async.bulk + mbarrier),
//                  so HBM reads overlap the arithmetic and the stores of the current row;
//   otherwise    : (rows that are not 16-byte aligned, or longer) a CTA stages the row in shared
//                  memory with plain loads, or re-reads it from L2.
// exp() is evaluated once per element and kept; it is ex2.approx((x - max) * log2 e) and the
// normalisation multiplies by 1/sum: both are within 2e-6 relative of the reference's expf and
// division (the parity tolerance for these outputs is 1e-5), and they cut the instruction count per
// element by 3x, which is what makes the long-row kernels memory-bound rather than issue-bound.
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

// e^x for x <= 0 as 2^(x * log2 e) on the special-function unit.
__device__ __forceinline__ float fast_exp(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x * 1.4426950408889634f));
    return y;
}

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
    static constexpr bool kCached = true;
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
    template <class F> __device__ __forceinline__ void store(float* __restrict__ out, F f) const {
        each([&](int64_t j, float w) { __stcs(out + j, f(j, w)); });
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
    static constexpr bool kCached = true;
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
    template <class F> __device__ __forceinline__ void store(float* __restrict__ out, F f) const {
        each([&](int64_t j, float w) { __stcs(out + j, f(j, w)); });
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
    static constexpr bool kCached = false;
    const float* row;
    float* red_f;
    double* red_d;
    int64_t cols;
    __device__ __forceinline__ void load(const float* __restrict__ r) { row = r; }
    template <class F> __device__ __forceinline__ void each(F f) const {
        for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) f(j, __ldg(row + j));
    }
    template <class F> __device__ __forceinline__ void update(F f) {
        for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) (void)f(j, __ldg(row + j));
    }
    template <class F> __device__ __forceinline__ void store(float* __restrict__ out, F f) const {
        each([&](int64_t j, float w) { __stcs(out + j, f(j, w)); });
    }
    __device__ __forceinline__ float rmax() const {
        float m = -INFINITY;
        for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) m = fmaxf(m, __ldg(row + j));
        return block_max(m, red_f);
    }
    __device__ __forceinline__ float rsum(float partial) const { return static_cast<float>(block_sum(static_cast<double>(partial), red_d)); }
    __device__ __forceinline__ bool leader() const { return threadIdx.x == 0; }
};

// A CTA of THREADS threads owns a row in registers.  VEC: thread t holds the 128-bit vectors
// t, t + THREADS, ... (cols % 4 == 0, 16-byte aligned rows); otherwise the elements t, t + THREADS, ...
template <int THREADS, int ITEMS, bool VEC>
struct CtaRow {
    static constexpr bool kCached = true;
    float v[ITEMS];
    float* red_f;
    double* red_d;
    int64_t cols;
    __device__ __forceinline__ int64_t index(int it) const {
        return VEC ? (static_cast<int64_t>(threadIdx.x + (it >> 2) * THREADS) << 2) + (it & 3) : threadIdx.x + static_cast<int64_t>(it) * THREADS;
    }
    // src: the row in global memory, or its copy in shared memory
    __device__ __forceinline__ void load(const float* __restrict__ src) {
        if (VEC) {
#pragma unroll
            for (int q = 0; q < ITEMS / 4; ++q) {
                const int64_t j = static_cast<int64_t>(threadIdx.x + q * THREADS) << 2;
                float4 t = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
                if (j < cols) t = *reinterpret_cast<const float4*>(src + j);
                v[4 * q] = t.x; v[4 * q + 1] = t.y; v[4 * q + 2] = t.z; v[4 * q + 3] = t.w;
            }
        } else {
#pragma unroll
            for (int it = 0; it < ITEMS; ++it) {
                const int64_t j = threadIdx.x + static_cast<int64_t>(it) * THREADS;
                v[it] = j < cols ? src[j] : -INFINITY;
            }
        }
    }
    template <class F> __device__ __forceinline__ void each(F f) const {
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) {
            const int64_t j = index(it);
            if (j < cols) f(j, v[it]);
        }
    }
    template <class F> __device__ __forceinline__ void update(F f) {
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) {
            const int64_t j = index(it);
            if (j < cols) v[it] = f(j, v[it]);
        }
    }
    // out[j] = f(j, value) for every owned element, as 128-bit stores when VEC
    template <class F> __device__ __forceinline__ void store(float* __restrict__ out, F f) const {
        if (VEC) {
#pragma unroll
            for (int q = 0; q < ITEMS / 4; ++q) {
                const int64_t j = static_cast<int64_t>(threadIdx.x + q * THREADS) << 2;
                if (j < cols) __stcs(reinterpret_cast<float4*>(out + j), make_float4(f(j, v[4 * q]), f(j + 1, v[4 * q + 1]), f(j + 2, v[4 * q + 2]), f(j + 3, v[4 * q + 3])));
            }
        } else {
            each([&](int64_t j, float w) { __stcs(out + j, f(j, w)); });
        }
    }
    __device__ __forceinline__ float rmax() const {
        float m = -INFINITY;
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) m = fmaxf(m, v[it]);
        return block_max(m, red_f);
    }
    __device__ __forceinline__ float rsum(float partial) const { return static_cast<float>(block_sum(static_cast<double>(partial), red_d)); }
    __device__ __forceinline__ bool leader() const { return threadIdx.x == 0; }
};

// ---- the row algorithms, written once over a holder --------------------------------------------
// Returns THIS THREAD's share of the row's loss for the CE forms (the caller adds the shares of all
// its threads), 0 otherwise.
// `src` is where the holder loads the row from (global memory, or a staged copy in shared memory).
template <int ALG, class Row>
__device__ __forceinline__ float process_loaded(Row& r, const RowArgs& A, int64_t row, bool& poison) {
    const int64_t cols = A.cols;
    const float* xrow = A.x + row * cols;
    float* orow = A.out ? A.out + row * cols : nullptr;
    if (ALG == ALG_SOFTMAX_BWD) {
        // holder caches y; g is streamed twice (second pass hits L1/L2)
        const float* grow = A.t + row * cols;
        float part = 0.0f;
        r.each([&](int64_t j, float y) { part += __ldg(grow + j) * y; });
        const float dot = r.rsum(part);
        r.store(orow, [&](int64_t j, float y) { return y * (__ldg(grow + j) - dot); });
        return 0.0f;
    }
    const float m = r.rmax();
    float part = 0.0f;
    // one exp per element: the holder keeps e = exp(x - max) in place of x where it can
    r.update([&](int64_t, float v) {
        const float e = fast_exp(v - m);
        part += e;
        return e;
    });
    const float s = r.rsum(part);
    const float inv = 1.0f / s;
    auto prob = [&](float w) { return (Row::kCached ? w : fast_exp(w - m)) * inv; };
    if (ALG == ALG_SOFTMAX) {
        r.store(orow, [&](int64_t, float w) { return prob(w); });
        return 0.0f;
    }
    if (ALG == ALG_CE_ONEHOT) {
        const float* trow = A.t + row * cols;
        float loss = 0.0f;
        r.each([&](int64_t j, float w) {
            float t = __ldcs(trow + j);
            if (t != 0.0f) {  // a zero target adds exactly zero: log(max(p,1e-10)) is finite
                float p = fmaxf(prob(w), 1e-10f);
                loss = fmaf(-t, logf(p), loss);
            }
        });
        return loss;
    }
    if (ALG == ALG_CE_BWD) {
        const float* trow = A.t + row * cols;
        const float g = A.gdev ? __ldg(A.gdev) : 1.0f;
        r.store(orow, [&](int64_t j, float w) {
            float d = prob(w) - __ldcs(trow + j);
            return d * g;
        });
        return 0.0f;
    }
    // index-label forms
    const int c = static_cast<int>(__ldg(A.t + row));
    const bool ok = (c >= 0 && c < static_cast<int>(cols));
    if (!ok) poison = true;
    // The thread that holds element c contributes the row's loss: no extra global read and no
    // per-row reduction on the critical path.
    float loss = 0.0f;
    if (ok) {
        r.each([&](int64_t j, float w) {
            if (static_cast<int>(j) == c) loss = -logf(fmaxf(prob(w), 1e-10f));
        });
    }
    if (ALG == ALG_CE_FUSED) {
        r.store(orow, [&](int64_t j, float w) { return prob(w) - (static_cast<int>(j) == c ? 1.0f : 0.0f); });
    }
    return loss;
}

template <int ALG, class Row>
__device__ __forceinline__ float process_row(Row& r, const RowArgs& A, int64_t row, const float* src, bool& poison) {
    r.load(src);
    return process_loaded<ALG>(r, A, row, poison);
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
        const int64_t rr = live ? row : A.rows - 1;
        const float l = process_row<ALG>(r, A, rr, A.x + rr * A.cols, p);
        if (live) {
            poison |= p;
            if (alg_has_loss<ALG>()) acc += static_cast<double>(l);
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
        float l = process_row<ALG>(r, A, row, A.x + row * A.cols, poison);
        if (alg_has_loss<ALG>()) acc += static_cast<double>(l);
    }
    if (alg_has_loss<ALG>()) {
        if (poison && A.bad && threadIdx.x == 0) *A.bad = 1;
        int any_poison = __syncthreads_or(poison ? 1 : 0);
        double total = block_sum(acc, red_d);
        grid_finish(any_poison ? NAN : total, scratch, loss_out, 0.0f, false, red_d);
    }
}

// ---- bulk asynchronous copy of one row into shared memory -----------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void row_bar_init(uint32_t bar) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void row_fetch(uint32_t dst, const float* src, uint32_t bytes, uint32_t bar) {
    // the previous contents were read through ordinary loads: order them before the async write
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar) : "memory");
}
// Bounded: gives up after ~2^22 polls and reports it (the caller poisons the result and leaves).
__device__ __forceinline__ bool row_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < (1u << 22); ++i) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

// A CTA per row, row in registers.  PREFETCH: while row r is processed from registers, row r + grid is
// already on its way into shared memory (one bulk copy, completion on an mbarrier), so the HBM read
// of the next row overlaps the arithmetic and the stores of this one.  Needs 16-byte aligned rows.
template <int ALG, int THREADS, int ITEMS, bool VEC, bool PREFETCH>
__global__ void __launch_bounds__(THREADS) cta_reg_rows_kernel(RowArgs A, ReduceScratch* scratch, float* loss_out) {
    extern __shared__ __align__(128) float stage[];
    __shared__ double red_d[33];
    __shared__ float red_f[33];
    __shared__ __align__(8) uint64_t bar;
    __shared__ int gave_up;
    CtaRow<THREADS, ITEMS, VEC> r;
    r.cols = A.cols;
    r.red_f = red_f;
    r.red_d = red_d;
    double acc = 0.0;
    bool poison = false;
    const uint32_t row_bytes = static_cast<uint32_t>(A.cols * sizeof(float));
    uint32_t parity = 0;
    int64_t row = blockIdx.x;
    if (PREFETCH) {
        if (threadIdx.x == 0) {
            gave_up = 0;
            row_bar_init(smem_addr(&bar));
            if (row < A.rows) row_fetch(smem_addr(stage), A.x + row * A.cols, row_bytes, smem_addr(&bar));
        }
        __syncthreads();
    }
    for (; row < A.rows; row += gridDim.x) {
        const float* src = A.x + row * A.cols;
        if (PREFETCH) {
            if (threadIdx.x == 0 && !row_wait(smem_addr(&bar), parity)) gave_up = 1;
            __syncthreads();
            if (gave_up) { poison = true; break; }
            parity ^= 1u;
            src = stage;
        }
        float l;
        if (PREFETCH) {
            // copy to registers first, then hand the staging buffer to the next row's copy
            r.load(src);
            __syncthreads();
            const int64_t next = row + gridDim.x;
            if (threadIdx.x == 0 && next < A.rows) row_fetch(smem_addr(stage), A.x + next * A.cols, row_bytes, smem_addr(&bar));
            l = process_loaded<ALG>(r, A, row, poison);
        } else {
            l = process_row<ALG>(r, A, row, src, poison);
        }
        if (alg_has_loss<ALG>()) acc += static_cast<double>(l);
    }
    if (alg_has_loss<ALG>()) {
        if (poison && A.bad && threadIdx.x == 0) *A.bad = 1;
        int any_poison = __syncthreads_or(poison ? 1 : 0);
        double total = block_sum(acc, red_d);
        grid_finish(any_poison ? NAN : total, scratch, loss_out, 0.0f, false, red_d);
    }
}

template <int ALG, int THREADS, int ITEMS, bool PREFETCH>
ctk_status launch_cta_reg(const RowArgs& A, ReduceScratch* s, float* loss_out, cudaStream_t st) {
    const bool vec = (A.cols % 4 == 0) && ((reinterpret_cast<uintptr_t>(A.x) & 15u) == 0) && (!A.out || (reinterpret_cast<uintptr_t>(A.out) & 15u) == 0);
    const size_t smem = PREFETCH ? static_cast<size_t>(A.cols) * sizeof(float) : 0;
    // resident CTAs per SM: by threads (2048) and by staging memory (~200 KiB)
    int per_sm = 2048 / THREADS;
    if (PREFETCH) {
        const int by_smem = static_cast<int>((200u * 1024u) / (smem + 1024));
        per_sm = per_sm < by_smem ? per_sm : by_smem;
        if (per_sm < 1) per_sm = 1;
    }
    int64_t cap = static_cast<int64_t>(ctk::sm_count()) * per_sm;
    if (!PREFETCH) cap = A.rows;  // one row per CTA, the hardware scheduler walks the rows in order
    int64_t grid = A.rows < cap ? A.rows : cap;
    if (alg_has_loss<ALG>() && grid > kMaxReduceBlocks) grid = kMaxReduceBlocks;
    if (grid > 0x7fffffff) grid = 0x7fffffff;
    if (PREFETCH) {
        CTK_REQUIRE(vec, "row kernel: the prefetching form needs 16-byte aligned rows");
        auto k = cta_reg_rows_kernel<ALG, THREADS, ITEMS, true, true>;
        static bool attr_set = false;
        if (!attr_set) {
            CTK_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 32768 * static_cast<int>(sizeof(float))));
            attr_set = true;
        }
        k<<<static_cast<unsigned>(grid), THREADS, smem, st>>>(A, s, loss_out);
    } else if (vec) {
        cta_reg_rows_kernel<ALG, THREADS, ITEMS, true, false><<<static_cast<unsigned>(grid), THREADS, 0, st>>>(A, s, loss_out);
    } else {
        cta_reg_rows_kernel<ALG, THREADS, ITEMS, false, false><<<static_cast<unsigned>(grid), THREADS, 0, st>>>(A, s, loss_out);
    }
    return CTK_OK;
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
    const bool aligned_rows = (c % 4 == 0) && ((reinterpret_cast<uintptr_t>(A.x) & 15u) == 0) && (!A.out || (reinterpret_cast<uintptr_t>(A.out) & 15u) == 0);
    ctk_status rc = CTK_OK;
    if (c <= 8) launch_reg<ALG, 8, 1>(A, s, loss_out, st);
    else if (c <= 16) launch_reg<ALG, 16, 1>(A, s, loss_out, st);
    else if (c <= 32) launch_reg<ALG, 32, 1>(A, s, loss_out, st);
    else if (c <= 64) launch_reg<ALG, 32, 2>(A, s, loss_out, st);
    else if (c <= 128) launch_reg<ALG, 32, 4>(A, s, loss_out, st);
    else if (c <= 1024) rc = launch_cta_reg<ALG, 128, 8, false>(A, s, loss_out, st);
    else if (c <= 4096) rc = launch_cta_reg<ALG, 256, 16, false>(A, s, loss_out, st);
    else if (c <= 8192 && aligned_rows) rc = launch_cta_reg<ALG, 512, 16, true>(A, s, loss_out, st);
    else if (c <= 16384 && aligned_rows) rc = launch_cta_reg<ALG, 512, 32, true>(A, s, loss_out, st);
    else if (c <= 32768 && aligned_rows) rc = launch_cta_reg<ALG, 512, 64, true>(A, s, loss_out, st);
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
    if (rc) return rc;
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
