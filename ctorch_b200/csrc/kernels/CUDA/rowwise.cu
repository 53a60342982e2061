// Row-wise Softmax and Softmax+CrossEntropy, forward and backward, for [rows, cols] fp32.
//
// HBM-bound.  Each row is read from HBM once and kept on chip while its max, exp-sum and outputs
// are computed:
//   cols <= 16   : a thread owns a row; a CTA moves its 512 rows between HBM and shared memory as one
//                  contiguous block, with bulk asynchronous copies through two buffers so that the
//                  load of the next block and the store of the previous one overlap the work on
//                  the current one (the 10-class layer);
//   cols <= 1024 : a warp owns a row, values live in registers (128-bit loads), reductions are warp
//                  shuffles; the loss-carrying forms run a resident grid in which every warp keeps
//                  its next two rows in flight;
//   cols <= 4096 : a CTA of 128/256 threads owns a row in registers, one barrier per reduction;
//   cols <= 32K  : one CTA per SM; a producer warp streams this CTA's rows through a 208 KiB ring of
//                  shared memory with bulk asynchronous copies (cp.async.bulk + mbarriers) and runs
//                  more than a row ahead, 512 consumer threads keep the current row in registers,
//                  so HBM reads never stop for the arithmetic and the stores of the current row;
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

constexpr int kRowThreads = 512;   // CTA-per-row kernels
constexpr int kSmemRowMaxCols = 48 * 1024;
constexpr int kConsumers = 512;    // consumer threads of the streamed long-row kernel

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

// ---- mbarrier / bulk-copy helpers of the two pipelined kernels ------------------------------------------
constexpr uint32_t kStreamWaitLimit = 1u << 22;

__device__ int g_row_status = 0;  // set when a bounded wait of a pipelined row kernel ran out

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void sbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void sbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool sbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool sbar_wait(uint32_t bar, uint32_t parity, volatile int* gave_up) {
    for (uint32_t i = 0; i < kStreamWaitLimit; ++i) {
        if (sbar_try(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *gave_up) return false;
    }
    *gave_up = 1;
    atomicExch(&g_row_status, 1);
    return false;
}
__device__ __forceinline__ void chunk_fetch(uint32_t dst, const float* src, uint32_t bytes, uint32_t bar) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar) : "memory");
}
// ---- row holders -----------------------------------------------------------------------------
// Every holder exposes: load(src), rmax(), rsum(partial), each(f) / update(f) / store(out, f) over
// the elements this thread owns, each2 / store2 that also hand f the matching element of a second
// operand row, and pick(c, w) -- whether this thread owns element c, and its value.

// Cross-warp reductions for a CTA (or the consumer threads of one): one barrier per reduction, the
// scratch alternates between two halves so a slow reader of the previous result is never overwritten.
struct CtaReducer {
    float* red;   // 64 floats of shared memory
    int flip;
    bool named;   // true: barrier 1 over kStreamConsumers threads; false: __syncthreads
    __device__ __forceinline__ void sync() const {
        if (named) asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory");
        else __syncthreads();
    }
    template <bool IS_MAX>
    __device__ __forceinline__ float run(float v, int nwarps) {
        v = IS_MAX ? warp_max(v) : warp_sum(v);
        float* buf = red + 32 * flip;
        flip ^= 1;
        const int lane = threadIdx.x & 31;
        if (lane == 0) buf[threadIdx.x >> 5] = v;
        sync();
        float t = lane < nwarps ? buf[lane] : (IS_MAX ? -INFINITY : 0.0f);
        return IS_MAX ? warp_max(t) : warp_sum(t);
    }
};

// Elements of one row held in registers by a group of LANES threads (a warp, or all threads of a
// CTA).  VEC: member t holds the 128-bit vectors t, t + LANES, ... (cols % 4 == 0, 16-byte aligned
// rows); otherwise the elements t, t + LANES, ...  Guards are per vector and in 32-bit arithmetic:
// the per-element index arithmetic is what otherwise makes these kernels issue-bound.
template <int LANES, int ITEMS, bool VEC>
struct StridedRow {
    static_assert(!VEC || ITEMS % 4 == 0, "vector form holds whole vectors");
    static constexpr bool kCached = true;
    static constexpr bool kRawRow = false;
    static constexpr int kSteps = VEC ? ITEMS / 4 : ITEMS;
    float v[ITEMS];
    int cols;
    int t;
    __device__ __forceinline__ int first(int s) const { return VEC ? (t + s * LANES) << 2 : t + s * LANES; }
    __device__ __forceinline__ void load(const float* __restrict__ src) {
#pragma unroll
        for (int s = 0; s < kSteps; ++s) {
            const int j = first(s);
            if (VEC) {
                float4 w = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
                if (j < cols) w = __ldcs(reinterpret_cast<const float4*>(src + j));
                v[4 * s] = w.x; v[4 * s + 1] = w.y; v[4 * s + 2] = w.z; v[4 * s + 3] = w.w;
            } else {
                v[s] = j < cols ? __ldcs(src + j) : -INFINITY;
            }
        }
    }
    template <class F> __device__ __forceinline__ void each(F f) const {
#pragma unroll
        for (int s = 0; s < kSteps; ++s) {
            const int j = first(s);
            if (j < cols) {
                if (VEC) { f(j, v[4 * s]); f(j + 1, v[4 * s + 1]); f(j + 2, v[4 * s + 2]); f(j + 3, v[4 * s + 3]); }
                else f(j, v[s]);
            }
        }
    }
    template <class F> __device__ __forceinline__ void update(F f) {
#pragma unroll
        for (int s = 0; s < kSteps; ++s) {
            const int j = first(s);
            if (j < cols) {
                if (VEC) { v[4 * s] = f(j, v[4 * s]); v[4 * s + 1] = f(j + 1, v[4 * s + 1]); v[4 * s + 2] = f(j + 2, v[4 * s + 2]); v[4 * s + 3] = f(j + 3, v[4 * s + 3]); }
                else v[s] = f(j, v[s]);
            }
        }
    }
    template <class F> __device__ __forceinline__ void store(float* __restrict__ out, F f) const {
#pragma unroll
        for (int s = 0; s < kSteps; ++s) {
            const int j = first(s);
            if (j < cols) {
                if (VEC) __stcs(reinterpret_cast<float4*>(out + j), make_float4(f(j, v[4 * s]), f(j + 1, v[4 * s + 1]), f(j + 2, v[4 * s + 2]), f(j + 3, v[4 * s + 3])));
                else __stcs(out + j, f(j, v[s]));
            }
        }
    }
    // aux rows are 16-byte aligned too in the vector form (the launchers check)
    template <class F> __device__ __forceinline__ void each2(const float* __restrict__ aux, F f) const {
#pragma unroll
        for (int s = 0; s < kSteps; ++s) {
            const int j = first(s);
            if (j < cols) {
                if (VEC) {
                    const float4 a = __ldg(reinterpret_cast<const float4*>(aux + j));
                    f(j, v[4 * s], a.x); f(j + 1, v[4 * s + 1], a.y); f(j + 2, v[4 * s + 2], a.z); f(j + 3, v[4 * s + 3], a.w);
                } else {
                    f(j, v[s], __ldg(aux + j));
                }
            }
        }
    }
    template <class F> __device__ __forceinline__ void store2(float* __restrict__ out, const float* __restrict__ aux, F f) const {
#pragma unroll
        for (int s = 0; s < kSteps; ++s) {
            const int j = first(s);
            if (j < cols) {
                if (VEC) {
                    const float4 a = __ldcs(reinterpret_cast<const float4*>(aux + j));
                    __stcs(reinterpret_cast<float4*>(out + j), make_float4(f(j, v[4 * s], a.x), f(j + 1, v[4 * s + 1], a.y), f(j + 2, v[4 * s + 2], a.z), f(j + 3, v[4 * s + 3], a.w)));
                } else {
                    __stcs(out + j, f(j, v[s], __ldcs(aux + j)));
                }
            }
        }
    }
    __device__ __forceinline__ bool pick(int c, float& w) const {
        bool mine = false;
#pragma unroll
        for (int s = 0; s < kSteps; ++s) {
            const int j = first(s);
            if (VEC) {
                if (j == (c & ~3)) {
                    const int k = c & 3;
                    w = k == 0 ? v[4 * s] : k == 1 ? v[4 * s + 1] : k == 2 ? v[4 * s + 2] : v[4 * s + 3];
                    mine = true;
                }
            } else if (j == c) {
                w = v[s];
                mine = true;
            }
        }
        return mine;
    }
    __device__ __forceinline__ float local_max() const {
        float m = -INFINITY;
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) m = fmaxf(m, v[it]);
        return m;
    }
};

// A warp owns the row: reductions are shuffles, no barrier and no shared memory anywhere.
template <int ITEMS, bool VEC>
struct WarpRow : StridedRow<32, ITEMS, VEC> {
    __device__ __forceinline__ float rmax() const { return warp_max(this->local_max()); }
    __device__ __forceinline__ float rsum(float partial) const { return warp_sum(partial); }
};

// All THREADS threads of a CTA own the row.
template <int THREADS, int ITEMS, bool VEC>
struct CtaRow : StridedRow<THREADS, ITEMS, VEC> {
    CtaReducer rd;
    __device__ __forceinline__ float rmax() { return rd.template run<true>(this->local_max(), THREADS / 32); }
    __device__ __forceinline__ float rsum(float partial) { return rd.template run<false>(partial, THREADS / 32); }
};

// Generic pick for the holders that walk their elements with each().
template <class Row>
__device__ __forceinline__ bool pick_by_each(const Row& r, int c, float& w) {
    bool mine = false;
    r.each([&](int64_t j, float x) {
        if (static_cast<int>(j) == c) { w = x; mine = true; }
    });
    return mine;
}

struct SmemRow {
    static constexpr bool kCached = true;
    static constexpr bool kRawRow = false;
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
    template <class F> __device__ __forceinline__ void each2(const float* __restrict__ aux, F f) const {
        each([&](int64_t j, float w) { f(j, w, __ldg(aux + j)); });
    }
    template <class F> __device__ __forceinline__ void store2(float* __restrict__ out, const float* __restrict__ aux, F f) const {
        store(out, [&](int64_t j, float w) { return f(j, w, __ldcs(aux + j)); });
    }
    __device__ __forceinline__ bool pick(int c, float& w) const { return pick_by_each(*this, c, w); }
    __device__ __forceinline__ float rmax() const {
        float m = -INFINITY;
        for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) m = fmaxf(m, buf[j]);
        return block_max(m, red_f);
    }
    __device__ __forceinline__ float rsum(float partial) const { return static_cast<float>(block_sum(static_cast<double>(partial), red_d)); }
};

// Row too long for shared memory: every pass re-reads it (L2 absorbs most of the re-reads).
struct GlobalRow {
    static constexpr bool kCached = false;
    static constexpr bool kRawRow = false;
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
    template <class F> __device__ __forceinline__ void each2(const float* __restrict__ aux, F f) const {
        each([&](int64_t j, float w) { f(j, w, __ldg(aux + j)); });
    }
    template <class F> __device__ __forceinline__ void store2(float* __restrict__ out, const float* __restrict__ aux, F f) const {
        store(out, [&](int64_t j, float w) { return f(j, w, __ldcs(aux + j)); });
    }
    __device__ __forceinline__ bool pick(int c, float& w) const { return pick_by_each(*this, c, w); }
    __device__ __forceinline__ float rmax() const {
        float m = -INFINITY;
        for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) m = fmaxf(m, __ldg(row + j));
        return block_max(m, red_f);
    }
    __device__ __forceinline__ float rsum(float partial) const { return static_cast<float>(block_sum(static_cast<double>(partial), red_d)); }
};

// ---- the row algorithms, written once over a holder --------------------------------------------
// Returns THIS THREAD's share of the row's loss for the CE forms (the caller adds the shares of all
// its threads), 0 otherwise.
// `src` is where the holder loads the row from (global memory, or a staged copy in shared memory).
template <int ALG> __host__ __device__ constexpr bool alg_has_loss() { return ALG == ALG_CE_ONEHOT || ALG == ALG_CE_INDEX || ALG == ALG_CE_FUSED; }
template <int ALG> __host__ __device__ constexpr bool alg_two_operands() { return ALG == ALG_SOFTMAX_BWD || ALG == ALG_CE_ONEHOT || ALG == ALG_CE_BWD; }
template <int ALG> __host__ __device__ constexpr bool alg_has_output() { return ALG != ALG_CE_ONEHOT && ALG != ALG_CE_INDEX; }
template <int ALG> __host__ __device__ constexpr bool alg_has_label() { return ALG == ALG_CE_INDEX || ALG == ALG_CE_FUSED; }

// The row's class label for the index forms, fetched BEFORE the row itself so that its latency
// overlaps the row's; 0 for the other algorithms.
template <int ALG>
__device__ __forceinline__ float row_label(const RowArgs& A, int64_t row) {
    return alg_has_label<ALG>() ? __ldg(A.t + row) : 0.0f;
}

template <int ALG, class Row>
__device__ __forceinline__ float process_loaded(Row& r, const RowArgs& A, int64_t row, float label, bool& poison) {
    const int64_t cols = A.cols;
    const float* xrow = A.x + row * cols;
    float* orow = A.out ? A.out + row * cols : nullptr;
    if (ALG == ALG_SOFTMAX_BWD) {
        // holder caches y; g is read twice (the second time out of L1/L2)
        const float* grow = A.t + row * cols;
        float part = 0.0f;
        r.each2(grow, [&](int64_t, float y, float g) { part += g * y; });
        const float dot = r.rsum(part);
        r.store2(orow, grow, [&](int64_t, float y, float g) { return y * (g - dot); });
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
        r.each2(trow, [&](int64_t, float w, float t) {
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
        r.store2(orow, trow, [&](int64_t, float w, float t) {
            float d = prob(w) - t;
            return d * g;
        });
        return 0.0f;
    }
    // index-label forms
    const int c = static_cast<int>(label);
    const bool ok = (c >= 0 && c < static_cast<int>(cols));
    if (!ok) poison = true;
    if constexpr (ALG == ALG_CE_INDEX && Row::kRawRow) {
        // The forward loss alone, with the row still readable: -log(max(e_c / s, 1e-10)) written as
        // min(log s - (x_c - max), -log 1e-10) -- no division, no search for element c among the
        // registers (the thread-per-row kernel is bound by instruction issue at ten columns).
        const float xc = ok ? r.raw(c) : m;
        return ok ? fminf(logf(s) - (xc - m), -logf(1e-10f)) : 0.0f;
    }
    // The thread that holds element c contributes the row's loss: no dependent global read and no
    // per-row reduction on the critical path.
    // (Select the element first and take ONE logarithm per thread and row: written inside the loop,
    // the logarithm is evaluated for every element once the compiler turns the branch into selects.)
    float wc = 0.0f;
    const bool mine = r.pick(c, wc);
    const float loss = (ok && mine) ? -logf(fmaxf(prob(wc), 1e-10f)) : 0.0f;
    if (ALG == ALG_CE_FUSED) {
        r.store(orow, [&](int64_t j, float w) { return prob(w) - (static_cast<int>(j) == c ? 1.0f : 0.0f); });
    }
    return loss;
}

template <int ALG, class Row>
__device__ __forceinline__ float process_row(Row& r, const RowArgs& A, int64_t row, const float* src, bool& poison) {
    const float label = row_label<ALG>(A, row);
    r.load(src);
    return process_loaded<ALG>(r, A, row, label, poison);
}

// CTAs of `kernel` that are resident on the whole device at once (asked of the runtime once per
// instantiation): the grid of the persistent forms, so that no CTA waits for another to finish.
template <class K>
int64_t resident_ctas(K kernel, int threads, size_t smem) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem) != cudaSuccess || per_sm < 1) per_sm = 1;
    return static_cast<int64_t>(ctk::sm_count()) * per_sm;
}

// ---- short rows (cols <= 16): a thread per row ------------------------------------------------------
// A CTA takes 512 consecutive rows, i.e. one contiguous block of 512 * cols floats: the block is
// copied to shared memory with coalesced 128-bit loads, every thread then owns one row in registers
// (no shuffles, no barriers inside the row), results go back to the shared tile and leave with
// coalesced 128-bit stores.  Where cols is a multiple of 4 (rows 16, 32, 48 or 64 bytes apart would
// put a warp's threads on 2 to 8 banks) a thread walks its row starting at column (row mod cols),
// which spreads the warp over the banks again.
constexpr int kTileThreads = 256;
constexpr int kTileRowsPerThread = 2;  // two rows per thread: twice the bytes in flight per resident thread
constexpr int kTileRows = kTileThreads * kTileRowsPerThread;

template <int MAXC, bool ROT>
struct TileRow {
    static constexpr bool kCached = true;
    static constexpr bool kRawRow = true;   // the row as loaded stays readable (raw()) while the holder works on its registers
    float v[MAXC];
    float* mine;        // this thread's row in the x / out tile
    const float* aux;   // this thread's row in the second operand's tile
    int cols, rot;
    __device__ __forceinline__ int col(int k) const {
        if (!ROT) return k;
        const int j = k + rot;
        return j >= cols ? j - cols : j;
    }
    __device__ __forceinline__ void load(const float*) {
        if constexpr (MAXC == 10 && !ROT) {
            // exactly ten columns (rows 40 bytes apart, 8-byte aligned): five 8-byte reads; a half-warp's
            // sixteen rows land on all 32 banks once
            const float2* p = reinterpret_cast<const float2*>(mine);
#pragma unroll
            for (int k = 0; k < 5; ++k) {
                const float2 t = p[k];
                v[2 * k] = t.x;
                v[2 * k + 1] = t.y;
            }
        } else {
#pragma unroll
            for (int k = 0; k < MAXC; ++k) v[k] = k < cols ? mine[col(k)] : -INFINITY;
        }
    }
    __device__ __forceinline__ float raw(int c) const { return mine[c]; }
    template <class F> __device__ __forceinline__ void each(F f) const {
#pragma unroll
        for (int k = 0; k < MAXC; ++k)
            if (k < cols) f(static_cast<int64_t>(col(k)), v[k]);
    }
    template <class F> __device__ __forceinline__ void update(F f) {
#pragma unroll
        for (int k = 0; k < MAXC; ++k)
            if (k < cols) v[k] = f(static_cast<int64_t>(col(k)), v[k]);
    }
    template <class F> __device__ __forceinline__ void store(float*, F f) const {
#pragma unroll
        for (int k = 0; k < MAXC; ++k)
            if (k < cols) { const int j = col(k); mine[j] = f(static_cast<int64_t>(j), v[k]); }
    }
    template <class F> __device__ __forceinline__ void each2(const float*, F f) const {
#pragma unroll
        for (int k = 0; k < MAXC; ++k)
            if (k < cols) { const int j = col(k); f(static_cast<int64_t>(j), v[k], aux[j]); }
    }
    template <class F> __device__ __forceinline__ void store2(float*, const float*, F f) const {
#pragma unroll
        for (int k = 0; k < MAXC; ++k)
            if (k < cols) { const int j = col(k); mine[j] = f(static_cast<int64_t>(j), v[k], aux[j]); }
    }
    __device__ __forceinline__ float rmax() const {
        float m = -INFINITY;
#pragma unroll
        for (int k = 0; k < MAXC; ++k) m = fmaxf(m, v[k]);
        return m;
    }
    __device__ __forceinline__ float rsum(float partial) const { return partial; }
    __device__ __forceinline__ bool pick(int c, float& w) const {
        // element c sits in register (c - rot) mod cols
        int k = ROT ? c - rot : c;
        if (k < 0) k += cols;
#pragma unroll
        for (int i = 0; i < MAXC; ++i)
            if (i == k) w = v[i];
        return true;
    }
};

// Contiguous n floats global <-> shared, 128-bit where the block starts on a 16-byte boundary.
__device__ __forceinline__ void tile_in(float* __restrict__ dst, const float* __restrict__ src, int n) {
    if ((reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
        const int n4 = n >> 2;
        for (int i = threadIdx.x; i < n4; i += kTileThreads) reinterpret_cast<float4*>(dst)[i] = __ldcs(reinterpret_cast<const float4*>(src) + i);
        for (int i = (n4 << 2) + threadIdx.x; i < n; i += kTileThreads) dst[i] = __ldcs(src + i);
    } else {
        for (int i = threadIdx.x; i < n; i += kTileThreads) dst[i] = __ldcs(src + i);
    }
}
__device__ __forceinline__ void tile_out(float* __restrict__ dst, const float* __restrict__ src, int n) {
    if ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
        const int n4 = n >> 2;
        for (int i = threadIdx.x; i < n4; i += kTileThreads) __stcs(reinterpret_cast<float4*>(dst) + i, reinterpret_cast<const float4*>(src)[i]);
        for (int i = (n4 << 2) + threadIdx.x; i < n; i += kTileThreads) __stcs(dst + i, src[i]);
    } else {
        for (int i = threadIdx.x; i < n; i += kTileThreads) __stcs(dst + i, src[i]);
    }
}

// Bulk store of a finished tile, shared -> global, and the waits that go with it.
__device__ __forceinline__ void tile_store_async(float* dst, uint32_t src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(reinterpret_cast<uint64_t>(dst)), "r"(src), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void tile_stores_done_reading() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tile_stores_done() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// A resident grid walks the tiles.  PIPE: whole tiles move with bulk asynchronous copies through two
// buffers -- tile i+1 is on its way in and tile i-1 on its way out while tile i is worked on -- so a
// handful of resident CTAs keep HBM busy (the kernel needs ~50 registers per thread, which rules out
// hiding latency by occupancy).  That needs 16-byte aligned operands; otherwise, and for the ragged
// last tile, a tile moves with ordinary coalesced loads and stores.
template <int ALG, int MAXC, bool ROT, bool PIPE>
__global__ void __launch_bounds__(kTileThreads) tile_rows_kernel(RowArgs A, ReduceScratch* scratch, float* loss_out) {
    extern __shared__ __align__(128) float tiles[];  // per buffer: [512 * cols] x / out, then [512 * cols] second operand
    __shared__ double red_d[33];
    __shared__ __align__(8) uint64_t full[2];
    __shared__ volatile int gave_up;
    // MAXC = 10 is instantiated for exactly ten columns (the 10-class rows of the MNIST-shaped models):
    // the column count is then a constant, and the per-element "k < cols" tests and row address
    // multiplications fold away -- the kernel was bound by instruction issue, not by HBM, at this width.
    const int cols = (MAXC == 10) ? 10 : static_cast<int>(A.cols);
    constexpr int kOperands = alg_two_operands<ALG>() ? 2 : 1;
    const int buf_floats = kTileRows * cols * kOperands;
    const uint32_t tile_bytes = static_cast<uint32_t>(kTileRows * cols * sizeof(float));
    TileRow<MAXC, ROT> r;
    r.cols = cols;
    r.rot = ROT ? static_cast<int>(threadIdx.x) % cols : 0;
    double acc = 0.0;
    bool poison = false;
    const int64_t full_tiles = A.rows / kTileRows;
    const int64_t all_tiles = (A.rows + kTileRows - 1) / kTileRows;

    auto labels_of = [&](int64_t tile, float (&lab)[kTileRowsPerThread]) {
#pragma unroll
        for (int u = 0; u < kTileRowsPerThread; ++u) {
            const int64_t row = tile * kTileRows + threadIdx.x + u * kTileThreads;
            lab[u] = row < A.rows ? row_label<ALG>(A, row) : 0.0f;
        }
    };
    // the rows of one tile that is in shared memory, in place
    auto work = [&](float* tile_x, int64_t row0, int rows_here, const float (&lab)[kTileRowsPerThread]) {
#pragma unroll
        for (int u = 0; u < kTileRowsPerThread; ++u) {
            const int lr = static_cast<int>(threadIdx.x) + u * kTileThreads;  // rows t and t + 256: same banks per warp
            if (lr < rows_here) {
                r.mine = tile_x + lr * cols;
                r.aux = tile_x + kTileRows * cols + lr * cols;
                r.load(nullptr);
                const float l = process_loaded<ALG>(r, A, row0 + lr, lab[u], poison);
                if (alg_has_loss<ALG>()) acc += static_cast<double>(l);
            }
        }
    };
    // one tile with ordinary loads and stores, through buffer 0
    auto plain_tile = [&](int64_t tile) {
        const int64_t row0 = tile * kTileRows;
        const int rows_here = static_cast<int>(A.rows - row0 < kTileRows ? A.rows - row0 : kTileRows);
        const int n = rows_here * cols;
        float lab[kTileRowsPerThread];
        labels_of(tile, lab);
        tile_in(tiles, A.x + row0 * cols, n);
        if (kOperands == 2) tile_in(tiles + kTileRows * cols, A.t + row0 * cols, n);
        __syncthreads();
        work(tiles, row0, rows_here, lab);
        __syncthreads();
        if (alg_has_output<ALG>()) tile_out(A.out + row0 * cols, tiles, n);
        __syncthreads();
    };

    if (PIPE) {
        auto fetch = [&](int64_t tile, int b) {  // thread 0 only
            const uint32_t bar = smem_addr(&full[b]);
            float* dst = tiles + b * buf_floats;
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(tile_bytes * kOperands) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(smem_addr(dst)), "l"(reinterpret_cast<uint64_t>(A.x + tile * kTileRows * cols)), "r"(tile_bytes), "r"(bar) : "memory");
            if (kOperands == 2)
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(smem_addr(dst + kTileRows * cols)), "l"(reinterpret_cast<uint64_t>(A.t + tile * kTileRows * cols)), "r"(tile_bytes), "r"(bar) : "memory");
        };
        const int64_t first = blockIdx.x;
        if (threadIdx.x == 0) {
            gave_up = 0;
            sbar_init(smem_addr(&full[0]), 1);
            sbar_init(smem_addr(&full[1]), 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            if (first < full_tiles) fetch(first, 0);
        }
        __syncthreads();
        float label[kTileRowsPerThread], next_label[kTileRowsPerThread];
        if (first < full_tiles) labels_of(first, label);
        int it = 0;
        for (int64_t tile = first; tile < full_tiles; tile += gridDim.x, ++it) {
            const int b = it & 1;
            float* tile_x = tiles + b * buf_floats;
            const int64_t next = tile + gridDim.x;
            if (next < full_tiles) {
                // the other buffer is still being read by the store of the previous tile: let that finish
                if (threadIdx.x == 0) { tile_stores_done_reading(); fetch(next, b ^ 1); }
                labels_of(next, next_label);
            }
            const bool landed = sbar_wait(smem_addr(&full[b]), static_cast<uint32_t>(it >> 1) & 1u, &gave_up);
            if (__syncthreads_or(landed ? 0 : 1)) { poison = true; break; }
            work(tile_x, tile * kTileRows, kTileRows, label);
            if (alg_has_output<ALG>()) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // results visible to the bulk store
            __syncthreads();
            if (alg_has_output<ALG>() && threadIdx.x == 0) tile_store_async(A.out + tile * kTileRows * cols, smem_addr(tile_x), tile_bytes);
#pragma unroll
            for (int u = 0; u < kTileRowsPerThread; ++u) label[u] = next_label[u];
        }
        if (threadIdx.x == 0) tile_stores_done_reading();
        __syncthreads();
        // the ragged last tile: one CTA, ordinary loads and stores
        if (all_tiles > full_tiles && static_cast<int64_t>(blockIdx.x) == full_tiles % gridDim.x && !poison) plain_tile(full_tiles);
        if (threadIdx.x == 0) tile_stores_done();
    } else {
        for (int64_t tile = blockIdx.x; tile < all_tiles; tile += gridDim.x) plain_tile(tile);
    }
    if (alg_has_loss<ALG>()) {
        if (poison && A.bad) *A.bad = 1;
        int any_poison = __syncthreads_or(poison ? 1 : 0);
        double total = block_sum(acc, red_d);
        grid_finish(any_poison ? NAN : total, scratch, loss_out, 0.0f, false, red_d);
    }
}

template <int ALG, int MAXC, bool ROT, bool PIPE>
ctk_status launch_tile_form(const RowArgs& A, ReduceScratch* s, float* loss_out, cudaStream_t st) {
    auto k = tile_rows_kernel<ALG, MAXC, ROT, PIPE>;
    constexpr int kOperands = alg_two_operands<ALG>() ? 2 : 1;
    const size_t smem = static_cast<size_t>(kTileRows) * A.cols * sizeof(float) * kOperands * (PIPE ? 2 : 1);
    static ctk::PerDeviceOnce attr;  // up to 128 KiB (two operands, two buffers, 16 columns): above the default limit
    if (attr.first())
        CTK_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, kTileRows * MAXC * kOperands * (PIPE ? 2 : 1) * static_cast<int>(sizeof(float))));
    int64_t grid = (A.rows + kTileRows - 1) / kTileRows;
    static int64_t resident[MAXC + 1] = {0};  // by column count (it sets the shared-memory need)
    if (!resident[A.cols]) resident[A.cols] = resident_ctas(k, kTileThreads, smem);
    if (grid > resident[A.cols]) grid = resident[A.cols];
    if (alg_has_loss<ALG>() && grid > kMaxReduceBlocks) grid = kMaxReduceBlocks;
    k<<<static_cast<unsigned>(grid), kTileThreads, smem, st>>>(A, s, loss_out);
    return CTK_OK;
}

template <int ALG, int MAXC>
ctk_status launch_tile(const RowArgs& A, ReduceScratch* s, float* loss_out, cudaStream_t st) {
    const bool aligned = ((reinterpret_cast<uintptr_t>(A.x) & 15u) == 0) && (!alg_has_output<ALG>() || (reinterpret_cast<uintptr_t>(A.out) & 15u) == 0) &&
                         (!alg_two_operands<ALG>() || (reinterpret_cast<uintptr_t>(A.t) & 15u) == 0);
    const bool rot = A.cols % 4 == 0;
    if (aligned) return rot ? launch_tile_form<ALG, MAXC, true, true>(A, s, loss_out, st) : launch_tile_form<ALG, MAXC, false, true>(A, s, loss_out, st);
    return rot ? launch_tile_form<ALG, MAXC, true, false>(A, s, loss_out, st) : launch_tile_form<ALG, MAXC, false, false>(A, s, loss_out, st);
}

// ---- rows up to 1024 columns: a warp per row ---------------------------------------------------------
// Each warp of a 128-thread CTA walks its own rows: the row sits in the warp's registers (up to 32
// values per lane, 128-bit loads when the rows are aligned), max and sum are five shuffles each, and
// nothing in the row's life touches shared memory or a barrier.  Rows of different warps overlap
// freely, so HBM latency is hidden by the ~32 rows in flight per SM.
constexpr int kWarpRowThreads = 128;

template <int ALG, int ITEMS, bool VEC>
__global__ void __launch_bounds__(kWarpRowThreads) warp_rows_kernel(RowArgs A, ReduceScratch* scratch, float* loss_out) {
    __shared__ double red_d[33];
    WarpRow<ITEMS, VEC> r;
    r.cols = static_cast<int>(A.cols);
    r.t = threadIdx.x & 31;
    constexpr int kWarps = kWarpRowThreads / 32;
    const int64_t first = static_cast<int64_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
    const int64_t step = static_cast<int64_t>(gridDim.x) * kWarps;
    double acc = 0.0;
    bool poison = false;
    if constexpr (!alg_has_loss<ALG>()) {
        // one row per warp (the launcher sizes the grid so); the other resident warps hide its latency
        for (int64_t row = first; row < A.rows; row += step) process_row<ALG>(r, A, row, A.x + row * A.cols, poison);
    } else {
        // Resident grid: a warp walks many rows, and the loads of its next TWO rows are in flight while
        // the current one is worked on, so the few warps that fit (the three register sets cost
        // occupancy) still keep ~8 KB each on their way from HBM.
        WarpRow<ITEMS, VEC> n1, n2;
        n1.cols = n2.cols = r.cols;
        n1.t = n2.t = r.t;
        float label = 0.0f, label1 = 0.0f, label2 = 0.0f;
        if (first < A.rows) { label = row_label<ALG>(A, first); r.load(A.x + first * A.cols); }
        if (first + step < A.rows) { label1 = row_label<ALG>(A, first + step); n1.load(A.x + (first + step) * A.cols); }
        for (int64_t row = first; row < A.rows; row += step) {
            const int64_t row2 = row + 2 * step;
            if (row2 < A.rows) {
                label2 = row_label<ALG>(A, row2);
                n2.load(A.x + row2 * A.cols);
            }
            const float l = process_loaded<ALG>(r, A, row, label, poison);
            acc += static_cast<double>(l);
#pragma unroll
            for (int it = 0; it < ITEMS; ++it) { r.v[it] = n1.v[it]; n1.v[it] = n2.v[it]; }
            label = label1;
            label1 = label2;
        }
        if (poison && A.bad) *A.bad = 1;
        int any_poison = __syncthreads_or(poison ? 1 : 0);
        double total = block_sum(acc, red_d);
        // A poisoned CTA contributes NaN so the final value is NaN whichever CTA finishes last.
        grid_finish(any_poison ? NAN : total, scratch, loss_out, 0.0f, false, red_d);
    }
}

// 16-byte alignment of every row of every operand the vector forms touch.
template <int ALG>
bool rows_aligned(const RowArgs& A) {
    return (A.cols % 4 == 0) && ((reinterpret_cast<uintptr_t>(A.x) & 15u) == 0) && (!A.out || (reinterpret_cast<uintptr_t>(A.out) & 15u) == 0) &&
           (!alg_two_operands<ALG>() || (reinterpret_cast<uintptr_t>(A.t) & 15u) == 0);
}

template <int ALG, int ITEMS, bool VEC>
void launch_warp_form(const RowArgs& A, ReduceScratch* s, float* loss_out, cudaStream_t st) {
    constexpr int kWarps = kWarpRowThreads / 32;
    auto k = warp_rows_kernel<ALG, ITEMS, VEC>;
    int64_t grid = (A.rows + kWarps - 1) / kWarps;
    if (alg_has_loss<ALG>()) {
        static const int64_t resident = resident_ctas(k, kWarpRowThreads, 0);
        if (grid > resident) grid = resident;
        if (grid > kMaxReduceBlocks) grid = kMaxReduceBlocks;
    }
    if (grid > 0x7fffffff) grid = 0x7fffffff;
    k<<<static_cast<unsigned>(grid), kWarpRowThreads, 0, st>>>(A, s, loss_out);
}

template <int ALG, int ITEMS>
void launch_warp(const RowArgs& A, ReduceScratch* s, float* loss_out, cudaStream_t st) {
    if constexpr (ITEMS % 4 == 0) {
        if (rows_aligned<ALG>(A)) {
            launch_warp_form<ALG, ITEMS, true>(A, s, loss_out, st);
            return;
        }
    }
    launch_warp_form<ALG, ITEMS, false>(A, s, loss_out, st);
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

// A CTA per row, row in registers, many CTAs per SM (the other resident CTAs hide each one's latency).
// Forms without a loss launch one CTA per row and let the hardware scheduler walk the rows; forms
// with a loss run a resident grid that strides over the rows, so the per-CTA finish of the loss
// (fp64 block sum + ticket) is paid once per ~30 rows rather than once per row.
template <int ALG, int THREADS, int ITEMS, bool VEC>
__global__ void __launch_bounds__(THREADS) cta_reg_rows_kernel(RowArgs A, ReduceScratch* scratch, float* loss_out) {
    __shared__ double red_d[33];
    __shared__ float red_f[64];
    CtaRow<THREADS, ITEMS, VEC> r;
    r.cols = static_cast<int>(A.cols);
    r.t = threadIdx.x;
    r.rd = CtaReducer{red_f, 0, false};
    double acc = 0.0;
    bool poison = false;
    for (int64_t row = blockIdx.x; row < A.rows; row += gridDim.x) {
        const float l = process_row<ALG>(r, A, row, A.x + row * A.cols, poison);
        if (alg_has_loss<ALG>()) acc += static_cast<double>(l);
    }
    if (alg_has_loss<ALG>()) {
        if (poison && A.bad && threadIdx.x == 0) *A.bad = 1;
        int any_poison = __syncthreads_or(poison ? 1 : 0);
        double total = block_sum(acc, red_d);
        grid_finish(any_poison ? NAN : total, scratch, loss_out, 0.0f, false, red_d);
    }
}

template <int ALG, int THREADS, int ITEMS, bool VEC>
void launch_cta_reg_form(const RowArgs& A, ReduceScratch* s, float* loss_out, cudaStream_t st) {
    auto k = cta_reg_rows_kernel<ALG, THREADS, ITEMS, VEC>;
    int64_t grid = A.rows;
    if (alg_has_loss<ALG>()) {
        static const int64_t resident = resident_ctas(k, THREADS, 0);
        if (grid > resident) grid = resident;
        if (grid > kMaxReduceBlocks) grid = kMaxReduceBlocks;
    }
    if (grid > 0x7fffffff) grid = 0x7fffffff;
    k<<<static_cast<unsigned>(grid), THREADS, 0, st>>>(A, s, loss_out);
}

template <int ALG, int THREADS, int ITEMS>
ctk_status launch_cta_reg(const RowArgs& A, ReduceScratch* s, float* loss_out, cudaStream_t st) {
    if (rows_aligned<ALG>(A)) launch_cta_reg_form<ALG, THREADS, ITEMS, true>(A, s, loss_out, st);
    else launch_cta_reg_form<ALG, THREADS, ITEMS, false>(A, s, loss_out, st);
    return CTK_OK;
}

// ---- streamed rows: long rows through a ring of bulk asynchronous copies ---------------------------
// One CTA per SM.  A producer warp walks this CTA's rows and copies them, 16 KiB at a time
// (cp.async.bulk, completion on an mbarrier), into a ring of 13 slots of shared memory; 512 consumer
// threads take each chunk as it lands (thread t owns vectors t and t + 512 of every chunk).  The
// row itself goes straight into registers, so its slots are free again at once and the producer runs
// up to 208 KiB -- more than a row -- ahead, across row boundaries: the reads of the following rows
// overlap the arithmetic and the stores of the current one without any occupancy to lean on.
// A second operand row (one-hot targets; the upstream gradient of the softmax backward, which is
// needed twice and streamed twice, the second time out of L2) flows through the same ring and is
// used from shared memory in place.
// Every wait is bounded; a wait that runs out raises a CTA-wide flag, the roles leave their loops,
// the producer lets its copies land, and the loss (or a flag word) reports the failure.
constexpr int kChunkBytes = 16384;
constexpr int kChunkFloats = kChunkBytes / 4;
constexpr int kRingSlots = 13;
constexpr int kStreamThreads = kConsumers + 32;
// How many operand rows per row of the problem pass through the ring, and from where.
template <int ALG> __host__ __device__ constexpr int alg_streams() {
    return ALG == ALG_SOFTMAX_BWD ? 3 : (ALG == ALG_CE_ONEHOT || ALG == ALG_CE_BWD) ? 2 : 1;
}

// Consumer side of the ring: hands out, chunk after chunk, the two 128-bit vectors this thread owns
// (vectors t and t + 512 of the chunk's 1024).
struct RingReader {
    uint32_t ring, full0, empty0;
    int slot;
    uint32_t phase;
    volatile int* gave_up;
    // Waits (bounded) for the next chunk, reads this thread's vectors as far as the chunk reaches
    // (`fill` beyond, and when the wait ran out), and hands the slot back to the producer.
    __device__ __forceinline__ void next(uint32_t chunk_bytes, float fill, float4& a, float4& b) {
        a = make_float4(fill, fill, fill, fill);
        b = a;
        const uint32_t bar = full0 + 8u * slot;
        bool ok = sbar_try(bar, phase);
        if (!ok) ok = sbar_wait(bar, phase, gave_up);
        const uint32_t off = 16u * threadIdx.x;
        const uint32_t src = ring + slot * kChunkBytes + off;
        if (ok && off < chunk_bytes)
            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(a.x), "=f"(a.y), "=f"(a.z), "=f"(a.w) : "r"(src) : "memory");
        if (ok && off + kChunkBytes / 2 < chunk_bytes)
            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(b.x), "=f"(b.y), "=f"(b.z), "=f"(b.w) : "r"(src + kChunkBytes / 2) : "memory");
        __syncwarp();
        if ((threadIdx.x & 31) == 0) sbar_arrive(empty0 + 8u * slot);
        if (++slot == kRingSlots) { slot = 0; phase ^= 1u; }
    }
};

// The row holder of the streamed kernel: the register layout of a 512-thread CTA row, filled from
// the ring, reductions over the consumer threads only, second operand from the ring.
template <int ITEMS>
struct StreamRow : StridedRow<kConsumers, ITEMS, true> {
    static_assert(ITEMS % 8 == 0, "a chunk carries two vectors per thread");
    static constexpr int kChunks = ITEMS / 8;
    RingReader* ring;
    CtaReducer rd;
    uint32_t row_bytes;
    __device__ __forceinline__ uint32_t chunk_bytes(int c) const {
        const uint32_t start = static_cast<uint32_t>(c) * kChunkBytes;
        return start >= row_bytes ? 0u : (row_bytes - start < static_cast<uint32_t>(kChunkBytes) ? row_bytes - start : kChunkBytes);
    }
    __device__ __forceinline__ void load_from_ring(float fill) {
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
            float4 a = make_float4(fill, fill, fill, fill), b = a;
            const uint32_t cb = chunk_bytes(c);
            if (cb) ring->next(cb, fill, a, b);
            float* w = this->v + 8 * c;
            w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
        }
    }
    __device__ __forceinline__ float rmax() { return rd.template run<true>(this->local_max(), kConsumers / 32); }
    __device__ __forceinline__ float rsum(float partial) { return rd.template run<false>(partial, kConsumers / 32); }
    // Index-label CrossEntropy forward needs only max, sum of exponentials and the labelled logit:
    // they are folded chunk by chunk as the chunks land (a running maximum, the running sum rescaled
    // when the maximum moves), nothing is kept, every slot goes back to the producer at once and the
    // copies never pause for a whole row's arithmetic.  Returns this thread's share of the loss.
    __device__ __forceinline__ float online_ce(int c, bool& poison) {
        const bool ok = c >= 0 && c < this->cols;
        if (!ok) poison = true;
        float m = -INFINITY, ssum = 0.0f, xc = 0.0f;
        bool mine = false;
#pragma unroll
        for (int ch = 0; ch < kChunks; ++ch) {
            const uint32_t cb = chunk_bytes(ch);
            if (cb) {
                float4 a, b;
                ring->next(cb, -INFINITY, a, b);
                const float cm = fmaxf(fmaxf(fmaxf(a.x, a.y), fmaxf(a.z, a.w)), fmaxf(fmaxf(b.x, b.y), fmaxf(b.z, b.w)));
                const float mn = fmaxf(m, cm);
                if (mn > -INFINITY) {
                    const float part = ((fast_exp(a.x - mn) + fast_exp(a.y - mn)) + (fast_exp(a.z - mn) + fast_exp(a.w - mn))) +
                                       ((fast_exp(b.x - mn) + fast_exp(b.y - mn)) + (fast_exp(b.z - mn) + fast_exp(b.w - mn)));
                    ssum = ssum * fast_exp(m - mn) + part;
                    m = mn;
                }
                const int k = c & 3, j0 = this->first(2 * ch), j1 = this->first(2 * ch + 1);
                if (j0 == (c & ~3)) { xc = k == 0 ? a.x : k == 1 ? a.y : k == 2 ? a.z : a.w; mine = true; }
                if (j1 == (c & ~3)) { xc = k == 0 ? b.x : k == 1 ? b.y : k == 2 ? b.z : b.w; mine = true; }
            }
        }
        const float row_max = rd.template run<true>(m, kConsumers / 32);
        const float s = rd.template run<false>(m > -INFINITY ? ssum * fast_exp(m - row_max) : 0.0f, kConsumers / 32);
        return (ok && mine) ? -logf(fmaxf(fast_exp(xc - row_max) * (1.0f / s), 1e-10f)) : 0.0f;
    }
    template <class F> __device__ __forceinline__ void each2(const float*, F f) {
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
            const uint32_t cb = chunk_bytes(c);
            if (cb) {
                float4 a, b;
                ring->next(cb, 0.0f, a, b);
                const float* w = this->v + 8 * c;
                const int j0 = this->first(2 * c), j1 = this->first(2 * c + 1);
                if (j0 < this->cols) { f(j0, w[0], a.x); f(j0 + 1, w[1], a.y); f(j0 + 2, w[2], a.z); f(j0 + 3, w[3], a.w); }
                if (j1 < this->cols) { f(j1, w[4], b.x); f(j1 + 1, w[5], b.y); f(j1 + 2, w[6], b.z); f(j1 + 3, w[7], b.w); }
            }
        }
    }
    template <class F> __device__ __forceinline__ void store2(float* __restrict__ out, const float*, F f) {
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
            const uint32_t cb = chunk_bytes(c);
            if (cb) {
                float4 a, b;
                ring->next(cb, 0.0f, a, b);
                const float* w = this->v + 8 * c;
                const int j0 = this->first(2 * c), j1 = this->first(2 * c + 1);
                if (j0 < this->cols) __stcs(reinterpret_cast<float4*>(out + j0), make_float4(f(j0, w[0], a.x), f(j0 + 1, w[1], a.y), f(j0 + 2, w[2], a.z), f(j0 + 3, w[3], a.w)));
                if (j1 < this->cols) __stcs(reinterpret_cast<float4*>(out + j1), make_float4(f(j1, w[4], b.x), f(j1 + 1, w[5], b.y), f(j1 + 2, w[6], b.z), f(j1 + 3, w[7], b.w)));
            }
        }
    }
};

template <int ALG, int ITEMS>
__global__ void __launch_bounds__(kStreamThreads, 1) streamed_rows_kernel(RowArgs A, ReduceScratch* scratch, float* loss_out) {
    extern __shared__ __align__(128) uint8_t ring_raw[];
    __shared__ __align__(8) uint64_t bars[2 * kRingSlots];
    __shared__ double red_d[33];
    __shared__ float red_f[64];
    __shared__ volatile int gave_up;
    const uint32_t ring = smem_addr(ring_raw), full0 = smem_addr(bars), empty0 = full0 + 8u * kRingSlots;
    const int tid = threadIdx.x;
    if (tid == 0) {
        gave_up = 0;
        for (int s = 0; s < kRingSlots; ++s) { sbar_init(full0 + 8u * s, 1); sbar_init(empty0 + 8u * s, kConsumers / 32); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const uint32_t row_bytes = static_cast<uint32_t>(A.cols * sizeof(float));
    const int nch = static_cast<int>((row_bytes + kChunkBytes - 1) / kChunkBytes);
    double acc = 0.0;
    bool poison = false;

    if (tid >= kConsumers) {
        // ------------------------------ producer ------------------------------
        if (tid == kConsumers) {
            int slot = 0;
            uint32_t phase = 0, issued = 0;
            bool ok = true;
            for (int64_t row = blockIdx.x; row < A.rows && ok; row += gridDim.x) {
                for (int s = 0; s < alg_streams<ALG>() && ok; ++s) {
                    const float* src = (s == 0 ? A.x : A.t) + row * A.cols;
                    for (int c = 0; c < nch; ++c) {
                        if (!sbar_wait(empty0 + 8u * slot, phase ^ 1u, &gave_up)) { ok = false; break; }
                        // (the consumers' reads of this slot are ordered before the copy by their arrival on
                        // the empty barrier and this wait: release / acquire)
                        const uint32_t left = row_bytes - static_cast<uint32_t>(c) * kChunkBytes;
                        chunk_fetch(ring + slot * kChunkBytes, src + static_cast<int64_t>(c) * kChunkFloats, left < static_cast<uint32_t>(kChunkBytes) ? left : kChunkBytes,
                                    full0 + 8u * slot);
                        ++issued;
                        if (++slot == kRingSlots) { slot = 0; phase ^= 1u; }
                    }
                }
            }
            if (!ok) {
                // let the copies still in flight land before this CTA's shared memory is given up
                const uint32_t pending = issued < static_cast<uint32_t>(kRingSlots) ? issued : kRingSlots;
                int s = slot;
                uint32_t ph = phase;
                for (uint32_t i = 0; i < pending; ++i) {
                    if (--s < 0) { s = kRingSlots - 1; ph ^= 1u; }
                    for (uint32_t spin = 0; spin < (1u << 16) && !sbar_try(full0 + 8u * s, ph); ++spin) __nanosleep(64);
                }
            }
        }
    } else {
        // ------------------------------ consumers ------------------------------
        RingReader reader{ring, full0, empty0, 0, 0u, &gave_up};
        StreamRow<ITEMS> r;
        r.cols = static_cast<int>(A.cols);
        r.t = tid;
        r.ring = &reader;
        r.rd = CtaReducer{red_f, 0, true};
        r.row_bytes = row_bytes;
        for (int64_t row = blockIdx.x; row < A.rows; row += gridDim.x) {
            const float label = row_label<ALG>(A, row);
            float l;
            if constexpr (ALG == ALG_CE_INDEX) {
                l = r.online_ce(static_cast<int>(label), poison);
            } else {
                r.load_from_ring(ALG == ALG_SOFTMAX_BWD ? 0.0f : -INFINITY);
                l = process_loaded<ALG>(r, A, row, label, poison);
            }
            if (alg_has_loss<ALG>()) acc += static_cast<double>(l);
            // leave together: the OR over all consumers of "a wait ran out" is taken at a barrier
            uint32_t any;
            asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.or.pred p, 1, %2, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(any) : "r"(static_cast<uint32_t>(gave_up)), "n"(kConsumers) : "memory");
            if (any) { poison = true; break; }
        }
    }
    __syncthreads();
    if (alg_has_loss<ALG>()) {
        if (poison && A.bad && tid == 0) *A.bad = 1;
        int any_poison = __syncthreads_or(poison ? 1 : 0);
        double total = block_sum(acc, red_d);
        grid_finish(any_poison ? NAN : total, scratch, loss_out, 0.0f, false, red_d);
    }
}

template <int ALG, int ITEMS>
ctk_status launch_streamed(const RowArgs& A, ReduceScratch* s, float* loss_out, cudaStream_t st) {
    auto k = streamed_rows_kernel<ALG, ITEMS>;
    constexpr int smem = kRingSlots * kChunkBytes;
    static ctk::PerDeviceOnce attr;  // raises the opt-in shared-memory limit once per device, per instantiation
    if (attr.first()) CTK_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    const int64_t sms = ctk::sm_count();
    const int64_t grid = A.rows < sms ? A.rows : sms;
    k<<<static_cast<unsigned>(grid), kStreamThreads, smem, st>>>(A, s, loss_out);
    return CTK_OK;
}

// ---- softmax down the columns of a row-major [rows, cols] matrix (dim 0) -----------------------------
// Tensor::softmax(0) of the reference (src/Tensor.cpp:1728-1743) and its backward rule
// (src/AutoDiff.cpp:1473-1484).  A CTA of 32 x 32 threads owns a strip of 32 columns: a warp reads one
// 128-byte row segment at a time, every thread keeps a running maximum and a rescaled running sum for
// its column over the rows it visits (one pass), the 32 row-lanes of a column are merged through
// shared memory, and a second pass writes exp(x - max) / sum.  12 bytes per element instead of the 8 of
// a kernel that could keep its strip on chip: this form is not on any benchmark path.
constexpr int kColTile = 32;

constexpr int kColDepth = 8;   // independent row loads a thread keeps in flight

__global__ void __launch_bounds__(kColTile * kColTile) softmax_cols_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t rows, int64_t cols) {
    __shared__ float sm_m[kColTile][kColTile + 1], sm_s[kColTile][kColTile + 1];
    const int tx = threadIdx.x, ty = threadIdx.y;
    const int64_t col = static_cast<int64_t>(blockIdx.x) * kColTile + tx;
    const int64_t step = static_cast<int64_t>(kColTile) * cols;
    float m = -INFINITY, sum = 0.0f;
    if (col < cols) {
        int64_t r = ty;
        const float* p = x + r * cols + col;
        for (; r + (kColDepth - 1) * kColTile < rows; r += kColDepth * kColTile, p += kColDepth * step) {
            float v[kColDepth];
#pragma unroll
            for (int u = 0; u < kColDepth; ++u) v[u] = __ldg(p + u * step);
            float mn = m;
#pragma unroll
            for (int u = 0; u < kColDepth; ++u) mn = fmaxf(mn, v[u]);
            if (mn > -INFINITY) {
                float part = 0.0f;
#pragma unroll
                for (int u = 0; u < kColDepth; ++u) part += fast_exp(v[u] - mn);
                sum = sum * fast_exp(m - mn) + part;
                m = mn;
            }
        }
        for (; r < rows; r += kColTile, p += step) {
            const float v = __ldg(p);
            const float mn = fmaxf(m, v);
            if (mn > -INFINITY) {
                sum = sum * fast_exp(m - mn) + fast_exp(v - mn);
                m = mn;
            }
        }
    }
    sm_m[ty][tx] = m;
    sm_s[ty][tx] = sum;
    __syncthreads();
    float cm = -INFINITY;
#pragma unroll 8
    for (int i = 0; i < kColTile; ++i) cm = fmaxf(cm, sm_m[i][tx]);
    float cs = 0.0f;
#pragma unroll 8
    for (int i = 0; i < kColTile; ++i) cs += sm_m[i][tx] > -INFINITY ? sm_s[i][tx] * fast_exp(sm_m[i][tx] - cm) : 0.0f;
    const float inv = 1.0f / cs;
    if (col < cols) {
        int64_t r = ty;
        const float* p = x + r * cols + col;
        float* q = y + r * cols + col;
        for (; r + (kColDepth - 1) * kColTile < rows; r += kColDepth * kColTile, p += kColDepth * step, q += kColDepth * step) {
            float v[kColDepth];
#pragma unroll
            for (int u = 0; u < kColDepth; ++u) v[u] = __ldg(p + u * step);
#pragma unroll
            for (int u = 0; u < kColDepth; ++u) q[u * step] = fast_exp(v[u] - cm) * inv;
        }
        for (; r < rows; r += kColTile, p += step, q += step) *q = fast_exp(__ldg(p) - cm) * inv;
    }
}

__global__ void __launch_bounds__(kColTile * kColTile) softmax_cols_backward_kernel(const float* __restrict__ y, const float* __restrict__ g, float* __restrict__ dx, int64_t rows, int64_t cols) {
    __shared__ float sm_d[kColTile][kColTile + 1];
    const int tx = threadIdx.x, ty = threadIdx.y;
    const int64_t col = static_cast<int64_t>(blockIdx.x) * kColTile + tx;
    const int64_t step = static_cast<int64_t>(kColTile) * cols;
    constexpr int D = kColDepth / 2;   // two arrays per row
    float dot = 0.0f;
    if (col < cols) {
        int64_t r = ty;
        int64_t i = r * cols + col;
        for (; r + (D - 1) * kColTile < rows; r += D * kColTile, i += D * step) {
            float a[D], b[D];
#pragma unroll
            for (int u = 0; u < D; ++u) {
                a[u] = __ldg(g + i + u * step);
                b[u] = __ldg(y + i + u * step);
            }
#pragma unroll
            for (int u = 0; u < D; ++u) dot += a[u] * b[u];
        }
        for (; r < rows; r += kColTile, i += step) dot += __ldg(g + i) * __ldg(y + i);
    }
    sm_d[ty][tx] = dot;
    __syncthreads();
    float cd = 0.0f;
#pragma unroll 8
    for (int i = 0; i < kColTile; ++i) cd += sm_d[i][tx];
    if (col < cols) {
        int64_t r = ty;
        int64_t i = r * cols + col;
        for (; r + (D - 1) * kColTile < rows; r += D * kColTile, i += D * step) {
            float a[D], b[D];
#pragma unroll
            for (int u = 0; u < D; ++u) {
                a[u] = __ldg(g + i + u * step);
                b[u] = __ldg(y + i + u * step);
            }
#pragma unroll
            for (int u = 0; u < D; ++u) dx[i + u * step] = b[u] * (a[u] - cd);
        }
        for (; r < rows; r += kColTile, i += step) dx[i] = __ldg(y + i) * (__ldg(g + i) - cd);
    }
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
    // the streamed kernel moves rows with 16-byte bulk copies and 128-bit stores
    const bool aligned_rows = (c % 4 == 0) && ((reinterpret_cast<uintptr_t>(A.x) & 15u) == 0) && (!A.out || (reinterpret_cast<uintptr_t>(A.out) & 15u) == 0) &&
                              (alg_streams<ALG>() == 1 || (reinterpret_cast<uintptr_t>(A.t) & 15u) == 0);
    ctk_status rc = CTK_OK;
    if (c <= 8) rc = launch_tile<ALG, 8>(A, s, loss_out, st);
    else if (c == 10) rc = launch_tile<ALG, 10>(A, s, loss_out, st);
    else if (c <= 12) rc = launch_tile<ALG, 12>(A, s, loss_out, st);
    else if (c <= 16) rc = launch_tile<ALG, 16>(A, s, loss_out, st);
    else if (c <= 32) launch_warp<ALG, 1>(A, s, loss_out, st);
    else if (c <= 64) launch_warp<ALG, 2>(A, s, loss_out, st);
    else if (c <= 128) launch_warp<ALG, 4>(A, s, loss_out, st);
    else if (c <= 256) launch_warp<ALG, 8>(A, s, loss_out, st);
    else if (c <= 512) launch_warp<ALG, 16>(A, s, loss_out, st);
    else if (c <= 1024) launch_warp<ALG, 32>(A, s, loss_out, st);
    else if (c <= 2048) rc = launch_cta_reg<ALG, 128, 16>(A, s, loss_out, st);
    else if (c <= 4096) rc = launch_cta_reg<ALG, 256, 16>(A, s, loss_out, st);
    else if (c <= 8192 && aligned_rows) rc = launch_streamed<ALG, 16>(A, s, loss_out, st);
    else if (c <= 16384 && aligned_rows) rc = launch_streamed<ALG, 32>(A, s, loss_out, st);
    else if (c <= 32768 && aligned_rows) rc = launch_streamed<ALG, 64>(A, s, loss_out, st);
    else {
        int64_t cap = static_cast<int64_t>(ctk::sm_count()) * (c <= 12 * 1024 ? 4 : 1);
        int grid = static_cast<int>(A.rows < cap ? A.rows : cap);
        if (grid > kMaxReduceBlocks) grid = kMaxReduceBlocks;
        if (c <= kSmemRowMaxCols) {
            size_t bytes = static_cast<size_t>(c) * sizeof(float);
            static ctk::PerDeviceOnce attr;  // raises the opt-in limit once per device, per instantiation
            if (attr.first())
                CTK_CUDA(cudaFuncSetAttribute(cta_rows_kernel<ALG, SmemRow>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              kSmemRowMaxCols * static_cast<int>(sizeof(float))));
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

ctk_status ctk_rowwise_status(int* status) {
    CTK_REQUIRE(status, "ctk_rowwise_status: null");
    CTK_CUDA(cudaDeviceSynchronize());
    CTK_CUDA(cudaMemcpyFromSymbol(status, g_row_status, sizeof(int)));
    if (*status != 0) mark_reduce_scratch_dirty();  // a CTA that gave up did not take its ticket
    return CTK_OK;
}

ctk_status ctk_softmax_rows_f32(const float* x, float* y, int64_t rows, int64_t cols, void* stream) {
    CTK_RANGE("ctk_softmax_rows_f32");
    CTK_REQUIRE((x && y) || rows == 0 || cols == 0, "ctk_softmax_rows_f32: null pointer");
    RowArgs A{x, nullptr, y, nullptr, nullptr, rows, cols};
    return launch_rows<ALG_SOFTMAX>("softmax_rows", A, nullptr, nullptr, stream);
}

ctk_status ctk_softmax_cols_f32(const float* x, float* y, int64_t rows, int64_t cols, void* stream) {
    CTK_RANGE("ctk_softmax_cols_f32");
    CTK_REQUIRE(rows >= 0 && cols >= 0, "ctk_softmax_cols_f32: negative shape");
    if (rows == 0 || cols == 0) return CTK_OK;
    CTK_REQUIRE(x && y, "ctk_softmax_cols_f32: null pointer");
    const int64_t grid = (cols + kColTile - 1) / kColTile;
    CTK_REQUIRE(grid <= 0x7fffffff, "ctk_softmax_cols_f32: too many columns");
    softmax_cols_kernel<<<static_cast<unsigned>(grid), dim3(kColTile, kColTile), 0, as_stream(stream)>>>(x, y, rows, cols);
    CTK_LAUNCH_CHECK("softmax_cols_kernel");
    return CTK_OK;
}

ctk_status ctk_softmax_backward_cols_f32(const float* y, const float* g, float* dx, int64_t rows, int64_t cols, void* stream) {
    CTK_RANGE("ctk_softmax_backward_cols_f32");
    CTK_REQUIRE(rows >= 0 && cols >= 0, "ctk_softmax_backward_cols_f32: negative shape");
    if (rows == 0 || cols == 0) return CTK_OK;
    CTK_REQUIRE(y && g && dx, "ctk_softmax_backward_cols_f32: null pointer");
    const int64_t grid = (cols + kColTile - 1) / kColTile;
    CTK_REQUIRE(grid <= 0x7fffffff, "ctk_softmax_backward_cols_f32: too many columns");
    softmax_cols_backward_kernel<<<static_cast<unsigned>(grid), dim3(kColTile, kColTile), 0, as_stream(stream)>>>(y, g, dx, rows, cols);
    CTK_LAUNCH_CHECK("softmax_cols_backward_kernel");
    return CTK_OK;
}

ctk_status ctk_softmax_backward_rows_f32(const float* y, const float* g, float* dx, int64_t rows, int64_t cols, void* stream) {
    CTK_RANGE("ctk_softmax_backward_rows_f32");
    CTK_REQUIRE((y && g && dx) || rows == 0 || cols == 0, "ctk_softmax_backward_rows_f32: null pointer");
    RowArgs A{y, g, dx, nullptr, nullptr, rows, cols};
    return launch_rows<ALG_SOFTMAX_BWD>("softmax_backward_rows", A, nullptr, nullptr, stream);
}

ctk_status ctk_ce_onehot_f32(const float* logits, const float* onehot, int64_t rows, int64_t cols, float* out,
                             void* scratch, void* stream) {
    CTK_RANGE("ctk_ce_onehot_f32");
    CTK_REQUIRE((logits && onehot) || rows == 0 || cols == 0, "ctk_ce_onehot_f32: null pointer");
    RowArgs A{logits, onehot, nullptr, nullptr, nullptr, rows, cols};
    return launch_rows<ALG_CE_ONEHOT>("ce_onehot", A, out, scratch, stream);
}

ctk_status ctk_ce_index_f32(const float* logits, const float* labels, int64_t rows, int64_t cols, float* out,
                            int* bad_label_flag, void* scratch, void* stream) {
    CTK_RANGE("ctk_ce_index_f32");
    CTK_REQUIRE((logits && labels) || rows == 0 || cols == 0, "ctk_ce_index_f32: null pointer");
    RowArgs A{logits, labels, nullptr, nullptr, bad_label_flag, rows, cols};
    return launch_rows<ALG_CE_INDEX>("ce_index", A, out, scratch, stream);
}

ctk_status ctk_ce_backward_f32(const float* logits, const float* onehot, const float* g_device, float* dlogits,
                               int64_t rows, int64_t cols, void* stream) {
    CTK_RANGE("ctk_ce_backward_f32");
    CTK_REQUIRE((logits && onehot && dlogits) || rows == 0 || cols == 0, "ctk_ce_backward_f32: null pointer");
    RowArgs A{logits, onehot, dlogits, g_device, nullptr, rows, cols};
    return launch_rows<ALG_CE_BWD>("ce_backward", A, nullptr, nullptr, stream);
}

ctk_status ctk_ce_fused_index_f32(const float* logits, const float* labels, int64_t rows, int64_t cols, float* out,
                                  float* dlogits, int* bad_label_flag, void* scratch, void* stream) {
    CTK_RANGE("ctk_ce_fused_index_f32");
    CTK_REQUIRE((logits && labels && dlogits) || rows == 0 || cols == 0, "ctk_ce_fused_index_f32: null pointer");
    RowArgs A{logits, labels, dlogits, nullptr, bad_label_flag, rows, cols};
    return launch_rows<ALG_CE_FUSED>("ce_fused_index", A, out, scratch, stream);
}

}  // extern "C"
