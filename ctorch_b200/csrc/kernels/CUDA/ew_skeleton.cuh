// Skeleton shared by every HBM-bound elementwise kernel of the library.
//
// Each CTA owns ONE contiguous tile of kEwThreads x kEwUnroll 128-bit vectors per array (16 KiB per
// array) and does it in two phases: issue all of the tile's loads, then compute and store.  The
// grid is simply ceil(vectors / tile): on B200 this ran a two-input add at 7.0 TB/s against
// 6.2-6.5 TB/s for the same loop on a persistent grid of 148 x k CTAs striding through memory and
// 4.6 TB/s when loads and stores of one vector were interleaved -- the block scheduler walking
// memory in order keeps DRAM pages open, and the two phases keep every load of a tile in flight at
// once.  Operands that are not 16-byte aligned take the element-wise kernel below.
//
// F is a functor: void operator()(const float* x /*NIN*/, float* y /*NOUT*/) const.
#pragma once
#include "common.cuh"

namespace ctk {

constexpr int kEwThreads = 256;
constexpr int kEwUnroll = 4;
constexpr int kEwTile = kEwThreads * kEwUnroll;  // vectors per CTA

enum { EW_STREAM = 0, EW_SCALAR = 1, EW_ROW = 2 };  // how an input is indexed

template <int NIN, int NOUT>
struct EwArgs {
    const float* in[NIN > 0 ? NIN : 1];
    int mode[NIN > 0 ? NIN : 1];
    float* out[NOUT];
    int64_t out_limit[NOUT];  // elements of out[k] to write (a broadcast operand's gradient is a prefix)
    int64_t n;                // result elements
    int64_t inner;            // period of EW_ROW inputs
};

// MODES packs the indexing mode of input k in bits [2k, 2k+2): a compile-time constant, so a kernel
// carries only the address arithmetic it needs (with run-time modes the compiler kept the 64-bit
// modulo of the row mode on every path, and the one-stream broadcast forms ran at 5.0 TB/s instead
// of 6.9).
template <int NIN, int NOUT, class F, int MODES>
__global__ void __launch_bounds__(kEwThreads) ew_vec_kernel(EwArgs<NIN, NOUT> A, F f) {
    const int64_t n4 = A.n >> 2;
    const int64_t base = static_cast<int64_t>(blockIdx.x) * kEwTile + threadIdx.x;
    float4 v[NIN > 0 ? NIN : 1][kEwUnroll];
    float s[NIN > 0 ? NIN : 1];
    bool any_row = false;
#pragma unroll
    for (int k = 0; k < NIN; ++k) {
        const int mode = (MODES >> (2 * k)) & 3;
        s[k] = (mode == EW_SCALAR) ? __ldg(A.in[k]) : 0.0f;
        any_row |= (mode == EW_ROW);
    }
    // position of this thread's first vector inside the row period (one 64-bit modulo per thread)
    const uint32_t inner32 = static_cast<uint32_t>(A.inner);
    const uint32_t row0 = any_row ? static_cast<uint32_t>((base << 2) % A.inner) : 0u;
    // phase 1: every load of the tile
#pragma unroll
    for (int u = 0; u < kEwUnroll; ++u) {
        const int64_t i4 = base + u * kEwThreads;
        if (i4 < n4) {
#pragma unroll
            for (int k = 0; k < NIN; ++k) {
                const int mode = (MODES >> (2 * k)) & 3;
                if (mode == EW_STREAM) v[k][u] = __ldcs(reinterpret_cast<const float4*>(A.in[k]) + i4);
                else if (mode == EW_ROW) v[k][u] = __ldg(reinterpret_cast<const float4*>(A.in[k] + (row0 + static_cast<uint32_t>(u * kEwThreads * 4)) % inner32));
                else v[k][u] = make_float4(s[k], s[k], s[k], s[k]);
            }
        }
    }
    // phase 2: compute and store
#pragma unroll
    for (int u = 0; u < kEwUnroll; ++u) {
        const int64_t i4 = base + u * kEwThreads;
        if (i4 < n4) {
            float4 r[NOUT];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float x[NIN > 0 ? NIN : 1], y[NOUT];
#pragma unroll
                for (int k = 0; k < NIN; ++k) x[k] = reinterpret_cast<const float*>(&v[k][u])[c];
                f(x, y);
#pragma unroll
                for (int k = 0; k < NOUT; ++k) reinterpret_cast<float*>(&r[k])[c] = y[k];
            }
            const int64_t i = i4 << 2;
#pragma unroll
            for (int k = 0; k < NOUT; ++k) {
                if (!A.out[k]) continue;
                if (i + 3 < A.out_limit[k]) __stcs(reinterpret_cast<float4*>(A.out[k] + i), r[k]);
                else {
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        if (i + c < A.out_limit[k]) A.out[k][i + c] = reinterpret_cast<const float*>(&r[k])[c];
                }
            }
        }
    }
    // the up-to-three elements after the last full vector
    if (blockIdx.x == gridDim.x - 1) {
        const int64_t i = (n4 << 2) + threadIdx.x;
        if (i < A.n) {
            float x[NIN > 0 ? NIN : 1], y[NOUT];
#pragma unroll
            for (int k = 0; k < NIN; ++k) {
                const int mode = (MODES >> (2 * k)) & 3;
                x[k] = (mode == EW_STREAM) ? A.in[k][i] : (mode == EW_ROW) ? __ldg(A.in[k] + (i % A.inner)) : s[k];
            }
            f(x, y);
#pragma unroll
            for (int k = 0; k < NOUT; ++k)
                if (A.out[k] && i < A.out_limit[k]) A.out[k][i] = y[k];
        }
    }
}

template <int NIN, int NOUT, class F>
__global__ void __launch_bounds__(kEwThreads) ew_scalar_kernel(EwArgs<NIN, NOUT> A, F f) {
    float s[NIN > 0 ? NIN : 1];
#pragma unroll
    for (int k = 0; k < NIN; ++k) s[k] = (A.mode[k] == EW_SCALAR) ? __ldg(A.in[k]) : 0.0f;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < A.n; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        float x[NIN > 0 ? NIN : 1], y[NOUT];
#pragma unroll
        for (int k = 0; k < NIN; ++k)
            x[k] = (A.mode[k] == EW_STREAM) ? A.in[k][i] : (A.mode[k] == EW_ROW) ? __ldg(A.in[k] + (i % A.inner)) : s[k];
        f(x, y);
#pragma unroll
        for (int k = 0; k < NOUT; ++k)
            if (A.out[k] && i < A.out_limit[k]) A.out[k][i] = y[k];
    }
}

inline bool ew_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Launches the vector kernel when every streamed pointer is 16-byte aligned (and row periods are a
// multiple of 4), else the element-wise one.
template <int NIN, int NOUT, class F>
ctk_status ew_launch(const char* name, EwArgs<NIN, NOUT> A, F f, cudaStream_t st) {
    if (A.n <= 0) return CTK_OK;
    bool vec = true;
    for (int k = 0; k < NIN; ++k) {
        if (A.mode[k] == EW_STREAM && !ew_aligned16(A.in[k])) vec = false;
        if (A.mode[k] == EW_ROW && (!ew_aligned16(A.in[k]) || A.inner % 4 != 0)) vec = false;
    }
    for (int k = 0; k < NOUT; ++k)
        if (A.out[k] && !ew_aligned16(A.out[k])) vec = false;
    // Instantiated mode patterns: all inputs streamed; the LAST input a broadcast scalar or a row
    // (the second operand of a binary op, the upstream scalar of a loss gradient, the source of a
    // fill / tile); the FIRST input a broadcast scalar (0-D left operand).  Anything else takes the
    // element-wise kernel.
    int packed = 0;
    for (int k = 0; k < NIN; ++k) packed |= (A.mode[k] & 3) << (2 * k);
    constexpr int kLast = NIN > 0 ? 2 * (NIN - 1) : 0;
    constexpr int kLastScalar = NIN > 0 ? (EW_SCALAR << kLast) : -1;
    constexpr int kLastRow = NIN > 0 ? (EW_ROW << kLast) : -2;
    constexpr int kFirstScalar = NIN > 1 ? EW_SCALAR : -3;
    if (vec && A.inner >= (int64_t(1) << 31)) vec = false;
    if (vec && packed != 0 && packed != kLastScalar && packed != kLastRow && packed != kFirstScalar) vec = false;
    if (vec) {
        const int64_t n4 = A.n >> 2;
        int64_t grid = (n4 + kEwTile - 1) / kEwTile;
        if (grid < 1) grid = 1;
        CTK_REQUIRE(grid < (int64_t(1) << 31), "elementwise kernel: too many elements for one launch");
        const unsigned g = static_cast<unsigned>(grid);
        if (packed == 0) ew_vec_kernel<NIN, NOUT, F, 0><<<g, kEwThreads, 0, st>>>(A, f);
        else if (packed == kLastScalar) ew_vec_kernel<NIN, NOUT, F, (NIN > 0 ? (EW_SCALAR << kLast) : 0)><<<g, kEwThreads, 0, st>>>(A, f);
        else if (packed == kLastRow) ew_vec_kernel<NIN, NOUT, F, (NIN > 0 ? (EW_ROW << kLast) : 0)><<<g, kEwThreads, 0, st>>>(A, f);
        else ew_vec_kernel<NIN, NOUT, F, (NIN > 1 ? EW_SCALAR : 0)><<<g, kEwThreads, 0, st>>>(A, f);
    } else {
        ew_scalar_kernel<NIN, NOUT, F><<<ctk_stream_grid(A.n, kEwThreads, 8), kEwThreads, 0, st>>>(A, f);
    }
    CTK_LAUNCH_CHECK(name);
    return CTK_OK;
}

}  // namespace ctk
