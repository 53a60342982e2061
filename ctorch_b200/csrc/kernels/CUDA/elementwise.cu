// Broadcast-aware elementwise kernels, forward and backward, for sm_100a.
//
// All of these are HBM-bound streams and share one skeleton (ew_skeleton.cuh): 128-bit coalesced
// loads with streaming hints, one 16 KiB tile per array per CTA, all loads of the tile issued before
// the first store.  This file is compiled with -fmad=false: every product and sum below is rounded
// on its own, as in the reference's chain of single-op kernels; the one intended fused multiply-add
// (the SGD update) calls fmaf explicitly.
//
// Reference semantics are restated per functor; file:line citations are relative to the reference.
#include <math.h>

#include "ew_skeleton.cuh"

namespace {
using namespace ctk;

// ---------------------------------------------------------------------------------------------
// functors
// ---------------------------------------------------------------------------------------------
template <int OP>
__device__ __forceinline__ float bin_op(float x, float y) {
    if (OP == CTK_OP_ADD) return x + y;  // Add_BASIC_kernel.cpp:48-68
    if (OP == CTK_OP_SUB) return x - y;  // Sub_BASIC_kernel.cpp:57-60
    if (OP == CTK_OP_MUL) return x * y;  // Mul_BASIC_kernel.cpp:58-61
    return x / y;                        // Div_BASIC_kernel.cpp:37-44 (IEEE quotient kept for y == 0)
}

template <int OP>
__device__ __forceinline__ float un_op(float x) {
    if (OP == CTK_OP_NEG) return -x;                           // Neg_BASIC_kernel.cpp:26-28
    if (OP == CTK_OP_RELU) return x > 0.0f ? x : 0.0f;         // ReLU_BASIC_kernel.cpp:23-25 (NaN -> 0)
    if (OP == CTK_OP_SIGMOID) return 1.0f / (1.0f + expf(-x)); // Sigmoid_BASIC_kernel.cpp:24-26
    if (OP == CTK_OP_TANH) {                                   // Tanh_BASIC_kernel.cpp:24-28
        float ep = expf(x), en = expf(-x);
        return (ep - en) / (ep + en);
    }
    if (OP == CTK_OP_SIN) return sinf(x);                      // Sin_BASIC_kernel.cpp
    return cosf(x);                                            // Cos_BASIC_kernel.cpp
}

template <int OP> struct BinaryF {
    __device__ __forceinline__ void operator()(const float* x, float* y) const { y[0] = bin_op<OP>(x[0], x[1]); }
};
template <int OP> struct UnaryF {
    __device__ __forceinline__ void operator()(const float* x, float* y) const { y[0] = un_op<OP>(x[0]); }
};
// src/Tensor.cpp:751-806 (t*s), :855-910 (t+s), :913-973 (t/s), :1427-1429 (s-t), :1450-1452 (s/t,
// evaluated on the materialised operand)
template <int KIND> struct ScalarF {
    float s;
    __device__ __forceinline__ void operator()(const float* x, float* y) const {
        if (KIND == 0) y[0] = x[0] * s;
        else if (KIND == 1) y[0] = x[0] + s;
        else if (KIND == 2) y[0] = x[0] / s;
        else if (KIND == 3) y[0] = s - x[0];
        else y[0] = s / x[0];
    }
};
// src/AutoDiff.cpp:1317-1416, one rounding per reference kernel call.  x[0] = g, x[1] = input.
template <int OP> struct UnaryBwdF {
    __device__ __forceinline__ void operator()(const float* x, float* y) const {
        const float g = x[0];
        if (OP == CTK_OP_NEG) { y[0] = -g; return; }
        const float v = x[1];
        if (OP == CTK_OP_RELU) y[0] = g * (v > 0.0f ? 1.0f : 0.0f);
        else if (OP == CTK_OP_SIGMOID) {
            float s = un_op<CTK_OP_SIGMOID>(v);
            float oms = 1.0f - s;
            float t = s * oms;
            y[0] = t * g;
        } else if (OP == CTK_OP_TANH) {
            float t = un_op<CTK_OP_TANH>(v);
            float t2 = t * t;
            float om = 1.0f - t2;
            y[0] = om * g;
        } else if (OP == CTK_OP_SIN) y[0] = cosf(v) * g;
        else y[0] = (-sinf(v)) * g;
    }
};
// Add :1216-1221, Sub :1222-1233 (x[0] = g); Mul :1234-1258, Div :1259-1316 (x = g, a, b) of
// src/AutoDiff.cpp.  y[0] = da, y[1] = db.
template <int OP> struct BinaryBwdF {
    __device__ __forceinline__ void operator()(const float* x, float* y) const {
        const float g = x[0];
        if (OP == CTK_OP_ADD) { y[0] = g; y[1] = g; }
        else if (OP == CTK_OP_SUB) { y[0] = g; y[1] = -g; }
        else if (OP == CTK_OP_MUL) { y[0] = x[2] * g; y[1] = x[1] * g; }
        else {
            y[0] = g / x[2];
            float na = -x[1];
            float t = na * g;
            float bb = x[2] * x[2];
            y[1] = t / bb;
        }
    }
};
struct FillF {
    float v;
    __device__ __forceinline__ void operator()(const float*, float* y) const { y[0] = v; }
};
struct CopyF {  // fill from a device scalar (input 0 is EW_SCALAR) and tile (input 0 is EW_ROW)
    __device__ __forceinline__ void operator()(const float* x, float* y) const { y[0] = x[0]; }
};
struct AccumulateF {  // src/AutoDiff.cpp:1868-1907
    __device__ __forceinline__ void operator()(const float* x, float* y) const { y[0] = x[0] + x[1]; }
};
struct SgdF {  // mnist/mnist.cpp:84-87 `p[i] -= g[i] * lr`, which g++ -O3 emits as one fused multiply-add
    float lr;
    __device__ __forceinline__ void operator()(const float* x, float* y) const { y[0] = fmaf(-x[1], lr, x[0]); }
};

struct GatherArgs {
    int64_t shape[8];
    int64_t stride[8];
    int rank;
};
__global__ void __launch_bounds__(kEwThreads) gather_nd_kernel(const float* __restrict__ src, float* __restrict__ dst, int64_t n, GatherArgs g) {
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        int64_t rem = i, off = 0;
        for (int j = g.rank - 1; j >= 0; --j) {
            const int64_t idx = rem % g.shape[j];
            rem /= g.shape[j];
            off += idx * g.stride[j];
        }
        dst[i] = __ldg(src + off);
    }
}

__global__ void __launch_bounds__(kEwThreads) onehot_kernel(const float* __restrict__ labels, int64_t rows, int64_t classes, float* __restrict__ out) {
    const int64_t n = rows * classes;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t r = i / classes, j = i - r * classes;
        out[i] = (static_cast<int>(__ldg(labels + r)) == static_cast<int>(j)) ? 1.0f : 0.0f;
    }
}

// dst[i] = float(src[i]) / divisor, IEEE division: the pixel normalisation of the IDX image reader
// (mnist/mnist_loader.cpp:38-40, `pixel / 255.0f`), done on the device so that images cross PCIe as
// bytes.  A byte has 256 values: every CTA divides each of them once into a table in shared memory, so
// the stream itself is one 4-byte load, four table reads and one 16-byte store per thread, with the
// lanes of a warp on consecutive addresses on both sides (128 B read, 512 B written per instruction),
// four of them in flight per thread.
__global__ void __launch_bounds__(kEwThreads) u8_to_f32_kernel(const uint8_t* __restrict__ src, int64_t n, float divisor, float* __restrict__ dst, int vec) {
    __shared__ float quotient[256];
    for (int v = threadIdx.x; v < 256; v += blockDim.x) quotient[v] = __fdiv_rn(static_cast<float>(v), divisor);
    __syncthreads();
    const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    int64_t done = 0;
    if (vec) {
        const int64_t n4 = n >> 2;
        const uint32_t* s = reinterpret_cast<const uint32_t*>(src);
        float4* d = reinterpret_cast<float4*>(dst);
        auto four = [&](uint32_t w) {
            return make_float4(quotient[w & 0xffu], quotient[(w >> 8) & 0xffu], quotient[(w >> 16) & 0xffu], quotient[w >> 24]);
        };
        int64_t i = tid;
        for (; i + 3 * stride < n4; i += 4 * stride) {
            uint32_t w[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) w[q] = __ldcs(s + i + q * stride);
#pragma unroll
            for (int q = 0; q < 4; ++q) __stcs(d + i + q * stride, four(w[q]));
        }
        for (; i < n4; i += stride) __stcs(d + i, four(__ldcs(s + i)));
        done = n4 << 2;
    }
    for (int64_t i = done + tid; i < n; i += stride) dst[i] = quotient[src[i]];
}

// out[r] = index of the first element of row r that is strictly greater than everything before it,
// starting from (`init`, index 0): the prediction loop of mnist/mnist.cpp:140-147 (init -1 on
// probabilities); init = -inf gives the plain first-maximum argmax.  A warp per row; a lane keeps
// its first maximum, lanes are merged preferring the larger value, then the smaller index.
__global__ void __launch_bounds__(kEwThreads) argmax_rows_kernel(const float* __restrict__ x, int64_t rows, int64_t cols, float init, float* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    for (int64_t r = warp; r < rows; r += nwarps) {
        const float* row = x + r * cols;
        float best = init;
        int64_t idx = 0;
        for (int64_t j = lane; j < cols; j += 32) {
            const float v = __ldg(row + j);
            if (v > best) { best = v; idx = j; }
        }
        // a lane that found nothing above `init` must not win with index 0 over a lane that did
        bool found = best > init;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int64_t oi = __shfl_xor_sync(0xffffffffu, idx, o);
            const bool of = __shfl_xor_sync(0xffffffffu, found ? 1 : 0, o) != 0;
            const bool take = of && (!found || ob > best || (ob == best && oi < idx));
            if (take) { best = ob; idx = oi; found = true; }
        }
        if (lane == 0) out[r] = found ? static_cast<float>(idx) : 0.0f;
    }
}

// The same for short rows (cols <= 16, the class probabilities of the MNIST application): a thread per
// row walks its few elements in order -- exactly the reference's loop, no shuffles; the 32 rows of a warp
// are neighbours in memory, so the lines one load instruction touches are used up by the next few.
__global__ void __launch_bounds__(kEwThreads) argmax_short_rows_kernel(const float* __restrict__ x, int64_t rows, int cols, float init, float* __restrict__ out) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; r < rows; r += stride) {
        const float* row = x + r * cols;
        float best = init;
        int idx = 0;
        for (int j = 0; j < cols; ++j) {
            const float v = __ldg(row + j);
            if (v > best) { best = v; idx = j; }
        }
        out[r] = static_cast<float>(idx);
    }
}

template <int NIN, int NOUT>
EwArgs<NIN, NOUT> make_args(int64_t n, int64_t inner = 1) {
    EwArgs<NIN, NOUT> A{};
    A.n = n;
    A.inner = inner < 1 ? 1 : inner;
    for (int k = 0; k < NOUT; ++k) A.out_limit[k] = n;
    return A;
}

}  // namespace

extern "C" {

ctk_status ctk_binary_f32(int op, const float* a, const float* b, float* out, int64_t n, int layout, int64_t inner, void* stream) {
    CTK_RANGE("ctk_binary_f32");
    CTK_REQUIRE(n >= 0, "ctk_binary_f32: negative size");
    if (n == 0) return CTK_OK;
    CTK_REQUIRE(a && b && out, "ctk_binary_f32: null pointer");
    CTK_REQUIRE(layout >= CTK_B_SAME && layout <= CTK_A_SCALAR, "ctk_binary_f32: unknown layout");
    CTK_REQUIRE(layout != CTK_B_ROW || (inner > 0 && n % inner == 0), "ctk_binary_f32: row layout needs n % inner == 0");
    auto A = make_args<2, 1>(n, inner);
    A.in[0] = a; A.in[1] = b; A.out[0] = out;
    A.mode[0] = (layout == CTK_A_SCALAR) ? EW_SCALAR : EW_STREAM;
    A.mode[1] = (layout == CTK_B_SCALAR) ? EW_SCALAR : (layout == CTK_B_ROW) ? EW_ROW : EW_STREAM;
    cudaStream_t st = as_stream(stream);
    switch (op) {
        case CTK_OP_ADD: return ew_launch("binary_add", A, BinaryF<CTK_OP_ADD>{}, st);
        case CTK_OP_SUB: return ew_launch("binary_sub", A, BinaryF<CTK_OP_SUB>{}, st);
        case CTK_OP_MUL: return ew_launch("binary_mul", A, BinaryF<CTK_OP_MUL>{}, st);
        case CTK_OP_DIV: return ew_launch("binary_div", A, BinaryF<CTK_OP_DIV>{}, st);
        default: return fail(CTK_ERR_INVALID, "ctk_binary_f32: op must be Add/Sub/Mul/Div");
    }
}

ctk_status ctk_unary_f32(int op, const float* a, float* out, int64_t n, void* stream) {
    CTK_RANGE("ctk_unary_f32");
    CTK_REQUIRE(n >= 0, "ctk_unary_f32: negative size");
    if (n == 0) return CTK_OK;
    CTK_REQUIRE(a && out, "ctk_unary_f32: null pointer");
    auto A = make_args<1, 1>(n);
    A.in[0] = a; A.mode[0] = EW_STREAM; A.out[0] = out;
    cudaStream_t st = as_stream(stream);
    switch (op) {
        case CTK_OP_NEG: return ew_launch("unary_neg", A, UnaryF<CTK_OP_NEG>{}, st);
        case CTK_OP_RELU: return ew_launch("unary_relu", A, UnaryF<CTK_OP_RELU>{}, st);
        case CTK_OP_SIGMOID: return ew_launch("unary_sigmoid", A, UnaryF<CTK_OP_SIGMOID>{}, st);
        case CTK_OP_TANH: return ew_launch("unary_tanh", A, UnaryF<CTK_OP_TANH>{}, st);
        case CTK_OP_SIN: return ew_launch("unary_sin", A, UnaryF<CTK_OP_SIN>{}, st);
        case CTK_OP_COS: return ew_launch("unary_cos", A, UnaryF<CTK_OP_COS>{}, st);
        default: return fail(CTK_ERR_INVALID, "ctk_unary_f32: op must be Neg/ReLU/Sigmoid/Tanh/Sin/Cos");
    }
}

ctk_status ctk_scalar_f32(int kind, const float* a, float s, float* out, int64_t n, void* stream) {
    CTK_RANGE("ctk_scalar_f32");
    CTK_REQUIRE(n >= 0, "ctk_scalar_f32: negative size");
    if (n == 0) return CTK_OK;
    CTK_REQUIRE(a && out, "ctk_scalar_f32: null pointer");
    auto A = make_args<1, 1>(n);
    A.in[0] = a; A.mode[0] = EW_STREAM; A.out[0] = out;
    cudaStream_t st = as_stream(stream);
    switch (kind) {
        case 0: return ew_launch("scalar_mul", A, ScalarF<0>{s}, st);
        case 1: return ew_launch("scalar_add", A, ScalarF<1>{s}, st);
        case 2: return ew_launch("scalar_div", A, ScalarF<2>{s}, st);
        case 3: return ew_launch("scalar_rsub", A, ScalarF<3>{s}, st);
        case 4: return ew_launch("scalar_rdiv", A, ScalarF<4>{s}, st);
        default: return fail(CTK_ERR_INVALID, "ctk_scalar_f32: kind must be 0..4");
    }
}

ctk_status ctk_fill_f32(float* p, float value, const float* value_device, int64_t n, void* stream) {
    CTK_RANGE("ctk_fill_f32");
    CTK_REQUIRE(n >= 0, "ctk_fill_f32: negative size");
    if (n == 0) return CTK_OK;
    CTK_REQUIRE(p, "ctk_fill_f32: null pointer");
    if (value_device) {
        auto A = make_args<1, 1>(n);
        A.in[0] = value_device; A.mode[0] = EW_SCALAR; A.out[0] = p;
        return ew_launch("fill_from", A, CopyF{}, as_stream(stream));
    }
    auto A = make_args<0, 1>(n);
    A.out[0] = p;
    return ew_launch("fill", A, FillF{value}, as_stream(stream));
}

ctk_status ctk_tile_f32(const float* src, int64_t src_n, float* dst, int64_t n, void* stream) {
    CTK_RANGE("ctk_tile_f32");
    CTK_REQUIRE(n >= 0 && src_n > 0, "ctk_tile_f32: bad size");
    if (n == 0) return CTK_OK;
    CTK_REQUIRE(src && dst, "ctk_tile_f32: null pointer");
    auto A = make_args<1, 1>(n, src_n);
    A.in[0] = src; A.mode[0] = EW_ROW; A.out[0] = dst;
    return ew_launch("tile", A, CopyF{}, as_stream(stream));
}

ctk_status ctk_onehot_f32(const float* labels, int64_t rows, int64_t classes, float* onehot, void* stream) {
    CTK_RANGE("ctk_onehot_f32");
    CTK_REQUIRE(rows >= 0 && classes >= 0, "ctk_onehot_f32: negative shape");
    if (rows == 0 || classes == 0) return CTK_OK;
    CTK_REQUIRE(labels && onehot, "ctk_onehot_f32: null pointer");
    onehot_kernel<<<ctk_stream_grid(rows * classes, kEwThreads, 8), kEwThreads, 0, as_stream(stream)>>>(labels, rows, classes, onehot);
    CTK_LAUNCH_CHECK("onehot_kernel");
    return CTK_OK;
}

ctk_status ctk_u8_to_f32(const uint8_t* src, int64_t n, float divisor, float* dst, void* stream) {
    CTK_RANGE("ctk_u8_to_f32");
    CTK_REQUIRE(n >= 0, "ctk_u8_to_f32: negative size");
    if (n == 0) return CTK_OK;
    CTK_REQUIRE(src && dst, "ctk_u8_to_f32: null pointer");
    const int vec = ((reinterpret_cast<uintptr_t>(src) & 3u) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) ? 1 : 0;
    u8_to_f32_kernel<<<ctk_stream_grid((n + 15) / 16, kEwThreads, 8), kEwThreads, 0, as_stream(stream)>>>(src, n, divisor, dst, vec);
    CTK_LAUNCH_CHECK("u8_to_f32_kernel");
    return CTK_OK;
}

ctk_status ctk_argmax_rows_f32(const float* x, int64_t rows, int64_t cols, float init, float* out_index, void* stream) {
    CTK_RANGE("ctk_argmax_rows_f32");
    CTK_REQUIRE(rows >= 0 && cols >= 0, "ctk_argmax_rows_f32: negative shape");
    if (rows == 0) return CTK_OK;
    CTK_REQUIRE(out_index && (x || cols == 0), "ctk_argmax_rows_f32: null pointer");
    if (cols >= 1 && cols <= 16) {
        argmax_short_rows_kernel<<<ctk_stream_grid(rows, kEwThreads, 8), kEwThreads, 0, as_stream(stream)>>>(x, rows, static_cast<int>(cols), init, out_index);
    } else {
        argmax_rows_kernel<<<ctk_stream_grid(rows * 32, kEwThreads, 8), kEwThreads, 0, as_stream(stream)>>>(x, rows, cols, init, out_index);
    }
    CTK_LAUNCH_CHECK("argmax_rows_kernel");
    return CTK_OK;
}

ctk_status ctk_gather_nd_f32(const float* src, float* dst, int rank, const int64_t* dst_shape, const int64_t* src_strides, void* stream) {
    CTK_RANGE("ctk_gather_nd_f32");
    CTK_REQUIRE(rank >= 0 && rank <= 8, "ctk_gather_nd_f32: rank must be 0..8");
    CTK_REQUIRE(src && dst && (rank == 0 || (dst_shape && src_strides)), "ctk_gather_nd_f32: null pointer");
    GatherArgs g{};
    g.rank = rank;
    int64_t n = 1;
    for (int j = 0; j < rank; ++j) {
        CTK_REQUIRE(dst_shape[j] >= 0 && src_strides[j] >= 0, "ctk_gather_nd_f32: negative extent or stride");
        g.shape[j] = dst_shape[j];
        g.stride[j] = src_strides[j];
        n *= dst_shape[j];
    }
    if (n == 0) return CTK_OK;
    gather_nd_kernel<<<ctk_stream_grid(n, kEwThreads, 8), kEwThreads, 0, as_stream(stream)>>>(src, dst, n, g);
    CTK_LAUNCH_CHECK("gather_nd_kernel");
    return CTK_OK;
}

ctk_status ctk_unary_backward_f32(int op, const float* x, const float* g, float* dx, int64_t n, void* stream) {
    CTK_RANGE("ctk_unary_backward_f32");
    CTK_REQUIRE(n >= 0, "ctk_unary_backward_f32: negative size");
    if (n == 0) return CTK_OK;
    CTK_REQUIRE(g && dx && (x || op == CTK_OP_NEG), "ctk_unary_backward_f32: null pointer");
    cudaStream_t st = as_stream(stream);
    if (op == CTK_OP_NEG) {
        auto A = make_args<1, 1>(n);
        A.in[0] = g; A.mode[0] = EW_STREAM; A.out[0] = dx;
        return ew_launch("unary_bwd_neg", A, UnaryBwdF<CTK_OP_NEG>{}, st);
    }
    auto A = make_args<2, 1>(n);
    A.in[0] = g; A.in[1] = x; A.mode[0] = A.mode[1] = EW_STREAM; A.out[0] = dx;
    switch (op) {
        case CTK_OP_RELU: return ew_launch("unary_bwd_relu", A, UnaryBwdF<CTK_OP_RELU>{}, st);
        case CTK_OP_SIGMOID: return ew_launch("unary_bwd_sigmoid", A, UnaryBwdF<CTK_OP_SIGMOID>{}, st);
        case CTK_OP_TANH: return ew_launch("unary_bwd_tanh", A, UnaryBwdF<CTK_OP_TANH>{}, st);
        case CTK_OP_SIN: return ew_launch("unary_bwd_sin", A, UnaryBwdF<CTK_OP_SIN>{}, st);
        case CTK_OP_COS: return ew_launch("unary_bwd_cos", A, UnaryBwdF<CTK_OP_COS>{}, st);
        default: return fail(CTK_ERR_INVALID, "ctk_unary_backward_f32: unsupported op");
    }
}

ctk_status ctk_binary_backward_f32(int op, const float* a, const float* b, const float* g, float* da, float* db,
                                   int64_t n, int layout, int64_t inner, void* stream) {
    CTK_RANGE("ctk_binary_backward_f32");
    CTK_REQUIRE(n >= 0, "ctk_binary_backward_f32: negative size");
    if (n == 0 || (!da && !db)) return CTK_OK;
    CTK_REQUIRE(g, "ctk_binary_backward_f32: null gradient");
    CTK_REQUIRE(layout >= CTK_B_SAME && layout <= CTK_B_ROW, "ctk_binary_backward_f32: layout must be same/scalar/row");
    CTK_REQUIRE(layout != CTK_B_ROW || (inner > 0 && n % inner == 0), "ctk_binary_backward_f32: row layout needs n % inner == 0");
    const bool needs = (op == CTK_OP_MUL || op == CTK_OP_DIV);
    CTK_REQUIRE(!needs || (a && b), "ctk_binary_backward_f32: Mul/Div need both operands");
    // A broadcast b receives the gradient's leading elements (row 0 / element 0): the reference's
    // grad-shape adjustment gathers with index 0 on the broadcast dims (src/AutoDiff.cpp:690-757).
    const int64_t nb = (layout == CTK_B_SAME) ? n : (layout == CTK_B_SCALAR) ? 1 : inner;
    cudaStream_t st = as_stream(stream);
    if (!needs) {
        auto A = make_args<1, 2>(n, inner);
        A.in[0] = g; A.mode[0] = EW_STREAM;
        A.out[0] = da; A.out[1] = db; A.out_limit[1] = nb;
        if (op == CTK_OP_ADD) return ew_launch("binary_bwd_add", A, BinaryBwdF<CTK_OP_ADD>{}, st);
        if (op == CTK_OP_SUB) return ew_launch("binary_bwd_sub", A, BinaryBwdF<CTK_OP_SUB>{}, st);
        return fail(CTK_ERR_INVALID, "ctk_binary_backward_f32: op must be Add/Sub/Mul/Div");
    }
    auto A = make_args<3, 2>(n, inner);
    A.in[0] = g; A.in[1] = a; A.in[2] = b;
    A.mode[0] = A.mode[1] = EW_STREAM;
    A.mode[2] = (layout == CTK_B_SCALAR) ? EW_SCALAR : (layout == CTK_B_ROW) ? EW_ROW : EW_STREAM;
    A.out[0] = da; A.out[1] = db; A.out_limit[1] = nb;
    if (op == CTK_OP_MUL) return ew_launch("binary_bwd_mul", A, BinaryBwdF<CTK_OP_MUL>{}, st);
    return ew_launch("binary_bwd_div", A, BinaryBwdF<CTK_OP_DIV>{}, st);
}

ctk_status ctk_accumulate_f32(float* dst, const float* src, int64_t n, void* stream) {
    CTK_RANGE("ctk_accumulate_f32");
    CTK_REQUIRE(n >= 0, "ctk_accumulate_f32: negative size");
    if (n == 0) return CTK_OK;
    CTK_REQUIRE(dst && src, "ctk_accumulate_f32: null pointer");
    auto A = make_args<2, 1>(n);
    A.in[0] = dst; A.in[1] = src; A.mode[0] = A.mode[1] = EW_STREAM; A.out[0] = dst;
    return ew_launch("accumulate", A, AccumulateF{}, as_stream(stream));
}

ctk_status ctk_sgd_update_f32(float* p, const float* g, float lr, int64_t n, void* stream) {
    CTK_RANGE("ctk_sgd_update_f32");
    CTK_REQUIRE(n >= 0, "ctk_sgd_update_f32: negative size");
    if (n == 0) return CTK_OK;
    CTK_REQUIRE(p && g, "ctk_sgd_update_f32: null pointer");
    auto A = make_args<2, 1>(n);
    A.in[0] = p; A.in[1] = g; A.mode[0] = A.mode[1] = EW_STREAM; A.out[0] = p;
    return ew_launch("sgd_update", A, SgdF{lr}, as_stream(stream));
}

}  // extern "C"
