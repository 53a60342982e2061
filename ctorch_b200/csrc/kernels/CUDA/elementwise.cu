// Broadcast-aware elementwise kernels, forward and backward, for sm_100a.
//
// All of these are HBM-bound streams: 128-bit coalesced loads/stores with streaming cache hints,
// four independent vectors in flight per thread, grids sized in whole waves of the SM count.
// This file is compiled with -fmad=false: every product and sum below is rounded on its own, as
// in the reference's chain of single-op kernels; the one intended fused multiply-add (the SGD
// update) calls fmaf explicitly.
//
// Reference semantics restated per functor; file:line citations are relative to the reference.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kCtasPerSm = 8;
constexpr int kUnroll = 4;

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

template <int KIND>
__device__ __forceinline__ float scalar_op(float x, float s) {
    if (KIND == 0) return x * s;  // src/Tensor.cpp:751-806
    if (KIND == 1) return x + s;  // :855-910
    if (KIND == 2) return x / s;  // :913-973
    if (KIND == 3) return s - x;  // :1427-1429
    return s / x;                 // :1450-1452 (evaluated on the materialised operand)
}

// src/AutoDiff.cpp:1317-1416, one rounding per reference kernel call.
template <int OP>
__device__ __forceinline__ float un_bwd(float x, float g) {
    if (OP == CTK_OP_NEG) return -g;
    if (OP == CTK_OP_RELU) return g * (x > 0.0f ? 1.0f : 0.0f);
    if (OP == CTK_OP_SIGMOID) {
        float s = un_op<CTK_OP_SIGMOID>(x);
        float oms = 1.0f - s;
        float t = s * oms;
        return t * g;
    }
    if (OP == CTK_OP_TANH) {
        float t = un_op<CTK_OP_TANH>(x);
        float t2 = t * t;
        float om = 1.0f - t2;
        return om * g;
    }
    if (OP == CTK_OP_SIN) return cosf(x) * g;
    return (-sinf(x)) * g;
}

__device__ __forceinline__ float4 ld_stream(const float* p) { return __ldcs(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ void st_stream(float* p, float4 v) { __stcs(reinterpret_cast<float4*>(p), v); }

#define CTK_APPLY4(r, expr_x, expr_y, expr_z, expr_w) \
    r.x = (expr_x); r.y = (expr_y); r.z = (expr_z); r.w = (expr_w)

// ---------------------------------------------------------------------------------------------
// generic streaming skeleton: F(i4, i) computes the float4 at vector index i4 / the scalar at i.
// ---------------------------------------------------------------------------------------------
template <class VecBody, class TailBody>
__device__ __forceinline__ void stream_loop(int64_t n, bool vec_ok, VecBody vec, TailBody tail) {
    const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
    if (vec_ok) {
        const int64_t n4 = n >> 2;
        int64_t i = tid;
        for (; i + (kUnroll - 1) * nthreads < n4; i += kUnroll * nthreads) {
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) vec(i + u * nthreads, u);
        }
        for (; i < n4; i += nthreads) vec(i, 0);
        for (int64_t j = (n4 << 2) + tid; j < n; j += nthreads) tail(j);
    } else {
        for (int64_t j = tid; j < n; j += nthreads) tail(j);
    }
}

template <int OP, int LAYOUT>
__global__ void __launch_bounds__(kThreads) binary_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                          float* __restrict__ out, int64_t n, int64_t inner, bool vec_ok) {
    const float s = (LAYOUT == CTK_B_SCALAR) ? __ldg(b) : (LAYOUT == CTK_A_SCALAR) ? __ldg(a) : 0.0f;
    auto vec = [&](int64_t i4, int) {
        const int64_t i = i4 << 2;
        float4 x, y, r;
        if (LAYOUT == CTK_A_SCALAR) x = make_float4(s, s, s, s); else x = ld_stream(a + i);
        if (LAYOUT == CTK_B_SAME || LAYOUT == CTK_A_SCALAR) y = ld_stream(b + i);
        else if (LAYOUT == CTK_B_SCALAR) y = make_float4(s, s, s, s);
        else y = __ldg(reinterpret_cast<const float4*>(b + (i % inner)));
        CTK_APPLY4(r, bin_op<OP>(x.x, y.x), bin_op<OP>(x.y, y.y), bin_op<OP>(x.z, y.z), bin_op<OP>(x.w, y.w));
        st_stream(out + i, r);
    };
    auto tail = [&](int64_t i) {
        float x = (LAYOUT == CTK_A_SCALAR) ? s : a[i];
        float y = (LAYOUT == CTK_B_SAME || LAYOUT == CTK_A_SCALAR) ? b[i] : (LAYOUT == CTK_B_SCALAR) ? s : __ldg(b + (i % inner));
        out[i] = bin_op<OP>(x, y);
    };
    stream_loop(n, vec_ok, vec, tail);
}

template <int OP>
__global__ void __launch_bounds__(kThreads) unary_kernel(const float* __restrict__ a, float* __restrict__ out, int64_t n, bool vec_ok) {
    auto vec = [&](int64_t i4, int) {
        const int64_t i = i4 << 2;
        float4 x = ld_stream(a + i), r;
        CTK_APPLY4(r, un_op<OP>(x.x), un_op<OP>(x.y), un_op<OP>(x.z), un_op<OP>(x.w));
        st_stream(out + i, r);
    };
    auto tail = [&](int64_t i) { out[i] = un_op<OP>(a[i]); };
    stream_loop(n, vec_ok, vec, tail);
}

template <int KIND>
__global__ void __launch_bounds__(kThreads) scalar_kernel(const float* __restrict__ a, float s, float* __restrict__ out, int64_t n, bool vec_ok) {
    auto vec = [&](int64_t i4, int) {
        const int64_t i = i4 << 2;
        float4 x = ld_stream(a + i), r;
        CTK_APPLY4(r, scalar_op<KIND>(x.x, s), scalar_op<KIND>(x.y, s), scalar_op<KIND>(x.z, s), scalar_op<KIND>(x.w, s));
        st_stream(out + i, r);
    };
    auto tail = [&](int64_t i) { out[i] = scalar_op<KIND>(a[i], s); };
    stream_loop(n, vec_ok, vec, tail);
}

template <int OP>
__global__ void __launch_bounds__(kThreads) unary_bwd_kernel(const float* __restrict__ x, const float* __restrict__ g,
                                                             float* __restrict__ dx, int64_t n, bool vec_ok) {
    auto vec = [&](int64_t i4, int) {
        const int64_t i = i4 << 2;
        float4 gg = ld_stream(g + i), r;
        float4 xx = (OP == CTK_OP_NEG) ? gg : ld_stream(x + i);
        CTK_APPLY4(r, un_bwd<OP>(xx.x, gg.x), un_bwd<OP>(xx.y, gg.y), un_bwd<OP>(xx.z, gg.z), un_bwd<OP>(xx.w, gg.w));
        st_stream(dx + i, r);
    };
    auto tail = [&](int64_t i) { dx[i] = un_bwd<OP>((OP == CTK_OP_NEG) ? 0.0f : x[i], g[i]); };
    stream_loop(n, vec_ok, vec, tail);
}

// Add :1216-1221, Sub :1222-1233, Mul :1234-1258, Div :1259-1316 of src/AutoDiff.cpp.  db for a
// broadcast b is the gradient's leading `nb` elements (first row / first element): the reference's
// grad-shape adjustment gathers with index 0, src/AutoDiff.cpp:690-757.
template <int OP>
__device__ __forceinline__ void bin_bwd(float a, float b, float g, float& ga, float& gb) {
    if (OP == CTK_OP_ADD) { ga = g; gb = g; }
    else if (OP == CTK_OP_SUB) { ga = g; gb = -g; }
    else if (OP == CTK_OP_MUL) { ga = b * g; gb = a * g; }
    else {
        ga = g / b;
        float na = -a;
        float t = na * g;
        float bb = b * b;
        gb = t / bb;
    }
}

template <int OP, int LAYOUT>
__global__ void __launch_bounds__(kThreads) binary_bwd_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                              const float* __restrict__ g, float* __restrict__ da,
                                                              float* __restrict__ db, int64_t n, int64_t inner, int64_t nb,
                                                              bool vec_ok) {
    constexpr bool kNeedsOperands = (OP == CTK_OP_MUL || OP == CTK_OP_DIV);
    const float s = (LAYOUT == CTK_B_SCALAR && kNeedsOperands) ? __ldg(b) : 0.0f;
    auto vec = [&](int64_t i4, int) {
        const int64_t i = i4 << 2;
        float4 gg = ld_stream(g + i), x = gg, y = gg, ra, rb;
        if (kNeedsOperands) {
            x = ld_stream(a + i);
            if (LAYOUT == CTK_B_SAME) y = ld_stream(b + i);
            else if (LAYOUT == CTK_B_SCALAR) y = make_float4(s, s, s, s);
            else y = __ldg(reinterpret_cast<const float4*>(b + (i % inner)));
        }
        bin_bwd<OP>(x.x, y.x, gg.x, ra.x, rb.x);
        bin_bwd<OP>(x.y, y.y, gg.y, ra.y, rb.y);
        bin_bwd<OP>(x.z, y.z, gg.z, ra.z, rb.z);
        bin_bwd<OP>(x.w, y.w, gg.w, ra.w, rb.w);
        if (da) st_stream(da + i, ra);
        if (db) {
            if (i + 3 < nb) st_stream(db + i, rb);
            else {
                if (i < nb) db[i] = rb.x;
                if (i + 1 < nb) db[i + 1] = rb.y;
                if (i + 2 < nb) db[i + 2] = rb.z;
            }
        }
    };
    auto tail = [&](int64_t i) {
        float x = 0.0f, y = 0.0f, ga, gb;
        if (kNeedsOperands) {
            x = a[i];
            y = (LAYOUT == CTK_B_SAME) ? b[i] : (LAYOUT == CTK_B_SCALAR) ? s : __ldg(b + (i % inner));
        }
        bin_bwd<OP>(x, y, g[i], ga, gb);
        if (da) da[i] = ga;
        if (db && i < nb) db[i] = gb;
    };
    stream_loop(n, vec_ok, vec, tail);
}

__global__ void __launch_bounds__(kThreads) fill_kernel(float* __restrict__ p, float v, const float* __restrict__ vdev, int64_t n, bool vec_ok) {
    const float val = vdev ? __ldg(vdev) : v;
    auto vec = [&](int64_t i4, int) { st_stream(p + (i4 << 2), make_float4(val, val, val, val)); };
    auto tail = [&](int64_t i) { p[i] = val; };
    stream_loop(n, vec_ok, vec, tail);
}

__global__ void __launch_bounds__(kThreads) tile_kernel(const float* __restrict__ src, int64_t src_n, float* __restrict__ dst, int64_t n, bool vec_ok) {
    auto vec = [&](int64_t i4, int) {
        const int64_t i = i4 << 2;
        st_stream(dst + i, __ldg(reinterpret_cast<const float4*>(src + (i % src_n))));
    };
    auto tail = [&](int64_t i) { dst[i] = __ldg(src + (i % src_n)); };
    stream_loop(n, vec_ok, vec, tail);
}

__global__ void __launch_bounds__(kThreads) accumulate_kernel(float* __restrict__ dst, const float* __restrict__ src, int64_t n, bool vec_ok) {
    auto vec = [&](int64_t i4, int) {
        const int64_t i = i4 << 2;
        float4 d = *reinterpret_cast<const float4*>(dst + i), s = ld_stream(src + i);
        d.x += s.x; d.y += s.y; d.z += s.z; d.w += s.w;
        *reinterpret_cast<float4*>(dst + i) = d;
    };
    auto tail = [&](int64_t i) { dst[i] += src[i]; };
    stream_loop(n, vec_ok, vec, tail);
}

// mnist/mnist.cpp:84-87 `p[i] -= g[i] * lr`, which g++ -O3 emits as one fused multiply-add.
__global__ void __launch_bounds__(kThreads) sgd_kernel(float* __restrict__ p, const float* __restrict__ g, float lr, int64_t n, bool vec_ok) {
    auto vec = [&](int64_t i4, int) {
        const int64_t i = i4 << 2;
        float4 w = *reinterpret_cast<const float4*>(p + i), d = ld_stream(g + i);
        w.x = fmaf(-d.x, lr, w.x); w.y = fmaf(-d.y, lr, w.y); w.z = fmaf(-d.z, lr, w.z); w.w = fmaf(-d.w, lr, w.w);
        *reinterpret_cast<float4*>(p + i) = w;
    };
    auto tail = [&](int64_t i) { p[i] = fmaf(-g[i], lr, p[i]); };
    stream_loop(n, vec_ok, vec, tail);
}

struct GatherArgs {
    int64_t shape[8];
    int64_t stride[8];
    int rank;
};
__global__ void __launch_bounds__(kThreads) gather_nd_kernel(const float* __restrict__ src, float* __restrict__ dst, int64_t n, GatherArgs g) {
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

__global__ void __launch_bounds__(kThreads) onehot_kernel(const float* __restrict__ labels, int64_t rows, int64_t classes, float* __restrict__ out) {
    const int64_t n = rows * classes;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t r = i / classes, j = i - r * classes;
        out[i] = (static_cast<int>(__ldg(labels + r)) == static_cast<int>(j)) ? 1.0f : 0.0f;
    }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int grid_for(int64_t n) { return ctk_stream_grid((n + 3) / 4, kThreads * kUnroll, kCtasPerSm); }

}  // namespace

#define CTK_DISPATCH_LAYOUT(KERNEL, OPV, ...)                                                              \
    switch (layout) {                                                                                      \
        case CTK_B_SAME: KERNEL<OPV, CTK_B_SAME><<<grid, kThreads, 0, st>>>(__VA_ARGS__); break;            \
        case CTK_B_SCALAR: KERNEL<OPV, CTK_B_SCALAR><<<grid, kThreads, 0, st>>>(__VA_ARGS__); break;        \
        case CTK_B_ROW: KERNEL<OPV, CTK_B_ROW><<<grid, kThreads, 0, st>>>(__VA_ARGS__); break;              \
        default: KERNEL<OPV, CTK_A_SCALAR><<<grid, kThreads, 0, st>>>(__VA_ARGS__); break;                  \
    }

extern "C" {

ctk_status ctk_binary_f32(int op, const float* a, const float* b, float* out, int64_t n, int layout, int64_t inner, void* stream) {
    CTK_REQUIRE(n >= 0, "ctk_binary_f32: negative size");
    if (n == 0) return CTK_OK;
    CTK_REQUIRE(a && b && out, "ctk_binary_f32: null pointer");
    CTK_REQUIRE(layout >= CTK_B_SAME && layout <= CTK_A_SCALAR, "ctk_binary_f32: unknown layout");
    CTK_REQUIRE(layout != CTK_B_ROW || (inner > 0 && n % inner == 0), "ctk_binary_f32: row layout needs n % inner == 0");
    bool vec_ok = aligned16(out) && (layout == CTK_A_SCALAR || aligned16(a)) &&
                  (layout == CTK_B_SCALAR || aligned16(b)) && (layout != CTK_B_ROW || inner % 4 == 0);
    cudaStream_t st = ctk::as_stream(stream);
    int grid = grid_for(n);
    switch (op) {
        case CTK_OP_ADD: CTK_DISPATCH_LAYOUT(binary_kernel, CTK_OP_ADD, a, b, out, n, inner, vec_ok); break;
        case CTK_OP_SUB: CTK_DISPATCH_LAYOUT(binary_kernel, CTK_OP_SUB, a, b, out, n, inner, vec_ok); break;
        case CTK_OP_MUL: CTK_DISPATCH_LAYOUT(binary_kernel, CTK_OP_MUL, a, b, out, n, inner, vec_ok); break;
        case CTK_OP_DIV: CTK_DISPATCH_LAYOUT(binary_kernel, CTK_OP_DIV, a, b, out, n, inner, vec_ok); break;
        default: return ctk::fail(CTK_ERR_INVALID, "ctk_binary_f32: op must be Add/Sub/Mul/Div");
    }
    CTK_LAUNCH_CHECK("binary_kernel");
    return CTK_OK;
}

ctk_status ctk_unary_f32(int op, const float* a, float* out, int64_t n, void* stream) {
    CTK_REQUIRE(n >= 0, "ctk_unary_f32: negative size");
    if (n == 0) return CTK_OK;
    CTK_REQUIRE(a && out, "ctk_unary_f32: null pointer");
    bool vec_ok = aligned16(a) && aligned16(out);
    cudaStream_t st = ctk::as_stream(stream);
    int grid = grid_for(n);
    switch (op) {
        case CTK_OP_NEG: unary_kernel<CTK_OP_NEG><<<grid, kThreads, 0, st>>>(a, out, n, vec_ok); break;
        case CTK_OP_RELU: unary_kernel<CTK_OP_RELU><<<grid, kThreads, 0, st>>>(a, out, n, vec_ok); break;
        case CTK_OP_SIGMOID: unary_kernel<CTK_OP_SIGMOID><<<grid, kThreads, 0, st>>>(a, out, n, vec_ok); break;
        case CTK_OP_TANH: unary_kernel<CTK_OP_TANH><<<grid, kThreads, 0, st>>>(a, out, n, vec_ok); break;
        case CTK_OP_SIN: unary_kernel<CTK_OP_SIN><<<grid, kThreads, 0, st>>>(a, out, n, vec_ok); break;
        case CTK_OP_COS: unary_kernel<CTK_OP_COS><<<grid, kThreads, 0, st>>>(a, out, n, vec_ok); break;
        default: return ctk::fail(CTK_ERR_INVALID, "ctk_unary_f32: op must be Neg/ReLU/Sigmoid/Tanh/Sin/Cos");
    }
    CTK_LAUNCH_CHECK("unary_kernel");
    return CTK_OK;
}

ctk_status ctk_scalar_f32(int kind, const float* a, float s, float* out, int64_t n, void* stream) {
    CTK_REQUIRE(n >= 0, "ctk_scalar_f32: negative size");
    if (n == 0) return CTK_OK;
    CTK_REQUIRE(a && out, "ctk_scalar_f32: null pointer");
    bool vec_ok = aligned16(a) && aligned16(out);
    cudaStream_t st = ctk::as_stream(stream);
    int grid = grid_for(n);
    switch (kind) {
        case 0: scalar_kernel<0><<<grid, kThreads, 0, st>>>(a, s, out, n, vec_ok); break;
        case 1: scalar_kernel<1><<<grid, kThreads, 0, st>>>(a, s, out, n, vec_ok); break;
        case 2: scalar_kernel<2><<<grid, kThreads, 0, st>>>(a, s, out, n, vec_ok); break;
        case 3: scalar_kernel<3><<<grid, kThreads, 0, st>>>(a, s, out, n, vec_ok); break;
        case 4: scalar_kernel<4><<<grid, kThreads, 0, st>>>(a, s, out, n, vec_ok); break;
        default: return ctk::fail(CTK_ERR_INVALID, "ctk_scalar_f32: kind must be 0..4");
    }
    CTK_LAUNCH_CHECK("scalar_kernel");
    return CTK_OK;
}

ctk_status ctk_fill_f32(float* p, float value, const float* value_device, int64_t n, void* stream) {
    CTK_REQUIRE(n >= 0, "ctk_fill_f32: negative size");
    if (n == 0) return CTK_OK;
    CTK_REQUIRE(p, "ctk_fill_f32: null pointer");
    fill_kernel<<<grid_for(n), kThreads, 0, ctk::as_stream(stream)>>>(p, value, value_device, n, aligned16(p));
    CTK_LAUNCH_CHECK("fill_kernel");
    return CTK_OK;
}

ctk_status ctk_tile_f32(const float* src, int64_t src_n, float* dst, int64_t n, void* stream) {
    CTK_REQUIRE(n >= 0 && src_n > 0, "ctk_tile_f32: bad size");
    if (n == 0) return CTK_OK;
    CTK_REQUIRE(src && dst, "ctk_tile_f32: null pointer");
    bool vec_ok = aligned16(src) && aligned16(dst) && src_n % 4 == 0;
    tile_kernel<<<grid_for(n), kThreads, 0, ctk::as_stream(stream)>>>(src, src_n, dst, n, vec_ok);
    CTK_LAUNCH_CHECK("tile_kernel");
    return CTK_OK;
}

ctk_status ctk_onehot_f32(const float* labels, int64_t rows, int64_t classes, float* onehot, void* stream) {
    CTK_REQUIRE(rows >= 0 && classes >= 0, "ctk_onehot_f32: negative shape");
    if (rows == 0 || classes == 0) return CTK_OK;
    CTK_REQUIRE(labels && onehot, "ctk_onehot_f32: null pointer");
    onehot_kernel<<<ctk_stream_grid(rows * classes, kThreads, kCtasPerSm), kThreads, 0, ctk::as_stream(stream)>>>(labels, rows, classes, onehot);
    CTK_LAUNCH_CHECK("onehot_kernel");
    return CTK_OK;
}

ctk_status ctk_gather_nd_f32(const float* src, float* dst, int rank, const int64_t* dst_shape, const int64_t* src_strides, void* stream) {
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
    gather_nd_kernel<<<ctk_stream_grid(n, kThreads, kCtasPerSm), kThreads, 0, ctk::as_stream(stream)>>>(src, dst, n, g);
    CTK_LAUNCH_CHECK("gather_nd_kernel");
    return CTK_OK;
}

ctk_status ctk_unary_backward_f32(int op, const float* x, const float* g, float* dx, int64_t n, void* stream) {
    CTK_REQUIRE(n >= 0, "ctk_unary_backward_f32: negative size");
    if (n == 0) return CTK_OK;
    CTK_REQUIRE(g && dx && (x || op == CTK_OP_NEG), "ctk_unary_backward_f32: null pointer");
    bool vec_ok = aligned16(g) && aligned16(dx) && (op == CTK_OP_NEG || aligned16(x));
    cudaStream_t st = ctk::as_stream(stream);
    int grid = grid_for(n);
    switch (op) {
        case CTK_OP_NEG: unary_bwd_kernel<CTK_OP_NEG><<<grid, kThreads, 0, st>>>(x, g, dx, n, vec_ok); break;
        case CTK_OP_RELU: unary_bwd_kernel<CTK_OP_RELU><<<grid, kThreads, 0, st>>>(x, g, dx, n, vec_ok); break;
        case CTK_OP_SIGMOID: unary_bwd_kernel<CTK_OP_SIGMOID><<<grid, kThreads, 0, st>>>(x, g, dx, n, vec_ok); break;
        case CTK_OP_TANH: unary_bwd_kernel<CTK_OP_TANH><<<grid, kThreads, 0, st>>>(x, g, dx, n, vec_ok); break;
        case CTK_OP_SIN: unary_bwd_kernel<CTK_OP_SIN><<<grid, kThreads, 0, st>>>(x, g, dx, n, vec_ok); break;
        case CTK_OP_COS: unary_bwd_kernel<CTK_OP_COS><<<grid, kThreads, 0, st>>>(x, g, dx, n, vec_ok); break;
        default: return ctk::fail(CTK_ERR_INVALID, "ctk_unary_backward_f32: unsupported op");
    }
    CTK_LAUNCH_CHECK("unary_bwd_kernel");
    return CTK_OK;
}

ctk_status ctk_binary_backward_f32(int op, const float* a, const float* b, const float* g, float* da, float* db,
                                   int64_t n, int layout, int64_t inner, void* stream) {
    CTK_REQUIRE(n >= 0, "ctk_binary_backward_f32: negative size");
    if (n == 0 || (!da && !db)) return CTK_OK;
    CTK_REQUIRE(g, "ctk_binary_backward_f32: null gradient");
    CTK_REQUIRE(layout >= CTK_B_SAME && layout <= CTK_B_ROW, "ctk_binary_backward_f32: layout must be same/scalar/row");
    CTK_REQUIRE(layout != CTK_B_ROW || (inner > 0 && n % inner == 0), "ctk_binary_backward_f32: row layout needs n % inner == 0");
    const bool needs = (op == CTK_OP_MUL || op == CTK_OP_DIV);
    CTK_REQUIRE(!needs || (a && b), "ctk_binary_backward_f32: Mul/Div need both operands");
    const int64_t nb = (layout == CTK_B_SAME) ? n : (layout == CTK_B_SCALAR) ? 1 : inner;
    bool vec_ok = aligned16(g) && (!da || aligned16(da)) && (!db || aligned16(db)) &&
                  (!needs || (aligned16(a) && (layout == CTK_B_SCALAR || aligned16(b)))) &&
                  (layout != CTK_B_ROW || inner % 4 == 0);
    cudaStream_t st = ctk::as_stream(stream);
    int grid = grid_for(n);
    switch (op) {
        case CTK_OP_ADD: CTK_DISPATCH_LAYOUT(binary_bwd_kernel, CTK_OP_ADD, a, b, g, da, db, n, inner, nb, vec_ok); break;
        case CTK_OP_SUB: CTK_DISPATCH_LAYOUT(binary_bwd_kernel, CTK_OP_SUB, a, b, g, da, db, n, inner, nb, vec_ok); break;
        case CTK_OP_MUL: CTK_DISPATCH_LAYOUT(binary_bwd_kernel, CTK_OP_MUL, a, b, g, da, db, n, inner, nb, vec_ok); break;
        case CTK_OP_DIV: CTK_DISPATCH_LAYOUT(binary_bwd_kernel, CTK_OP_DIV, a, b, g, da, db, n, inner, nb, vec_ok); break;
        default: return ctk::fail(CTK_ERR_INVALID, "ctk_binary_backward_f32: op must be Add/Sub/Mul/Div");
    }
    CTK_LAUNCH_CHECK("binary_bwd_kernel");
    return CTK_OK;
}

ctk_status ctk_accumulate_f32(float* dst, const float* src, int64_t n, void* stream) {
    CTK_REQUIRE(n >= 0, "ctk_accumulate_f32: negative size");
    if (n == 0) return CTK_OK;
    CTK_REQUIRE(dst && src, "ctk_accumulate_f32: null pointer");
    accumulate_kernel<<<grid_for(n), kThreads, 0, ctk::as_stream(stream)>>>(dst, src, n, aligned16(dst) && aligned16(src));
    CTK_LAUNCH_CHECK("accumulate_kernel");
    return CTK_OK;
}

ctk_status ctk_sgd_update_f32(float* p, const float* g, float lr, int64_t n, void* stream) {
    CTK_REQUIRE(n >= 0, "ctk_sgd_update_f32: negative size");
    if (n == 0) return CTK_OK;
    CTK_REQUIRE(p && g, "ctk_sgd_update_f32: null pointer");
    sgd_kernel<<<grid_for(n), kThreads, 0, ctk::as_stream(stream)>>>(p, g, lr, n, aligned16(p) && aligned16(g));
    CTK_LAUNCH_CHECK("sgd_kernel");
    return CTK_OK;
}

}  // extern "C"
