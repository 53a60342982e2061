// Element-wise comparisons (float -> bool), dtype conversion out of float, typed fills and uniform
// random numbers: the host loops of src/Tensor.cpp:985-1309, 1462-1591 (comparisons), 199-243
// (to(DType)), 422-450 (ones) and 458-479 (rand) as HBM-bound streaming kernels.
//
// One tile of 256 threads x 4 vectors of four floats per CTA, grid = number of tiles, all loads of the
// tile issued before the first use, streaming cache hints -- the shape of the float elementwise
// skeleton, with narrower or wider stores.  A scalar kernel takes unaligned pointers and the last
// n % 4 elements.
#include <math.h>

#include <type_traits>

#include "common.cuh"

namespace {
using namespace ctk;

constexpr int kThreads = 256, kUnroll = 4;

template <int CMP>
__device__ __forceinline__ unsigned char cmp1(float x, float y) {
    if (CMP == CTK_CMP_GT) return x > y;
    if (CMP == CTK_CMP_LT) return x < y;
    if (CMP == CTK_CMP_EQ) return x == y;
    if (CMP == CTK_CMP_GE) return x >= y;
    if (CMP == CTK_CMP_LE) return x <= y;
    return x != y;
}
// FORM: 0 a ? b, 1 a ? s, 2 s ? a
template <int CMP, int FORM>
__device__ __forceinline__ unsigned char cmp_form(float a, float b, float s) {
    if (FORM == CTK_CMP_TENSOR) return cmp1<CMP>(a, b);
    if (FORM == CTK_CMP_SCALAR_RIGHT) return cmp1<CMP>(a, s);
    return cmp1<CMP>(s, a);
}

template <int CMP, int FORM>
__global__ void __launch_bounds__(kThreads) compare_vec_kernel(const float4* __restrict__ a, const float4* __restrict__ b, float s,
                                                               uchar4* __restrict__ out, int64_t n4) {
    const int64_t base = static_cast<int64_t>(blockIdx.x) * (kThreads * kUnroll) + threadIdx.x;
    float4 va[kUnroll], vb[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        const int64_t i = base + u * kThreads;
        if (i < n4) {
            va[u] = __ldcs(a + i);
            if (FORM == CTK_CMP_TENSOR) vb[u] = __ldcs(b + i);
        }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        const int64_t i = base + u * kThreads;
        if (i < n4) {
            uchar4 r;
            r.x = cmp_form<CMP, FORM>(va[u].x, vb[u].x, s);
            r.y = cmp_form<CMP, FORM>(va[u].y, vb[u].y, s);
            r.z = cmp_form<CMP, FORM>(va[u].z, vb[u].z, s);
            r.w = cmp_form<CMP, FORM>(va[u].w, vb[u].w, s);
            __stcs(out + i, r);
        }
    }
}
template <int CMP, int FORM>
__global__ void __launch_bounds__(kThreads) compare_scalar_kernel(const float* __restrict__ a, const float* __restrict__ b, float s,
                                                                  unsigned char* __restrict__ out, int64_t first, int64_t n) {
    for (int64_t i = first + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        out[i] = cmp_form<CMP, FORM>(a[i], FORM == CTK_CMP_TENSOR ? b[i] : 0.0f, s);
}

template <int CMP, int FORM>
ctk_status launch_compare(const float* a, const float* b, float s, unsigned char* out, int64_t n, cudaStream_t st) {
    const bool aligned = ((reinterpret_cast<uintptr_t>(a) | (FORM == CTK_CMP_TENSOR ? reinterpret_cast<uintptr_t>(b) : 0)) & 15u) == 0 &&
                         (reinterpret_cast<uintptr_t>(out) & 3u) == 0;
    const int64_t n4 = aligned ? n / 4 : 0;
    if (n4 > 0) {
        const int64_t per_cta = kThreads * kUnroll;
        compare_vec_kernel<CMP, FORM><<<static_cast<unsigned>((n4 + per_cta - 1) / per_cta), kThreads, 0, st>>>(
            reinterpret_cast<const float4*>(a), reinterpret_cast<const float4*>(b), s, reinterpret_cast<uchar4*>(out), n4);
        CTK_LAUNCH_CHECK("compare_vec_kernel");
    }
    if (n4 * 4 < n) {
        compare_scalar_kernel<CMP, FORM><<<ctk_stream_grid(n - n4 * 4, kThreads, 8), kThreads, 0, st>>>(a, b, s, out, n4 * 4, n);
        CTK_LAUNCH_CHECK("compare_scalar_kernel");
    }
    return CTK_OK;
}
template <int CMP>
ctk_status compare_form(int form, const float* a, const float* b, float s, unsigned char* out, int64_t n, cudaStream_t st) {
    switch (form) {
        case CTK_CMP_TENSOR: return launch_compare<CMP, CTK_CMP_TENSOR>(a, b, s, out, n, st);
        case CTK_CMP_SCALAR_RIGHT: return launch_compare<CMP, CTK_CMP_SCALAR_RIGHT>(a, b, s, out, n, st);
        case CTK_CMP_SCALAR_LEFT: return launch_compare<CMP, CTK_CMP_SCALAR_LEFT>(a, b, s, out, n, st);
        default: return fail(CTK_ERR_INVALID, "ctk_compare_f32: form must be tensor / scalar right / scalar left");
    }
}

// ---- float -> other dtypes (src/Tensor.cpp:199-243: static_cast per element) ------------------------
template <typename T> __device__ __forceinline__ T conv1(float x);
template <> __device__ __forceinline__ double conv1<double>(float x) { return static_cast<double>(x); }
template <> __device__ __forceinline__ int conv1<int>(float x) { return static_cast<int>(x); }                    // toward zero
template <> __device__ __forceinline__ long long conv1<long long>(float x) { return static_cast<long long>(x); }  // toward zero
template <> __device__ __forceinline__ unsigned char conv1<unsigned char>(float x) { return x != 0.0f; }          // static_cast<bool>

__device__ __forceinline__ void store4(double* dst, int64_t i4, float4 v) {
    double2* d = reinterpret_cast<double2*>(dst) + 2 * i4;
    __stcs(d, make_double2(conv1<double>(v.x), conv1<double>(v.y)));
    __stcs(d + 1, make_double2(conv1<double>(v.z), conv1<double>(v.w)));
}
__device__ __forceinline__ void store4(int* dst, int64_t i4, float4 v) {
    __stcs(reinterpret_cast<int4*>(dst) + i4, make_int4(conv1<int>(v.x), conv1<int>(v.y), conv1<int>(v.z), conv1<int>(v.w)));
}
__device__ __forceinline__ void store4(long long* dst, int64_t i4, float4 v) {
    longlong2* d = reinterpret_cast<longlong2*>(dst) + 2 * i4;
    __stcs(d, make_longlong2(conv1<long long>(v.x), conv1<long long>(v.y)));
    __stcs(d + 1, make_longlong2(conv1<long long>(v.z), conv1<long long>(v.w)));
}
__device__ __forceinline__ void store4(unsigned char* dst, int64_t i4, float4 v) {
    __stcs(reinterpret_cast<uchar4*>(dst) + i4,
           make_uchar4(conv1<unsigned char>(v.x), conv1<unsigned char>(v.y), conv1<unsigned char>(v.z), conv1<unsigned char>(v.w)));
}

template <typename T>
__global__ void __launch_bounds__(kThreads) cast_vec_kernel(const float4* __restrict__ src, T* __restrict__ dst, int64_t n4) {
    const int64_t base = static_cast<int64_t>(blockIdx.x) * (kThreads * kUnroll) + threadIdx.x;
    float4 v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        const int64_t i = base + u * kThreads;
        v[u] = i < n4 ? __ldcs(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (sizeof(T) == 8) {
        // 8-byte results: a lane's four values are 32 bytes, so its two 16-byte stores would each
        // leave every other half-sector of the instruction's span untouched.  Lanes trade values so
        // that store 1 covers the warp's first 512 bytes and store 2 the second: lane L writes the
        // values of vector L/2 (first half) and of vector 16 + L/2 (second half).
        const int lane = threadIdx.x & 31;
        const int half = lane & 1;
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int64_t w0 = base + u * kThreads - lane;  // the warp's first vector
#pragma unroll
            for (int part = 0; part < 2; ++part) {
                const int from = part * 16 + (lane >> 1);
                const float x = __shfl_sync(0xffffffffu, v[u].x, from), y = __shfl_sync(0xffffffffu, v[u].y, from);
                const float z = __shfl_sync(0xffffffffu, v[u].z, from), w = __shfl_sync(0xffffffffu, v[u].w, from);
                if (w0 + from < n4) {
                    T* d = dst + 4 * (w0 + from) + 2 * half;
                    const T e0 = conv1<T>(half ? z : x), e1 = conv1<T>(half ? w : y);
                    if (sizeof(T) == 8 && std::is_same<T, double>::value) __stcs(reinterpret_cast<double2*>(d), make_double2(static_cast<double>(e0), static_cast<double>(e1)));
                    else __stcs(reinterpret_cast<longlong2*>(d), make_longlong2(static_cast<long long>(e0), static_cast<long long>(e1)));
                }
            }
        }
        return;
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        const int64_t i = base + u * kThreads;
        if (i < n4) store4(dst, i, v[u]);
    }
}
template <typename T>
__global__ void __launch_bounds__(kThreads) cast_scalar_kernel(const float* __restrict__ src, T* __restrict__ dst, int64_t first, int64_t n) {
    for (int64_t i = first + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        dst[i] = conv1<T>(src[i]);
}
template <typename T>
ctk_status launch_cast(const float* src, T* dst, int64_t n, cudaStream_t st) {
    const bool aligned = (reinterpret_cast<uintptr_t>(src) & 15u) == 0 && (reinterpret_cast<uintptr_t>(dst) & (4 * sizeof(T) > 16 ? 15u : 4 * sizeof(T) - 1)) == 0;
    const int64_t n4 = aligned ? n / 4 : 0;
    if (n4 > 0) {
        const int64_t per_cta = kThreads * kUnroll;
        cast_vec_kernel<T><<<static_cast<unsigned>((n4 + per_cta - 1) / per_cta), kThreads, 0, st>>>(reinterpret_cast<const float4*>(src), dst, n4);
        CTK_LAUNCH_CHECK("cast_vec_kernel");
    }
    if (n4 * 4 < n) {
        cast_scalar_kernel<T><<<ctk_stream_grid(n - n4 * 4, kThreads, 8), kThreads, 0, st>>>(src, dst, n4 * 4, n);
        CTK_LAUNCH_CHECK("cast_scalar_kernel");
    }
    return CTK_OK;
}

// ---- typed fill (ones() of the non-float dtypes) --------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads) fill_typed_kernel(T* __restrict__ dst, T v, int64_t n) {
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<int64_t>(gridDim.x) * blockDim.x) dst[i] = v;
}

// ---- uniform [0, 1) -------------------------------------------------------------------------------------
// Counter-based: element i of a call is a function of (seed, offset + i) alone, so the values do not
// depend on the launch shape.  One splitmix64 finaliser per PAIR of counters (c >> 1); the even counter
// takes bits 40-63 of it, the odd one bits 16-39: 24 bits each, so 1.0 is never produced, and the
// 64-bit multiplies -- the kernel is bound by them, not by its stores, otherwise -- are shared by two
// elements.
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__device__ __forceinline__ uint64_t pair_hash(uint64_t key, uint64_t pair) { return mix64(key + pair * 0x9E3779B97F4A7C15ull); }
__device__ __forceinline__ float hi24(uint64_t z) { return static_cast<float>(static_cast<uint32_t>(z >> 40)) * 5.9604644775390625e-08f; }
__device__ __forceinline__ float lo24(uint64_t z) { return static_cast<float>(static_cast<uint32_t>(z >> 16) & 0xFFFFFFu) * 5.9604644775390625e-08f; }
__device__ __forceinline__ float uniform_at(uint64_t key, uint64_t c) {
    const uint64_t z = pair_hash(key, c >> 1);
    return (c & 1) ? lo24(z) : hi24(z);
}
// dst 16-byte aligned; vector v holds counters offset + 4v .. offset + 4v + 3
__global__ void __launch_bounds__(kThreads) rand_uniform_vec_kernel(float4* __restrict__ dst, int64_t n4, uint64_t key, uint64_t offset) {
    const int64_t base = static_cast<int64_t>(blockIdx.x) * (kThreads * kUnroll) + threadIdx.x;
    const bool odd = offset & 1;  // the same for every thread
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        const int64_t i = base + u * kThreads;
        if (i >= n4) continue;
        const uint64_t c = offset + 4 * static_cast<uint64_t>(i);
        const uint64_t z0 = pair_hash(key, c >> 1), z1 = pair_hash(key, (c >> 1) + 1);
        float4 v;
        if (!odd) {
            v = make_float4(hi24(z0), lo24(z0), hi24(z1), lo24(z1));
        } else {
            const uint64_t z2 = pair_hash(key, (c >> 1) + 2);
            v = make_float4(lo24(z0), hi24(z1), lo24(z1), hi24(z2));
        }
        __stcs(dst + i, v);
    }
}
__global__ void __launch_bounds__(kThreads) rand_uniform_scalar_kernel(float* __restrict__ dst, int64_t first, int64_t n, uint64_t key, uint64_t offset) {
    for (int64_t i = first + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        dst[i] = uniform_at(key, offset + static_cast<uint64_t>(i));
}
static uint64_t host_mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

}  // namespace

extern "C" {

ctk_status ctk_compare_f32(int cmp, int form, const float* a, const float* b, float scalar, unsigned char* out, int64_t n, void* stream) {
    CTK_RANGE("ctk_compare_f32");
    CTK_REQUIRE(n >= 0, "ctk_compare_f32: negative size");
    if (n == 0) return CTK_OK;
    CTK_REQUIRE(a && out && (form != CTK_CMP_TENSOR || b), "ctk_compare_f32: null pointer");
    cudaStream_t st = as_stream(stream);
    switch (cmp) {
        case CTK_CMP_GT: return compare_form<CTK_CMP_GT>(form, a, b, scalar, out, n, st);
        case CTK_CMP_LT: return compare_form<CTK_CMP_LT>(form, a, b, scalar, out, n, st);
        case CTK_CMP_EQ: return compare_form<CTK_CMP_EQ>(form, a, b, scalar, out, n, st);
        case CTK_CMP_GE: return compare_form<CTK_CMP_GE>(form, a, b, scalar, out, n, st);
        case CTK_CMP_LE: return compare_form<CTK_CMP_LE>(form, a, b, scalar, out, n, st);
        case CTK_CMP_NE: return compare_form<CTK_CMP_NE>(form, a, b, scalar, out, n, st);
        default: return fail(CTK_ERR_INVALID, "ctk_compare_f32: cmp must be GT/LT/EQ/GE/LE/NE");
    }
}

ctk_status ctk_cast_f32(int dtype, const float* src, void* dst, int64_t n, void* stream) {
    CTK_RANGE("ctk_cast_f32");
    CTK_REQUIRE(n >= 0, "ctk_cast_f32: negative size");
    if (n == 0) return CTK_OK;
    CTK_REQUIRE(src && dst, "ctk_cast_f32: null pointer");
    cudaStream_t st = as_stream(stream);
    switch (dtype) {
        case CTK_DTYPE_F64: return launch_cast<double>(src, static_cast<double*>(dst), n, st);
        case CTK_DTYPE_I32: return launch_cast<int>(src, static_cast<int*>(dst), n, st);
        case CTK_DTYPE_I64: return launch_cast<long long>(src, static_cast<long long*>(dst), n, st);
        case CTK_DTYPE_BOOL: return launch_cast<unsigned char>(src, static_cast<unsigned char*>(dst), n, st);
        default: return fail(CTK_ERR_INVALID, "ctk_cast_f32: dtype must be double / int32 / int64 / bool");
    }
}

ctk_status ctk_fill_dtype(int dtype, void* dst, double value, int64_t n, void* stream) {
    CTK_RANGE("ctk_fill_dtype");
    CTK_REQUIRE(n >= 0, "ctk_fill_dtype: negative size");
    if (n == 0) return CTK_OK;
    CTK_REQUIRE(dst, "ctk_fill_dtype: null pointer");
    cudaStream_t st = as_stream(stream);
    const int grid = ctk_stream_grid(n, kThreads, 8);
    switch (dtype) {
        case CTK_DTYPE_F32: fill_typed_kernel<float><<<grid, kThreads, 0, st>>>(static_cast<float*>(dst), static_cast<float>(value), n); break;
        case CTK_DTYPE_F64: fill_typed_kernel<double><<<grid, kThreads, 0, st>>>(static_cast<double*>(dst), value, n); break;
        case CTK_DTYPE_I32: fill_typed_kernel<int><<<grid, kThreads, 0, st>>>(static_cast<int*>(dst), static_cast<int>(value), n); break;
        case CTK_DTYPE_I64: fill_typed_kernel<long long><<<grid, kThreads, 0, st>>>(static_cast<long long*>(dst), static_cast<long long>(value), n); break;
        case CTK_DTYPE_BOOL: fill_typed_kernel<unsigned char><<<grid, kThreads, 0, st>>>(static_cast<unsigned char*>(dst), value != 0.0, n); break;
        default: return fail(CTK_ERR_INVALID, "ctk_fill_dtype: unknown dtype");
    }
    CTK_LAUNCH_CHECK("fill_typed_kernel");
    return CTK_OK;
}

ctk_status ctk_rand_uniform_f32(float* dst, int64_t n, uint64_t seed, uint64_t offset, void* stream) {
    CTK_RANGE("ctk_rand_uniform_f32");
    CTK_REQUIRE(n >= 0, "ctk_rand_uniform_f32: negative size");
    if (n == 0) return CTK_OK;
    CTK_REQUIRE(dst, "ctk_rand_uniform_f32: null pointer");
    cudaStream_t st = as_stream(stream);
    const uint64_t key = host_mix64(seed ^ 0x9E3779B97F4A7C15ull);
    const int64_t n4 = (reinterpret_cast<uintptr_t>(dst) & 15u) == 0 ? n / 4 : 0;
    if (n4 > 0) {
        const int64_t per_cta = kThreads * kUnroll;
        rand_uniform_vec_kernel<<<static_cast<unsigned>((n4 + per_cta - 1) / per_cta), kThreads, 0, st>>>(reinterpret_cast<float4*>(dst), n4, key, offset);
        CTK_LAUNCH_CHECK("rand_uniform_vec_kernel");
    }
    if (n4 * 4 < n) {
        rand_uniform_scalar_kernel<<<ctk_stream_grid(n - n4 * 4, kThreads, 8), kThreads, 0, st>>>(dst, n4 * 4, n, key, offset);
        CTK_LAUNCH_CHECK("rand_uniform_scalar_kernel");
    }
    return CTK_OK;
}

}  // extern "C"
