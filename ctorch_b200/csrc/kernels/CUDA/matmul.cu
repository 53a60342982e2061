// MatMul for sm_100a: C[m,n] = sum_l A[i*sa0 + l*sa1] * B[l*sb0 + j*sb1], fp32 in / fp32 out.
//
// Replaces MatMul_BASIC_kernel (src/kernels/CPU-BASIC/MatMul_BASIC_kernel.cpp:13-57).  Strides are
// taken as that kernel reads them, so C = A.B, dA = dC.B^T and dB = A^T.dC (src/AutoDiff.cpp:
// 1702-1704, 1808-1810, where B^T / A^T are stride-swapped views) are one entry point.
//
// Tensor-core path (the product): persistent, warp-specialised tcgen05 kernels.
//   warp 0     : TMA producer -- per-CTA cp.async.bulk.tensor loads into 128B-swizzled shared
//                memory, a ring of stages guarded by full/empty mbarriers;
//   warp 1     : MMA issuer -- one elected lane issues tcgen05.mma.kind::tf32 from shared-memory
//                descriptors into a TMEM accumulator, tcgen05.commit frees the stage; owns the TMEM
//                allocation (two accumulators, so the epilogue of tile i overlaps the main loop of
//                tile i+1);
//   warps 2..5 : epilogue -- tcgen05.ld the accumulator (each warp its 32-lane quarter), store C.
//   Two kernels share that skeleton: the CTA-pair kernel (a cluster of two CTAs, cta_group::2,
//   M=256 N=256 K=8 per instruction, each CTA staging half of A's rows and half of B's columns) for
//   every product with m, n > 128, and the single-CTA kernel (M=128, N in {64,128,256}) for the rest.
//   Either operand may be K-major (row of K contiguous) or MN-major (row of M/N contiguous): the
//   major-ness goes into the instruction descriptor and the shared-memory descriptors, no
//   transposed copy is made.  M/N/K tails are zero-filled by TMA and masked at the store.
//   The tiles of a last wave that would occupy at most half the machine are computed as two halves
//   of K each, by two CTAs (pairs): the first half stores its sum, the second adds its own to it once
//   a flag says the first is done -- a fixed order, so the result is the same from call to call.
//   The sum over k is kept in TMEM for at most 2048 terms at a time (fewer for narrow tiles); longer
//   sums are added up in fp32 by the epilogue (the tensor core truncates when it adds into its
//   accumulator).
//   TF32 mode multiplies the fp32 operands as they are (the tensor core reads the top 19 bits).
//   The fp32-accurate mode (CTK_MATMUL_3XTF32) multiplies hi.hi + lo.hi + hi.lo, hi the TF32 part of an
//   operand and lo = x - hi: hi.hi as kind::tf32, the two small terms as kind::tf32 too ("3xTF32") or, by
//   default, as kind::f16 on bf16 roundings of their factors, into the same TMEM accumulator; the dropped
//   term lo.lo is ~2^-20 of the product, i.e. fp32-level accuracy.  Where TMA can read the operand itself
//   it IS hi (the tensor core ignores the low 13 mantissa bits) and only the small terms' arrays are
//   written -- to a scratch buffer or one the caller keeps with the operand; elsewhere hi = tf32(x)
//   rounded to nearest goes into an array of its own (see SplitOut).  MN-major operands whose contiguous
//   extent is a multiple of 64 are fetched as 3-D tensors, one copy per array and stage.
//   Narrow outputs (N <= 16, long K) and short contractions (K <= 16) do not use the tensor cores at all:
//   see narrow_rows_kernel / narrow_cols_kernel and skinny_k_kernel.
//   Every mbarrier wait is bounded; a wait that runs out sets a device status word, the CTA drains
//   its copies, frees its TMEM and returns.
//
// CUDA-core path: a plain fp32-FMA tiled kernel for operands without a unit stride, for TF32 mode on
// operands TMA cannot address in place, and on request (mode FP32_SIMT).
#include <cuda.h>
#include <cuda_bf16.h>
#include <math.h>
#include <cstdlib>

#include <mutex>
#include <vector>

#include "common.cuh"

namespace {
using namespace ctk;

__device__ int g_tc_status = 0;  // first bounded wait that ran out: (role << 8) | barrier id, else 0

// ================================================================================================
// CUDA-core path
// ================================================================================================
constexpr int SM_TILE = 64, SM_BK = 16, SM_THREADS = 256;

__global__ void __launch_bounds__(SM_THREADS) simt_matmul_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                                  float* __restrict__ c, int64_t m, int64_t n, int64_t k,
                                                                  int64_t sa0, int64_t sa1, int64_t sb0, int64_t sb1) {
    __shared__ float As[SM_BK][SM_TILE + 4];
    __shared__ float Bs[SM_BK][SM_TILE + 4];
    const int tid = threadIdx.x;
    const int64_t m0 = static_cast<int64_t>(blockIdx.y) * SM_TILE, n0 = static_cast<int64_t>(blockIdx.x) * SM_TILE;
    const int tx = tid % 16, ty = tid / 16;  // 16 x 16 threads, 4 x 4 outputs each
    float acc[4][4] = {};
    const bool a_kfast = (sa1 == 1), b_nfast = (sb1 == 1);
    for (int64_t k0 = 0; k0 < k; k0 += SM_BK) {
        // A tile: 64 rows x 16 k, each thread 4 elements; the fastest-varying thread index follows
        // the contiguous dimension so global loads coalesce for both major-nesses.
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            int i, l;
            if (a_kfast) { l = tid % SM_BK; i = tid / SM_BK + r * (SM_THREADS / SM_BK); }
            else { i = tid % SM_TILE; l = tid / SM_TILE + r * (SM_THREADS / SM_TILE); }
            const int64_t gi = m0 + i, gl = k0 + l;
            As[l][i] = (gi < m && gl < k) ? __ldg(a + gi * sa0 + gl * sa1) : 0.0f;
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            int j, l;
            if (b_nfast) { j = tid % SM_TILE; l = tid / SM_TILE + r * (SM_THREADS / SM_TILE); }
            else { l = tid % SM_BK; j = tid / SM_BK + r * (SM_THREADS / SM_BK); }
            const int64_t gj = n0 + j, gl = k0 + l;
            Bs[l][j] = (gj < n && gl < k) ? __ldg(b + gl * sb0 + gj * sb1) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int l = 0; l < SM_BK; ++l) {
            float av[4], bv[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) { av[u] = As[l][ty * 4 + u]; bv[u] = Bs[l][tx * 4 + u]; }
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int v = 0; v < 4; ++v) acc[u][v] = fmaf(av[u], bv[v], acc[u][v]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int64_t gi = m0 + ty * 4 + u;
        if (gi >= m) continue;
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            const int64_t gj = n0 + tx * 4 + v;
            if (gj < n) c[gi * n + gj] = acc[u][v];
        }
    }
}

// ================================================================================================
// hi/lo split for 3xTF32
// ================================================================================================
// x with its low 13 mantissa bits cleared: the value the tensor core uses when it is handed x as a TF32 operand.
__device__ __forceinline__ float to_tf32_trunc(float x) { return __uint_as_float(__float_as_uint(x) & 0xFFFFE000u); }
__device__ __forceinline__ float to_tf32_rna(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

// Where the split of an [outer, inner] operand goes: arrays of pitch `pitch` elements (a multiple
// of 8, so that rows of every array start on 16 bytes whatever the source pitch was; pad columns are
// never read: the tensor maps' extent stays `inner`).
//   correction terms on the TF32 path (variant 0):  hi = tf32(x) and lo = tf32(x - hi), fp32 each;
//   correction terms on the bf16 path (variant 1):  hi = tf32(x) as fp32, h16 = bf16(hi), l16 = bf16(x - hi).
// Where hi comes from.  The tensor core reads the top 19 bits of an fp32 operand and ignores the rest
// (measured: a TF32 product of raw operands equals, bit for bit, the product of the same operands with
// their low 13 mantissa bits cleared).  So where TMA can read the operand itself -- 16-byte aligned, rows a
// multiple of 16 bytes apart -- hi needs no array: the operand IS hi = trunc(x), the split has
// SplitOut::hi == nullptr and keeps only the small terms of x - trunc(x) (4 bytes per element written
// instead of 8).  Elsewhere (the 10-wide layer's 40-byte rows) hi = x rounded to nearest is written to
// an array of its own as before.  [hi: 4 B, or none][p2: lo 4 B | h16 2 B + l16 2 B].
struct SplitOut {
    float* hi = nullptr;
    void* p2 = nullptr;  // lo (fp32) or h16 (bf16)
    void* p3 = nullptr;  // l16 (bf16), variant 1 only
    int variant = 0;
    int64_t pitch = 0;
};
__device__ __forceinline__ uint2 pack_bf16x4(float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 r;
    r.x = *reinterpret_cast<const uint32_t*>(&a);
    r.y = *reinterpret_cast<const uint32_t*>(&b);
    return r;
}
// The split of four consecutive elements x, stored at element offset `off` (a multiple of 4) of each array.
template <bool STREAMING>
__device__ __forceinline__ void store_split4(const SplitOut& o, int64_t off, float4 x) {
    float4 h, l;
    if (o.hi != nullptr) {
        h.x = to_tf32_rna(x.x); h.y = to_tf32_rna(x.y); h.z = to_tf32_rna(x.z); h.w = to_tf32_rna(x.w);
        if (STREAMING) __stcs(reinterpret_cast<float4*>(o.hi + off), h);
        else *reinterpret_cast<float4*>(o.hi + off) = h;
    } else {  // the operand itself is read as hi: what the tensor core sees of it
        h.x = to_tf32_trunc(x.x); h.y = to_tf32_trunc(x.y); h.z = to_tf32_trunc(x.z); h.w = to_tf32_trunc(x.w);
    }
    l.x = x.x - h.x; l.y = x.y - h.y; l.z = x.z - h.z; l.w = x.w - h.w;  // exact in fp32
    if (o.variant == 0) {
        l.x = to_tf32_rna(l.x); l.y = to_tf32_rna(l.y); l.z = to_tf32_rna(l.z); l.w = to_tf32_rna(l.w);
        if (STREAMING) __stcs(reinterpret_cast<float4*>(static_cast<float*>(o.p2) + off), l);
        else *reinterpret_cast<float4*>(static_cast<float*>(o.p2) + off) = l;
    } else {
        const uint2 h16 = pack_bf16x4(h), l16 = pack_bf16x4(l);
        if (STREAMING) {
            __stcs(reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(o.p2) + off), h16);
            __stcs(reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(o.p3) + off), l16);
        } else {
            *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(o.p2) + off) = h16;
            *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(o.p3) + off) = l16;
        }
    }
}
__device__ __forceinline__ void store_split1(const SplitOut& o, int64_t off, float x) {
    const float h = o.hi != nullptr ? to_tf32_rna(x) : to_tf32_trunc(x);
    if (o.hi != nullptr) o.hi[off] = h;
    if (o.variant == 0) {
        static_cast<float*>(o.p2)[off] = to_tf32_rna(x - h);
    } else {
        static_cast<__nv_bfloat16*>(o.p2)[off] = __float2bfloat16_rn(h);
        static_cast<__nv_bfloat16*>(o.p3)[off] = __float2bfloat16_rn(x - h);
    }
}

// x viewed as [outer, inner] with row pitch ld_in -> its split with row pitch out.pitch.
// One tile of 256 x 4 vectors per CTA: with this many bytes in flight per CTA and the hardware block
// scheduler walking memory in order, streaming kernels on B200 run above the plain-copy rate.
constexpr int SPLIT_THREADS = 256, SPLIT_UNROLL = 4;
__global__ void __launch_bounds__(SPLIT_THREADS) split_tf32_vec_kernel(const float* __restrict__ x, SplitOut out, int64_t outer, int64_t inner4, int64_t ld_in) {
    const int64_t total = outer * inner4;
    const int64_t base = static_cast<int64_t>(blockIdx.x) * (SPLIT_THREADS * SPLIT_UNROLL) + threadIdx.x;
    float4 v[SPLIT_UNROLL];
    int64_t r[SPLIT_UNROLL], c4[SPLIT_UNROLL];
#pragma unroll
    for (int u = 0; u < SPLIT_UNROLL; ++u) {
        const int64_t i = base + u * SPLIT_THREADS;
        if (i < total) {
            r[u] = i / inner4;
            c4[u] = i - r[u] * inner4;
            v[u] = __ldg(reinterpret_cast<const float4*>(x + r[u] * ld_in) + c4[u]);
        }
    }
#pragma unroll
    for (int u = 0; u < SPLIT_UNROLL; ++u) {
        const int64_t i = base + u * SPLIT_THREADS;
        if (i < total) store_split4<false>(out, r[u] * out.pitch + 4 * c4[u], v[u]);
    }
}
// The SGD update of a weight matrix with its split rewritten in the same pass: p -= g*lr as in
// ctk_sgd_update_f32 (one fused multiply-add), then the split of the NEW value for the product the
// weights enter next.  p viewed [outer, inner] with pitch ld_in, g contiguous.
__global__ void __launch_bounds__(SPLIT_THREADS) sgd_split_vec_kernel(float* __restrict__ p, const float* __restrict__ g, float lr, SplitOut out,
                                                                      int64_t outer, int64_t inner4, int64_t ld_in) {
    const int64_t total = outer * inner4;
    const int64_t base = static_cast<int64_t>(blockIdx.x) * (SPLIT_THREADS * SPLIT_UNROLL) + threadIdx.x;
    float4 v[SPLIT_UNROLL], d[SPLIT_UNROLL];
    int64_t r[SPLIT_UNROLL], c4[SPLIT_UNROLL];
#pragma unroll
    for (int u = 0; u < SPLIT_UNROLL; ++u) {
        const int64_t i = base + u * SPLIT_THREADS;
        if (i < total) {
            r[u] = i / inner4;
            c4[u] = i - r[u] * inner4;
            v[u] = *(reinterpret_cast<const float4*>(p + r[u] * ld_in) + c4[u]);
            d[u] = __ldcs(reinterpret_cast<const float4*>(g) + i);
        }
    }
#pragma unroll
    for (int u = 0; u < SPLIT_UNROLL; ++u) {
        const int64_t i = base + u * SPLIT_THREADS;
        if (i < total) {
            float4 x;
            x.x = fmaf(-d[u].x, lr, v[u].x); x.y = fmaf(-d[u].y, lr, v[u].y); x.z = fmaf(-d[u].z, lr, v[u].z); x.w = fmaf(-d[u].w, lr, v[u].w);
            *(reinterpret_cast<float4*>(p + r[u] * ld_in) + c4[u]) = x;
            store_split4<false>(out, r[u] * out.pitch + 4 * c4[u], x);
        }
    }
}
// Any pitch, any alignment (e.g. the 10-class layer's rows of 40 bytes): one element per thread.
__global__ void __launch_bounds__(SPLIT_THREADS) split_tf32_scalar_kernel(const float* __restrict__ x, SplitOut out, int64_t outer, int64_t inner, int64_t ld_in) {
    const int64_t total = outer * inner;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t r = i / inner, c = i - r * inner;
        store_split1(out, r * out.pitch + c, __ldg(x + r * ld_in + c));
    }
}

// ================================================================================================
// tcgen05 path
// ================================================================================================
namespace tc {

constexpr int BM = 128;
constexpr int BK = 32;               // 32 fp32 = 128 bytes = one swizzle row
constexpr int UMMA_K = 8;            // K of one tcgen05.mma.kind::tf32
constexpr int THREADS = 192;         // warp 0 TMA, warp 1 MMA, warps 2-5 epilogue
constexpr int SMEM_BUDGET = 200 * 1024;
constexpr uint32_t WAIT_LIMIT = 1u << 20;  // polls per bounded wait (each poll may itself block a few us)
// Longest run of k accumulated in TMEM before the sum moves to fp32 (see Params::chunk_kb), by tile
// width.  The error of a chunk grows with its length -- measured on N(0,1) operands, normwise against
// the largest entry: 3.0e-5 at 4096, 1.5e-5 at 2048, 0.8e-5 at 1024; several times that where the
// products of a sum share a sign or nearly cancel, as in the weight gradients of an untrained network.
// Its cost is one more drain of the accumulator, during which the tensor pipe idles ~3.4 us per
// 128 x 256 accumulator: one full training step of 784-4096-4096-4096-10 at batch 8192 ran 6.01 ms with
// 4096, 6.29 ms with 2048 and 6.65 ms with 1024 for the wide tiles, its logits 6.2e-5 / 3.3e-5 / 1.9e-5
// from float64.  2048 keeps every gradient of that step within 1e-4 with room to spare; the narrow tiles
// of the 10-class layer, whose weight gradient adds products of one sign that nearly cancel in the end,
// use 1024 (at 256 the layer's two products cost 0.4 ms of a 5.3 ms step in drains alone).
constexpr int chunk_k_for(int bn) { return bn >= 256 ? 2048 : 1024; }
// (With the correction terms on the bf16 path an accumulator sees four instructions per 16 terms instead
// of six -- K = 16 per bf16 instruction -- i.e. two thirds of the truncations: at 4096^3 its error is
// 1.0e-5 where the TF32 corrections give 1.6e-5 with the same chunks.)

template <int BN, int TERMS>
struct Cfg {
    static constexpr int A_BYTES = BM * BK * 4;
    static constexpr int B_BYTES = BN * BK * 4;
    static constexpr int STAGE_BYTES = (TERMS == 1 ? 1 : 2) * (A_BYTES + B_BYTES);  // fp32 tiles, plus as many bytes of lo / 16-bit copies
    static constexpr int STAGES_RAW = SMEM_BUDGET / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
    static constexpr int TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;  // two accumulators, power of two
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;  // + slack for 1024-byte alignment
    static_assert(STAGES >= 2, "need at least two stages");
    static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0 && TMEM_COLS <= 512, "TMEM columns must be a power of two <= 512");
};

struct Params {
    int64_t m, n, k;
    int tiles_m, tiles_n, num_kb;
    float* c;
    int vec_store;    // n % 4 == 0 and c 16-byte aligned
    int whole_tiles;  // tiles [0, whole_tiles) are computed whole; each later tile as two K-halves
    // One word per (halved tile, CTA of the pair, epilogue warp), zero at launch: the warp that owns
    // these rows in the FIRST half sets it after its last store; the same warp of the second half
    // waits for it before it reads C.
    int* half_flags;
    // The tensor core adds each K=8 step into its fp32 accumulator with truncation, so the error of a
    // sum kept in TMEM grows in proportion to the number of steps (measured, normwise against the
    // result's largest entry, N(0,1) operands: 3e-5 after 4096 terms, 5e-4 after 65536).  A tile's
    // k-blocks are therefore accumulated in chunks of at most chunk_kb blocks; every chunk starts
    // from a zero accumulator and the epilogue adds the chunks in fp32 with round-to-nearest
    // (C += chunk, same thread, in order; the running sum waits in L2).
    int chunk_kb;
    // Epilogue of the fused forms (all optional; whole tiles only): c = [relu](acc + bias[col]), then
    // c *= (mask > 0 ? 1 : 0) with mask an [m, n] array of pitch n (ReLU's backward rule applied to a
    // gradient product), and the split of c written next to it (SplitOut: [m, out.pitch] arrays) for the
    // products c enters next.
    const float* bias;
    int relu;
    const float* mask;
    SplitOut out;  // out.p2 == nullptr: no split
    // An MN-major operand whose contiguous extent is a multiple of 64 comes with 3-D tensor maps
    // {128 bytes of the MN index, k, 128-byte group}: one copy per array and stage fetches all of a tile's
    // column groups (box {32 | 64 elements, 32, groups}) where the 2-D maps need one copy per group.
    int a_grouped, b_grouped;
};

// A unit of work: a whole output tile, or one K-half of a tile of the last, partly filled wave.
// Halves let twice as many SMs work on that wave.  The first half (part 0) writes its sum to C like
// a whole tile would; the second (part 1) adds its chunks to what part 0 left there, after part 0's
// flag.  Units 2t and 2t+1 are neighbours in the unit order, so the two halves of a tile run on
// different CTAs (pairs) at the same time whenever the grid has more than one; a wait never points
// at work queued behind the waiter.
struct Unit {
    int tile, kb0, kb1;
    bool half;
    int part;   // halves: 0 = first half of K, 1 = second
    int slot;   // halves: index of the tile among the halved ones
};
__device__ __forceinline__ int unit_count(const Params& P) {
    const int tiles = P.tiles_m * P.tiles_n;
    return P.whole_tiles + 2 * (tiles - P.whole_tiles);
}
__device__ __forceinline__ Unit unit_of(int u, const Params& P) {
    if (u < P.whole_tiles) return Unit{u, 0, P.num_kb, false, 0, 0};
    const int v = u - P.whole_tiles;
    const int mid = (P.num_kb + 1) >> 1;
    return (v & 1) ? Unit{P.whole_tiles + (v >> 1), mid, P.num_kb, true, 1, v >> 1} : Unit{P.whole_tiles + (v >> 1), 0, mid, true, 0, v >> 1};
}
// Second half: wait (bounded) until the first half's warp for the same rows has published its sum.
__device__ __forceinline__ bool wait_first_half(const int* flag, int lane, volatile int* abort_flag, int code) {
    int ok = 1;
    if (lane == 0) {
        ok = 0;
        for (uint32_t i = 0; i < (1u << 22); ++i) {
            int v;
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
            if (v != 0) { ok = 1; break; }
            if ((i & 63u) == 63u) {
                if (*abort_flag) break;
                __nanosleep(128);
            }
        }
        if (!ok && !*abort_flag) {
            *abort_flag = 1;
            atomicCAS(&g_tc_status, 0, code);
        }
    }
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
// First half: every lane's stores of this warp's rows are done; make them visible, then raise the flag.
__device__ __forceinline__ void publish_first_half(int* flag, int lane) {
    __threadfence();
    __syncwarp();
    if (lane == 0) asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(flag), "r"(1) : "memory");
}

// Tile order.  Tiles are numbered band by band: a band is TILE_BAND tile columns wide and is walked
// row after row, so the tiles that run at the same time (one wave of the persistent grid) form a
// compact block of about 9 x 8 tiles instead of a few full tile rows.  A wave then reads ~17 instead
// of ~21 operand panels, and -- what matters for DRAM -- a band's B panels (8 x 256 columns) stay in
// L2 while A streams past them once per band, where row-major order re-read all of B for every wave.
constexpr int TILE_BAND = 8;
__host__ __device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
    const int band = tile / (TILE_BAND * tiles_m);
    const int first_col = band * TILE_BAND;
    const int width = tiles_n - first_col < TILE_BAND ? tiles_n - first_col : TILE_BAND;
    const int r = tile - band * (TILE_BAND * tiles_m);
    tm = r / width;
    tn = first_col + r % width;
}

// ---- PTX wrappers --------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  On running out (or when another role already gave up) records `code` and raises
// the CTA-wide abort flag; every role then leaves its loops and the CTA tears down normally.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code, uint32_t limit = WAIT_LIMIT) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u) {
            if (*abort_flag) return false;
            __nanosleep(64);
        }
    }
    *abort_flag = 1;
    atomicCAS(&g_tc_status, 0, code);
    return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor (sm_100 format): start address >> 4 in bits [0,14), leading byte
// offset >> 4 in [16,30), stride byte offset >> 4 in [32,46), version 1 in [46,48), swizzle code
// in [61,64).
//   K-major tile  [rows][32 fp32], 128-byte swizzle (16-byte chunks XOR row%8, code 2): rows 128 B
//                 apart, 8-row groups 1024 B apart -> SBO = 1024; a K=8 step advances the start
//                 address by 32 B inside the swizzle row.
//   MN-major tile [k][32 fp32 of M/N] in 32-wide column groups.  For 32-bit operands the tensor
//                 core only takes the "128-byte swizzle with 32-byte atoms" layout (32-byte chunks
//                 XOR k%4, code 1; TMA writes it with SWIZZLE_128B_ATOM_32B): 4 k-rows (512 B) form
//                 one atom -> SBO = 512, column groups are 4096 B apart -> LBO = 4096; a K=8 step
//                 advances the start address by 1024 B.
//   16-bit operands (the bf16 copies of the correction terms):
//   K-major tile  [rows][32 bf16] = 64-byte rows, 64-byte swizzle (16-byte chunks XOR (row/2)%4, code
//                 4): 8-row groups 512 B apart -> SBO = 512; a K=16 step advances the start address by 32 B.
//   MN-major tile [k][64 bf16 of M/N] in 64-wide column groups, plain 128-byte swizzle (code 2): 8 k-rows
//                 (1024 B) form one atom -> SBO = 1024, column groups are 4096 B apart -> LBO = 4096; a
//                 K=16 step advances the start address by 2048 B.
constexpr uint32_t kSwizzle128B = 2, kSwizzle128BAtom32B = 1, kSwizzle64B = 4;
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t swizzle_code) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(swizzle_code) << 61;
    return d;
}

// Instruction descriptor: D fp32 (bits [4,6) = 1), A/B format in [7,10) and [10,13) (kind::tf32: 2 =
// TF32; kind::f16: 1 = BF16), A/B major-ness in bits 15/16 (1 = MN-major), N >> 3 in [17,23), M >> 4
// in [24,29).
constexpr uint32_t kFmtTF32 = 2, kFmtBF16 = 1;
__host__ __device__ constexpr uint32_t make_idesc_fmt(uint32_t fmt, int m, int n, bool a_mn_major, bool b_mn_major) {
    return (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(a_mn_major) << 15) |
           (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
           (static_cast<uint32_t>(m >> 4) << 24);
}
__host__ __device__ constexpr uint32_t make_idesc(int n, bool a_mn_major, bool b_mn_major) { return make_idesc_fmt(kFmtTF32, BM, n, a_mn_major, b_mn_major); }

// ---- one pipeline stage: where the operand tiles sit, how they are loaded, how they are multiplied ----
// TERMS = 1: TF32, the fp32 operands as they are.
// TERMS = 3: 3xTF32 -- hi = tf32(x), lo = tf32(x - hi) of both operands; lo.hi + hi.lo + hi.hi.
// TERMS = 2: TF32 + 2 x BF16 -- hi as above, and 16-bit copies h16 = bf16(hi), l16 = bf16(x - hi):
//            l16.h16 + h16.l16 on the bf16 path (twice the TF32 rate) + hi.hi on the TF32 path.  The two
//            correction terms are 2^-11 of the main one, so rounding their factors to bf16 (2^-9) leaves
//            2^-20 of the product, the order of the lo.lo term every variant drops; the stage holds the
//            same 8 bytes per operand element as TERMS = 3, the tensor pipe does 2 units of work instead of 3.
// Stage layout (A_B / B_B = bytes of one fp32 tile): TERMS 3: [A hi][A lo][B hi][B lo];
// TERMS 2: [A hi][A h16][A l16][B hi][B h16][B l16]; TERMS 1: [A][B].
template <int TERMS, int A_B, int B_B>
struct StageLayout {
    static constexpr int BYTES = (TERMS == 1 ? 1 : 2) * (A_B + B_B);
    static constexpr uint32_t a_hi = 0, a_lo = A_B;                 // TERMS 3
    static constexpr uint32_t a_h16 = A_B, a_l16 = A_B + A_B / 2;   // TERMS 2
    static constexpr uint32_t b_hi = (TERMS == 1 ? 1 : 2) * A_B;
    static constexpr uint32_t b_lo = b_hi + B_B;
    static constexpr uint32_t b_h16 = b_hi + B_B, b_l16 = b_hi + B_B + B_B / 2;
};

// The loads of one stage.  maps: a[0..2], b[0..2] = {hi, lo, -} (TERMS 3) or {hi, h16, l16} (TERMS 2).
// tma(dst, map, c0, c1) issues one tiled copy whose completion is counted on the stage's barrier.
template <int TERMS, bool A_MN, bool B_MN, int A_ROWS, int B_ROWS, typename Tma, typename Tma3>
__device__ __forceinline__ void load_stage(uint32_t base, const CUtensorMap* const (&ma)[3], const CUtensorMap* const (&mb)[3], int m0, int n0, int k0,
                                           bool a_grouped, bool b_grouped, Tma tma, Tma3 tma3) {
    using L = StageLayout<TERMS, A_ROWS * BK * 4, B_ROWS * BK * 4>;
    // wide: elements per 128-byte column group (32 fp32, 64 bf16)
    auto tile = [&](uint32_t dst, const CUtensorMap* map, bool mn, bool grouped, int rows, int r0, int wide) {
        if (!mn) {
            tma(dst, map, k0, r0);
        } else if (grouped) {
            tma3(dst, map, 0, k0, r0 / wide);
        } else {
            for (int g = 0; g < rows / wide; ++g) tma(dst + g * 4096, map, r0 + wide * g, k0);
        }
    };
    tile(base + L::a_hi, ma[0], A_MN, a_grouped, A_ROWS, m0, 32);
    tile(base + L::b_hi, mb[0], B_MN, b_grouped, B_ROWS, n0, 32);
    if (TERMS == 3) {
        tile(base + L::a_lo, ma[1], A_MN, a_grouped, A_ROWS, m0, 32);
        tile(base + L::b_lo, mb[1], B_MN, b_grouped, B_ROWS, n0, 32);
    }
    if (TERMS == 2) {
        tile(base + L::a_h16, ma[1], A_MN, a_grouped, A_ROWS, m0, 64);
        tile(base + L::a_l16, ma[2], A_MN, a_grouped, A_ROWS, m0, 64);
        tile(base + L::b_h16, mb[1], B_MN, b_grouped, B_ROWS, n0, 64);
        tile(base + L::b_l16, mb[2], B_MN, b_grouped, B_ROWS, n0, 64);
    }
}

// The MMAs of one k-block (32 terms of the sum) into the accumulator at d_tmem; fresh: this k-block
// opens a new accumulator (its first instruction overwrites).  The small terms go first.
// mma32 / mma16(d, a_desc, b_desc, idesc, accumulate) issue kind::tf32 / kind::f16.
template <int TERMS, bool A_MN, bool B_MN, int A_ROWS, int B_ROWS, typename Mma32, typename Mma16>
__device__ __forceinline__ void issue_kblock(uint32_t base, uint32_t d_tmem, uint32_t idesc32, uint32_t idesc16, bool fresh, Mma32 mma32, Mma16 mma16) {
    using L = StageLayout<TERMS, A_ROWS * BK * 4, B_ROWS * BK * 4>;
    constexpr uint32_t a_lbo = A_MN ? 4096u : 0u, b_lbo = B_MN ? 4096u : 0u;
    uint32_t acc = fresh ? 0u : 1u;
    if (TERMS == 2) {
        constexpr uint32_t a_sbo = A_MN ? 1024u : 512u, b_sbo = B_MN ? 1024u : 512u;
        constexpr uint32_t a_sw = A_MN ? kSwizzle128B : kSwizzle64B, b_sw = B_MN ? kSwizzle128B : kSwizzle64B;
#pragma unroll
        for (int ks = 0; ks < BK / 16; ++ks) {
            const uint32_t a_step = A_MN ? ks * 2048u : ks * 32u, b_step = B_MN ? ks * 2048u : ks * 32u;
            const uint64_t a_h = make_desc(base + L::a_h16 + a_step, a_lbo, a_sbo, a_sw), a_l = make_desc(base + L::a_l16 + a_step, a_lbo, a_sbo, a_sw);
            const uint64_t b_h = make_desc(base + L::b_h16 + b_step, b_lbo, b_sbo, b_sw), b_l = make_desc(base + L::b_l16 + b_step, b_lbo, b_sbo, b_sw);
            mma16(d_tmem, a_l, b_h, idesc16, acc);
            mma16(d_tmem, a_h, b_l, idesc16, 1u);
            acc = 1u;
        }
    }
    constexpr uint32_t a_sbo = A_MN ? 512u : 1024u, b_sbo = B_MN ? 512u : 1024u;
    constexpr uint32_t a_sw = A_MN ? kSwizzle128BAtom32B : kSwizzle128B, b_sw = B_MN ? kSwizzle128BAtom32B : kSwizzle128B;
#pragma unroll
    for (int ks = 0; ks < BK / UMMA_K; ++ks) {
        const uint32_t a_step = A_MN ? ks * 1024u : ks * 32u, b_step = B_MN ? ks * 1024u : ks * 32u;
        const uint64_t a_hi = make_desc(base + L::a_hi + a_step, a_lbo, a_sbo, a_sw);
        const uint64_t b_hi = make_desc(base + L::b_hi + b_step, b_lbo, b_sbo, b_sw);
        if (TERMS == 3) {
            const uint64_t a_lo = make_desc(base + L::a_lo + a_step, a_lbo, a_sbo, a_sw);
            const uint64_t b_lo = make_desc(base + L::b_lo + b_step, b_lbo, b_sbo, b_sw);
            mma32(d_tmem, a_lo, b_hi, idesc32, acc);
            mma32(d_tmem, a_hi, b_lo, idesc32, 1u);
            acc = 1u;
        }
        mma32(d_tmem, a_hi, b_hi, idesc32, acc);
        acc = 1u;
    }
}

// One 32-column chunk of one accumulator row (this lane's) on its way to memory.
constexpr int STAGE_PITCH = 36;  // floats per staged row: 16-byte aligned, conflict-free for 128-bit accesses
using EpilogueStage = float[32][STAGE_PITCH];

// What a lane prefetches for one whole 32 x 32 chunk in the layout it STORES in (row sub + 4i of the
// chunk, 16 bytes at column c4): the eight pieces of the fourth array the chunk's epilogue reads -- the
// running sum of the earlier K-chunks, or else the mask (the ReLU output whose backward rule the
// epilogue applies).  Loaded one chunk ahead of their use, so that their DRAM latency overlaps the
// TMEM load and staging of the chunk before.
struct SideRegs {
    float4 v[8];
};
__device__ __forceinline__ bool chunk_is_whole(const Params& P, int64_t col0) {
    return P.vec_store && col0 + 32 <= P.n;
}
// first / last: this is the unit's first / last K-chunk.  Two arrays may be read beside the accumulator:
// the running sum parked in C by the chunks before (every chunk but the first) and the mask (the last
// chunk).  Each has its own registers, so both are in flight a column chunk ahead.
__device__ __forceinline__ void load_pieces(const float* arr, const Params& P, int64_t row_base, int lane, int64_t col0, SideRegs& out, bool coherent) {
    const int sub = lane >> 3, c4 = (lane & 7) * 4;
    const float* src = arr + (row_base + sub) * P.n + col0 + c4;
    const int64_t step = 4 * P.n;
    const int rows_left = static_cast<int>(P.m - row_base < 32 ? P.m - row_base : 32);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        if (i * 4 + sub < rows_left) {
            // (a running sum may have been written by another SM -- the first half of a halved tile -- so it is read from L2)
            out.v[i] = coherent ? __ldcg(reinterpret_cast<const float4*>(src + i * step)) : __ldcs(reinterpret_cast<const float4*>(src + i * step));
        } else {
            out.v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
}
__device__ __forceinline__ void load_side(const Params& P, bool first, bool last, int64_t row_base, int lane, int64_t col0, SideRegs& sum, SideRegs& mask) {
    if (!chunk_is_whole(P, col0)) return;
    if (!first) load_pieces(P.c, P, row_base, lane, col0, sum, true);
    if (last && P.mask != nullptr) load_pieces(P.mask, P, row_base, lane, col0, mask, false);
}

// One 32 x 32 chunk of an accumulator leaves the CTA.  Each lane holds 32 columns of ITS row (the
// shape tcgen05.ld.32x32b delivers), so a direct store would write 16 bytes to each of 32 different
// lines per instruction.  Whole chunks therefore go through `stage` (one per epilogue warp): the lane
// writes its row there, and the warp reads it back with 8 lanes across a row, so that every store
// instruction writes 4 complete 128-byte lines.  All epilogue arithmetic happens in that store
// layout, one fp32 operation per element and step, in this order: + running sum of the earlier
// K-chunks; on the last chunk + bias, ReLU, x (mask > 0), store, hi/lo split of what was stored.
__device__ __forceinline__ void emit_chunk(const Params& P, bool half, bool first, bool last, int64_t row_base, int lane, int64_t col0,
                                           uint32_t (&r)[32], EpilogueStage& stage, const SideRegs& sd, const SideRegs& mk) {
    if (col0 >= P.n) return;  // same for the whole warp
    const int64_t row = row_base + lane;
    if (chunk_is_whole(P, col0)) {
        // lane -> (row sub + 4i of the chunk, 16 bytes at column c4): addresses once, then a fixed step
        const int sub = lane >> 3, c4 = (lane & 7) * 4;
        const int rows_left = static_cast<int>(P.m - row_base < 32 ? P.m - row_base : 32);
        float* cdst = P.c + (row_base + sub) * P.n + col0 + c4;
        const int64_t cstep = 4 * P.n;
        // A whole tile's running sum never leaves this warp before the last chunk, so it need not be in
        // C's layout: piece i of a lane's OWN accumulator row is parked at the address the final store
        // uses for its piece i -- the same coalesced lines, without the trip through shared memory (whose
        // bandwidth the tensor core's operand reads need).  Only the last chunk transposes.
        const bool parked = !half && rows_left == 32;
        if (parked && !first) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                r[4 * i] = __float_as_uint(__fadd_rn(__uint_as_float(r[4 * i]), sd.v[i].x));
                r[4 * i + 1] = __float_as_uint(__fadd_rn(__uint_as_float(r[4 * i + 1]), sd.v[i].y));
                r[4 * i + 2] = __float_as_uint(__fadd_rn(__uint_as_float(r[4 * i + 2]), sd.v[i].z));
                r[4 * i + 3] = __float_as_uint(__fadd_rn(__uint_as_float(r[4 * i + 3]), sd.v[i].w));
            }
        }
        if (parked && !last) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                *reinterpret_cast<float4*>(cdst + i * cstep) =
                    make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]), __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
            return;
        }
        const bool add_old = !first && !parked;  // (a parked sum has been added above)
#pragma unroll
        for (int v = 0; v < 8; ++v)
            *reinterpret_cast<float4*>(&stage[lane][4 * v]) =
                make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]), __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
        __syncwarp();
        const bool plain = !add_old && (!last || (P.bias == nullptr && !P.relu && P.mask == nullptr && P.out.p2 == nullptr));
        if (plain && last) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (i * 4 + sub < rows_left) __stcs(reinterpret_cast<float4*>(cdst + i * cstep), *reinterpret_cast<const float4*>(&stage[i * 4 + sub][c4]));
        } else if (plain) {  // the first of several chunks: read again by the next one, so no streaming hint
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (i * 4 + sub < rows_left) *reinterpret_cast<float4*>(cdst + i * cstep) = *reinterpret_cast<const float4*>(&stage[i * 4 + sub][c4]);
        } else {
            const bool biased = last && P.bias != nullptr, relu = last && P.relu, masked = last && P.mask != nullptr, split = last && P.out.p2 != nullptr;
            const int64_t soff = (row_base + sub) * P.out.pitch + col0 + c4, sstep = 4 * P.out.pitch;
            float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
            if (biased) bv = __ldg(reinterpret_cast<const float4*>(P.bias + col0 + c4));  // Add_BASIC_kernel's [N,H] + [H]
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (i * 4 + sub >= rows_left) continue;
                float4 x = *reinterpret_cast<const float4*>(&stage[i * 4 + sub][c4]);
                if (add_old) {  // the chunks before this one
                    const float4 o = sd.v[i];
                    x.x = __fadd_rn(x.x, o.x); x.y = __fadd_rn(x.y, o.y); x.z = __fadd_rn(x.z, o.z); x.w = __fadd_rn(x.w, o.w);
                }
                if (biased) { x.x += bv.x; x.y += bv.y; x.z += bv.z; x.w += bv.w; }
                if (relu) {    // ReLU_BASIC_kernel (NaN -> 0)
                    x.x = x.x > 0.0f ? x.x : 0.0f; x.y = x.y > 0.0f ? x.y : 0.0f; x.z = x.z > 0.0f ? x.z : 0.0f; x.w = x.w > 0.0f ? x.w : 0.0f;
                }
                if (masked) {  // g * (y > 0 ? 1 : 0): the backward rule of ReLU, y its output
                    const float4 y = mk.v[i];
                    x.x *= y.x > 0.0f ? 1.0f : 0.0f; x.y *= y.y > 0.0f ? 1.0f : 0.0f;
                    x.z *= y.z > 0.0f ? 1.0f : 0.0f; x.w *= y.w > 0.0f ? 1.0f : 0.0f;
                }
                if (last) __stcs(reinterpret_cast<float4*>(cdst + i * cstep), x);
                else *reinterpret_cast<float4*>(cdst + i * cstep) = x;  // read again by the next chunk: keep it in L2
                if (split) store_split4<true>(P.out, soff + i * sstep, x);
            }
        }
        __syncwarp();  // the stage is free again
        return;
    }
    if (row >= P.m) return;
    float* crow = P.c + row * P.n;
    // a ragged chunk (or an unaligned C): element by element, the same operations in the same order
#pragma unroll
    for (int v = 0; v < 32; ++v)
        if (col0 + v < P.n) {
            float x = __uint_as_float(r[v]);
            if (!first) x = __fadd_rn(x, __ldcg(crow + col0 + v));
            if (last) {
                if (P.bias != nullptr) x += __ldg(P.bias + col0 + v);
                if (P.relu) x = x > 0.0f ? x : 0.0f;
                if (P.mask != nullptr) x *= P.mask[row * P.n + col0 + v] > 0.0f ? 1.0f : 0.0f;
            }
            crow[col0 + v] = x;
            if (last && P.out.p2 != nullptr) store_split1(P.out, row * P.out.pitch + col0 + v, x);
        }
}

// ---- the kernel ----------------------------------------------------------------------------------
// A_MN / B_MN: operand is MN-major (its M/N index is the contiguous one).  Tensor maps describe the
// operand as a 2-D array {contiguous dim, other dim}; box = {32, rows} for a K-major operand and
// {32, 32} per 32-wide column group for an MN-major one.
template <int BN, int TERMS, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(THREADS, 1)
tcgen05_matmul_kernel(const __grid_constant__ CUtensorMap map_a0, const __grid_constant__ CUtensorMap map_a1, const __grid_constant__ CUtensorMap map_a2,
                      const __grid_constant__ CUtensorMap map_b0, const __grid_constant__ CUtensorMap map_b1, const __grid_constant__ CUtensorMap map_b2,
                      const Params P) {
    using C = Cfg<BN, TERMS>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bars[2 * 8 + 4];  // full[8], empty[8], tmem_full[2], tmem_empty[2]
    __shared__ uint32_t tmem_base_slot;
    __shared__ __align__(16) EpilogueStage stages[4];  // one per epilogue warp
    __shared__ volatile int abort_flag;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (8 + s); };
    auto tfull_bar = [&](int a) { return bar0 + 8u * (16 + a); };
    auto tempty_bar = [&](int a) { return bar0 + 8u * (18 + a); };
    auto stage_addr = [&](int s) { return smem_base + s * C::STAGE_BYTES; };  // (layout inside: StageLayout)
    const CUtensorMap* const maps_a[3] = {&map_a0, &map_a1, &map_a2};
    const CUtensorMap* const maps_b[3] = {&map_b0, &map_b1, &map_b2};

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_tmap(&map_a0);
        prefetch_tmap(&map_b0);
        if (TERMS >= 2) { prefetch_tmap(&map_a1); prefetch_tmap(&map_b1); }
        if (TERMS == 2) { prefetch_tmap(&map_a2); prefetch_tmap(&map_b2); }
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_slot), C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    const int num_units = unit_count(P);

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            uint32_t issued = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
                const Unit U = unit_of(u, P);
                int tm, tn;
                tile_coords(U.tile, P.tiles_m, P.tiles_n, tm, tn);
                const int m0 = tm * BM, n0 = tn * BN;
                for (int kb = U.kb0; kb < U.kb1; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, &abort_flag, 0x100 | stage)) { ok = false; break; }
                    mbar_expect_tx(full_bar(stage), C::STAGE_BYTES);
                    const uint32_t fb = full_bar(stage);
                    load_stage<TERMS, A_MN, B_MN, BM, BN>(stage_addr(stage), maps_a, maps_b, m0, n0, kb * BK, P.a_grouped != 0, P.b_grouped != 0,
                                                         [&](uint32_t dst, const CUtensorMap* map, int c0, int c1) { tma_load_2d(dst, map, fb, c0, c1); },
                                                         [&](uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2) { tma_load_3d(dst, map, fb, c0, c1, c2); });
                    ++issued;
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) {
                // Gave up: let the copies already issued land before the CTA's shared memory goes away.
                const uint32_t pending = issued < static_cast<uint32_t>(C::STAGES) ? issued : C::STAGES;
                int s = stage;
                uint32_t ph = phase;
                for (uint32_t i = 0; i < pending; ++i) {
                    if (--s < 0) { s = C::STAGES - 1; ph ^= 1u; }
                    for (uint32_t spin = 0; spin < (1u << 16) && !mbar_try_wait(full_bar(s), ph); ++spin) __nanosleep(64);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BN, A_MN, B_MN), idesc16 = make_idesc_fmt(kFmtBF16, BM, BN, A_MN, B_MN);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
                const Unit U = unit_of(u, P);
                const int chunk_kb = P.chunk_kb;
                for (int c0 = U.kb0; c0 < U.kb1 && ok; c0 += chunk_kb) {  // one accumulator per K-chunk
                const int c1 = c0 + chunk_kb < U.kb1 ? c0 + chunk_kb : U.kb1;
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, &abort_flag, 0x200 | (18 + acc))) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
                for (int kb = c0; kb < c1; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, &abort_flag, 0x200 | stage)) { ok = false; break; }
                    tc_fence_after();
                    issue_kblock<TERMS, A_MN, B_MN, BM, BN>(stage_addr(stage), d_tmem, idesc, idesc16, kb == c0, tc_mma_tf32, tc_mma_f16);
                    tc_commit(empty_bar(stage));  // arrives when the MMAs above have read the stage
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                tc_commit(tfull_bar(acc));        // this chunk's accumulator is complete
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
                }
            }
        }
    } else {
        // ------------------------------ epilogue ------------------------------
        const int quarter = warp & 3;  // TMEM lanes this warp may read: [32*quarter, 32*quarter+32)
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
            const Unit U = unit_of(u, P);
            int tm, tn;
            tile_coords(U.tile, P.tiles_m, P.tiles_n, tm, tn);
            const int64_t m0 = static_cast<int64_t>(tm) * BM, n0 = static_cast<int64_t>(tn) * BN;
            const int64_t row_base = m0 + quarter * 32;
            const int chunk_kb = P.chunk_kb;
            int* half_flag = U.half ? P.half_flags + (U.slot * 2 + 0) * 4 + quarter : nullptr;
            // second half of K: its sums are added to what the first half stored
            if (U.half && U.part == 1 && !wait_first_half(half_flag, lane, &abort_flag, 0xA00 | quarter)) { ok = false; break; }
#pragma unroll 1
            for (int c0 = U.kb0; c0 < U.kb1 && ok; c0 += chunk_kb) {  // one accumulator per K-chunk
            const bool first = c0 == U.kb0 && U.part == 0, last = c0 + chunk_kb >= U.kb1;
            SideRegs sd_now, sd_next, mk_now, mk_next;
            load_side(P, first, last, row_base, lane, n0, sd_next, mk_next);  // column chunk 0's, while the accumulator is still being computed
            if (!mbar_wait(tfull_bar(acc), acc_phase, &abort_flag, 0x300 | (16 + acc))) { ok = false; break; }
            tc_fence_after();
#pragma unroll 1
            for (int cc = 0; cc < BN / 32; ++cc) {
                uint32_t r[32];
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * BN + cc * 32);
                tmem_ld32(taddr, r);
                sd_now = sd_next;
                mk_now = mk_next;
                const int64_t col0 = n0 + cc * 32;
                if (cc + 1 < BN / 32) load_side(P, first, last, row_base, lane, col0 + 32, sd_next, mk_next);
                tmem_ld_wait();
                emit_chunk(P, U.half, first, last, row_base, lane, col0, r, stages[warp - 2], sd_now, mk_now);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
            if (ok && U.half && U.part == 0) publish_first_half(half_flag, lane);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ---- CTA-pair variant --------------------------------------------------------------------------------
// Two CTAs of a cluster (ranks 0 and 1, on neighbouring SMs) compute one 256 x 256 tile with
// tcgen05.mma.cta_group::2 (M=256, N=256, K=8).  Each CTA stages its own 128 rows of A and its own
// 128 columns of B, so a 128 x 256 accumulator costs 32 KB of shared-memory fill and read per
// k-block instead of 48 KB: the single-CTA kernel is bound by shared-memory bandwidth, this one is
// not, and each B tile crosses L2 once per 256 rows of C instead of once per 128.
//   * both producers load with cp.async.bulk.tensor...cta_group::2 (each CTA its own half; no
//     load is shared between CTAs) and signal the full barrier of rank 0, whose producer posts the
//     expected byte count of both halves;
//   * rank 0's warp 1 issues the MMAs; tcgen05.commit signals the empty / accumulator-full
//     barriers of both CTAs;
//   * the epilogue warps of both CTAs read their own TMEM (lanes = their 128 rows) and arrive on
//     rank 0's accumulator-empty barrier (count 8);
//   * TMEM is allocated and freed with cta_group::2 by warp 1 of both CTAs; a cluster barrier after
//     set-up and before tear-down keeps either CTA from touching a peer that is not there.
namespace pair {

constexpr int BN = 256;     // tile width of the pair
constexpr int BN_CTA = 128; // columns of B each CTA stages

template <int TERMS>
struct Cfg {
    static constexpr int A_BYTES = BM * BK * 4;
    static constexpr int B_BYTES = BN_CTA * BK * 4;
    static constexpr int STAGE_BYTES = (TERMS == 1 ? 1 : 2) * (A_BYTES + B_BYTES);  // per CTA
    static constexpr int STAGES_RAW = SMEM_BUDGET / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
    static constexpr int TMEM_COLS = 512;  // two 256-column accumulators
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;
    static_assert(STAGES >= 2, "need at least two stages");
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Address of the same shared-memory object in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    __syncwarp();
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Bounded wait that also orders this thread after the (possibly remote) arrivals' earlier writes.
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if ((i & 255u) == 255u) {
            if (*abort_flag) return false;
            __nanosleep(64);
        }
    }
    *abort_flag = 1;
    atomicCAS(&g_tc_status, 0, code);
    return false;
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// Per-CTA load of this CTA's half; the completion bytes go to the barrier at `cluster_bar`
// (a shared::cluster address: rank 0's full barrier).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t cluster_bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, uint32_t cluster_bar, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// Arrives on the barrier at this shared-memory offset in both CTAs of the pair once the MMAs
// issued so far have completed.
__device__ __forceinline__ void tc_commit_both(uint32_t bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(mask) : "memory");
}
__device__ __forceinline__ void tc_mma_tf32_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_mma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// M = 256 across the pair.
__host__ __device__ constexpr uint32_t make_idesc_pair(bool a_mn_major, bool b_mn_major) { return make_idesc_fmt(kFmtTF32, 2 * BM, BN, a_mn_major, b_mn_major); }

// P.tiles_m / P.tiles_n count 256 x 256 tiles.  Grid = 2 x number of resident clusters.
template <int TERMS, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(THREADS, 1)
tcgen05_matmul_pair_kernel(const __grid_constant__ CUtensorMap map_a0, const __grid_constant__ CUtensorMap map_a1, const __grid_constant__ CUtensorMap map_a2,
                           const __grid_constant__ CUtensorMap map_b0, const __grid_constant__ CUtensorMap map_b1, const __grid_constant__ CUtensorMap map_b2,
                           const Params P) {
    using C = Cfg<TERMS>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bars[2 * 8 + 4];  // full[8], empty[8], tmem_full[2], tmem_empty[2]
    __shared__ uint32_t tmem_base_slot;
    __shared__ __align__(16) EpilogueStage stages[4];  // one per epilogue warp
    __shared__ volatile int abort_flag;

    const uint32_t rank = cluster_ctarank();      // 0 = issues the MMAs
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (8 + s); };
    auto tfull_bar = [&](int a) { return bar0 + 8u * (16 + a); };
    auto tempty_bar = [&](int a) { return bar0 + 8u * (18 + a); };
    auto stage_addr = [&](int s) { return smem_base + s * C::STAGE_BYTES; };  // (layout inside: StageLayout)
    const CUtensorMap* const maps_a[3] = {&map_a0, &map_a1, &map_a2};
    const CUtensorMap* const maps_b[3] = {&map_b0, &map_b1, &map_b2};
    const uint32_t peer_abort = map_to_cta(smem_u32(const_cast<int*>(&abort_flag)), rank ^ 1u);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 8); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_tmap(&map_a0);
        prefetch_tmap(&map_b0);
        if (TERMS >= 2) { prefetch_tmap(&map_a1); prefetch_tmap(&map_b1); }
        if (TERMS == 2) { prefetch_tmap(&map_a2); prefetch_tmap(&map_b2); }
    }
    if (warp == 1) {
        tmem_alloc2(smem_u32(&tmem_base_slot), C::TMEM_COLS);
        tmem_relinquish2();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peer's barriers exist before anything is signalled across
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    const int num_units = unit_count(P);
    const int first_unit = blockIdx.x >> 1, unit_step = gridDim.x >> 1;
    // Unit number `seq` of this pair: first_unit + seq * unit_step (num_units once the pair has run out).
    auto unit_at = [&](uint32_t seq) -> int {
        const int64_t v = static_cast<int64_t>(first_unit) + static_cast<int64_t>(seq) * unit_step;
        return v < num_units ? static_cast<int>(v) : num_units;
    };

    if (warp == 0) {
        // ------------------------------ TMA producer (both CTAs) ------------------------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            uint32_t issued = 0;
            bool ok = true;
            for (uint32_t seq = 0; ok; ++seq) {
                const int u = unit_at(seq);
                if (u >= num_units) break;
                const Unit U = unit_of(u, P);
                int tm, tn;
                tile_coords(U.tile, P.tiles_m, P.tiles_n, tm, tn);
                const int m0 = tm * (2 * BM) + static_cast<int>(rank) * BM;
                const int n0 = tn * BN + static_cast<int>(rank) * BN_CTA;
                for (int kb = U.kb0; kb < U.kb1; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, &abort_flag, 0x500 | stage)) { ok = false; break; }
                    if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * C::STAGE_BYTES);
                    const uint32_t fb = map_to_cta(full_bar(stage), 0);
                    load_stage<TERMS, A_MN, B_MN, BM, BN_CTA>(stage_addr(stage), maps_a, maps_b, m0, n0, kb * BK, P.a_grouped != 0, P.b_grouped != 0,
                                                             [&](uint32_t dst, const CUtensorMap* map, int c0, int c1) { tma_load_2d_pair(dst, map, fb, c0, c1); },
                                                             [&](uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2) { tma_load_3d_pair(dst, map, fb, c0, c1, c2); });
                    ++issued;
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            if (ok) {
                // Tail: every stage this CTA filled has been released, i.e. the MMAs that read it are
                // done and no arrival on this CTA's empty barriers is still on its way.
                const uint32_t pending = issued < static_cast<uint32_t>(C::STAGES) ? issued : C::STAGES;
                for (uint32_t i = 0; i < pending && ok; ++i) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, &abort_flag, 0x580 | stage)) ok = false;
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) {
                // Gave up.  The completion of this CTA's copies is counted on rank 0's barriers, so
                // there is nothing local to wait on: give the copies in flight a bounded ~2 ms to land.
                st_cluster_u32(peer_abort, 1u);
                for (int i = 0; i < 2048; ++i) __nanosleep(1000);
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer (rank 0 only) ------------------------------
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = make_idesc_pair(A_MN, B_MN), idesc16 = make_idesc_fmt(kFmtBF16, 2 * BM, BN, A_MN, B_MN);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (uint32_t seq = 0; ok; ++seq) {
                const int u = unit_at(seq);
                if (u >= num_units) break;
                const Unit U = unit_of(u, P);
                const int chunk_kb = P.chunk_kb;
                for (int c0 = U.kb0; c0 < U.kb1 && ok; c0 += chunk_kb) {  // one accumulator per K-chunk
                const int c1 = c0 + chunk_kb < U.kb1 ? c0 + chunk_kb : U.kb1;
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, &abort_flag, 0x600 | (18 + acc))) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
                for (int kb = c0; kb < c1; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, &abort_flag, 0x600 | stage)) { ok = false; break; }
                    tc_fence_after();
                    issue_kblock<TERMS, A_MN, B_MN, BM, BN_CTA>(stage_addr(stage), d_tmem, idesc, idesc16, kb == c0, tc_mma_tf32_pair, tc_mma_f16_pair);
                    tc_commit_both(empty_bar(stage));  // both CTAs' stage is free once these MMAs have read it
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                tc_commit_both(tfull_bar(acc));        // this chunk's accumulator is complete, in both CTAs' TMEM
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
                }
            }
            if (!ok) st_cluster_u32(peer_abort, 1u);
        }
    } else {
        // ------------------------------ epilogue (both CTAs) ------------------------------
        const int quarter = warp & 3;
        const uint32_t tempty0 = map_to_cta(tempty_bar(0), 0), tempty1 = map_to_cta(tempty_bar(1), 0);
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (uint32_t seq = 0; ok; ++seq) {
            const int u = unit_at(seq);
            if (u >= num_units) break;
            const Unit U = unit_of(u, P);
            int tm, tn;
            tile_coords(U.tile, P.tiles_m, P.tiles_n, tm, tn);
            const int64_t m0 = static_cast<int64_t>(tm) * (2 * BM) + static_cast<int64_t>(rank) * BM;
            const int64_t n0 = static_cast<int64_t>(tn) * BN;
            const int64_t row_base = m0 + quarter * 32;
            const int chunk_kb = P.chunk_kb;
            int* half_flag = U.half ? P.half_flags + (U.slot * 2 + static_cast<int>(rank)) * 4 + quarter : nullptr;
            // second half of K: its sums are added to what the first half stored
            if (U.half && U.part == 1 && !wait_first_half(half_flag, lane, &abort_flag, 0xA00 | quarter)) { ok = false; break; }
#pragma unroll 1
            for (int c0 = U.kb0; c0 < U.kb1 && ok; c0 += chunk_kb) {  // one accumulator per K-chunk
            const bool first = c0 == U.kb0 && U.part == 0, last = c0 + chunk_kb >= U.kb1;
            SideRegs sd_now, sd_next, mk_now, mk_next;
            load_side(P, first, last, row_base, lane, n0, sd_next, mk_next);  // column chunk 0's, while the accumulator is still being computed
            if (!mbar_wait(tfull_bar(acc), acc_phase, &abort_flag, 0x700 | (16 + acc))) { ok = false; break; }
            tc_fence_after();
#pragma unroll 1
            for (int cc = 0; cc < BN / 32; ++cc) {
                uint32_t r[32];
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * BN + cc * 32);
                tmem_ld32(taddr, r);
                sd_now = sd_next;
                mk_now = mk_next;
                const int64_t col0 = n0 + cc * 32;
                if (cc + 1 < BN / 32) load_side(P, first, last, row_base, lane, col0 + 32, sd_next, mk_next);
                tmem_ld_wait();
                emit_chunk(P, U.half, first, last, row_base, lane, col0, r, stages[warp - 2], sd_now, mk_now);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc ? tempty1 : tempty0);
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
            if (ok && U.half && U.part == 0) publish_first_half(half_flag, lane);
        }
        if (!ok && lane == 0) st_cluster_u32(peer_abort, 1u);
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // neither CTA leaves (or frees TMEM) while the other may still signal it
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc2(tmem_base, C::TMEM_COLS);
    }
}

}  // namespace pair

// ---- self-test of the bounded wait -------------------------------------------------------------------
// One CTA waits, with the kernels' own wait routine and a short limit, on a barrier that nothing ever
// arrives on.  The wait has to run out, record its code in the status word, raise the abort flag and
// let the kernel return normally -- the path a real time-out would take -- without any fault.
__global__ void wait_timeout_selftest_kernel(int* observed) {
    __shared__ uint64_t bar;
    __shared__ volatile int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    bool ok = true;
    if (threadIdx.x == 0) ok = mbar_wait(smem_u32(&bar), 0u, &abort_flag, 0x7e57, 1u << 12);
    __syncthreads();
    // a second role sees the flag and gives up at once instead of running out itself
    if (threadIdx.x == 32) ok = mbar_wait(smem_u32(&bar), 0u, &abort_flag, 0x7e58, 1u << 30);
    __syncthreads();
    if (threadIdx.x == 0) { observed[0] = ok ? 1 : 0; observed[1] = abort_flag; }
    if (threadIdx.x == 32) observed[2] = ok ? 1 : 0;
}

// ---- host side -------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
std::mutex g_encode_mu;

ctk_status get_encoder(EncodeTiledFn* out) {
    std::lock_guard<std::mutex> lock(g_encode_mu);
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        CTK_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
        if (!fn || q != cudaDriverEntryPointSuccess) return fail(CTK_ERR_CUDA, "cuTensorMapEncodeTiled not available from the driver");
        g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    *out = g_encode;
    return CTK_OK;
}

// Encoded tensor maps, remembered.  An encoding is a pure function of (base, extents, pitch, box, layout),
// and cuTensorMapEncodeTiled costs about a microsecond -- six of them per product is most of the host time
// of a small product called again and again on the same buffers (the layers of a small network).  A small
// direct-mapped table per thread; a colliding or new key is simply encoded again.
struct MapKey {
    const void* base;
    int64_t inner, outer, ld;
    int box_outer, flags;  // flags: bit 0 MN-major, bit 1 bf16
    int groups;            // > 0: an MN-major operand as a 3-D tensor, `groups` 128-byte column groups per box
    bool operator==(const MapKey& o) const {
        return base == o.base && inner == o.inner && outer == o.outer && ld == o.ld && box_outer == o.box_outer && flags == o.flags && groups == o.groups;
    }
};
struct MapSlot {
    MapKey key{nullptr, 0, 0, 0, 0, -1, 0};
    CUtensorMap map;
};
constexpr int kMapSlots = 256;
thread_local MapSlot t_map_cache[kMapSlots];

ctk_status encode_map(CUtensorMap* map, const MapKey& k) {
    uint64_t h = reinterpret_cast<uintptr_t>(k.base) >> 4;
    h ^= static_cast<uint64_t>(k.inner) * 0x9E3779B97F4A7C15ull ^ static_cast<uint64_t>(k.outer) * 0xC2B2AE3D27D4EB4Full ^
         static_cast<uint64_t>(k.ld) * 0x165667B19E3779F9ull ^ static_cast<uint64_t>((k.box_outer * 4 + k.flags) * 16 + k.groups);
    MapSlot& slot = t_map_cache[(h ^ (h >> 29)) % kMapSlots];
    if (slot.key == k) {
        *map = slot.map;
        return CTK_OK;
    }
    EncodeTiledFn enc;
    ctk_status st = get_encoder(&enc);
    if (st) return st;
    const bool mn_major = (k.flags & 1) != 0, bf16 = (k.flags & 2) != 0;
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(k.inner), static_cast<cuuint64_t>(k.outer)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(k.ld) * (bf16 ? 2 : 4)};
    cuuint32_t estr[2] = {1u, 1u};
    cuuint32_t box[2];
    CUtensorMapSwizzle swz;
    if (!bf16) {
        box[0] = 32u;
        box[1] = static_cast<cuuint32_t>(k.box_outer);
        swz = mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B;
    } else {
        box[0] = mn_major ? 64u : 32u;
        box[1] = static_cast<cuuint32_t>(mn_major ? 32 : k.box_outer);
        swz = mn_major ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
    }
    CUresult r;
    if (k.groups > 0) {
        // {128 bytes along MN, k, column group}: group g of row kk starts g * 128 bytes into the row
        const cuuint64_t wide = box[0];
        cuuint64_t dims3[3] = {wide, static_cast<cuuint64_t>(k.outer), static_cast<cuuint64_t>(k.inner) / wide};
        cuuint64_t strides3[2] = {strides[0], 128u};
        cuuint32_t box3[3] = {box[0], box[1], static_cast<cuuint32_t>(k.groups)};
        cuuint32_t estr3[3] = {1u, 1u, 1u};
        r = enc(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(k.base), dims3, strides3, box3, estr3,
                CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else {
        r = enc(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(k.base), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (r != CUDA_SUCCESS) return fail(CTK_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(r)));
    slot.key = k;
    slot.map = *map;
    return CTK_OK;
}

// 2-D fp32 tensor {inner (contiguous), outer} with row pitch ld elements; box {32, box_outer};
// 128-byte swizzle (16-byte chunks for a K-major operand, 32-byte atoms for an MN-major one);
// out-of-range elements read as zero.
// groups > 0 (MN-major only): the 3-D form, `groups` column groups of 32 elements per box.
ctk_status make_map(CUtensorMap* map, const float* base, int64_t inner, int64_t outer, int64_t ld, int box_outer, bool mn_major, int groups = 0) {
    return encode_map(map, MapKey{base, inner, outer, ld, box_outer, mn_major ? 1 : 0, mn_major ? groups : 0});
}

// The same operand as bf16 ([outer, ld] elements of 2 bytes): box {32, box_outer} with the 64-byte
// swizzle for a K-major operand (a k-block is 32 elements = 64 bytes), {64, 32} with the 128-byte
// swizzle per 64-wide column group for an MN-major one.
// groups > 0 (MN-major only): the 3-D form, `groups` column groups of 64 elements per box.
ctk_status make_map16(CUtensorMap* map, const void* base, int64_t inner, int64_t outer, int64_t ld, int box_outer, bool mn_major, int groups = 0) {
    return encode_map(map, MapKey{base, inner, outer, ld, box_outer, (mn_major ? 1 : 0) | 2, mn_major ? groups : 0});
}

// One operand as the tensor-core path sees it.
struct Operand {
    const float* p;
    bool mn_major;   // the M/N index is the contiguous one
    int64_t mn, k;   // extents
    int64_t ld;      // pitch of the non-contiguous dim, in elements
    int64_t inner() const { return mn_major ? mn : k; }
    int64_t outer() const { return mn_major ? k : mn; }
};

bool tma_ok(const Operand& o) {
    return (reinterpret_cast<uintptr_t>(o.p) & 15u) == 0 && o.ld % 4 == 0 && o.ld >= o.inner() && o.inner() % 4 == 0;
}

template <int BN, int TERMS, bool A_MN, bool B_MN>
ctk_status launch_tc(const CUtensorMap maps[6], const Params& P, cudaStream_t st) {
    using C = Cfg<BN, TERMS>;
    auto kernel = tcgen05_matmul_kernel<BN, TERMS, A_MN, B_MN>;
    static ctk::PerDeviceOnce attr;  // the attribute belongs to the (kernel, device) pair
    if (attr.first()) CTK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    const int units = P.whole_tiles + 2 * (P.tiles_m * P.tiles_n - P.whole_tiles);
    const int sms = ctk::sm_count();
    const int grid = units < sms ? units : sms;  // persistent: one CTA per SM
    kernel<<<grid, THREADS, C::SMEM_BYTES, st>>>(maps[0], maps[1], maps[2], maps[3], maps[4], maps[5], P);
    CTK_LAUNCH_CHECK("tcgen05_matmul_kernel");
    return CTK_OK;
}

template <int BN, int TERMS>
ctk_status launch_tc_major(bool a_mn, bool b_mn, const CUtensorMap maps[6], const Params& P, cudaStream_t st) {
    if (a_mn && b_mn) return launch_tc<BN, TERMS, true, true>(maps, P, st);
    if (a_mn) return launch_tc<BN, TERMS, true, false>(maps, P, st);
    if (b_mn) return launch_tc<BN, TERMS, false, true>(maps, P, st);
    return launch_tc<BN, TERMS, false, false>(maps, P, st);
}

int pick_bn(int64_t n) { return n > 128 ? 256 : (n > 64 ? 128 : 64); }

// Number of CTA pairs resident on the device (all instantiations of the pair kernel use the same
// threads and shared memory, so one of them is asked).
ctk_status resident_pairs(int* out);

// ---- CTA-pair launch ----
// Resident clusters of two per device, asked of the driver once (the kernels differ only in code, not in resources).
template <int TERMS, bool A_MN, bool B_MN>
ctk_status launch_pair(const CUtensorMap maps[6], const Params& P, cudaStream_t st) {
    using C = pair::Cfg<TERMS>;
    auto kernel = pair::tcgen05_matmul_pair_kernel<TERMS, A_MN, B_MN>;
    static int max_clusters[64] = {0};
    int dev = 0;
    CTK_CUDA(cudaGetDevice(&dev));
    CTK_REQUIRE(dev >= 0 && dev < 64, "device ordinal out of range");
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (!max_clusters[dev]) {
        CTK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
        cfg.gridDim = dim3(2 * static_cast<unsigned>(ctk::sm_count()));
        int n = 0;
        CTK_CUDA(cudaOccupancyMaxActiveClusters(&n, kernel, &cfg));
        CTK_REQUIRE(n > 0, "the device cannot hold a cluster of two CTAs of the MatMul kernel");
        max_clusters[dev] = n;
    }
    const int units = P.whole_tiles + 2 * (P.tiles_m * P.tiles_n - P.whole_tiles);
    const int clusters = units < max_clusters[dev] ? units : max_clusters[dev];
    cfg.gridDim = dim3(2 * static_cast<unsigned>(clusters));
    CTK_CUDA(cudaLaunchKernelEx(&cfg, kernel, maps[0], maps[1], maps[2], maps[3], maps[4], maps[5], P));
    CTK_LAUNCH_CHECK("tcgen05_matmul_pair_kernel");
    return CTK_OK;
}

ctk_status resident_pairs(int* out) {
    static int pairs[64] = {0};
    int dev = 0;
    CTK_CUDA(cudaGetDevice(&dev));
    CTK_REQUIRE(dev >= 0 && dev < 64, "device ordinal out of range");
    if (!pairs[dev]) {
        using C = pair::Cfg<3>;
        auto kernel = pair::tcgen05_matmul_pair_kernel<3, false, false>;
        CTK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
        cudaLaunchConfig_t cfg = {};
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.gridDim = dim3(2 * static_cast<unsigned>(ctk::sm_count()));
        cfg.blockDim = dim3(THREADS);
        cfg.dynamicSmemBytes = C::SMEM_BYTES;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        CTK_CUDA(cudaOccupancyMaxActiveClusters(&n, kernel, &cfg));
        CTK_REQUIRE(n > 0, "the device cannot hold a cluster of two CTAs of the MatMul kernel");
        pairs[dev] = n;
    }
    *out = pairs[dev];
    return CTK_OK;
}

template <int TERMS>
ctk_status launch_pair_major(bool a_mn, bool b_mn, const CUtensorMap maps[6], const Params& P, cudaStream_t st) {
    if (a_mn && b_mn) return launch_pair<TERMS, true, true>(maps, P, st);
    if (a_mn) return launch_pair<TERMS, true, false>(maps, P, st);
    if (b_mn) return launch_pair<TERMS, false, true>(maps, P, st);
    return launch_pair<TERMS, false, false>(maps, P, st);
}

}  // namespace tc

// Classifies one operand: returns false if neither stride is 1.
bool classify(const float* p, int64_t mn, int64_t k, int64_t s_mn, int64_t s_k, tc::Operand* o) {
    o->p = p; o->mn = mn; o->k = k;
    if (s_k == 1 && (s_mn >= k || mn == 1)) { o->mn_major = false; o->ld = (mn == 1 && s_mn < k) ? k : s_mn; return true; }
    if (s_mn == 1 && (s_k >= mn || k == 1)) { o->mn_major = true; o->ld = (k == 1 && s_k < mn) ? mn : s_k; return true; }
    return false;
}

// ---- a short contraction (K <= 16) with a large output: CUDA cores, bound by the output's bytes ------
// dX of a layer with few outputs (the 10-class layer: [B,10].[10,H]) has one k-block per tile, so on the
// tensor-core kernel nothing hides the epilogue and its four warps per SM cannot keep HBM busy.  Here a
// thread keeps the K values of its four output columns in registers and walks down the rows: per row
// one broadcast read of A's K values, 4K multiply-adds, one 16-byte store (plus the mask read and the
// two split stores of the fused forms).  Products and sums are rounded one by one in l order -- the
// arithmetic of MatMul_BASIC_kernel.cpp:41-50 as g++ compiles it, so this path is bit-identical to it.
// A: [m, k] contiguous; B: [n, k] contiguous (the t() view of an [n, k] array as the right operand).
constexpr int SK_MAXK = 16, SK_THREADS = 128, SK_ROWS = 32;
__global__ void __launch_bounds__(SK_THREADS) skinny_k_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c,
                                                             int64_t m, int64_t n, int k, const float* __restrict__ mask,
                                                             SplitOut out) {
    const int64_t j0 = (static_cast<int64_t>(blockIdx.x) * SK_THREADS + threadIdx.x) * 4;
    const bool live = j0 < n;  // (no early return: every thread takes part in staging A)
    float bw[4][SK_MAXK];
#pragma unroll
    for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int l = 0; l < SK_MAXK; ++l) bw[q][l] = (live && l < k) ? __ldg(b + (j0 + q) * k + l) : 0.0f;
    const int64_t r0 = static_cast<int64_t>(blockIdx.y) * SK_ROWS;
    const int rows_here = static_cast<int>(m - r0 < SK_ROWS ? m - r0 : SK_ROWS);
    // this CTA's rows of A, once, through shared memory (every thread reads all of them)
    __shared__ float a_sm[SK_ROWS][SK_MAXK];
    for (int i = threadIdx.x; i < SK_ROWS * SK_MAXK; i += SK_THREADS) {
        const int rr = i / SK_MAXK, l = i % SK_MAXK;
        a_sm[rr][l] = (rr < rows_here && l < k) ? __ldg(a + (r0 + rr) * k + l) : 0.0f;
    }
    __syncthreads();
    if (!live) return;
    constexpr int G = 8;  // rows in flight per thread: their mask reads are issued together, then their stores
    for (int rb = 0; rb < rows_here; rb += G) {
        float4 y[G];
        if (mask != nullptr) {
#pragma unroll
            for (int g = 0; g < G; ++g)
                if (rb + g < rows_here) y[g] = __ldcs(reinterpret_cast<const float4*>(mask + (r0 + rb + g) * n + j0));
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            if (rb + g >= rows_here) break;
            const int64_t r = r0 + rb + g;
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int l = 0; l < SK_MAXK; ++l)
                if (l < k) {
                    const float av = a_sm[rb + g][l];
#pragma unroll
                    for (int q = 0; q < 4; ++q) acc[q] = __fadd_rn(acc[q], __fmul_rn(av, bw[q][l]));
                }
            float4 x = make_float4(acc[0], acc[1], acc[2], acc[3]);
            if (mask != nullptr) {
                x.x *= y[g].x > 0.0f ? 1.0f : 0.0f; x.y *= y[g].y > 0.0f ? 1.0f : 0.0f;
                x.z *= y[g].z > 0.0f ? 1.0f : 0.0f; x.w *= y[g].w > 0.0f ? 1.0f : 0.0f;
            }
            __stcs(reinterpret_cast<float4*>(c + r * n + j0), x);
            if (out.p2 != nullptr) store_split4<true>(out, r * out.pitch + j0, x);
        }
    }
}
// The shapes that take it: 3xTF32 mode, K <= 16, both operands K-major and contiguous, whole 16-byte
// pieces, and an output of at least 2^20 elements (small products stay on the tensor-core kernel).
static bool skinny_k_ok(const float* a, const float* b, const float* c, int64_t m, int64_t n, int64_t k, int64_t sa0, int64_t sa1, int64_t sb0,
                        int64_t sb1, int md) {
    return md == CTK_MATMUL_3XTF32 && k >= 1 && k <= SK_MAXK && sa1 == 1 && sa0 == k && sb0 == 1 && sb1 == k && n % 4 == 0 &&
           m * n >= (int64_t(1) << 20) && (m + SK_ROWS - 1) / SK_ROWS <= 65535 && (c == nullptr || (reinterpret_cast<uintptr_t>(c) & 15u) == 0) &&
           a != nullptr && b != nullptr;
}

// ---- a narrow output (N <= 16) over a long contraction: CUDA cores, bound by A's bytes ---------------
// The 10-class layer: logits = H.W ([B,H].[H,10]) and dW = H^T.dY ([H,B].[B,10]).  On the tensor-core
// kernel these are 64-wide tiles of which ten columns are used, a handful of tiles each walking the whole
// contraction, and A has to be read as its 8-byte split.  Here A is read once as fp32 (16-byte loads, the
// next ones always in flight while the current ones are multiplied), B sits in shared memory, every
// product is an fp32 FMA and the sums are fp32 -- closer to the float64 result than the reference's own
// sequential fp32 loop.  Both kernels split the contraction over the grid's y dimension; the partial
// results land in a workspace [parts][m][n] and narrow_sum_kernel adds them in part order (a fixed order:
// two calls give the same bits).  With one part they write C themselves.
//   narrow_rows_kernel: A [m, k] with unit stride along k.  A CTA keeps its 512 k of B transposed in shared
//     memory for its whole life and walks down a range of rows; a warp takes four rows at a time, a lane
//     four consecutive k per load (the same four k of B in one 16-byte read), and the lanes' sums are
//     folded across the warp, halving the values a lane holds at every step.
//   narrow_cols_kernel: A [m, k] with unit stride along m (the t() view of a [k, m] array).  A thread owns
//     four consecutive m and walks down its part of k, B's rows broadcast from shared memory.
constexpr int SN_MAXN = 16, SN_THREADS = 256, SN_WARPS = SN_THREADS / 32, SN_WARP_ROWS = 4;
constexpr int SN_KS = 512, SN_PITCH = SN_KS + 4;   // k per CTA; the pad spreads the transposed staging writes over the banks
template <int NP>
__global__ void __launch_bounds__(SN_THREADS, NP <= 12 ? 2 : 1) narrow_rows_kernel(const float* __restrict__ a, int64_t lda, const float* __restrict__ b, int64_t sb0, int64_t sb1,
                                                                float* __restrict__ part, int64_t m, int n, int64_t k, int64_t rows_per_cta) {
    __shared__ __align__(16) float bt[NP * SN_PITCH];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t k0 = static_cast<int64_t>(blockIdx.y) * SN_KS;
    const int kc = static_cast<int>(k - k0 < SN_KS ? k - k0 : SN_KS);
    const int64_t row_begin = static_cast<int64_t>(blockIdx.x) * rows_per_cta;
    const int64_t row_end = row_begin + rows_per_cta < m ? row_begin + rows_per_cta : m;
    float* out = part + static_cast<int64_t>(blockIdx.y) * m * n;
    // rows [r, r + 4) at k-step t (k = k0 + 4 lane + 128 t): four 16-byte loads; past the end zeros / the last row again
    auto load = [&](int64_t r, int t, float4 (&dst)[SN_WARP_ROWS]) {
        const int kk = 4 * lane + 128 * t;
#pragma unroll
        for (int q = 0; q < SN_WARP_ROWS; ++q) {
            const int64_t row = r + q < m ? r + q : m - 1;
            dst[q] = (kk < kc && r < row_end) ? __ldcs(reinterpret_cast<const float4*>(a + row * lda + k0 + kk)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    float4 a0[SN_WARP_ROWS], a1[SN_WARP_ROWS];
    int64_t r = row_begin + warp * SN_WARP_ROWS;
    load(r, 0, a0);   // in flight while B is staged
    for (int i = threadIdx.x; i < SN_KS * NP; i += SN_THREADS) {
        const int kk = i / NP, j = i - kk * NP;
        bt[j * SN_PITCH + kk] = (j < n && kk < kc) ? __ldg(b + (k0 + kk) * sb0 + j * sb1) : 0.0f;
    }
    __syncthreads();
    float acc[SN_WARP_ROWS * NP];
    auto fold = [&](const float4 (&av)[SN_WARP_ROWS], int t) {
        const int kk = 4 * lane + 128 * t;
#pragma unroll
        for (int j = 0; j < NP; ++j) {
            const float4 bv = *reinterpret_cast<const float4*>(&bt[j * SN_PITCH + kk]);
#pragma unroll
            for (int q = 0; q < SN_WARP_ROWS; ++q) {
                float v = acc[q * NP + j];
                v = fmaf(av[q].x, bv.x, v);
                v = fmaf(av[q].y, bv.y, v);
                v = fmaf(av[q].z, bv.z, v);
                v = fmaf(av[q].w, bv.w, v);
                acc[q * NP + j] = v;
            }
        }
    };
    for (; r < row_end; r += SN_WARPS * SN_WARP_ROWS) {
#pragma unroll
        for (int i = 0; i < SN_WARP_ROWS * NP; ++i) acc[i] = 0.0f;
        load(r, 1, a1); fold(a0, 0);
        load(r, 2, a0); fold(a1, 1);
        load(r, 3, a1); fold(a0, 2);
        load(r + SN_WARPS * SN_WARP_ROWS, 0, a0); fold(a1, 3);   // the next four rows' first loads
        // fold the lanes: at each step a lane hands half of its values to its partner and adds the partner's
        // other half to the half it keeps; after four steps lane pair p holds values [p V/16, (p+1) V/16)
        constexpr int V = SN_WARP_ROWS * NP;
        int cnt = V;
#pragma unroll
        for (int o = 16; o >= 2; o >>= 1) {
            cnt >>= 1;
            const bool upper = (lane & o) != 0;
#pragma unroll
            for (int i = 0; i < cnt; ++i) {
                const float send = upper ? acc[i] : acc[i + cnt];
                const float keep = upper ? acc[i + cnt] : acc[i];
                acc[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
            }
        }
        constexpr int MINE = V / 16;
#pragma unroll
        for (int i = 0; i < MINE; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], 1);
        if ((lane & 1) == 0) {
#pragma unroll
            for (int i = 0; i < MINE; ++i) {
                const int idx = (lane >> 1) * MINE + i;
                const int q = idx / NP, j = idx - q * NP;
                if (j < n && r + q < row_end) out[(r + q) * n + j] = acc[i];
            }
        }
    }
}

constexpr int SG_THREADS = 128, SG_KC = 128, SG_DEPTH = 4;
template <int NP>
__global__ void __launch_bounds__(SG_THREADS) narrow_cols_kernel(const float* __restrict__ a, int64_t lda, const float* __restrict__ b, int64_t sb0, int64_t sb1,
                                                                float* __restrict__ part, int64_t m, int n, int64_t k, int64_t k_per_part) {
    __shared__ __align__(16) float bs[SG_KC * NP];
    const int64_t i0 = (static_cast<int64_t>(blockIdx.x) * SG_THREADS + threadIdx.x) * 4;
    const bool live = i0 < m;   // (m is a multiple of 4; no early return: every thread takes part in staging B)
    const int64_t kb = static_cast<int64_t>(blockIdx.y) * k_per_part;
    const int64_t ke = kb + k_per_part < k ? kb + k_per_part : k;
    float acc[4][NP];
#pragma unroll
    for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int j = 0; j < NP; ++j) acc[q][j] = 0.0f;
    auto fold = [&](const float4& av, int kk) {
#pragma unroll
        for (int j4 = 0; j4 < NP / 4; ++j4) {
            const float4 bv = *reinterpret_cast<const float4*>(&bs[kk * NP + 4 * j4]);
            const float bj[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                acc[0][4 * j4 + t] = fmaf(av.x, bj[t], acc[0][4 * j4 + t]);
                acc[1][4 * j4 + t] = fmaf(av.y, bj[t], acc[1][4 * j4 + t]);
                acc[2][4 * j4 + t] = fmaf(av.z, bj[t], acc[2][4 * j4 + t]);
                acc[3][4 * j4 + t] = fmaf(av.w, bj[t], acc[3][4 * j4 + t]);
            }
        }
    };
    // rows [kr, kr + SG_DEPTH) of A (zeros past this part's end)
    const float* col = a + (live ? i0 : 0);
    auto load = [&](int64_t kr, float4 (&dst)[SG_DEPTH]) {
#pragma unroll
        for (int u = 0; u < SG_DEPTH; ++u)
            dst[u] = (live && kr + u < ke) ? __ldcs(reinterpret_cast<const float4*>(col + (kr + u) * lda)) : make_float4(0.f, 0.f, 0.f, 0.f);
    };
    float4 x0[SG_DEPTH], x1[SG_DEPTH];
    load(kb, x0);   // in flight while B is staged
    for (int64_t k0 = kb; k0 < ke; k0 += SG_KC) {
        const int kc = static_cast<int>(ke - k0 < SG_KC ? ke - k0 : SG_KC);
        __syncthreads();
        for (int i = threadIdx.x; i < SG_KC * NP; i += SG_THREADS) {
            const int kk = i / NP, j = i - kk * NP;
            bs[i] = (j < n && kk < kc) ? __ldg(b + (k0 + kk) * sb0 + j * sb1) : 0.0f;
        }
        __syncthreads();
        // (rows past kc multiply zeros of A with zeros of B)
        for (int kk = 0; kk < SG_KC; kk += 2 * SG_DEPTH) {
            load(k0 + kk + SG_DEPTH, x1);
#pragma unroll
            for (int u = 0; u < SG_DEPTH; ++u) fold(x0[u], kk + u);
            load(k0 + kk + 2 * SG_DEPTH, x0);
#pragma unroll
            for (int u = 0; u < SG_DEPTH; ++u) fold(x1[u], kk + SG_DEPTH + u);
            if (kk + 2 * SG_DEPTH >= kc) break;   // (x0 now holds zeros, or the next chunk's first rows)
        }
    }
    if (live) {
        float* o = part + static_cast<int64_t>(blockIdx.y) * m * n + i0 * n;
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
            for (int j = 0; j < NP; ++j)
                if (j < n) o[q * n + j] = acc[q][j];
    }
}

__global__ void __launch_bounds__(256) narrow_sum_kernel(const float* __restrict__ part, int parts, int64_t count, float* __restrict__ c) {
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        float v = 0.0f;
        int s = 0;
        for (; s + 8 <= parts; s += 8) {   // eight loads in flight, added in part order
            float x[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) x[u] = __ldcs(part + (s + u) * count + i);
#pragma unroll
            for (int u = 0; u < 8; ++u) v += x[u];
        }
        for (; s < parts; ++s) v += __ldcs(part + s * count + i);
        c[i] = v;
    }
}

// The shapes that take it: fp32-accurate mode, N <= 16, A with a unit stride and whole 16-byte pieces
// along it, and an A of at least 2^20 elements with a contraction of at least 256 (smaller products
// stay on the tensor-core kernel).  Returns 0 (no), 1 (A along k: narrow_rows) or 2 (A along m: narrow_cols).
static int narrow_n_form(const float* a, const float* b, int64_t m, int64_t n, int64_t k, int64_t sa0, int64_t sa1, int md) {
    if (md != CTK_MATMUL_3XTF32 || n < 1 || n > SN_MAXN || k < 256 || m * k < (int64_t(1) << 20) || a == nullptr || b == nullptr) return 0;
    if ((reinterpret_cast<uintptr_t>(a) & 15u) != 0) return 0;
    if (sa1 == 1 && sa0 >= k && sa0 % 4 == 0 && k % 4 == 0 && (k + SN_KS - 1) / SN_KS <= 65535) return 1;
    if (sa0 == 1 && sa1 >= m && sa1 % 4 == 0 && m % 4 == 0 && (m / 4 + SG_THREADS - 1) / SG_THREADS < (int64_t(1) << 31)) return 2;
    return 0;
}

// How narrow_cols splits the contraction: enough parts for about four CTAs per SM, each at least 64 long
// and a multiple of 2 * SG_DEPTH.
static void narrow_cols_parts(int64_t m, int64_t k, int* parts, int64_t* k_per_part) {
    const int64_t col_ctas = (m / 4 + SG_THREADS - 1) / SG_THREADS;
    int64_t want = (4 * static_cast<int64_t>(ctk::sm_count()) + col_ctas - 1) / col_ctas;
    if (want > k / 64) want = k / 64;
    if (want < 1) want = 1;
    if (want > 65535) want = 65535;
    int64_t per = (k + want - 1) / want;
    per = (per + 2 * SG_DEPTH - 1) / (2 * SG_DEPTH) * (2 * SG_DEPTH);
    *k_per_part = per;
    *parts = static_cast<int>((k + per - 1) / per);
}

template <int NP>
static ctk_status launch_narrow(int form, const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k, int64_t sa0, int64_t sa1,
                                int64_t sb0, int64_t sb1, void* workspace, cudaStream_t st) {
    int parts = 1;
    int64_t per = k;
    if (form == 1) parts = static_cast<int>((k + SN_KS - 1) / SN_KS);
    else narrow_cols_parts(m, k, &parts, &per);
    float* part = c;
    if (parts > 1) {
        void* ws = workspace;   // (a caller's workspace is sized for the operands' splits: at least 8 bytes per element of A)
        if (!ws) {
            ctk_status rc = device_scratch(1, static_cast<size_t>(parts) * m * n * sizeof(float), &ws);
            if (rc) return rc;
        }
        part = static_cast<float*>(ws);
    }
    if (form == 1) {
        // row ranges: about two resident CTAs per SM in all, whole groups of SN_WARPS x SN_WARP_ROWS rows
        constexpr int64_t kGroup = SN_WARPS * SN_WARP_ROWS;
        int64_t row_ctas = (2 * static_cast<int64_t>(ctk::sm_count()) + parts - 1) / parts;
        if (row_ctas < 1) row_ctas = 1;
        int64_t rows_per_cta = ((m + row_ctas - 1) / row_ctas + kGroup - 1) / kGroup * kGroup;
        row_ctas = (m + rows_per_cta - 1) / rows_per_cta;
        dim3 grid(static_cast<unsigned>(row_ctas), static_cast<unsigned>(parts));
        narrow_rows_kernel<NP><<<grid, SN_THREADS, 0, st>>>(a, sa0, b, sb0, sb1, part, m, static_cast<int>(n), k, rows_per_cta);
        CTK_LAUNCH_CHECK("narrow_rows_kernel");
    } else {
        dim3 grid(static_cast<unsigned>((m / 4 + SG_THREADS - 1) / SG_THREADS), static_cast<unsigned>(parts));
        narrow_cols_kernel<NP><<<grid, SG_THREADS, 0, st>>>(a, sa1, b, sb0, sb1, part, m, static_cast<int>(n), k, per);
        CTK_LAUNCH_CHECK("narrow_cols_kernel");
    }
    if (parts > 1) {
        narrow_sum_kernel<<<ctk_stream_grid(m * n, 256, 8), 256, 0, st>>>(part, parts, m * n, c);
        CTK_LAUNCH_CHECK("narrow_sum_kernel");
    }
    return CTK_OK;
}

int g_default_mode = CTK_MATMUL_3XTF32;
// Which tensor-core path carries the two correction terms of mode CTK_MATMUL_3XTF32:
// 0 = TF32 (three TF32 products), 1 = bf16 (one TF32 product + two bf16 products; the default).
// (CTORCH_MATMUL_CORRECTION=tf32 | bf16 in the environment sets the start value.)
int g_correction = [] {
    const char* e = std::getenv("CTORCH_MATMUL_CORRECTION");
    if (e && e[0] == 't') return 0;
    if (e && e[0] == 'b') return 1;
    return 1;  // measured on B200: 14-19 % faster training steps and a smaller error (1.0e-5 against 1.6e-5 at 4096^3)
}();
int g_pairing = 0;  // 0: CTA pairs where the shape allows, 1: single-CTA kernel only
// MN-major operands as 3-D tensor maps (one copy per array and stage).  CTORCH_MATMUL_GROUPED_MAPS=0 keeps the 2-D maps.
bool g_grouped_maps = [] {
    const char* e = std::getenv("CTORCH_MATMUL_GROUPED_MAPS");
    return !(e && e[0] == '0');
}();
int g_split_tail = 1;  // K-halves for the tiles of a last wave that fills at most half the machine: 0 never, 1 where the contraction is long enough to pay, 2 wherever the shape allows
// ---- optional per-launch timing of the tensor-core kernel ----
struct TcProfile {
    static constexpr int kMax = 8192;
    bool on = false;
    std::vector<cudaEvent_t> ev;  // 2 per launch, created on demand, reused
    std::vector<double> flops;
    int used = 0;
};
TcProfile g_prof;
std::mutex g_prof_mu;

// Returns the event pair for the next launch, or false when profiling is off / the record is full.
bool prof_begin(double flops, cudaStream_t st, cudaEvent_t* stop) {
    std::lock_guard<std::mutex> lock(g_prof_mu);
    if (!g_prof.on || g_prof.used >= TcProfile::kMax) return false;
    const int i = g_prof.used;
    while (static_cast<int>(g_prof.ev.size()) < 2 * (i + 1)) {
        cudaEvent_t e;
        if (cudaEventCreate(&e) != cudaSuccess) return false;
        g_prof.ev.push_back(e);
    }
    if (static_cast<int>(g_prof.flops.size()) <= i) g_prof.flops.resize(i + 1);
    g_prof.flops[i] = flops;
    g_prof.used = i + 1;
    cudaEventRecord(g_prof.ev[2 * i], st);
    *stop = g_prof.ev[2 * i + 1];
    return true;
}

int resolve_mode(int mode) { return mode < 0 ? g_default_mode : mode; }

// 0 = tcgen05, 1 = SIMT.
// TF32 mode reads the caller's operands in place, so both must be addressable by TMA (unit stride in
// one dim, the other pitch a multiple of 16 bytes, 16-byte aligned base).  3xTF32 mode reads its own
// hi/lo copies, which are laid out for TMA whatever the source pitch: a unit stride is enough, so
// the 10-wide layer (40-byte rows) also runs on the tensor cores.
int choose_path(const float* a, const float* b, int64_t m, int64_t n, int64_t k, int64_t sa0, int64_t sa1, int64_t sb0,
                int64_t sb1, int mode, tc::Operand* oa, tc::Operand* ob) {
    const int md = resolve_mode(mode);
    if (md == CTK_MATMUL_FP32_SIMT) return 1;
    tc::Operand A, B;
    if (!classify(a, m, k, sa0, sa1, &A) || !classify(b, n, k, sb1, sb0, &B)) return 1;
    if (md == CTK_MATMUL_TF32) {
        if (!tc::tma_ok(A) || !tc::tma_ok(B)) return 1;
        if (n < 16 || k < 8) return 1;  // a tile of mostly padding: not worth a pass over unsplit operands
    }
    if (oa) *oa = A;
    if (ob) *ob = B;
    return 0;
}

// The three arrays of a split inside one buffer (256-byte aligned start, `outer` rows of `pitch` elements).
// in_place: the operand itself serves as hi (see SplitOut): the first array's room stays unused.
SplitOut split_layout(void* buf, int64_t outer, int64_t pitch, int variant, bool in_place) {
    SplitOut o;
    float* first = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(buf) + 255u) & ~static_cast<uintptr_t>(255u));
    o.hi = in_place ? nullptr : first;
    o.variant = variant;
    o.pitch = pitch;
    if (variant == 0) {
        o.p2 = first + outer * pitch;
    } else {
        __nv_bfloat16* h16 = reinterpret_cast<__nv_bfloat16*>(first + outer * pitch);
        o.p2 = h16;
        o.p3 = h16 + outer * pitch;
    }
    return o;
}
// Whether the array at p ([.., inner] with row pitch ld elements) can be read by TMA as it is, so that it
// serves as the hi part of its own split.  CTORCH_MATMUL_HI_IN_PLACE=0 in the environment: never.
bool g_hi_in_place = [] {
    const char* e = std::getenv("CTORCH_MATMUL_HI_IN_PLACE");
    return !(e && e[0] == '0');
}();
bool hi_in_place(const void* p, int64_t inner, int64_t ld) {
    return g_hi_in_place && (reinterpret_cast<uintptr_t>(p) & 15u) == 0 && ld % 4 == 0 && ld >= inner && inner % 4 == 0;
}
// The value a kept split's valid flag has when it holds the split of this variant, with or without hi.
int split_tag(int variant, bool in_place) { return 1 + variant + (in_place ? 2 : 0); }
int64_t split_pitch_of(int64_t inner) { return (inner + 7) / 8 * 8; }

// ---- flags of the K-halved tiles ------------------------------------------------------------------
// A launch with halved tiles needs 8 words per such tile (2 CTAs x 4 epilogue warps), zero when it
// starts.  They live in a ring of slots inside the module (no allocation: the entry point that must not
// allocate uses them too); every launch takes the next slot and clears it on its own stream first.  A
// slot comes round again after kHalfSlots launches with halved tiles -- far more than can be in flight.
constexpr int kHalfTilesMax = 128, kHalfSlots = 256;
static __device__ int g_half_flags[kHalfSlots][kHalfTilesMax * 8];
int* g_half_flags_ptr[64] = {nullptr};
std::mutex g_half_mu;
unsigned g_half_next = 0;

ctk_status half_flag_slot(int** out) {
    int dev = 0;
    CTK_CUDA(cudaGetDevice(&dev));
    CTK_REQUIRE(dev >= 0 && dev < 64, "device ordinal out of range");
    std::lock_guard<std::mutex> lock(g_half_mu);
    if (!g_half_flags_ptr[dev]) {
        void* p = nullptr;
        CTK_CUDA(cudaGetSymbolAddress(&p, g_half_flags));
        CTK_REQUIRE(p != nullptr, "cudaGetSymbolAddress returned a null address for the half-tile flags");
        g_half_flags_ptr[dev] = static_cast<int*>(p);
    }
    *out = g_half_flags_ptr[dev] + static_cast<size_t>(g_half_next++ % kHalfSlots) * (kHalfTilesMax * 8);
    return CTK_OK;
}

// ---- fixed scratch for callers that must not allocate -------------------------------------------
// Some hosts cannot let a library allocate device memory behind their back: code running inside a
// CUDA stream capture (an allocation there is either illegal or becomes part of the graph), services
// that hand the whole GPU to their own arena allocator at start-up and treat any later cudaMalloc as
// a bug, and latency-sensitive loops where a growing workspace would mean a device synchronisation
// in the middle of a step.  For them the hi/lo split of the 3xTF32 product can live in this
// fixed-size array, which is part of the loaded module: every GPU that loads the library holds these
// 16 MiB (+1 KiB) until the process exits.
constexpr size_t kStaticWorkspaceBytes = (16u << 20) + 1024;  // 4 Mi split floats + the 1 KiB alignment slack
static __device__ __align__(256) unsigned char g_static_workspace[kStaticWorkspaceBytes];

// In host code the name above is only a handle for the runtime, not an address a kernel could use:
// the device address is looked up once per device (with that device current) and cached.
void* g_static_workspace_ptr[64] = {nullptr};
std::mutex g_static_workspace_mu;

ctk_status static_workspace(void** out) {
    int dev = 0;
    CTK_CUDA(cudaGetDevice(&dev));
    CTK_REQUIRE(dev >= 0 && dev < 64, "device ordinal out of range");
    std::lock_guard<std::mutex> lock(g_static_workspace_mu);
    if (!g_static_workspace_ptr[dev]) {
        void* p = nullptr;
        CTK_CUDA(cudaGetSymbolAddress(&p, g_static_workspace));
        CTK_REQUIRE(p != nullptr, "cudaGetSymbolAddress returned a null address for the static workspace");
        g_static_workspace_ptr[dev] = p;
    }
    *out = g_static_workspace_ptr[dev];
    return CTK_OK;
}

}  // namespace

extern "C" {

ctk_status ctk_set_matmul_mode(int mode) {
    CTK_REQUIRE(mode >= CTK_MATMUL_3XTF32 && mode <= CTK_MATMUL_FP32_SIMT, "ctk_set_matmul_mode: unknown mode");
    g_default_mode = mode;
    return CTK_OK;
}
int ctk_get_matmul_mode(void) { return g_default_mode; }

// Which path carries the two correction terms of the fp32-accurate mode (CTK_MATMUL_3XTF32): 0 = TF32
// (lo.hi + hi.lo + hi.hi, all TF32), 1 = bf16 (l16.h16 + h16.l16 in bf16 + hi.hi in TF32).  Process-wide;
// a kept split made under the other setting is not reused (its valid flag holds the setting's tag).
ctk_status ctk_set_matmul_correction(int bf16) {
    CTK_REQUIRE(bf16 == 0 || bf16 == 1, "ctk_set_matmul_correction: 0 (TF32 correction terms) or 1 (bf16 correction terms)");
    g_correction = bf16;
    return CTK_OK;
}
int ctk_get_matmul_correction(void) { return g_correction; }
// The value a kept split's valid flag has when the buffer holds a split made under the current setting.
int ctk_matmul_split_tag(void) { return split_tag(g_correction, false); }
// The same for the split of the array at p ([.., inner], row pitch ld elements): 2 more when the array itself
// serves as the split's hi part (16-byte aligned rows), which is how the epilogues and the SGD update write it.
int ctk_matmul_split_tag_for(const void* p, int64_t inner, int64_t ld) { return split_tag(g_correction, hi_in_place(p, inner, ld)); }

ctk_status ctk_set_matmul_tail_split(int on) {
    CTK_REQUIRE(on >= 0 && on <= 2, "ctk_set_matmul_tail_split: 0, 1 or 2");
    g_split_tail = on;
    return CTK_OK;
}

ctk_status ctk_set_matmul_pairing(int pairing) {
    CTK_REQUIRE(pairing == 0 || pairing == 1, "ctk_set_matmul_pairing: 0 (CTA pairs where possible) or 1 (single-CTA kernel only)");
    g_pairing = pairing;
    return CTK_OK;
}

// Split copies have their contiguous extent padded to a multiple of 8 elements; which extent that is
// depends on the operand's major-ness, so the larger of the two possibilities is reserved.
static int64_t padded_elems(int64_t mn, int64_t k) {
    const int64_t a = mn * ((k + 7) / 8 * 8), b = k * ((mn + 7) / 8 * 8);
    return a > b ? a : b;
}
size_t ctk_matmul_workspace_bytes(int64_t m, int64_t n, int64_t k, int mode) {
    if (resolve_mode(mode) != CTK_MATMUL_3XTF32) return 0;
    return static_cast<size_t>(2 * (padded_elems(m, k) + padded_elems(n, k))) * sizeof(float) + 1024;
}

int ctk_matmul_path(const float* a, const float* b, int64_t m, int64_t n, int64_t k, int64_t sa0, int64_t sa1,
                    int64_t sb0, int64_t sb1, int mode) {
    if (skinny_k_ok(a, b, nullptr, m, n, k, sa0, sa1, sb0, sb1, resolve_mode(mode))) return 2;
    if (narrow_n_form(a, b, m, n, k, sa0, sa1, resolve_mode(mode))) return 3;
    return choose_path(a, b, m, n, k, sa0, sa1, sb0, sb1, mode, nullptr, nullptr);
}

ctk_status ctk_matmul_profile_enable(int on) {
    std::lock_guard<std::mutex> lock(g_prof_mu);
    g_prof.on = on != 0;
    g_prof.used = 0;
    return CTK_OK;
}

ctk_status ctk_matmul_profile_read(int64_t* launches, double* total_ms, double* total_flops) {
    CTK_REQUIRE(launches && total_ms && total_flops, "ctk_matmul_profile_read: null");
    CTK_CUDA(cudaDeviceSynchronize());
    std::lock_guard<std::mutex> lock(g_prof_mu);
    double ms = 0.0, fl = 0.0;
    for (int i = 0; i < g_prof.used; ++i) {
        float t = 0.0f;
        CTK_CUDA(cudaEventElapsedTime(&t, g_prof.ev[2 * i], g_prof.ev[2 * i + 1]));
        ms += t;
        fl += g_prof.flops[i];
    }
    *launches = g_prof.used;
    *total_ms = ms;
    *total_flops = fl;
    g_prof.used = 0;
    return CTK_OK;
}

// Runs the bounded-wait self-test: returns through `result` {wait returned ok (0 expected), abort flag
// (1 expected), second waiter ok (0 expected), status word (0x7e57 expected)} and clears the status
// word again.  No MatMul may be in flight.
ctk_status ctk_matmul_selftest_wait_timeout(int result[4]) {
    CTK_RANGE("ctk_matmul_selftest_wait_timeout");
    CTK_REQUIRE(result, "ctk_matmul_selftest_wait_timeout: null");
    CTK_CUDA(cudaDeviceSynchronize());
    int saved = 0;
    CTK_CUDA(cudaMemcpyFromSymbol(&saved, g_tc_status, sizeof(int)));
    const int zero = 0;
    CTK_CUDA(cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int)));
    int* dev = nullptr;
    CTK_CUDA(cudaMalloc(&dev, 3 * sizeof(int)));
    tc::wait_timeout_selftest_kernel<<<1, 64>>>(dev);
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemcpy(result, dev, 3 * sizeof(int), cudaMemcpyDeviceToHost);
    cudaFree(dev);
    CTK_CUDA(e);
    CTK_CUDA(cudaMemcpyFromSymbol(&result[3], g_tc_status, sizeof(int)));
    CTK_CUDA(cudaMemcpyToSymbol(g_tc_status, &saved, sizeof(int)));
    return CTK_OK;
}

ctk_status ctk_matmul_status(int* status) {
    CTK_REQUIRE(status, "ctk_matmul_status: null");
    CTK_CUDA(cudaDeviceSynchronize());
    CTK_CUDA(cudaMemcpyFromSymbol(status, g_tc_status, sizeof(int)));
    return CTK_OK;
}

// A caller-kept split of one operand: `buf` holds hi then lo ([outer, pitch] each), `valid` says
// whether it matches the operand's current contents (0: the product fills it and sets 1).
struct KeptSplit {
    void* buf;
    int* valid;
};

// What a fused call adds to the product: c = [relu](a.b + bias) and, optionally, c's own hi/lo split
// (layout of a K-major [m, n] operand) for the products c enters next.
struct FusedEpilogue {
    const float* bias = nullptr;
    int relu = 0;
    const float* mask = nullptr;
    void* c_split = nullptr;
};

static ctk_status matmul_impl(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k, int64_t sa0,
                              int64_t sa1, int64_t sb0, int64_t sb1, int mode, void* workspace, KeptSplit ka, KeptSplit kb, void* stream,
                              FusedEpilogue fe = FusedEpilogue()) {
    CTK_REQUIRE(m >= 0 && n >= 0 && k >= 0, "ctk_matmul_f32: negative extent");
    if (m == 0 || n == 0) return CTK_OK;
    CTK_REQUIRE(c, "ctk_matmul_f32: null output");
    cudaStream_t st = as_stream(stream);
    if (k == 0) {
        CTK_CUDA(cudaMemsetAsync(c, 0, static_cast<size_t>(m * n) * sizeof(float), st));
        return CTK_OK;
    }
    CTK_REQUIRE(a && b, "ctk_matmul_f32: null operand");
    const int md = resolve_mode(mode);
    CTK_REQUIRE(md >= CTK_MATMUL_3XTF32 && md <= CTK_MATMUL_FP32_SIMT, "ctk_matmul_f32: unknown mode");
    CTK_REQUIRE(m < (int64_t(1) << 31) && n < (int64_t(1) << 31) && k < (int64_t(1) << 31), "ctk_matmul_f32: extent >= 2^31");

    if (fe.bias == nullptr && !fe.relu && skinny_k_ok(a, b, c, m, n, k, sa0, sa1, sb0, sb1, md) &&
        (fe.mask == nullptr || (reinterpret_cast<uintptr_t>(fe.mask) & 15u) == 0)) {
        SplitOut so;
        if (fe.c_split) so = split_layout(fe.c_split, m, split_pitch_of(n), g_correction, hi_in_place(c, n, n));
        dim3 grid(static_cast<unsigned>((n / 4 + SK_THREADS - 1) / SK_THREADS), static_cast<unsigned>((m + SK_ROWS - 1) / SK_ROWS));
        skinny_k_kernel<<<grid, SK_THREADS, 0, st>>>(a, b, c, m, n, static_cast<int>(k), fe.mask, so);
        CTK_LAUNCH_CHECK("skinny_k_kernel");
        return CTK_OK;
    }

    const bool fused = fe.bias != nullptr || fe.relu || fe.mask != nullptr || fe.c_split != nullptr;
    if (!fused) {
        const int form = narrow_n_form(a, b, m, n, k, sa0, sa1, md);
        if (form != 0) {
            if (n <= 4) return launch_narrow<4>(form, a, b, c, m, n, k, sa0, sa1, sb0, sb1, workspace, st);
            if (n <= 8) return launch_narrow<8>(form, a, b, c, m, n, k, sa0, sa1, sb0, sb1, workspace, st);
            if (n <= 12) return launch_narrow<12>(form, a, b, c, m, n, k, sa0, sa1, sb0, sb1, workspace, st);
            return launch_narrow<16>(form, a, b, c, m, n, k, sa0, sa1, sb0, sb1, workspace, st);
        }
    }
    tc::Operand A, B;
    if (choose_path(a, b, m, n, k, sa0, sa1, sb0, sb1, md, &A, &B) == 1) {
        if (fused) return fail(CTK_ERR_INVALID, "fused MatMul: the operands need the tensor-core path (a unit stride each)");
        dim3 grid(static_cast<unsigned>((n + SM_TILE - 1) / SM_TILE), static_cast<unsigned>((m + SM_TILE - 1) / SM_TILE));
        CTK_REQUIRE(grid.y <= 65535u, "ctk_matmul_f32: m too large for the CUDA-core path");
        simt_matmul_kernel<<<grid, SM_THREADS, 0, st>>>(a, b, c, m, n, k, sa0, sa1, sb0, sb1);
        CTK_LAUNCH_CHECK("simt_matmul_kernel");
        return CTK_OK;
    }

    const int variant = g_correction;
    const int terms = (md == CTK_MATMUL_3XTF32) ? (variant == 1 ? 2 : 3) : 1;
    // the operand itself as the hi part of its split, where TMA can read it
    const bool a_in_place = terms != 1 && hi_in_place(A.p, A.inner(), A.ld), b_in_place = terms != 1 && hi_in_place(B.p, B.inner(), B.ld);
    const int a_tag = split_tag(variant, a_in_place), b_tag = split_tag(variant, b_in_place);  // what a kept split's valid flag must say
    SplitOut sa, sb;
    int64_t a_ld = A.ld, b_ld = B.ld;   // pitch of the split's arrays (of the operand itself in TF32 mode)
    if (terms != 1) {
        const int64_t a_pitch = split_pitch_of(A.inner()), b_pitch = split_pitch_of(B.inner());
        void *abuf = ka.buf, *bbuf = kb.buf;
        if (!abuf || !bbuf) {
            void* ws = workspace;
            if (!ws) {
                ctk_status rc = device_scratch(1, ctk_matmul_workspace_bytes(m, n, k, md), &ws);
                if (rc) return rc;
            }
            const SplitOut first = split_layout(ws, A.outer(), a_pitch, variant, false);
            if (!abuf) abuf = ws;
            if (!bbuf) bbuf = first.hi + 2 * A.outer() * a_pitch;  // behind A's 8 bytes per element
        }
        sa = split_layout(abuf, A.outer(), a_pitch, variant, a_in_place);
        sb = split_layout(bbuf, B.outer(), b_pitch, variant, b_in_place);
        auto split = [&](const tc::Operand& O, const SplitOut& out) -> ctk_status {
            const bool vec = (reinterpret_cast<uintptr_t>(O.p) & 15u) == 0 && O.ld % 4 == 0 && O.inner() % 4 == 0;
            if (vec) {
                const int64_t total = O.outer() * (O.inner() / 4);
                const int64_t per_cta = SPLIT_THREADS * SPLIT_UNROLL;
                split_tf32_vec_kernel<<<static_cast<unsigned>((total + per_cta - 1) / per_cta), SPLIT_THREADS, 0, st>>>(O.p, out, O.outer(), O.inner() / 4, O.ld);
            } else {
                split_tf32_scalar_kernel<<<ctk_stream_grid(O.outer() * O.inner(), SPLIT_THREADS, 8), SPLIT_THREADS, 0, st>>>(O.p, out, O.outer(), O.inner(), O.ld);
            }
            CTK_LAUNCH_CHECK("split_tf32_kernel");
            return CTK_OK;
        };
        ctk_status rc2;
        if (!(ka.buf && ka.valid && *ka.valid == a_tag)) {
            if ((rc2 = split(A, sa))) return rc2;
            if (ka.buf && ka.valid) *ka.valid = a_tag;
        }
        if (!(kb.buf && kb.valid && *kb.valid == b_tag)) {
            if ((rc2 = split(B, sb))) return rc2;
            if (kb.buf && kb.valid) *kb.valid = b_tag;
        }
        a_ld = a_pitch; b_ld = b_pitch;
    }

    const int bn = tc::pick_bn(n);
    // Two CTAs per 256 x 256 tile once there is more than one 128-row block to pair up.
    const bool paired = (g_pairing == 0) && bn == 256 && m > tc::BM;
    CUtensorMap maps[6];  // a: {hi | x, lo | h16, l16}, b: the same
    const int a_box = A.mn_major ? tc::BK : tc::BM;
    const int b_rows = paired ? tc::pair::BN_CTA : bn;
    const int b_box = B.mn_major ? tc::BK : b_rows;
    ctk_status rc;
    const float* a32 = (terms == 1 || a_in_place) ? A.p : sa.hi;
    const float* b32 = (terms == 1 || b_in_place) ? B.p : sb.hi;
    const int64_t a_ld32 = (terms == 1 || a_in_place) ? A.ld : a_ld, b_ld32 = (terms == 1 || b_in_place) ? B.ld : b_ld;
    // MN-major operands with whole 128-byte groups along MN: one 3-D copy per array and stage instead of
    // one per group (g_grouped_maps goes false for good if the driver refuses such a map)
    bool a_grouped = g_grouped_maps && A.mn_major && A.inner() % 64 == 0;
    bool b_grouped = g_grouped_maps && B.mn_major && B.inner() % 64 == 0 && b_rows >= 64;
    auto encode_all = [&]() -> ctk_status {
        const int ag32 = a_grouped ? tc::BM / 32 : 0, ag16 = a_grouped ? tc::BM / 64 : 0;
        const int bg32 = b_grouped ? b_rows / 32 : 0, bg16 = b_grouped ? b_rows / 64 : 0;
        ctk_status e;
        if ((e = tc::make_map(&maps[0], a32, A.inner(), A.outer(), a_ld32, a_box, A.mn_major, ag32))) return e;
        if ((e = tc::make_map(&maps[3], b32, B.inner(), B.outer(), b_ld32, b_box, B.mn_major, bg32))) return e;
        if (terms == 3) {
            if ((e = tc::make_map(&maps[1], static_cast<const float*>(sa.p2), A.inner(), A.outer(), a_ld, a_box, A.mn_major, ag32))) return e;
            if ((e = tc::make_map(&maps[4], static_cast<const float*>(sb.p2), B.inner(), B.outer(), b_ld, b_box, B.mn_major, bg32))) return e;
            maps[2] = maps[1];
            maps[5] = maps[4];
        } else if (terms == 2) {
            if ((e = tc::make_map16(&maps[1], sa.p2, A.inner(), A.outer(), a_ld, tc::BM, A.mn_major, ag16))) return e;
            if ((e = tc::make_map16(&maps[2], sa.p3, A.inner(), A.outer(), a_ld, tc::BM, A.mn_major, ag16))) return e;
            if ((e = tc::make_map16(&maps[4], sb.p2, B.inner(), B.outer(), b_ld, b_rows, B.mn_major, bg16))) return e;
            if ((e = tc::make_map16(&maps[5], sb.p3, B.inner(), B.outer(), b_ld, b_rows, B.mn_major, bg16))) return e;
        } else {
            maps[1] = maps[2] = maps[0];
            maps[4] = maps[5] = maps[3];
        }
        return CTK_OK;
    };
    rc = encode_all();
    if (rc && (a_grouped || b_grouped)) {
        g_grouped_maps = false;
        a_grouped = b_grouped = false;
        rc = encode_all();
    }
    if (rc) return rc;

    tc::Params P;
    P.m = m; P.n = n; P.k = k;
    const int tile_m = paired ? 2 * tc::BM : tc::BM;
    P.tiles_m = static_cast<int>((m + tile_m - 1) / tile_m);
    P.tiles_n = static_cast<int>((n + bn - 1) / bn);
    P.num_kb = static_cast<int>((k + tc::BK - 1) / tc::BK);
    P.chunk_kb = tc::chunk_k_for(tc::pick_bn(n)) / tc::BK;
    P.c = c;
    P.vec_store = (n % 4 == 0) && ((reinterpret_cast<uintptr_t>(c) & 15u) == 0);
    P.bias = fe.bias;
    P.relu = fe.relu;
    P.mask = fe.mask;
    P.a_grouped = a_grouped ? 1 : 0;
    P.b_grouped = b_grouped ? 1 : 0;
    P.out = SplitOut();
    P.out.pitch = split_pitch_of(n);
    if (fe.c_split) P.out = split_layout(fe.c_split, m, split_pitch_of(n), variant, hi_in_place(c, n, n));
    CTK_REQUIRE(static_cast<int64_t>(P.tiles_m) * P.tiles_n < (int64_t(1) << 30), "ctk_matmul_f32: too many tiles");
    // The last wave: when at most half of the SMs (or CTA pairs) would have a tile, its tiles are
    // computed as two K-halves each (the second added to the first, in that order), so that twice as
    // many work on it.
    {
        const int tiles = P.tiles_m * P.tiles_n;
        int workers = ctk::sm_count();
        if (paired && (rc = tc::resident_pairs(&workers))) return rc;
        P.whole_tiles = tiles;
        const int tail = tiles % workers;
        // (a fused epilogue needs the whole sum)
        P.half_flags = nullptr;
        // (the second half's epilogue starts after the first's -- about 12 us more at the end of the kernel,
        // and the flags are cleared by one more node on the stream -- so halves pay once half of the
        // contraction takes longer than that: from 96 k-blocks of three or two terms, 192 of one)
        const int min_kb = g_split_tail == 2 ? 16 : (terms == 1 ? 192 : 96);
        if (g_split_tail && !fused && P.num_kb >= min_kb && tail > 0 && 2 * tail <= workers && tail <= kHalfTilesMax) {
            int* flags = nullptr;
            if ((rc = half_flag_slot(&flags))) return rc;
            CTK_CUDA(cudaMemsetAsync(flags, 0, static_cast<size_t>(tail) * 8 * sizeof(int), st));
            P.half_flags = flags;
            P.whole_tiles = tiles - tail;
        }
    }

 #define CTK_TC(BN_)                                                                                 \
    (terms == 3 ? tc::launch_tc_major<BN_, 3>(A.mn_major, B.mn_major, maps, P, st)                  \
     : terms == 2 ? tc::launch_tc_major<BN_, 2>(A.mn_major, B.mn_major, maps, P, st)                \
                  : tc::launch_tc_major<BN_, 1>(A.mn_major, B.mn_major, maps, P, st))
    cudaEvent_t stop_ev;
    const bool timed = prof_begin(2.0 * static_cast<double>(m) * static_cast<double>(n) * static_cast<double>(k), st, &stop_ev);
    if (paired)
        rc = terms == 3   ? tc::launch_pair_major<3>(A.mn_major, B.mn_major, maps, P, st)
             : terms == 2 ? tc::launch_pair_major<2>(A.mn_major, B.mn_major, maps, P, st)
                          : tc::launch_pair_major<1>(A.mn_major, B.mn_major, maps, P, st);
    else
        rc = (bn == 256) ? CTK_TC(256) : (bn == 128) ? CTK_TC(128) : CTK_TC(64);
    if (timed) cudaEventRecord(stop_ev, st);
    return rc;
#undef CTK_TC
}

ctk_status ctk_matmul_f32(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k, int64_t sa0,
                          int64_t sa1, int64_t sb0, int64_t sb1, int mode, void* workspace, void* stream) {
    CTK_RANGE("ctk_matmul_f32");
    return matmul_impl(a, b, c, m, n, k, sa0, sa1, sb0, sb1, mode, workspace, KeptSplit{nullptr, nullptr}, KeptSplit{nullptr, nullptr}, stream);
}

// hi + lo of an operand with extents (mn, k), whichever of the two is contiguous, + alignment slack.
size_t ctk_matmul_split_bytes(int64_t mn, int64_t k) { return static_cast<size_t>(2 * padded_elems(mn, k)) * sizeof(float) + 256; }

// The 3xTF32 product with the hi/lo split of either operand kept by the caller between calls.
// An operand that enters several products unchanged (an activation in its layer's forward product
// and again, transposed, in the weight-gradient product; an upstream gradient in both backward
// products) is then split once instead of once per product: 12 bytes of HBM traffic per element saved
// each time.  a_split / b_split: device buffers of ctk_matmul_split_bytes(m, k) / (n, k) bytes, or
// NULL to use the workspace for that operand; *a_valid / *b_valid: 0 = fill the buffer in this call
// (set to 1 on return), 1 = the buffer already holds the split of exactly these values, viewed with
// exactly this shape and these strides.  Keeping that promise is the caller's job: the buffer must
// be discarded when the operand's memory is written.
ctk_status ctk_matmul_3xtf32_kept_f32(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k, int64_t sa0,
                                      int64_t sa1, int64_t sb0, int64_t sb1, void* a_split, int* a_valid, void* b_split,
                                      int* b_valid, void* workspace, void* stream) {
    CTK_RANGE("ctk_matmul_3xtf32_kept_f32");
    CTK_REQUIRE((!a_split || a_valid) && (!b_split || b_valid), "ctk_matmul_3xtf32_kept_f32: a split buffer needs its valid flag");
    return matmul_impl(a, b, c, m, n, k, sa0, sa1, sb0, sb1, CTK_MATMUL_3XTF32, workspace, KeptSplit{a_split, a_valid}, KeptSplit{b_split, b_valid}, stream);
}

// c = [relu](a.b + bias[col]) in one launch, with c's own hi/lo split written by the same epilogue.
// The bias add and the ReLU are the single fp32 operations of Add_BASIC_kernel's [N,H] + [H] form and
// of ReLU_BASIC_kernel applied to the rounded accumulator, so the result equals MatMul, Add, ReLU run
// one after the other bit for bit; what is saved is their two passes over c and the read of the later
// split.  mask (an [m, n] array of pitch n, or NULL) multiplies the result by (mask > 0 ? 1 : 0), the
// single operation of ReLU's backward rule with mask the ReLU's output: a gradient product g.W^T that
// feeds that rule leaves the kernel already masked and split.  bias: n floats or NULL; c_split:
// ctk_matmul_split_bytes(m, n) bytes or NULL (valid for c viewed as [m, n] with pitch n afterwards).
// Needs the tensor-core path for both operands.
ctk_status ctk_matmul_3xtf32_fused_f32(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k, int64_t sa0,
                                       int64_t sa1, int64_t sb0, int64_t sb1, void* a_split, int* a_valid, void* b_split,
                                       int* b_valid, const float* bias, int relu, const float* mask, void* c_split, void* workspace,
                                       void* stream) {
    CTK_RANGE("ctk_matmul_3xtf32_fused_f32");
    CTK_REQUIRE((!a_split || a_valid) && (!b_split || b_valid), "ctk_matmul_3xtf32_fused_f32: a split buffer needs its valid flag");
    CTK_REQUIRE(m > 0 && n > 0 && k > 0, "ctk_matmul_3xtf32_fused_f32: empty product");
    FusedEpilogue fe;
    fe.bias = bias;
    fe.relu = relu ? 1 : 0;
    fe.mask = mask;
    fe.c_split = c_split;
    return matmul_impl(a, b, c, m, n, k, sa0, sa1, sb0, sb1, CTK_MATMUL_3XTF32, workspace, KeptSplit{a_split, a_valid}, KeptSplit{b_split, b_valid}, stream, fe);
}

// p -= g*lr (ctk_sgd_update_f32's arithmetic) and, in the same pass, the hi/lo split of the updated p
// into `split` -- a buffer of ctk_matmul_split_bytes(inner, outer) bytes that ctk_matmul_3xtf32_kept_f32
// then takes as valid for p viewed as [outer, inner] with pitch ld (or, transposed, with the strides
// swapped).  Saves the split's own read of the weights before their next product.  p and g 16-byte
// aligned, inner and ld multiples of 4, g contiguous; anything else is refused (CTK_ERR_INVALID) and the
// caller runs the plain update.
ctk_status ctk_sgd_update_split_f32(float* p, const float* g, float lr, int64_t outer, int64_t inner, int64_t ld, void* split, void* stream) {
    CTK_RANGE("ctk_sgd_update_split_f32");
    CTK_REQUIRE(outer >= 0 && inner >= 0 && ld >= inner, "ctk_sgd_update_split_f32: bad extents");
    if (outer == 0 || inner == 0) return CTK_OK;
    CTK_REQUIRE(p && g && split, "ctk_sgd_update_split_f32: null pointer");
    CTK_REQUIRE(((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g)) & 15u) == 0 && inner % 4 == 0 && ld % 4 == 0,
                "ctk_sgd_update_split_f32: needs 16-byte aligned rows (use ctk_sgd_update_f32)");
    const SplitOut out = split_layout(split, outer, split_pitch_of(inner), g_correction, hi_in_place(p, inner, ld));
    const int64_t total = outer * (inner / 4);
    const int64_t per_cta = SPLIT_THREADS * SPLIT_UNROLL;
    sgd_split_vec_kernel<<<static_cast<unsigned>((total + per_cta - 1) / per_cta), SPLIT_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
        p, g, lr, out, outer, inner / 4, ld);
    CTK_LAUNCH_CHECK("sgd_split_vec_kernel");
    return CTK_OK;
}

// 3xTF32 MatMul that allocates nothing: same arguments and same result as ctk_matmul_f32 in mode
// CTK_MATMUL_3XTF32, with the hi/lo split kept in the library's fixed 16 MiB array instead of a
// workspace that is allocated or passed in.
//   - Operands whose split does not fit -- 2*(m*k + k*n) floats may take at most 16 MiB, which
//     1024x1024 by 1024x1024 just reaches -- are refused with CTK_ERR_LIMIT; nothing is launched.
//   - One-time set-up happens inside calls: the first call on a device looks up the array's device
//     address; the first call of each shape class on a device (tile width from n, major-ness of each
//     operand, CTA pairs or not) sets that kernel instantiation's shared-memory attribute and, for
//     pairs, queries the occupancy.  Make one call per shape class outside any stream capture first.
//   - `stream` must belong to the device that is current at the call.
//   - No byte of the array has to be zero on entry: each call writes the part it reads before it
//     reads it, so stale contents of the previous call do not matter.
//   - All calls on one GPU share the one array: two calls whose kernels may overlap (different
//     streams, no ordering between them) race on it.  Order them on the GPU.
//   - Launch timing (ctk_matmul_profile_enable) creates events on demand, so it must be off.
ctk_status ctk_matmul_3xtf32_noalloc_f32(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k,
                                         int64_t sa0, int64_t sa1, int64_t sb0, int64_t sb1, void* stream) {
    CTK_RANGE("ctk_matmul_3xtf32_noalloc_f32");
    CTK_REQUIRE(m >= 0 && n >= 0 && k >= 0, "ctk_matmul_3xtf32_noalloc_f32: negative extent");
    const size_t need = ctk_matmul_workspace_bytes(m, n, k, CTK_MATMUL_3XTF32);
    if (need > kStaticWorkspaceBytes)
        return fail(CTK_ERR_LIMIT, "ctk_matmul_3xtf32_noalloc_f32: operands need " + std::to_string(need) +
                                       " bytes of split scratch, the fixed array holds " + std::to_string(kStaticWorkspaceBytes) +
                                       " (2*(m*k + k*n) floats may take at most 16 MiB); use ctk_matmul_f32 with a workspace instead");
    {
        std::lock_guard<std::mutex> lock(g_prof_mu);
        if (g_prof.on) return fail(CTK_ERR_INVALID, "ctk_matmul_3xtf32_noalloc_f32: switch launch timing off first (it creates events)");
    }
    void* ws = nullptr;
    ctk_status rc = static_workspace(&ws);
    if (rc) return rc;
    return matmul_impl(a, b, c, m, n, k, sa0, sa1, sb0, sb1, CTK_MATMUL_3XTF32, ws, KeptSplit{nullptr, nullptr}, KeptSplit{nullptr, nullptr}, stream);
}

}  // extern "C"
