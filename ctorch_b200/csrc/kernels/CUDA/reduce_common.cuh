// Device helpers shared by the scalar reductions and the row-wise loss kernels: warp/block
// reductions by shuffle, and the single-launch "last block finishes" grid reduction.
#pragma once
#include "common.cuh"

namespace ctk {

constexpr int kMaxReduceBlocks = 16384;

// Layout of the reduction scratch: kMaxReduceBlocks per-block partial sums, then a ticket counter.
struct ReduceScratch {
    double partials[kMaxReduceBlocks];
    unsigned int ticket;
    unsigned int pad[3];
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over the CTA; result valid in every thread.  `smem` holds at least 33 doubles.
__device__ __forceinline__ double block_sum(double v, double* smem) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    if (warp == 0) {
        double t = lane < nwarps ? smem[lane] : 0.0;
        t = warp_sum(t);
        if (lane == 0) smem[32] = t;
    }
    __syncthreads();
    return smem[32];
}
__device__ __forceinline__ float block_max(float v, float* smem) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? smem[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) smem[32] = t;
    }
    __syncthreads();
    return smem[32];
}

// Every CTA contributes `cta_total` (valid in thread 0).  The CTA that takes the last ticket adds
// the partials in a fixed order (so the result does not depend on scheduling), writes
// out = float(total) * post_scale or float(total) / post_div, and rewinds the ticket for the next
// launch.  All threads of every CTA must call this.
__device__ __forceinline__ void grid_finish(double cta_total, ReduceScratch* s, float* out, float post_div,
                                            bool poison, double* smem) {
    __shared__ bool is_last;
    if (threadIdx.x == 0) {
        s->partials[blockIdx.x] = cta_total;
        __threadfence();
        unsigned int t = atomicAdd(&s->ticket, 1u);
        is_last = (t == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    double acc = 0.0;
    for (unsigned int i = threadIdx.x; i < gridDim.x; i += blockDim.x) acc += __ldcg(&s->partials[i]);
    acc = block_sum(acc, smem);
    if (threadIdx.x == 0) {
        float r = static_cast<float>(acc);
        if (post_div != 0.0f) r = r / post_div;
        *out = poison ? NAN : r;
        s->ticket = 0;
    }
}

ctk_status reduce_scratch(void* user, cudaStream_t st, ReduceScratch** out);
// A kernel left the library's own scratch block with a ticket it did not rewind: zero it before the next use.
void mark_reduce_scratch_dirty();

}  // namespace ctk
