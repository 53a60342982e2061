/*
 * ctorch_b200 -- C ABI of the B200 (sm_100a) kernel library behind CTorch's reserved
 * DeviceType::kCUDA slot.
 *
 * This is the boundary the reference's `*_CUDA_kernel(const Tensor&, ...)` adapters bind to
 * (prototypes reserved in the reference at src/kernels/kernels.h:42-242, dispatched by
 * include/Ctorch_Scheduler.h:86-166).  Plain pointers and sizes only: every pointer named
 * "device" is a CUDA device pointer of the current device, every `stream` is a cudaStream_t
 * passed as void* (NULL = the legacy default stream).
 *
 * Conventions
 *   - every function returns 0 on success or a non-zero ctk_status; ctk_last_error() gives the
 *     message of the calling thread's last failure;
 *   - launches are asynchronous on `stream`; nothing synchronises unless its comment says so;
 *   - all data are fp32 (the reference path is fp32 only); labels are floats holding integers,
 *     as in the reference;
 *   - operator codes are the numeric values of the reference's `enum class op`
 *     (include/Ctools.h:175-209), so an adapter can pass `static_cast<int>(op)`;
 *   - there is no CPU fallback anywhere: without a usable CUDA device every call fails with
 *     CTK_ERR_CUDA.
 */
#ifndef CTORCH_B200_H
#define CTORCH_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int ctk_status;
enum {
    CTK_OK = 0,
    CTK_ERR_INVALID = 1,  /* bad argument (shape, stride, mode, null pointer)      */
    CTK_ERR_CUDA = 2,     /* a CUDA runtime / driver call failed                   */
    CTK_ERR_NCCL = 3,     /* an NCCL call failed                                   */
    CTK_ERR_KERNEL = 4,   /* a kernel reported a bounded wait that ran out         */
    CTK_ERR_LIMIT = 5     /* size beyond a documented maximum                      */
};

/* Values of the reference's `enum class op` that this library implements. */
enum {
    CTK_OP_ADD = 0, CTK_OP_SUB = 1, CTK_OP_NEG = 2, CTK_OP_MUL = 3, CTK_OP_DIV = 4,
    CTK_OP_MATMUL = 5, CTK_OP_DOT = 6, CTK_OP_COS = 7, CTK_OP_SIN = 8, CTK_OP_RELU = 11,
    CTK_OP_TANH = 12, CTK_OP_SIGMOID = 13, CTK_OP_SOFTMAX = 14, CTK_OP_MSE = 17, CTK_OP_MAE = 18,
    CTK_OP_CE = 19, CTK_OP_SUM = 21
};

/* Layout of the operands of a binary elementwise op with n result elements. */
enum {
    CTK_B_SAME = 0,   /* a[n], b[n]                                                       */
    CTK_B_SCALAR = 1, /* a[n], b[1]           (reference: b.numel()==1 / 0-D operand)     */
    CTK_B_ROW = 2,    /* a[n/inner, inner], b[inner]   (reference: [N,H] op [H])           */
    CTK_A_SCALAR = 3  /* a[1], b[n]           (reference: 0-D left operand of Sub/Mul)     */
};

/* MatMul precision modes (north star: 3xTF32 for fp32-level accuracy, plain TF32). */
enum { CTK_MATMUL_3XTF32 = 0, CTK_MATMUL_TF32 = 1, CTK_MATMUL_FP32_SIMT = 2 };

/* ------------------------------------------------------------------------------------------- */
/* Errors, device, memory, streams, events.                                                     */
/* Replaces the host-only allocation of the reference's Storage (include/Storage.h:77, 88-93,   */
/* 175-181): device allocation from a stream-ordered pool plus pinned host staging.             */
/* ------------------------------------------------------------------------------------------- */
const char* ctk_last_error(void);
int ctk_version(void);
ctk_status ctk_device_count(int* count);
ctk_status ctk_set_device(int ordinal);
ctk_status ctk_get_device(int* ordinal);
ctk_status ctk_device_sync(void);
/* SM count, total and free device memory of the current device (any pointer may be NULL). */
ctk_status ctk_device_info(int* sm_count, size_t* total_bytes, size_t* free_bytes);

ctk_status ctk_malloc(void** device_ptr, size_t bytes);      /* pooled; bytes==0 gives NULL    */
/* Grows the pool's backing memory to at least `bytes` now, so that a training loop's first steps do
 * not stop for the driver to map memory piece by piece.  Synchronises the device. */
ctk_status ctk_pool_reserve(size_t bytes);
/* For buffers a caller keeps and recycles itself over many steps: plain device allocations outside
 * the pool (they would fragment it).  Both calls synchronise the device. */
ctk_status ctk_malloc_longlived(void** device_ptr, size_t bytes);
ctk_status ctk_free_longlived(void* device_ptr);
ctk_status ctk_free(void* device_ptr);
ctk_status ctk_malloc_host(void** pinned_ptr, size_t bytes); /* page-locked staging memory     */
ctk_status ctk_free_host(void* pinned_ptr);
ctk_status ctk_memcpy_h2d(void* device_dst, const void* host_src, size_t bytes, void* stream);
ctk_status ctk_memcpy_d2h(void* host_dst, const void* device_src, size_t bytes, void* stream);
ctk_status ctk_memcpy_d2d(void* device_dst, const void* device_src, size_t bytes, void* stream);
ctk_status ctk_memset(void* device_ptr, int byte_value, size_t bytes, void* stream);

ctk_status ctk_stream_create(void** stream);
/* non_blocking != 0: the stream does not synchronise with the legacy default stream. */
ctk_status ctk_stream_create_ex(void** stream, int non_blocking);
/* The same with the device's greatest (high_priority != 0) or least stream priority: pending blocks of a
 * higher-priority stream are placed first whenever SMs become free. */
ctk_status ctk_stream_create_priority(void** stream, int non_blocking, int high_priority);
ctk_status ctk_stream_destroy(void* stream);
ctk_status ctk_stream_sync(void* stream);
/* Stream capture (no counterpart in the reference): the work this thread issues to `stream` between
 * begin and end is recorded instead of run, and comes back as an executable graph that replays it
 * with one launch.  `stream` must be a created stream (the default stream cannot be captured); nothing
 * that allocates or synchronises may be called in between.  kernels_in_graph is added to
 * ctk_launch_count() per replay. */
ctk_status ctk_stream_begin_capture(void* stream);
ctk_status ctk_stream_end_capture(void* stream, void** graph_exec);
ctk_status ctk_graph_launch(void* graph_exec, void* stream, int kernels_in_graph);
ctk_status ctk_graph_destroy(void* graph_exec);
ctk_status ctk_event_create(void** event);
ctk_status ctk_event_destroy(void* event);
ctk_status ctk_event_record(void* event, void* stream);
ctk_status ctk_event_sync(void* event);
ctk_status ctk_event_elapsed_ms(void* start_event, void* stop_event, float* ms);
ctk_status ctk_stream_wait_event(void* stream, void* event);
/* *is_pinned = 1 if host_ptr lies in page-locked (or registered) host memory. */
ctk_status ctk_host_is_pinned(const void* host_ptr, int* is_pinned);
/* Number of kernels this library has launched in this process (bench bookkeeping). */
uint64_t ctk_launch_count(void);

/* ------------------------------------------------------------------------------------------- */
/* Elementwise, forward.                                                                        */
/* ------------------------------------------------------------------------------------------- */
/* out = a (op) b, op in {ADD,SUB,MUL,DIV}.  Replaces Add/Sub/Mul/Div_BASIC_kernel
 * (src/kernels/CPU-BASIC/Add_BASIC_kernel.cpp:11-71, Sub_..:12-62, Mul_..:13-63, Div_..:12-47).
 * `inner` is only read for CTK_B_ROW.  Division is IEEE (x/0 = inf, 0/0 = NaN), as the reference
 * stores. */
ctk_status ctk_binary_f32(int op, const float* a, const float* b, float* out, int64_t n, int layout,
                          int64_t inner, void* stream);
/* out = op(a), op in {NEG,RELU,SIGMOID,TANH,SIN,COS}.  Replaces Neg/ReLU/Sigmoid/Tanh/Sin/
 * Cos_BASIC_kernel (src/kernels/CPU-BASIC/*.cpp).  Tanh uses the reference's
 * (e^x - e^-x)/(e^x + e^-x), not tanhf. */
ctk_status ctk_unary_f32(int op, const float* a, float* out, int64_t n, void* stream);
/* Tensor-op-float forms that the reference computes with host loops, not through the scheduler
 * (src/Tensor.cpp:751-973, 1416-1453).  kind: 0 a*s, 1 a+s, 2 a/s, 3 s-a, 4 s/a. */
ctk_status ctk_scalar_f32(int kind, const float* a, float s, float* out, int64_t n, void* stream);
/* p[i] = value.  Replaces Tensor::zero/ones host loops (src/Tensor.cpp:390-455) and the 0-D
 * gradient fill of AutoDiff::check_and_adjust_grad_shape (src/AutoDiff.cpp:579-627).
 * If value_device is non-NULL the value is read from that device scalar instead. */
ctk_status ctk_fill_f32(float* p, float value, const float* value_device, int64_t n, void* stream);
/* dst[i] = src[i % src_n]: Tensor::broadcast_to for a trailing-dims broadcast
 * (src/Tensor.cpp:289-387) and the lower-rank tiling of the grad-shape adjustment
 * (src/AutoDiff.cpp:633-687). */
ctk_status ctk_tile_f32(const float* src, int64_t src_n, float* dst, int64_t n, void* stream);

/* onehot[r, j] = (j == (int)labels[r]) ? 1 : 0 for labels stored as floats: the host loop of
 * mnist/mnist.cpp:67-72, for labels that already live on the device. */
ctk_status ctk_onehot_f32(const float* labels, int64_t rows, int64_t classes, float* onehot, void* stream);

/* dst[i] = (float)src[i] / divisor (IEEE division): the pixel normalisation of the IDX image reader
 * (mnist/mnist_loader.cpp:34-41, `pixel / 255.0f`) on the device, so images cross PCIe as bytes. */
ctk_status ctk_u8_to_f32(const uint8_t* src, int64_t n, float divisor, float* dst, void* stream);

/* out_index[r] = first index j of row r with x[r,j] greater than `init` and than every earlier
 * element, 0 if there is none: the prediction loop of mnist/mnist.cpp:140-147 (init = -1 on
 * probabilities); init = -INFINITY is the plain first-maximum argmax.  Indices as floats, like
 * the labels they are compared with. */
ctk_status ctk_argmax_rows_f32(const float* x, int64_t rows, int64_t cols, float init, float* out_index, void* stream);

/* ---- comparisons, dtype conversion, typed fill, random numbers -------------------------------- */
enum { CTK_CMP_GT = 0, CTK_CMP_LT = 1, CTK_CMP_EQ = 2, CTK_CMP_GE = 3, CTK_CMP_LE = 4, CTK_CMP_NE = 5 };
enum { CTK_CMP_TENSOR = 0, CTK_CMP_SCALAR_RIGHT = 1, CTK_CMP_SCALAR_LEFT = 2 };
/* the values of the reference's `enum class DType` (include/Ctools.h:163-169) */
enum { CTK_DTYPE_F32 = 0, CTK_DTYPE_F64 = 1, CTK_DTYPE_I32 = 2, CTK_DTYPE_I64 = 3, CTK_DTYPE_BOOL = 4 };

/* out[i] = a[i] cmp b[i] (form TENSOR: Tensor::operator>, <, ==, >=, <=, != on two tensors,
 * src/Tensor.cpp:1119-1309), a[i] cmp scalar (SCALAR_RIGHT: the float forms, :985-1116) or
 * scalar cmp a[i] (SCALAR_LEFT: the free operators, :1462-1591), as bytes 0/1 -- the reference's
 * kBool tensors.  IEEE comparisons: anything against NaN is false except !=. */
ctk_status ctk_compare_f32(int cmp, int form, const float* a, const float* b, float scalar,
                           unsigned char* out, int64_t n, void* stream);
/* dst[i] = static_cast<T>(src[i]) for T = double, int32_t, int64_t, bool: Tensor::to(DType) out of
 * float (src/Tensor.cpp:199-243).  Integers truncate toward zero; values outside the target's range and
 * NaN are undefined behaviour in the reference (x86 yields INT_MIN) and saturate / give 0 here. */
ctk_status ctk_cast_f32(int dtype, const float* src, void* dst, int64_t n, void* stream);
/* dst[i] = value converted to the dtype: Tensor::ones / zero for every dtype (src/Tensor.cpp:390-450). */
ctk_status ctk_fill_dtype(int dtype, void* dst, double value, int64_t n, void* stream);
/* dst[i] = uniform in [0, 1): Tensor::rand (src/Tensor.cpp:458-479).  The reference draws from a
 * thread-local mt19937 seeded by std::random_device, so no sequence of it can be reproduced; here
 * element i is a pure function of (seed, offset + i) -- a counter-based generator (one splitmix64
 * finaliser per pair of counters, 24 bits of it each), identical for any launch shape, never 1.0. */
ctk_status ctk_rand_uniform_f32(float* dst, int64_t n, uint64_t seed, uint64_t offset, void* stream);

/* out[j] = sum over r of x[r, j] for a contiguous [rows, cols] array.  No counterpart in the reference,
 * whose gradient of a broadcast [H] operand is row 0 of the upstream gradient (src/AutoDiff.cpp:690-757);
 * this is the sum an opt-in "exact broadcast gradient" mode uses instead.  Two passes in fixed order:
 * the same bits from call to call. */
ctk_status ctk_colsum_f32(const float* x, int64_t rows, int64_t cols, float* out, void* stream);

/* out = number of i with (int)a[i] == (int)b[i] (as a float): the comparison of predicted and true
 * labels of mnist/mnist.cpp:150-153.  Exact up to 2^24 matches. */
ctk_status ctk_count_matches_f32(const float* a, const float* b, int64_t n, float* out, void* scratch, void* stream);

/* dst[r] = src[sum_j r_j * src_strides[j]] over the row-major index r of dst_shape (rank <= 8, a
 * stride of 0 repeats index 0): the gather of AutoDiff::check_and_adjust_grad_shape's broadcast
 * branch (src/AutoDiff.cpp:690-890), which takes index 0 on every broadcast dim. */
ctk_status ctk_gather_nd_f32(const float* src, float* dst, int rank, const int64_t* dst_shape,
                             const int64_t* src_strides, void* stream);

/* ------------------------------------------------------------------------------------------- */
/* Elementwise, backward (the per-op rules of AutoDiff::backward, src/AutoDiff.cpp:1216-1416),  */
/* each fused into one pass; intermediate roundings follow the reference's operator chain.      */
/* ------------------------------------------------------------------------------------------- */
/* dx = g * d op(x)/dx for op in {NEG,RELU,SIGMOID,TANH,SIN,COS}. */
ctk_status ctk_unary_backward_f32(int op, const float* x, const float* g, float* dx, int64_t n, void* stream);
/* da, db (either may be NULL) for op in {ADD,SUB,MUL,DIV}; g has n elements.  For CTK_B_ROW db has
 * `inner` elements and receives ROW 0 of the full gradient, for CTK_B_SCALAR db has one element
 * and receives element 0: the reference's grad-shape adjustment gathers with index 0 on the
 * broadcast dims, it does not sum (src/AutoDiff.cpp:690-757). */
ctk_status ctk_binary_backward_f32(int op, const float* a, const float* b, const float* g, float* da,
                                   float* db, int64_t n, int layout, int64_t inner, void* stream);
/* dst[i] += src[i]: the gradient accumulation loop (src/AutoDiff.cpp:1868-1907). */
ctk_status ctk_accumulate_f32(float* dst, const float* src, int64_t n, void* stream);
/* p[i] = fma(-g[i], lr, p[i]): the SGD loop of mnist/mnist.cpp:80-92 (one rounding, as compiled). */
ctk_status ctk_sgd_update_f32(float* p, const float* g, float lr, int64_t n, void* stream);

/* ------------------------------------------------------------------------------------------- */
/* Reductions to a scalar and row-wise losses.                                                  */
/* `out` is a DEVICE scalar.  `scratch` is device memory of at least ctk_reduce_scratch_bytes() */
/* bytes that no other running kernel uses; pass NULL to use the library's per-device scratch   */
/* (allocated on first use; calls that share it must be ordered on the GPU).                    */
/* ------------------------------------------------------------------------------------------- */
size_t ctk_reduce_scratch_bytes(void);
/* Tensor::sum (src/Tensor.cpp:638-666). */
ctk_status ctk_sum_f32(const float* a, int64_t n, float* out, void* scratch, void* stream);
/* Dot_BASIC_kernel (src/kernels/CPU-BASIC/Dot_BASIC_kernel.cpp:12-46). */
ctk_status ctk_dot_f32(const float* a, const float* b, int64_t n, float* out, void* scratch, void* stream);
/* MSE_BASIC_kernel / MAE_BASIC_kernel (:12-46 each): mean over ALL elements. */
ctk_status ctk_mse_f32(const float* a, const float* b, int64_t n, float* out, void* scratch, void* stream);
ctk_status ctk_mae_f32(const float* a, const float* b, int64_t n, float* out, void* scratch, void* stream);
/* dp = ((p - t) * 2 / n) * g and dp = (sign(p - t) / n) * g (src/AutoDiff.cpp:1491-1516,
 * 1602-1642); g is a device scalar (the upstream 0-D gradient). */
ctk_status ctk_mse_backward_f32(const float* p, const float* t, const float* g_device, float* dp, int64_t n, void* stream);
ctk_status ctk_mae_backward_f32(const float* p, const float* t, const float* g_device, float* dp, int64_t n, void* stream);

/* Synchronises the device and reads the row kernels' status word (no counterpart in the reference):
 * 0, or 1 once a bounded wait of the long-row kernel (rows of 4097..32768 floats, streamed through
 * shared memory with asynchronous copies) ran out; the outputs of that launch are then invalid and
 * its loss, if any, is NaN. */
ctk_status ctk_rowwise_status(int* status);
/* Row softmax over the last dim of [rows, cols]: Softmax_BASIC_kernel
 * (src/kernels/CPU-BASIC/Softmax_BASIC_kernel.cpp:16-101) == Tensor::softmax row path
 * (src/Tensor.cpp:1712-1727). */
ctk_status ctk_softmax_rows_f32(const float* x, float* y, int64_t rows, int64_t cols, void* stream);
/* Softmax down the columns (dim 0) of a row-major [rows, cols] matrix: Tensor::softmax(0)
 * (src/Tensor.cpp:1728-1743), and its backward dx = y * (g - sum_i g_i y_i) per column
 * (src/AutoDiff.cpp:1473-1484). */
ctk_status ctk_softmax_cols_f32(const float* x, float* y, int64_t rows, int64_t cols, void* stream);
ctk_status ctk_softmax_backward_cols_f32(const float* y, const float* g, float* dx, int64_t rows, int64_t cols, void* stream);
/* dx = y * (g - sum_j g_j y_j) per row, from the saved OUTPUT y (src/AutoDiff.cpp:1417-1490). */
ctk_status ctk_softmax_backward_rows_f32(const float* y, const float* g, float* dx, int64_t rows, int64_t cols, void* stream);
/* Softmax + cross entropy SUMMED over rows, clamp max(p, 1e-10): CrossEntropy_BASIC_kernel
 * one-hot path (CrossEntropy_BASIC_kernel.cpp:36-66) and index-label path (:88-120). */
ctk_status ctk_ce_onehot_f32(const float* logits, const float* onehot, int64_t rows, int64_t cols,
                             float* out, void* scratch, void* stream);
/* An out-of-range label makes the reference return an empty tensor; here *out becomes NaN and
 * the device word `bad_label_flag` (may be NULL) is set to 1. */
ctk_status ctk_ce_index_f32(const float* logits, const float* labels, int64_t rows, int64_t cols,
                            float* out, int* bad_label_flag, void* scratch, void* stream);
/* dlogits = (softmax(logits) - onehot) * g (src/AutoDiff.cpp:1517-1601); g is a device scalar,
 * or NULL for 1. */
ctk_status ctk_ce_backward_f32(const float* logits, const float* onehot, const float* g_device,
                               float* dlogits, int64_t rows, int64_t cols, void* stream);
/* Forward and backward in one pass over the logits, index labels: loss (summed) to *out and
 * dlogits = softmax - onehot(label).  Checked against the one-hot reference path. */
ctk_status ctk_ce_fused_index_f32(const float* logits, const float* labels, int64_t rows, int64_t cols,
                                  float* out, float* dlogits, int* bad_label_flag, void* scratch, void* stream);

/* ------------------------------------------------------------------------------------------- */
/* MatMul.  Replaces MatMul_BASIC_kernel (src/kernels/CPU-BASIC/MatMul_BASIC_kernel.cpp:13-57): */
/* C[i,j] = sum_l A[i*sa0 + l*sa1] * B[l*sb0 + j*sb1], C row-major [m,n]; strides in ELEMENTS,   */
/* exactly as that kernel reads them, so the stride-swapped views made by Tensor::t() (used by   */
/* the backward rule for dA = dC.B^T and dB = A^T.dC, src/AutoDiff.cpp:1702-1704, 1808-1810)     */
/* need no copy.                                                                                 */
/*   mode  CTK_MATMUL_3XTF32: three tcgen05 TF32 products of an exact hi/lo split, fp32 TMEM      */
/*         accumulation (fp32-level accuracy);  CTK_MATMUL_TF32: one TF32 product;                */
/*         CTK_MATMUL_FP32_SIMT: fp32 FMA on CUDA cores (also taken automatically when an         */
/*         operand cannot be addressed by TMA: a stride-1 dim is required and the other stride    */
/*         must be a multiple of 4 elements, base 16-byte aligned);  -1: the process default.     */
/*   workspace: device scratch for the hi/lo split, at least ctk_matmul_workspace_bytes() bytes;  */
/*         NULL uses the library's per-device workspace (grown on demand; calls sharing it must   */
/*         be ordered on the GPU).                                                                */
/* ------------------------------------------------------------------------------------------- */
ctk_status ctk_set_matmul_mode(int mode);
int ctk_get_matmul_mode(void);
/* Tile scheduling of the tensor-core path (no counterpart in the reference): 0 (default) computes   */
/* 256 x 256 tiles on pairs of CTAs (tcgen05 cta_group::2) whenever m > 128 and n > 128, 1 keeps     */
/* every product on the single-CTA kernel.  Both kernels accumulate k in the same order in fp32   */
/* TMEM, so the result does not depend on the choice.                                              */
ctk_status ctk_set_matmul_pairing(int pairing);
/* The fp32-accurate mode CTK_MATMUL_3XTF32 multiplies hi = tf32(x) parts on the TF32 path and adds two    */
/* correction terms lo.hi + hi.lo, lo = x - hi.  0: the corrections run on the TF32 path too (three TF32    */
/* products per fp32 product, "3xTF32").  1 (default): they run on the bf16 path -- their factors rounded  */
/* to bf16, which leaves 2^-20 of the product, the order of the lo.lo term both variants drop -- at twice   */
/* the TF32 rate: two units of tensor-core work per product instead of three, same bytes per operand      */
/* element; measured error at 4096^3 against float64: 1.0e-5 (bf16 path) / 1.6e-5 (TF32 path), normwise.  */
/* Process-wide; CTORCH_MATMUL_CORRECTION=tf32|bf16 in the environment sets the start value.  A split kept by the caller carries in its valid flag the tag of the setting it was made  */
/* under (ctk_matmul_split_tag: 1 or 2); a buffer with another tag is filled again.                        */
/* Where the operand itself can be read by TMA (16-byte aligned, rows a multiple of 16 bytes apart) it serves */
/* as the hi part of its own split -- the tensor core reads the top 19 bits of an fp32 word, i.e. hi =     */
/* x truncated -- and only the terms of x - hi are written (tag + 2; CTORCH_MATMUL_HI_IN_PLACE=0 switches   */
/* that off).  ctk_matmul_split_tag_for(p, inner, ld): the tag of a split of the array at p ([.., inner]    */
/* elements, row pitch ld) as ctk_matmul_3xtf32_fused_f32 and ctk_sgd_update_split_f32 write it.            */
ctk_status ctk_set_matmul_correction(int bf16);
int ctk_get_matmul_correction(void);
int ctk_matmul_split_tag(void);
int ctk_matmul_split_tag_for(const void* p, int64_t inner, int64_t ld);
/* 1 (default): when the last wave of output tiles would occupy at most half of the SMs (or CTA    */
/* pairs) -- which includes every product with few tiles, like the 10-class layer -- each of its   */
/* tiles is computed as two halves of K by two CTAs (pairs); the second half is added to the first   */
/* after a flag, always in that order, so repeated calls give the same bits -- where the contraction  */
/* is long enough for that to pay (the second half's epilogue runs after the first's: from K = 3072 */
/* in the fp32-accurate mode, 6144 in TF32 mode).  2: from K = 512, whatever it costs (tests).       */
/* 0: every tile whole.                                                                              */
ctk_status ctk_set_matmul_tail_split(int on);
/* Self-test of the kernels' bounded waits (no counterpart in the reference): one CTA waits with a  */
/* short limit on a barrier nothing arrives on.  result = {first wait ok (expected 0), CTA abort     */
/* flag (1), second waiter ok (0: it leaves as soon as it sees the flag), status word (0x7e57)}.    */
/* The kernel returns normally; the status word is restored afterwards.                            */
ctk_status ctk_matmul_selftest_wait_timeout(int result[4]);
size_t ctk_matmul_workspace_bytes(int64_t m, int64_t n, int64_t k, int mode);
ctk_status ctk_matmul_f32(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k,
                          int64_t sa0, int64_t sa1, int64_t sb0, int64_t sb1, int mode,
                          void* workspace, void* stream);
/* No counterpart in the reference.  The 3xTF32 product with the hi/lo split of either operand kept
 * by the caller between calls: an operand that enters several products unchanged (an activation
 * in its layer's forward product and, transposed, in the weight-gradient product; an upstream
 * gradient in both backward products; the weights a tape holds) is split once, not once per
 * product.  a_split / b_split: device buffers of ctk_matmul_split_bytes(m, k) / (n, k) bytes, or
 * NULL (that operand is split into the workspace as usual).  *a_valid / *b_valid: 0 = fill the
 * buffer in this call (set to 1 on return); 1 = it already holds the split of exactly these
 * values viewed with exactly these extents and strides (a transposed view of the same memory
 * counts as the same).  The caller discards the buffer when the operand's memory is written.
 * Operands the tensor cores cannot take (no unit stride) run on the CUDA cores; the flags are
 * then left alone. */
size_t ctk_matmul_split_bytes(int64_t mn, int64_t k);
ctk_status ctk_matmul_3xtf32_kept_f32(const float* a, const float* b, float* c, int64_t m, int64_t n,
                                      int64_t k, int64_t sa0, int64_t sa1, int64_t sb0, int64_t sb1,
                                      void* a_split, int* a_valid, void* b_split, int* b_valid,
                                      void* workspace, void* stream);
/* No counterpart in the reference (there the three are separate kernels: MatMul_BASIC_kernel, the
 * [N,H] + [H] form of Add_BASIC_kernel, ReLU_BASIC_kernel).  c = [relu](a.b + bias[col]) in one launch:
 * the epilogue of the 3xTF32 product adds the bias to the rounded fp32 accumulator, applies
 * x > 0 ? x : 0, stores c and -- if c_split is given -- c's own hi/lo split for the products c enters
 * next.  Bit-identical to the three kernels run in sequence (on whole tiles: this call never cuts a
 * tile's K in two).  mask, an [m, n] array of pitch n or NULL, multiplies the result by
 * (mask > 0 ? 1 : 0) before it is stored and split: with mask the output of a ReLU this is the ReLU's
 * backward rule (AutoDiff.cpp:1320-1371) applied to a gradient product g.W^T in its epilogue.
 * bias: n floats or NULL; relu: 0/1;
 * c_split: ctk_matmul_split_bytes(m, n) bytes or NULL; the other arguments as in
 * ctk_matmul_3xtf32_kept_f32.  Fails with CTK_ERR_INVALID if an operand has no unit stride. */
ctk_status ctk_matmul_3xtf32_fused_f32(const float* a, const float* b, float* c, int64_t m, int64_t n,
                                       int64_t k, int64_t sa0, int64_t sa1, int64_t sb0, int64_t sb1,
                                       void* a_split, int* a_valid, void* b_split, int* b_valid,
                                       const float* bias, int relu, const float* mask, void* c_split,
                                       void* workspace, void* stream);
/* The SGD loop of mnist/mnist.cpp:80-92 on a weight matrix, with the hi/lo split of the updated
 * weights written in the same pass: p = fma(-g, lr, p) exactly as ctk_sgd_update_f32, then hi/lo of the
 * new p into `split` (ctk_matmul_split_bytes(inner, outer) bytes), which ctk_matmul_3xtf32_kept_f32
 * accepts as valid for p viewed [outer, inner] with pitch ld, or its t() view.  p, g 16-byte aligned,
 * inner % 4 == 0, ld % 4 == 0, g contiguous; otherwise CTK_ERR_INVALID and nothing is launched. */
ctk_status ctk_sgd_update_split_f32(float* p, const float* g, float lr, int64_t outer, int64_t inner,
                                    int64_t ld, void* split, void* stream);
/* No counterpart in the reference.  The 3xTF32 product for callers that must not allocate device
 * memory (inside a stream capture, under an arena allocator that owns the whole GPU, or in a loop
 * that cannot afford a workspace growing under it): identical arguments and result to
 * ctk_matmul_f32(..., CTK_MATMUL_3XTF32, ...), but the hi/lo split lives in a fixed 16 MiB array that
 * is part of the library (held by every GPU that loads it).  Limit: the 2*(m*k + k*n) split floats
 * may take at most 16 MiB (1024x1024 by 1024x1024 just fits), otherwise CTK_ERR_LIMIT and nothing runs.
 * One-time set-up: the first call on a device looks up the array's address, and the first call of each
 * SHAPE CLASS on a device (tile width 64 / 128 / 256 from n, each operand's major-ness, CTA pairs or
 * not from m > 128) sets that kernel's shared-memory attribute and, for CTA pairs, asks the occupancy.
 * Make one call per shape class you will use outside any stream capture first.  `stream` must belong
 * to the device that is current at the call (the array's address is looked up for the current device).
 * Calls that may overlap on the GPU race on the shared array; launch timing must be off. */
ctk_status ctk_matmul_3xtf32_noalloc_f32(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k,
                                         int64_t sa0, int64_t sa1, int64_t sb0, int64_t sb1, void* stream);
/* Which path ctk_matmul_f32 would take: 0 tcgen05, 1 SIMT (an operand without a unit stride, or on
 * request), 2 the short-contraction kernel (3xTF32 mode, K <= 16, both operands K-major and contiguous,
 * n % 4 == 0, at least 2^20 outputs: one thread per four output columns on the CUDA cores, products and
 * sums rounded one by one in l order -- bit-identical to MatMul_BASIC_kernel.cpp:41-50 -- and bound by
 * the output's bytes; takes the mask and split forms of ctk_matmul_3xtf32_fused_f32, not bias / ReLU),
 * 3 the narrow-output kernels (3xTF32 mode, n <= 16, k >= 256, at least 2^20 elements of A, A 16-byte
 * aligned with a unit stride and whole 16-byte pieces along it, no fused epilogue: A read once as fp32
 * on the CUDA cores, fp32 FMAs and fp32 sums in a fixed order, bound by A's bytes -- the 10-class
 * layer's logits and weight gradient; within the mode's 1e-4 of MatMul_BASIC_kernel.cpp:41-50, not
 * bit-identical to it). */
int ctk_matmul_path(const float* a, const float* b, int64_t m, int64_t n, int64_t k,
                    int64_t sa0, int64_t sa1, int64_t sb0, int64_t sb1, int mode);
/* Per-launch timing of the tensor-core kernel with CUDA events on the launching stream (off by
 * default).  ctk_matmul_profile_read synchronises, returns the number of launches timed since the
 * last enable/read, their summed duration and their summed algorithmic flops (2*m*n*k each), and
 * clears the record.  At most 8192 launches are kept per interval. */
ctk_status ctk_matmul_profile_enable(int on);
ctk_status ctk_matmul_profile_read(int64_t* launches, double* total_ms, double* total_flops);
/* Device status word of the tensor-core kernel's bounded waits: 0 = none ran out.  Reading it
 * synchronises the device. */
ctk_status ctk_matmul_status(int* status);

/* ------------------------------------------------------------------------------------------- */
/* Data-parallel gradient exchange (no counterpart in the reference, which is single-process):  */
/* one NCCL communicator per process, fp32 sum.                                                  */
/* ------------------------------------------------------------------------------------------- */
#define CTK_COMM_ID_BYTES 128
ctk_status ctk_comm_unique_id(void* id_out_128_bytes);
ctk_status ctk_comm_init_rank(void** comm, const void* id_128_bytes, int world_size, int rank);
/* The same with an upper bound on the CTAs a collective may occupy (max_ctas) and on those of its
 * in-switch part (nvls_ctas); 0 = NCCL's choice.  The collectives share the SMs with the persistent
 * MatMul kernels of backward. */
ctk_status ctk_comm_init_rank_config(void** comm, const void* id_128_bytes, int world_size, int rank, int max_ctas, int nvls_ctas);
ctk_status ctk_comm_info(void* comm, int* world_size, int* rank, int* nccl_version);
ctk_status ctk_comm_destroy(void* comm);
/* Device memory allocated by NCCL's allocator and registered with the communicator (symmetric != 0:
 * as a symmetric window), so collectives on it run out of user memory.  Collective calls: every rank
 * makes them, with the same sizes, in the same order. */
ctk_status ctk_comm_alloc(void* comm, size_t bytes, int symmetric, void** device_ptr);
ctk_status ctk_comm_free(void* comm, void* device_ptr);
ctk_status ctk_allreduce_sum_f32(void* comm, float* device_buf, int64_t n, void* stream);
/* recv[0, count) = sum over ranks of send[rank*count, (rank+1)*count); send holds world*count floats. */
ctk_status ctk_reduce_scatter_sum_f32(void* comm, const float* send, float* recv, int64_t count, void* stream);
/* recv[r*count, (r+1)*count) = rank r's send[0, count). */
ctk_status ctk_allgather_f32(void* comm, const float* send, float* recv, int64_t count, void* stream);
/* Failure detection.  ctk_comm_wait blocks the host until `event` has completed, polling the event and
 * ncclCommGetAsyncError, for at most timeout_ms: a peer that died or never joined would otherwise leave
 * the collective -- and a plain stream synchronisation -- waiting for ever.  On an asynchronous error
 * or at the deadline the communicator is aborted (ncclCommAbort ends its kernels) and CTK_ERR_NCCL is
 * returned; the CUDA context stays usable, the communicator does not.  ctk_comm_abort does the abort
 * alone.  ctk_watchdog_wait is the loop underneath with the three steps as callbacks (query: 1 done,
 * 0 pending, < 0 error; health: 0 fine; abort: called once before an error is returned), which is how
 * the loop is tested without a GPU. */
typedef int (*ctk_watch_fn)(void* user);
ctk_status ctk_comm_wait(void* comm, void* event, int timeout_ms);
ctk_status ctk_comm_abort(void* comm);
ctk_status ctk_watchdog_wait(ctk_watch_fn query, ctk_watch_fn health, ctk_watch_fn abort_fn, void* user, int timeout_ms, int poll_us);

#ifdef __cplusplus
}
#endif
#endif /* CTORCH_B200_H */
