/* TEST INFRASTRUCTURE ONLY -- the parity oracle.  Never linked into, imported by or called from
 * the product path; only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg use it.
 *
 * A plain-C, single-threaded restatement of the CTorch reference's CPU-BASIC arithmetic and of the
 * AutoDiff rules that the MLP training step exercises.  Each function names the reference
 * file:line it follows (paths relative to the reference checkout).  Where g++ -O3 on an FMA
 * machine contracts the reference's `s += a*b` into one fused multiply-add, the restatement calls
 * fmaf() explicitly (the library is built with -ffp-contract=off, so nothing else is fused).
 *
 * Parity pinned: every function here is checked bit-for-bit (libm-dependent ones to 1e-6) against
 * the unmodified reference library (oracle/_ref, built from the reference's own sources) and
 * against the committed fixtures in tests/golden/, which that library produced.
 *
 * Operator codes are the numeric values of the reference's `enum class op`
 * (include/Ctools.h:175-209).
 */
#ifndef CTORCH_ORACLE_H
#define CTORCH_ORACLE_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    ORC_ADD = 0, ORC_SUB = 1, ORC_NEG = 2, ORC_MUL = 3, ORC_DIV = 4, ORC_MATMUL = 5, ORC_DOT = 6,
    ORC_COS = 7, ORC_SIN = 8, ORC_RELU = 11, ORC_TANH = 12, ORC_SIGMOID = 13, ORC_SOFTMAX = 14,
    ORC_MSE = 17, ORC_MAE = 18, ORC_CE = 19, ORC_SUM = 21
};

/* Broadcast layout of the second operand of a binary elementwise op. */
enum {
    ORC_B_SAME = 0,   /* b has a's shape                                             */
    ORC_B_SCALAR = 1, /* b has one element                                           */
    ORC_B_ROW = 2,    /* a is [n/inner, inner], b is [inner]                         */
    ORC_A_SCALAR = 3  /* a has one element, result has b's shape (n = b's numel)     */
};

/* ---- forward ---- */
void orc_binary(int op, const float* a, const float* b, float* out, int64_t n, int bmode, int64_t inner);
void orc_unary(int op, const float* a, float* out, int64_t n);
/* kind: 0 t*s, 1 t+s, 2 t/s, 3 s-t, 4 s/t */
void orc_scalar(int kind, const float* a, int64_t n, float s, float* out);
void orc_matmul(const float* a, const float* b, float* c, int64_t m, int64_t k, int64_t n,
                int64_t sa0, int64_t sa1, int64_t sb0, int64_t sb1);
/* Selected rows of the same product: c_rows[r, :] = row rows[r] of A·B. */
void orc_matmul_rows(const float* a, const float* b, float* c_rows, const int64_t* rows, int64_t n_rows,
                     int64_t k, int64_t n, int64_t sa0, int64_t sa1, int64_t sb0, int64_t sb1);
/* Selected entries of the same product: out[e] = (A·B)[rows[e], cols[e]]. */
void orc_matmul_entries(const float* a, const float* b, float* out, const int64_t* rows, const int64_t* cols,
                        int64_t count, int64_t k, int64_t sa0, int64_t sa1, int64_t sb0, int64_t sb1);
float orc_sum(const float* a, int64_t n);
float orc_dot(const float* a, const float* b, int64_t n);
float orc_mse(const float* a, const float* b, int64_t n);
float orc_mae(const float* a, const float* b, int64_t n);
void orc_softmax_rows(const float* in, float* out, int64_t rows, int64_t cols);
float orc_ce_onehot(const float* logits, const float* onehot, int64_t rows, int64_t cols);
/* returns 0 and writes *loss, or 1 if a label is out of range (the reference returns an empty tensor) */
int orc_ce_index(const float* logits, const float* labels, int64_t rows, int64_t cols, float* loss);

/* ---- backward (AutoDiff rules) ---- */
void orc_grad_unary(int op, const float* x, const float* g, float* dx, int64_t n);
void orc_softmax_backward_rows(const float* y, const float* g, float* dx, int64_t rows, int64_t cols);
/* da/db may be NULL.  For ORC_B_ROW db has `inner` elements and receives row 0 of the full gradient
 * (the reference's grad-shape adjustment gathers, it does not sum).  For ORC_B_SCALAR db has one
 * element and receives element 0 of the full gradient, for the same reason. */
void orc_grad_binary(int op, const float* a, const float* b, const float* g, float* da, float* db,
                     int64_t n, int bmode, int64_t inner);
void orc_ce_backward(const float* logits, const float* onehot, float g, float* dlogits, int64_t rows, int64_t cols);
void orc_mse_backward(const float* p, const float* t, float g, float* dp, int64_t n);
void orc_mae_backward(const float* p, const float* t, float g, float* dp, int64_t n);

/* ---- the MLP training step (mnist/mnist.cpp:44-92) for `replicas` summed-gradient replicas ----
 * Same argument meaning as ref_mlp_train in ref_shim.cpp. */
int orc_mlp_train(int n_layers, const int64_t* dims, int64_t batch, int steps, int replicas,
                  const float* x, const float* labels, int n_batches, float* params, float lr,
                  float* losses, const int* grad_steps, int n_grad_steps, float* grads_out,
                  float* logits_out);

#ifdef __cplusplus
}
#endif
#endif
