/* TEST INFRASTRUCTURE ONLY -- see ctorch_oracle.h.  Plain-C restatement of the CTorch reference's
 * CPU-BASIC arithmetic; each function cites the reference file:line it follows. */
#include "ctorch_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------------------------------ */
/* forward                                                                                    */
/* ------------------------------------------------------------------------------------------ */

static inline float bin1(int op, float x, float y) {
    switch (op) {
        case ORC_ADD: return x + y; /* src/kernels/CPU-BASIC/Add_BASIC_kernel.cpp:48-68 */
        case ORC_SUB: return x - y; /* Sub_BASIC_kernel.cpp:57-60 */
        case ORC_MUL: return x * y; /* Mul_BASIC_kernel.cpp:58-61 */
        case ORC_DIV: return x / y; /* Div_BASIC_kernel.cpp:37-44: IEEE quotient is stored even for y == 0 */
        default: return NAN;
    }
}

/* Add: same / scalar b / [N,H]+[H] (Add_BASIC_kernel.cpp:21-69).  Sub and Mul broadcast only by
 * materialising a 0-D operand (Sub_BASIC_kernel.cpp:23-45, Mul_BASIC_kernel.cpp:24-46); the other
 * layouts are evaluated here on the materialised operand, which is what the same loop would give. */
void orc_binary(int op, const float* a, const float* b, float* out, int64_t n, int bmode, int64_t inner) {
    for (int64_t i = 0; i < n; ++i) {
        float x = (bmode == ORC_A_SCALAR) ? a[0] : a[i];
        float y = (bmode == ORC_B_SAME || bmode == ORC_A_SCALAR) ? b[i] : (bmode == ORC_B_SCALAR) ? b[0] : b[i % inner];
        out[i] = bin1(op, x, y);
    }
}

static inline float un1(int op, float x) {
    switch (op) {
        case ORC_NEG: return -x;                      /* Neg_BASIC_kernel.cpp:26-28 */
        case ORC_RELU: return x > 0.0f ? x : 0.0f;    /* ReLU_BASIC_kernel.cpp:23-25: std::max(0.0f, x) (NaN -> 0) */
        case ORC_SIGMOID: return 1.0f / (1.0f + expf(-x)); /* Sigmoid_BASIC_kernel.cpp:24-26 */
        case ORC_TANH: {                              /* Tanh_BASIC_kernel.cpp:24-28: not tanhf */
            float ep = expf(x), en = expf(-x);
            return (ep - en) / (ep + en);
        }
        case ORC_SIN: return sinf(x);                 /* Sin_BASIC_kernel.cpp */
        case ORC_COS: return cosf(x);                 /* Cos_BASIC_kernel.cpp */
        default: return NAN;
    }
}

void orc_unary(int op, const float* a, float* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = un1(op, a[i]);
}

/* src/Tensor.cpp:751-806 (t*s), 855-910 (t+s), 913-973 (t/s), 1427-1429 (s-t), 1450-1452 (s/t). */
void orc_scalar(int kind, const float* a, int64_t n, float s, float* out) {
    for (int64_t i = 0; i < n; ++i) {
        float x = a[i];
        switch (kind) {
            case 0: out[i] = x * s; break;
            case 1: out[i] = x + s; break;
            case 2: out[i] = x / s; break;
            case 3: out[i] = s - x; break;
            case 4: out[i] = s / x; break;
            default: out[i] = NAN;
        }
    }
}

/* MatMul_BASIC_kernel.cpp:42-54: ijk loop, fp32 accumulator, k ascending, stride-aware.  Product
 * and sum are rounded separately (g++ -O3 does not fuse across the data<float>() calls). */
void orc_matmul(const float* a, const float* b, float* c, int64_t m, int64_t k, int64_t n,
                int64_t sa0, int64_t sa1, int64_t sb0, int64_t sb1) {
    for (int64_t i = 0; i < m; ++i)
        for (int64_t j = 0; j < n; ++j) {
            float sum = 0.0f;
            for (int64_t l = 0; l < k; ++l) sum += a[i * sa0 + l * sa1] * b[l * sb0 + j * sb1];
            c[i * n + j] = sum;
        }
}

/* Selected rows of the same product.  Every entry is the recurrence of MatMul_BASIC_kernel.cpp:42-54
 * (sum = 0; for l ascending: sum += a*b, product and sum rounded separately).  Where B's rows are
 * contiguous the loops are interchanged (l outside, j inside): each entry still sees exactly the
 * same sequence of operations, only the entries of a row advance together, which lets a full row
 * of an 8192^3 or 784 x 65536 x 4096 product finish in a fraction of a second. */
void orc_matmul_rows(const float* a, const float* b, float* c_rows, const int64_t* rows, int64_t n_rows,
                     int64_t k, int64_t n, int64_t sa0, int64_t sa1, int64_t sb0, int64_t sb1) {
    for (int64_t r = 0; r < n_rows; ++r) {
        const int64_t i = rows[r];
        float* out = c_rows + r * n;
        if (sb1 == 1) {
            for (int64_t j = 0; j < n; ++j) out[j] = 0.0f;
            for (int64_t l = 0; l < k; ++l) {
                const float av = a[i * sa0 + l * sa1];
                const float* brow = b + l * sb0;
                for (int64_t j = 0; j < n; ++j) out[j] += av * brow[j];
            }
            continue;
        }
        for (int64_t j = 0; j < n; ++j) {
            float sum = 0.0f;
            for (int64_t l = 0; l < k; ++l) sum += a[i * sa0 + l * sa1] * b[l * sb0 + j * sb1];
            out[j] = sum;
        }
    }
}

/* Selected entries (rows[e], cols[e]) of the same product, the same recurrence per entry: the
 * sampled check of products the CPU cannot finish in full (4096^3 and up). */
void orc_matmul_entries(const float* a, const float* b, float* out, const int64_t* rows, const int64_t* cols,
                        int64_t count, int64_t k, int64_t sa0, int64_t sa1, int64_t sb0, int64_t sb1) {
    for (int64_t e = 0; e < count; ++e) {
        const float* ap = a + rows[e] * sa0;
        const float* bp = b + cols[e] * sb1;
        float sum = 0.0f;
        for (int64_t l = 0; l < k; ++l) sum += ap[l * sa1] * bp[l * sb0];
        out[e] = sum;
    }
}

/* src/Tensor.cpp:638-666: sequential fp32 sum. */
float orc_sum(const float* a, int64_t n) {
    float s = 0.0f;
    for (int64_t i = 0; i < n; ++i) s += a[i];
    return s;
}

/* Dot_BASIC_kernel.cpp:37-40 */
float orc_dot(const float* a, const float* b, int64_t n) {
    float s = 0.0f;
    for (int64_t i = 0; i < n; ++i) s += a[i] * b[i];
    return s;
}

/* MSE_BASIC_kernel.cpp:35-41 */
float orc_mse(const float* a, const float* b, int64_t n) {
    float s = 0.0f;
    for (int64_t i = 0; i < n; ++i) {
        float d = a[i] - b[i];
        s = fmaf(d, d, s);
    }
    return s / (float)n;
}

/* MAE_BASIC_kernel.cpp:35-41 */
float orc_mae(const float* a, const float* b, int64_t n) {
    float s = 0.0f;
    for (int64_t i = 0; i < n; ++i) s += fabsf(a[i] - b[i]);
    return s / (float)n;
}

/* Softmax_BASIC_kernel.cpp:70-91 == src/Tensor.cpp:1712-1727: max, e = exp(x - max), sequential
 * sum, divide. */
void orc_softmax_rows(const float* in, float* out, int64_t rows, int64_t cols) {
    for (int64_t i = 0; i < rows; ++i) {
        const float* x = in + i * cols;
        float* y = out + i * cols;
        float mx = x[0];
        for (int64_t j = 1; j < cols; ++j)
            if (x[j] > mx) mx = x[j];
        float sum = 0.0f;
        for (int64_t j = 0; j < cols; ++j) {
            float e = expf(x[j] - mx);
            y[j] = e;
            sum += e;
        }
        if (sum > 0.0f)
            for (int64_t j = 0; j < cols; ++j) y[j] /= sum;
    }
}

/* CrossEntropy_BASIC_kernel.cpp:41-66: per row softmax (exp evaluated twice), clamp at 1e-10,
 * loss -= t*log(p), summed over rows AND classes, no mean. */
float orc_ce_onehot(const float* logits, const float* onehot, int64_t rows, int64_t cols) {
    float ce = 0.0f;
    for (int64_t i = 0; i < rows; ++i) {
        const float* x = logits + i * cols;
        const float* t = onehot + i * cols;
        float mx = x[0];
        for (int64_t j = 1; j < cols; ++j)
            if (x[j] > mx) mx = x[j];
        float es = 0.0f;
        for (int64_t j = 0; j < cols; ++j) es += expf(x[j] - mx);
        for (int64_t j = 0; j < cols; ++j) {
            float p = expf(x[j] - mx) / es;
            p = p > 1e-10f ? p : 1e-10f;
            ce = fmaf(-t[j], logf(p), ce);
        }
    }
    return ce;
}

/* CrossEntropy_BASIC_kernel.cpp:88-120: index labels stored as floats. */
int orc_ce_index(const float* logits, const float* labels, int64_t rows, int64_t cols, float* loss) {
    float ce = 0.0f;
    for (int64_t i = 0; i < rows; ++i) {
        int c = (int)labels[i];
        if (c < 0 || c >= (int)cols) return 1;
        const float* x = logits + i * cols;
        float mx = x[0];
        for (int64_t j = 1; j < cols; ++j)
            if (x[j] > mx) mx = x[j];
        float es = 0.0f;
        for (int64_t j = 0; j < cols; ++j) es += expf(x[j] - mx);
        float p = expf(x[c] - mx) / es;
        p = p > 1e-10f ? p : 1e-10f;
        ce -= logf(p);
    }
    *loss = ce;
    return 0;
}

/* ------------------------------------------------------------------------------------------ */
/* backward: the per-op rules of src/AutoDiff.cpp:1216-1855.  The rules are written with Tensor  */
/* operators, so every intermediate is rounded to fp32 on its own (one kernel call each).        */
/* ------------------------------------------------------------------------------------------ */

void orc_grad_unary(int op, const float* x, const float* g, float* dx, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
        switch (op) {
            case ORC_NEG: dx[i] = -g[i]; break;                              /* :1317 */
            case ORC_RELU: dx[i] = g[i] * (x[i] > 0.0f ? 1.0f : 0.0f); break; /* :1327-1371 */
            case ORC_SIGMOID: {                                              /* :1377-1383 */
                float s = un1(ORC_SIGMOID, x[i]);
                float oms = 1.0f - s;
                float t = s * oms;
                dx[i] = t * g[i];
                break;
            }
            case ORC_TANH: {                                                 /* :1389-1398 */
                float t = un1(ORC_TANH, x[i]);
                float t2 = t * t;
                float om = 1.0f - t2;
                dx[i] = om * g[i];
                break;
            }
            case ORC_SIN: dx[i] = cosf(x[i]) * g[i]; break;                  /* :1399-1407 */
            case ORC_COS: dx[i] = (-sinf(x[i])) * g[i]; break;               /* :1408-1416 */
            case ORC_SUM: dx[i] = g[0]; break;                               /* :1850-1855 + :579-627 */
            default: dx[i] = NAN;
        }
    }
}

/* src/AutoDiff.cpp:1455-1466: uses the saved OUTPUT y. */
void orc_softmax_backward_rows(const float* y, const float* g, float* dx, int64_t rows, int64_t cols) {
    for (int64_t i = 0; i < rows; ++i) {
        float dot = 0.0f;
        /* g++ -O3 vectorises this in-order reduction eight wide with separately rounded products
         * and fuses only the scalar remainder loop; restated so the pin stays bit-exact. */
        const int64_t body = cols & ~(int64_t)7;
        for (int64_t j = 0; j < body; ++j) dot += g[i * cols + j] * y[i * cols + j];
        for (int64_t j = body; j < cols; ++j) dot = fmaf(g[i * cols + j], y[i * cols + j], dot);
        for (int64_t j = 0; j < cols; ++j) {
            int64_t idx = i * cols + j;
            dx[idx] = y[idx] * (g[idx] - dot);
        }
    }
}

/* Add :1216-1221, Sub :1222-1233, Mul :1234-1258, Div :1259-1316, then the grad-shape adjustment
 * :562-1049 whose "can_broadcast" branch (:690-890) GATHERS with index 0 on the extra leading
 * dims -- a [B,H] gradient sent to an [H] operand is its first row, and a gradient sent to a
 * one-element operand is its first element. */
void orc_grad_binary(int op, const float* a, const float* b, const float* g, float* da, float* db,
                     int64_t n, int bmode, int64_t inner) {
    const int64_t nb = (bmode == ORC_B_SAME) ? n : (bmode == ORC_B_SCALAR) ? 1 : inner;
    for (int64_t i = 0; i < n; ++i) {
        float bi = (bmode == ORC_B_SAME) ? b[i] : (bmode == ORC_B_SCALAR) ? b[0] : b[i % inner];
        float ga, gb;
        switch (op) {
            case ORC_ADD: ga = g[i]; gb = g[i]; break;
            case ORC_SUB: ga = g[i]; gb = -g[i]; break;
            case ORC_MUL: ga = bi * g[i]; gb = a[i] * g[i]; break;
            case ORC_DIV: {
                ga = g[i] / bi;
                float na = -a[i];
                float t = na * g[i];
                float bb = bi * bi;
                gb = t / bb;
                break;
            }
            default: ga = gb = NAN;
        }
        if (da) da[i] = ga;
        if (db && i < nb) db[i] = gb;
    }
}

/* src/AutoDiff.cpp:1537-1574: softmax recomputed on the host (exp evaluated twice), minus the
 * one-hot target (Sub kernel), times the upstream scalar (operator*(float)). */
void orc_ce_backward(const float* logits, const float* onehot, float g, float* dlogits, int64_t rows, int64_t cols) {
    for (int64_t i = 0; i < rows; ++i) {
        const float* x = logits + i * cols;
        float mx = x[0];
        for (int64_t j = 1; j < cols; ++j)
            if (x[j] > mx) mx = x[j];
        float es = 0.0f;
        for (int64_t j = 0; j < cols; ++j) es += expf(x[j] - mx);
        for (int64_t j = 0; j < cols; ++j) {
            float p = expf(x[j] - mx) / es;
            float d = p - onehot[i * cols + j];
            dlogits[i * cols + j] = d * g;
        }
    }
}

/* src/AutoDiff.cpp:1491-1516: (((p - t) * 2) / n) * g */
void orc_mse_backward(const float* p, const float* t, float g, float* dp, int64_t n) {
    const float fn = (float)n;
    for (int64_t i = 0; i < n; ++i) {
        float d = p[i] - t[i];
        float d2 = d * 2.0f;
        float c = d2 / fn;
        dp[i] = c * g;
    }
}

/* src/AutoDiff.cpp:1602-1642: (sign(p - t) / n) * g */
void orc_mae_backward(const float* p, const float* t, float g, float* dp, int64_t n) {
    const float fn = (float)n;
    for (int64_t i = 0; i < n; ++i) {
        float d = p[i] - t[i];
        float s = d > 0.0f ? 1.0f : (d < 0.0f ? -1.0f : 0.0f);
        float c = s / fn;
        dp[i] = c * g;
    }
}

/* ------------------------------------------------------------------------------------------ */
/* The MLP training step, mnist/mnist.cpp:44-92, with the AutoDiff behaviours that define the   */
/* reference's numbers:                                                                         */
/*   - loss is the SUM of per-row cross entropies (CrossEntropy_BASIC_kernel.cpp:31,64);         */
/*   - the bias gradient is ROW 0 of the upstream gradient (src/AutoDiff.cpp:690-757);           */
/*   - dX = g . W0^T uses the copy of W taken when W was first registered as a leaf              */
/*     (src/AutoDiff.cpp:286-290 never refreshed, :1651), while forward uses the live W;         */
/*   - the first layer's input gets no gradient (requires_grad false, :1191-1192);               */
/*   - p -= g*lr compiles to one fused multiply-add.                                             */
/* ------------------------------------------------------------------------------------------ */
int orc_mlp_train(int n_layers, const int64_t* dims, int64_t batch, int steps, int replicas,
                  const float* x, const float* labels, int n_batches, float* params, float lr,
                  float* losses, const int* grad_steps, int n_grad_steps, float* grads_out,
                  float* logits_out) {
    int64_t n_params = 0, max_w = 0;
    for (int l = 0; l < n_layers; ++l) {
        n_params += dims[l] * dims[l + 1] + dims[l + 1];
        if (dims[l + 1] > max_w) max_w = dims[l + 1];
        if (dims[l] > max_w) max_w = dims[l];
    }
    const int64_t classes = dims[n_layers];
    /* per replica: live params; shared: the initial snapshot (identical for every replica) */
    float* snap = (float*)malloc(sizeof(float) * n_params);
    float* live = (float*)malloc(sizeof(float) * n_params * replicas);
    float* gsum = (float*)malloc(sizeof(float) * n_params);
    float* gtmp = (float*)malloc(sizeof(float) * n_params);
    float** act = (float**)malloc(sizeof(float*) * (n_layers + 1)); /* act[l+1] = pre-activation a_l */
    float** hid = (float**)malloc(sizeof(float*) * (n_layers + 1)); /* hid[l] = input of layer l     */
    float* gcur = (float*)malloc(sizeof(float) * batch * max_w);
    float* gnext = (float*)malloc(sizeof(float) * batch * max_w);
    float* onehot = (float*)malloc(sizeof(float) * batch * classes);
    memcpy(snap, params, sizeof(float) * n_params);
    for (int r = 0; r < replicas; ++r) memcpy(live + (int64_t)r * n_params, params, sizeof(float) * n_params);
    hid[0] = NULL;
    for (int l = 0; l < n_layers; ++l) {
        act[l + 1] = (float*)malloc(sizeof(float) * batch * dims[l + 1]);
        hid[l + 1] = (float*)malloc(sizeof(float) * batch * dims[l + 1]);
    }
    for (int s = 0; s < steps; ++s) {
        memset(gsum, 0, sizeof(float) * n_params);
        for (int r = 0; r < replicas; ++r) {
            float* P = live + (int64_t)r * n_params;
            const int64_t bi = s % n_batches;
            const float* xb = x + (((int64_t)r * n_batches + bi) * batch) * dims[0];
            const float* yb = labels + ((int64_t)r * n_batches + bi) * batch;
            /* forward */
            const float* h = xb;
            int64_t off = 0;
            for (int l = 0; l < n_layers; ++l) {
                const int64_t in = dims[l], out = dims[l + 1];
                const float* W = P + off;
                const float* b = W + in * out;
                off += in * out + out;
                float* a = act[l + 1];
                orc_matmul(h, W, a, batch, in, out, in, 1, out, 1);
                orc_binary(ORC_ADD, a, b, a, batch * out, ORC_B_ROW, out);
                if (l + 1 < n_layers) {
                    orc_unary(ORC_RELU, a, hid[l + 1], batch * out);
                    h = hid[l + 1];
                } else {
                    h = a;
                }
            }
            for (int64_t i = 0; i < batch; ++i) {
                int lab = (int)yb[i];
                for (int64_t j = 0; j < classes; ++j) onehot[i * classes + j] = (j == lab) ? 1.0f : 0.0f;
            }
            losses[(int64_t)s * replicas + r] = orc_ce_onehot(act[n_layers], onehot, batch, classes);
            if (logits_out && s == steps - 1)
                memcpy(logits_out + (int64_t)r * batch * classes, act[n_layers], sizeof(float) * batch * classes);
            /* backward */
            orc_ce_backward(act[n_layers], onehot, 1.0f, gcur, batch, classes);
            int64_t end = n_params;
            for (int l = n_layers - 1; l >= 0; --l) {
                const int64_t in = dims[l], out = dims[l + 1];
                const int64_t woff = end - (in * out + out);
                end = woff;
                float* dW = gtmp + woff;
                float* db = dW + in * out;
                memcpy(db, gcur, sizeof(float) * out); /* first row only */
                const float* hin = (l == 0) ? xb : hid[l];
                orc_matmul(hin, gcur, dW, in, batch, out, 1, in, out, 1); /* hin^T . g */
                if (l > 0) {
                    const float* W0 = snap + woff;
                    orc_matmul(gcur, W0, gnext, batch, out, in, out, 1, 1, out); /* g . W0^T */
                    const float* apre = act[l];
                    for (int64_t i = 0; i < batch * in; ++i) gcur[i] = gnext[i] * (apre[i] > 0.0f ? 1.0f : 0.0f);
                }
            }
            if (replicas == 1) memcpy(gsum, gtmp, sizeof(float) * n_params);
            else for (int64_t i = 0; i < n_params; ++i) gsum[i] += gtmp[i];
        }
        for (int q = 0; q < n_grad_steps; ++q)
            if (grad_steps[q] == s) memcpy(grads_out + (int64_t)q * n_params, gsum, sizeof(float) * n_params);
        for (int r = 0; r < replicas; ++r) {
            float* P = live + (int64_t)r * n_params;
            for (int64_t i = 0; i < n_params; ++i) P[i] = fmaf(-gsum[i], lr, P[i]);
        }
    }
    memcpy(params, live, sizeof(float) * n_params);
    for (int l = 0; l < n_layers; ++l) {
        free(act[l + 1]);
        free(hid[l + 1]);
    }
    free(snap); free(live); free(gsum); free(gtmp); free(act); free(hid); free(gcur); free(gnext); free(onehot);
    return 0;
}
