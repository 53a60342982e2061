// TEST INFRASTRUCTURE ONLY -- never linked into, imported by or called from the product path.
//
// A C-ABI window onto the UNMODIFIED CTorch reference library.  This file is compiled together
// with the reference's own translation units (src/Tensor.cpp, src/AutoDiff.cpp, src/Ctools.cpp,
// src/kernels/CPU-BASIC/*.cpp) where they lie in the reference checkout; it contains no reference
// code itself.  Every entry point builds reference `Tensor` objects from caller buffers, drives the
// reference's public API (operators, Tensor methods, AutoDiff) and copies the result back, so the
// numbers that come out are the reference's own CPU-BASIC results.
//
// Used for: (1) pinning the plain-C restatement in oracle/ctorch_oracle.c, (2) generating the
// golden fixtures under tests/golden/, (3) the timed CPU baseline ("kind": "reference").
//
// Conventions: every function returns 0 on success, 1 if the reference threw (message available
// from ref_last_error()).  Operator codes are the numeric values of the reference's `enum class op`
// (include/Ctools.h:175-209).

#include <cstdint>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "Tensor.h"
#include "mnist_loader.h"
#include "AutoDiff.h"
#include "Ctorch_Error.h"
#include "../src/kernels/kernels.h"

namespace {

std::string g_err;

Tensor make(const float* src, const int64_t* shape, int rank) {
    std::vector<size_t> s(shape, shape + rank);
    Tensor t(ShapeTag{}, s, DType::kFloat, DeviceType::kCPU);
    if (src && t.numel() > 0) std::memcpy(t.data<float>(), src, t.numel() * sizeof(float));
    return t;
}

Tensor make2d(const float* src, int64_t r, int64_t c) {
    int64_t s[2] = {r, c};
    return make(src, s, 2);
}

int64_t copy_out(const Tensor& t, float* dst) {
    int64_t n = static_cast<int64_t>(t.numel());
    if (dst && n > 0 && t.data<float>()) std::memcpy(dst, t.data<float>(), n * sizeof(float));
    return n;
}

template <typename F>
int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return 1;
    } catch (...) {
        g_err = "unknown exception";
        return 1;
    }
}

Tensor apply_unary(const Tensor& x, int opc) {
    switch (static_cast<op>(opc)) {
        case op::Neg: return -x;
        case op::ReLU: return x.relu();
        case op::Sigmoid: return x.sigmoid();
        case op::Tanh: return x.tanh();
        case op::Sin: return x.sin();
        case op::Cos: return x.cos();
        case op::Softmax: return x.softmax(-1);
        case op::Sum: return x.sum();
        default: throw std::runtime_error("ref_shim: unsupported unary op");
    }
}

Tensor apply_binary(const Tensor& a, const Tensor& b, int opc) {
    switch (static_cast<op>(opc)) {
        case op::Add: return a + b;
        case op::Sub: return a - b;
        case op::Mul: return a * b;
        case op::Div: return a / b;
        case op::MatMul: return a.matmul(b);
        case op::Dot: return a.dot(b);
        case op::MSE: return a.mse_loss(b);
        case op::MAE: return a.mae_loss(b);
        case op::CE: return a.cross_entropy(b);
        default: throw std::runtime_error("ref_shim: unsupported binary op");
    }
}

}  // namespace

extern "C" {

const char* ref_last_error() { return g_err.c_str(); }

// Touch both singletons (the first log call sleeps 500 ms) and silence tracing.
int ref_init() {
    return guarded([] {
        static bool done = false;
        if (done) return;
        Ctorch_Error::setPrintLevel(PrintLevel::MINIUM);
        Tensor a({1.0f}), b({2.0f});
        Tensor c = a + b;
        (void)c;
        done = true;
    });
}

// out = op(a) ; returns numel via *out_numel.
int ref_unary(int opc, const float* a, const int64_t* shape, int rank, float* out, int64_t* out_numel) {
    return guarded([&] {
        Tensor x = make(a, shape, rank);
        Tensor y = apply_unary(x, opc);
        int64_t n = copy_out(y, out);
        if (out_numel) *out_numel = n;
    });
}

// The registered-but-unreachable Softmax kernel (src/kernels/CPU-BASIC/Softmax_BASIC_kernel.cpp).
int ref_softmax_kernel(const float* a, const int64_t* shape, int rank, float* out) {
    return guarded([&] {
        Tensor x = make(a, shape, rank);
        Tensor y = Softmax_BASIC_kernel(x);
        copy_out(y, out);
    });
}

int ref_binary(int opc, const float* a, const int64_t* ashape, int arank, const float* b,
               const int64_t* bshape, int brank, float* out, int64_t* out_numel) {
    return guarded([&] {
        Tensor x = make(a, ashape, arank);
        Tensor y = make(b, bshape, brank);
        Tensor z = apply_binary(x, y, opc);
        int64_t n = copy_out(z, out);
        if (out_numel) *out_numel = n;
    });
}

// kind: 0 t*s, 1 t+s, 2 t/s, 3 s-t, 4 s/t, 5 s*t, 6 s+t   (src/Tensor.cpp:751-973, 1416-1453)
int ref_scalar(int kind, const float* a, int64_t n, float s, float* out) {
    return guarded([&] {
        int64_t shape[1] = {n};
        Tensor x = make(a, shape, 1);
        Tensor y;
        switch (kind) {
            case 0: y = x * s; break;
            case 1: y = x + s; break;
            case 2: y = x / s; break;
            case 3: y = s - x; break;
            case 4: y = s / x; break;
            case 5: y = s * x; break;
            case 6: y = s + x; break;
            default: throw std::runtime_error("ref_shim: bad scalar kind");
        }
        copy_out(y, out);
    });
}

// C[m,n] = A·B where A is stored [m,k] (ta=0) or stored [k,m] and viewed through t() (ta=1);
// likewise B stored [k,n] (tb=0) or [n,k] viewed through t() (tb=1).
int ref_matmul(const float* a, const float* b, int64_t m, int64_t k, int64_t n, int ta, int tb, float* out) {
    return guarded([&] {
        Tensor A = ta ? make2d(a, k, m).t() : make2d(a, m, k);
        Tensor B = tb ? make2d(b, n, k).t() : make2d(b, k, n);
        Tensor C = A.matmul(B);
        copy_out(C, out);
    });
}

// dx = d(sum_i g_i * op(x)_i)/dx through the reference's AutoDiff.  g has the shape of op(x)
// (one element for Sum).
int ref_grad_unary(int opc, const float* x, const int64_t* shape, int rank, const float* g, float* dx) {
    return guarded([&] {
        AutoDiff ctx;
        AutoDiffContext::Guard guard(&ctx);
        Tensor X = make(x, shape, rank);
        X.requires_grad(true);
        Tensor Y = apply_unary(X, opc);
        Tensor G;
        if (Y.sizes().empty()) {
            G = Tensor(g[0]);
        } else {
            std::vector<int64_t> ys(Y.sizes().begin(), Y.sizes().end());
            G = make(g, ys.data(), static_cast<int>(ys.size()));
        }
        {
            AutoDiffContext::Guard off(nullptr);
            ctx.backward(Y, G);
        }
        Tensor D = grad(X);
        copy_out(D, dx);
    });
}

// da, db = gradients of sum(g * op(a,b)) (either may be null to skip).  g has the result's shape
// (one element for the 0-D losses).
int ref_grad_binary(int opc, const float* a, const int64_t* ashape, int arank, const float* b,
                    const int64_t* bshape, int brank, const float* g, float* da, float* db) {
    return guarded([&] {
        AutoDiff ctx;
        AutoDiffContext::Guard guard(&ctx);
        Tensor A = make(a, ashape, arank);
        Tensor B = make(b, bshape, brank);
        if (da) A.requires_grad(true);
        if (db) B.requires_grad(true);
        Tensor Y = apply_binary(A, B, opc);
        Tensor G;
        if (Y.sizes().empty()) {
            G = Tensor(g[0]);
        } else {
            std::vector<int64_t> ys(Y.sizes().begin(), Y.sizes().end());
            G = make(g, ys.data(), static_cast<int>(ys.size()));
        }
        {
            AutoDiffContext::Guard off(nullptr);
            ctx.backward(Y, G);
        }
        if (da) copy_out(grad(A), da);
        if (db) copy_out(grad(B), db);
    });
}

// The training step of mnist/mnist.cpp:44-92 generalised to any layer list, for `replicas`
// independent model replicas that sum their gradients element-wise before the SGD update
// (replicas = 1 is exactly the reference program's step).
//
//   dims[0..n_layers]        layer widths (dims[0] = input features, dims[n_layers] = classes)
//   x       [replicas][n_batches][batch][dims[0]]   step s uses batch s % n_batches
//   labels  [replicas][n_batches][batch]            class indices stored as floats
//   params  W1,b1,W2,b2,... packed, in/out (identical start for every replica)
//   losses  [steps][replicas]
//   grad_steps/n_grad_steps  steps whose (replica-summed) gradients are copied to grads_out
//   grads_out [n_grad_steps][packed params]
//   logits_out [replicas][batch][classes] of the LAST step (may be null)
int ref_mlp_train(int n_layers, const int64_t* dims, int64_t batch, int steps, int replicas,
                  const float* x, const float* labels, int n_batches, float* params, float lr,
                  float* losses, const int* grad_steps, int n_grad_steps, float* grads_out,
                  float* logits_out) {
    return guarded([&] {
        struct Replica {
            std::unique_ptr<AutoDiff> ctx;
            std::vector<Tensor> W, b;
        };
        int64_t n_params = 0;
        for (int l = 0; l < n_layers; ++l) n_params += dims[l] * dims[l + 1] + dims[l + 1];
        std::vector<Replica> reps(replicas);
        for (auto& r : reps) {
            r.ctx = std::make_unique<AutoDiff>();
            const float* p = params;
            for (int l = 0; l < n_layers; ++l) {
                r.W.push_back(make2d(p, dims[l], dims[l + 1]));
                p += dims[l] * dims[l + 1];
                int64_t bs[1] = {dims[l + 1]};
                r.b.push_back(make(p, bs, 1));
                p += dims[l + 1];
            }
        }
        const int64_t classes = dims[n_layers];
        std::vector<float> gsum(n_params), gtmp(n_params);
        for (int s = 0; s < steps; ++s) {
            std::fill(gsum.begin(), gsum.end(), 0.0f);
            for (int r = 0; r < replicas; ++r) {
                Replica& R = reps[r];
                AutoDiffContext::Guard guard(R.ctx.get());
                AutoDiff* ctx = AutoDiffContext::current();
                for (int l = 0; l < n_layers; ++l) {
                    ctx->make_leaf(R.W[l], true);
                    ctx->make_leaf(R.b[l], true);
                }
                for (int l = 0; l < n_layers; ++l) {
                    R.W[l].requires_grad(true);
                    R.b[l].requires_grad(true);
                }
                for (int l = 0; l < n_layers; ++l) {
                    ctx->zero_grad(R.W[l]);
                    ctx->zero_grad(R.b[l]);
                }
                const int64_t bi = s % n_batches;
                const float* xb = x + ((static_cast<int64_t>(r) * n_batches + bi) * batch) * dims[0];
                const float* yb = labels + (static_cast<int64_t>(r) * n_batches + bi) * batch;
                Tensor X = make2d(xb, batch, dims[0]);
                Tensor h = X;
                // Temporaries are move-assigned so tensor ids (the graph keys) survive, exactly as
                // in the reference program's `Tensor h1 = (x.matmul(W1) + b1).relu();`.
                for (int l = 0; l < n_layers; ++l) {
                    if (l + 1 < n_layers)
                        h = (h.matmul(R.W[l]) + R.b[l]).relu();
                    else
                        h = h.matmul(R.W[l]) + R.b[l];
                }
                Tensor onehot = make2d(nullptr, batch, classes);
                for (int64_t i = 0; i < batch; ++i) {
                    int lab = static_cast<int>(yb[i]);
                    for (int64_t j = 0; j < classes; ++j)
                        onehot.data<float>()[i * classes + j] = (j == lab) ? 1.0f : 0.0f;
                }
                Tensor loss = h.cross_entropy(onehot);
                losses[static_cast<int64_t>(s) * replicas + r] = loss.item<float>();
                backward(loss);
                if (logits_out && s == steps - 1)
                    copy_out(h, logits_out + static_cast<int64_t>(r) * batch * classes);
                float* gp = gtmp.data();
                for (int l = 0; l < n_layers; ++l) {
                    gp += copy_out(grad(R.W[l]), gp);
                    gp += copy_out(grad(R.b[l]), gp);
                }
                if (replicas == 1) {
                    gsum = gtmp;
                } else {
                    for (int64_t i = 0; i < n_params; ++i) gsum[i] += gtmp[i];
                }
            }
            for (int q = 0; q < n_grad_steps; ++q)
                if (grad_steps[q] == s)
                    std::memcpy(grads_out + static_cast<int64_t>(q) * n_params, gsum.data(),
                                n_params * sizeof(float));
            for (auto& R : reps) {
                const float* gp = gsum.data();
                for (int l = 0; l < n_layers; ++l) {
                    float* w = R.W[l].data<float>();
                    for (size_t i = 0; i < R.W[l].numel(); ++i) w[i] -= gp[i] * lr;
                    gp += R.W[l].numel();
                    float* bb = R.b[l].data<float>();
                    for (size_t i = 0; i < R.b[l].numel(); ++i) bb[i] -= gp[i] * lr;
                    gp += R.b[l].numel();
                }
            }
        }
        float* p = params;
        for (int l = 0; l < n_layers; ++l) {
            p += copy_out(reps[0].W[l], p);
            p += copy_out(reps[0].b[l], p);
        }
    });
}

// Tensor::softmax(dim) (src/Tensor.cpp:1645-1803) and, if g and dx are given, the gradient of
// sum(g * softmax(x, dim)) through the reference's backward rule (src/AutoDiff.cpp:1417-1490).
int ref_softmax_dim(const float* x, const int64_t* shape, int rank, int dim, float* out, const float* g, float* dx) {
    return guarded([&] {
        AutoDiff ctx;
        AutoDiffContext::Guard guard(&ctx);
        Tensor X = make(x, shape, rank);
        X.requires_grad(g != nullptr);
        Tensor Y = X.softmax(dim);
        copy_out(Y, out);
        if (g && dx) {
            std::vector<int64_t> ys(Y.sizes().begin(), Y.sizes().end());
            Tensor G = make(g, ys.data(), static_cast<int>(ys.size()));
            {
                AutoDiffContext::Guard off(nullptr);
                ctx.backward(Y, G);
            }
            copy_out(grad(X), dx);
        }
    });
}

// MNISTLoader of the reference (mnist/mnist_loader.{h,cpp}, compiled from where it lies): the
// training pair (test = 0) or the test pair (test = 1) of directory `dir`.  Sizes always come back;
// data is copied only when the caller's capacities (in elements) suffice.
int ref_mnist_load(const char* dir, int test, float* images, int64_t cap_images, int64_t* n_images,
                   int64_t* image_size, float* labels, int64_t cap_labels, int64_t* n_labels) {
    return guarded([&] {
        MNISTLoader loader(dir);
        Tensor im, lb;
        if (test) loader.load_test_data(im, lb);
        else loader.load_training_data(im, lb);
        *n_images = static_cast<int64_t>(im.shape()[0]);
        *image_size = static_cast<int64_t>(im.shape()[1]);
        *n_labels = static_cast<int64_t>(lb.shape()[0]);
        if (images && cap_images >= static_cast<int64_t>(im.numel())) copy_out(im, images);
        if (labels && cap_labels >= static_cast<int64_t>(lb.numel())) copy_out(lb, labels);
    });
}

// The comparison operators of the reference (src/Tensor.cpp:985-1309 members, 1462-1591 free
// functions): cmp 0 >, 1 <, 2 ==, 3 >=, 4 <=, 5 !=; form 0 tensor ? tensor, 1 tensor ? scalar,
// 2 scalar ? tensor.  out: numel bytes of the kBool result.
int ref_compare(int cmp, int form, const float* a, const float* b, float s, const int64_t* shape, int rank, unsigned char* out) {
    return guarded([&] {
        Tensor A = make(a, shape, rank);
        Tensor R;
        if (form == 0) {
            Tensor B = make(b, shape, rank);
            switch (cmp) {
                case 0: R = A > B; break;
                case 1: R = A < B; break;
                case 2: R = A == B; break;
                case 3: R = A >= B; break;
                case 4: R = A <= B; break;
                default: R = A != B; break;
            }
        } else if (form == 1) {
            switch (cmp) {
                case 0: R = A > s; break;
                case 1: R = A < s; break;
                case 2: R = A == s; break;
                case 3: R = A >= s; break;
                case 4: R = A <= s; break;
                default: R = A != s; break;
            }
        } else {
            switch (cmp) {
                case 0: R = s > A; break;
                case 1: R = s < A; break;
                case 2: R = s == A; break;
                case 3: R = s >= A; break;
                case 4: R = s <= A; break;
                default: R = s != A; break;
            }
        }
        // (Tensor::data<bool>() does not link: the library instantiates checkDType for the four numeric
        // types only, src/Tensor.cpp:1605-1608.  Storage::data is a header template.)
        const bool* r = R.storage().data<bool>();
        for (size_t i = 0; i < R.numel(); ++i) out[i] = r[i] ? 1 : 0;
    });
}

// Tensor::to(DType) of the reference (src/Tensor.cpp:199-243) out of a float tensor; dtype 1 double,
// 2 int32, 3 int64, 4 bool.  out: numel elements of the target type.
int ref_cast(int dtype, const float* a, int64_t n, void* out) {
    return guarded([&] {
        int64_t shape[1] = {n};
        Tensor A = make(a, shape, 1);
        Tensor R = A.to(static_cast<DType>(dtype));
        switch (dtype) {
            case 1: std::memcpy(out, R.data<double>(), n * sizeof(double)); break;
            case 2: std::memcpy(out, R.data<int32_t>(), n * sizeof(int32_t)); break;
            case 3: std::memcpy(out, R.data<int64_t>(), n * sizeof(int64_t)); break;
            default: {
                const bool* r = R.storage().data<bool>();
                for (int64_t i = 0; i < n; ++i) static_cast<unsigned char*>(out)[i] = r[i] ? 1 : 0;
            }
        }
    });
}

// Tensor::operator[] (src/Tensor.cpp:175-189) on a 1-D tensor, read back through item().
int ref_index(const float* a, int64_t n, int64_t index, float* out) {
    return guarded([&] {
        int64_t shape[1] = {n};
        Tensor A = make(a, shape, 1);
        *out = A[static_cast<size_t>(index)].item<float>();
    });
}

// Tensor::ones (src/Tensor.cpp:422-450) on a tensor of the given dtype, returned as doubles.
int ref_ones(int dtype, int64_t n, double* out) {
    return guarded([&] {
        Tensor A(ShapeTag{}, std::vector<size_t>{static_cast<size_t>(n)}, static_cast<DType>(dtype), DeviceType::kCPU);
        A.ones();
        for (int64_t i = 0; i < n; ++i) {
            switch (dtype) {
                case 0: out[i] = A.data<float>()[i]; break;
                case 1: out[i] = A.data<double>()[i]; break;
                case 2: out[i] = A.data<int32_t>()[i]; break;
                case 3: out[i] = static_cast<double>(A.data<int64_t>()[i]); break;
                default: out[i] = A.storage().data<bool>()[i] ? 1.0 : 0.0; break;
            }
        }
    });
}

}  // extern "C"
