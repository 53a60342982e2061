// The `*_CUDA_kernel` adapters registered on DeviceType::kCUDA: validate like the CPU-BASIC kernel
// of the same operator, allocate the result (never zero-filled: the kernel writes every element),
// call the C ABI, throw on any CUDA error.  Names and signatures are those the reference reserves in
// src/kernels/kernels.h:42-242; each function cites the CPU-BASIC kernel whose contract it keeps.
//
// Operand rules kept from the reference: the result has a's shape (b's when a is the 0-D operand),
// a fresh id and requires_grad == false; only MatMul accepts strided views.  Where the reference
// throws or reads out of bounds on a broadcast it does not support ([N,H] - [H], x / scalar), the
// device kernel evaluates the NumPy-style broadcast instead.
#include "Ctorch_Error.h"
#include "Tensor.h"
#include <cstdlib>

#include "ctorch_b200.h"
#include "kernels.h"

namespace ctorch {

namespace {

void require_device(const Tensor& t, const char* who) {
    if (t.device() != DeviceType::kCUDA)
        Ctorch_Error::throwException(ErrorPlatform::kCUDA, ErrorType::DEVICE_COMPAT, std::string(who) + ": operand is not on the CUDA device");
}
void require_float(const Tensor& t, const char* who) {
    if (t.dtype() != DType::kFloat) Ctorch_Error::throwException(ErrorPlatform::kCUDA, ErrorType::DATATYPE, std::string(who) + ": only float32 is supported");
}
void require_contiguous(const Tensor& t, const char* who) {
    if (!t.is_contiguous()) Ctorch_Error::throwException(ErrorPlatform::kCUDA, ErrorType::TENSOR_STATE, std::string(who) + ": contiguous operand expected");
}
bool host_scalar(const Tensor& t) { return t.device() == DeviceType::kCPU && t.numel() == 1; }

Tensor empty_like(const Tensor& t) { return Tensor(ShapeTag{}, t.sizes(), t.dtype(), DeviceType::kCUDA, false); }

// Add_BASIC_kernel.cpp:21-34 (same / b.numel()==1 / [N,H]+[H]); Sub/Mul_BASIC_kernel.cpp:23-46
// (0-D operand on either side).  `kind_*`: the ctk_scalar_f32 kinds for a host scalar on the right
// and on the left.
Tensor binary(const Tensor& a, const Tensor& b, int opc, const char* who, int kind_b_scalar, int kind_a_scalar) {
    if (a.dtype() != b.dtype()) Ctorch_Error::log(ErrorLevel::ERROR, ErrorPlatform::kCUDA, ErrorType::DATATYPE, std::string(who) + ": tensor dtypes differ");
    require_float(a, who);
    void* st = current_stream();
    // host 0-D operand (what Tensor(float) makes): an immediate
    if (host_scalar(b) && a.device() == DeviceType::kCUDA) {
        require_contiguous(a, who);
        Tensor r = empty_like(a);
        // a - s is evaluated as a + (-s): the same IEEE result
        const float s = kind_b_scalar < 0 ? -b.item<float>() : b.item<float>();
        cuda_check(ctk_scalar_f32(kind_b_scalar < 0 ? 1 : kind_b_scalar, a.data<float>(), s, r.data<float>(), static_cast<int64_t>(a.numel()), st), who);
        return r;
    }
    if (host_scalar(a) && b.device() == DeviceType::kCUDA) {
        require_contiguous(b, who);
        Tensor r = empty_like(b);
        cuda_check(ctk_scalar_f32(kind_a_scalar, b.data<float>(), a.item<float>(), r.data<float>(), static_cast<int64_t>(b.numel()), st), who);
        return r;
    }
    require_device(a, who);
    require_device(b, who);
    require_contiguous(a, who);
    require_contiguous(b, who);
    int layout;
    int64_t inner = 1;
    const Tensor* shape_of = &a;
    if (a.sizes() == b.sizes()) layout = CTK_B_SAME;
    else if (b.numel() == 1) layout = CTK_B_SCALAR;
    else if (a.dim() == 0) { layout = CTK_A_SCALAR; shape_of = &b; }
    else if (b.dim() == 1 && a.dim() == 2 && b.sizes()[0] == a.sizes()[1]) { layout = CTK_B_ROW; inner = static_cast<int64_t>(b.numel()); }
    else Ctorch_Error::throwException(ErrorPlatform::kCUDA, ErrorType::DIMENSION, std::string(who) + ": tensor shapes do not match and cannot be broadcast");
    Tensor r = empty_like(*shape_of);
    cuda_check(ctk_binary_f32(opc, a.data<float>(), b.data<float>(), r.data<float>(), static_cast<int64_t>(r.numel()), layout, inner, st), who);
    return r;
}

Tensor unary(const Tensor& a, int opc, const char* who) {
    require_device(a, who);
    require_float(a, who);
    require_contiguous(a, who);
    Tensor r = empty_like(a);
    cuda_check(ctk_unary_f32(opc, a.data<float>(), r.data<float>(), static_cast<int64_t>(a.numel()), current_stream()), who);
    return r;
}

Tensor scalar_result() { return Tensor(ShapeTag{}, {}, DType::kFloat, DeviceType::kCUDA, false); }

}  // namespace

Tensor Add_CUDA_kernel(const Tensor& a, const Tensor& b) { return binary(a, b, CTK_OP_ADD, "CUDA Add_Kernel", 1, 1); }   // Add_BASIC_kernel.cpp:11-71
Tensor Sub_CUDA_kernel(const Tensor& a, const Tensor& b) { return binary(a, b, CTK_OP_SUB, "CUDA Sub_Kernel", -1, 3); }  // Sub_BASIC_kernel.cpp:12-62
Tensor Mul_CUDA_kernel(const Tensor& a, const Tensor& b) { return binary(a, b, CTK_OP_MUL, "CUDA Mul_Kernel", 0, 0); }   // Mul_BASIC_kernel.cpp:13-63
Tensor Div_CUDA_kernel(const Tensor& a, const Tensor& b) { return binary(a, b, CTK_OP_DIV, "CUDA Div_Kernel", 2, 4); }   // Div_BASIC_kernel.cpp:12-47

Tensor Neg_CUDA_kernel(const Tensor& a) { return unary(a, CTK_OP_NEG, "CUDA Neg_Kernel"); }              // Neg_BASIC_kernel.cpp:11-31
Tensor ReLU_CUDA_kernel(const Tensor& a) { return unary(a, CTK_OP_RELU, "CUDA ReLU_Kernel"); }           // ReLU_BASIC_kernel.cpp:12-28
Tensor Sigmoid_CUDA_kernel(const Tensor& a) { return unary(a, CTK_OP_SIGMOID, "CUDA Sigmoid_Kernel"); }  // Sigmoid_BASIC_kernel.cpp:13-29
Tensor Tanh_CUDA_kernel(const Tensor& a) { return unary(a, CTK_OP_TANH, "CUDA Tanh_Kernel"); }           // Tanh_BASIC_kernel.cpp:13-31
Tensor Sin_CUDA_kernel(const Tensor& a) { return unary(a, CTK_OP_SIN, "CUDA Sin_Kernel"); }              // Sin_BASIC_kernel.cpp:13-28
Tensor Cos_CUDA_kernel(const Tensor& a) { return unary(a, CTK_OP_COS, "CUDA Cos_Kernel"); }              // Cos_BASIC_kernel.cpp:13-27

// MatMul_BASIC_kernel.cpp:13-57: 2-D only, inner dims must agree, strides honoured.
Tensor MatMul_CUDA_kernel(const Tensor& a, const Tensor& b) {
    const char* who = "CUDA MatMul_Kernel";
    require_device(a, who);
    require_device(b, who);
    require_float(a, who);
    if (a.dtype() != b.dtype()) Ctorch_Error::log(ErrorLevel::ERROR, ErrorPlatform::kCUDA, ErrorType::DATATYPE, "CUDA MatMul_Kernel: tensor dtypes differ");
    if (a.shape().size() != 2 || b.shape().size() != 2) Ctorch_Error::throwException(ErrorPlatform::kCUDA, ErrorType::DIMENSION, "MatMul supports 2-D tensors only");
    if (a.shape()[1] != b.shape()[0]) Ctorch_Error::throwException(ErrorPlatform::kCUDA, ErrorType::DIMENSION, "MatMul: inner dimensions do not match");
    const int64_t m = static_cast<int64_t>(a.shape()[0]), k = static_cast<int64_t>(a.shape()[1]), n = static_cast<int64_t>(b.shape()[1]);
    Tensor r(ShapeTag{}, {static_cast<size_t>(m), static_cast<size_t>(n)}, a.dtype(), DeviceType::kCUDA, false);
    const int64_t sa0 = static_cast<int64_t>(a.strides()[0]), sa1 = static_cast<int64_t>(a.strides()[1]);
    const int64_t sb0 = static_cast<int64_t>(b.strides()[0]), sb1 = static_cast<int64_t>(b.strides()[1]);
    // CTORCH_KEEP_SPLITS=0 in the environment switches the kept splits off (they cost up to twice the
    // operand's size in device memory for as long as the operand lives).
    static const bool keep_splits = [] {
        const char* e = std::getenv("CTORCH_KEEP_SPLITS");
        return !(e && e[0] == '0');
    }();
    // (path 3, a narrow output on the CUDA cores, reads the operands as they are: nothing to keep)
    if (!keep_splits || ctk_get_matmul_mode() != CTK_MATMUL_3XTF32 || m < 2 || n < 2 || k < 2 ||
        ctk_matmul_path(a.data<float>(), b.data<float>(), m, n, k, sa0, sa1, sb0, sb1, CTK_MATMUL_3XTF32) == 3) {
        cuda_check(ctk_matmul_f32(a.data<float>(), b.data<float>(), r.data<float>(), m, n, k, sa0, sa1, sb0, sb1, -1, nullptr, current_stream()), who);
        return r;
    }
    // 3xTF32: the hi/lo split of each operand stays with the operand's buffer (Storage drops it when
    // the buffer is written), so X in X.W and X^T.dY, dY in dY.W^T and X^T.dY, and the weights the
    // tape holds are each split once.  The view is named by its contiguous ("inner") extent, the
    // other extent and its pitch, so a t() view of the same memory finds the same split.
    KeptSplit* ka = operand_split(a, m, k, sa0, sa1);
    // one split per buffer: when both operands are views of the same buffer only A's is kept
    KeptSplit* kb = (b.storage().raw() == a.storage().raw()) ? nullptr : operand_split(b, n, k, sb1, sb0);
    cuda_check(ctk_matmul_3xtf32_kept_f32(a.data<float>(), b.data<float>(), r.data<float>(), m, n, k, sa0, sa1, sb0, sb1, ka ? ka->buf : nullptr,
                                          ka ? &ka->valid : nullptr, kb ? kb->buf : nullptr, kb ? &kb->valid : nullptr, nullptr, current_stream()),
               who);
    return r;
}

// Dot_BASIC_kernel.cpp:12-46
Tensor Dot_CUDA_kernel(const Tensor& a, const Tensor& b) {
    const char* who = "CUDA Dot_Kernel";
    require_device(a, who);
    require_device(b, who);
    require_contiguous(a, who);
    require_contiguous(b, who);
    if (a.numel() != b.numel()) Ctorch_Error::throwException(ErrorPlatform::kCUDA, ErrorType::DIMENSION, "CUDA Dot_Kernel: element counts differ");
    Tensor r = scalar_result();
    cuda_check(ctk_dot_f32(a.data<float>(), b.data<float>(), static_cast<int64_t>(a.numel()), r.data<float>(), nullptr, current_stream()), who);
    return r;
}

// MSE_BASIC_kernel.cpp:12-46 / MAE_BASIC_kernel.cpp:12-46: mean over all elements -> 0-D.
static Tensor mean_loss(const Tensor& a, const Tensor& b, bool mse, const char* who) {
    require_device(a, who);
    require_device(b, who);
    require_contiguous(a, who);
    require_contiguous(b, who);
    if (a.sizes() != b.sizes()) Ctorch_Error::throwException(ErrorPlatform::kCUDA, ErrorType::DIMENSION, std::string(who) + ": tensor shapes differ");
    if (a.numel() == 0) Ctorch_Error::throwException(ErrorPlatform::kCUDA, ErrorType::DIMENSION, std::string(who) + ": empty input");
    Tensor r = scalar_result();
    const int64_t n = static_cast<int64_t>(a.numel());
    cuda_check(mse ? ctk_mse_f32(a.data<float>(), b.data<float>(), n, r.data<float>(), nullptr, current_stream())
                   : ctk_mae_f32(a.data<float>(), b.data<float>(), n, r.data<float>(), nullptr, current_stream()),
               who);
    return r;
}
Tensor MSE_CUDA_kernel(const Tensor& a, const Tensor& b) { return mean_loss(a, b, true, "CUDA MSE_Kernel"); }
Tensor MAE_CUDA_kernel(const Tensor& a, const Tensor& b) { return mean_loss(a, b, false, "CUDA MAE_Kernel"); }

// Softmax_BASIC_kernel.cpp:16-101: 1-D or 2-D (rows), float only.
Tensor Softmax_CUDA_kernel(const Tensor& a) {
    const char* who = "CUDA Softmax_Kernel";
    require_device(a, who);
    require_float(a, who);
    require_contiguous(a, who);
    const size_t dim = a.sizes().size();
    if (dim == 0) Ctorch_Error::throwException(ErrorPlatform::kCUDA, ErrorType::DIMENSION, "CUDA Softmax_Kernel: scalars are not supported");
    if (dim > 2) Ctorch_Error::throwException(ErrorPlatform::kCUDA, ErrorType::DIMENSION, "CUDA Softmax_Kernel: only 1-D / 2-D tensors");
    const int64_t rows = dim == 1 ? 1 : static_cast<int64_t>(a.sizes()[0]);
    const int64_t cols = static_cast<int64_t>(a.sizes()[dim - 1]);
    Tensor r = empty_like(a);
    cuda_check(ctk_softmax_rows_f32(a.data<float>(), r.data<float>(), rows, cols, current_stream()), who);
    return r;
}

// CrossEntropy_BASIC_kernel.cpp:14-130: one-hot targets of the logits' shape (1-D/2-D) or index
// labels [B] for logits [B,C]; anything else logs an error and returns an empty tensor.  An index
// out of range makes the loss NaN here (the reference returns an empty tensor; checking on the host
// would cost a device synchronisation per call).
Tensor CrossEntropy_CUDA_kernel(const Tensor& a, const Tensor& b) {
    const char* who = "CUDA CrossEntropy_Kernel";
    require_device(a, who);
    require_device(b, who);
    require_contiguous(a, who);
    require_contiguous(b, who);
    void* st = current_stream();
    if (a.sizes() == b.sizes() && (a.dim() == 1 || a.dim() == 2)) {
        const int64_t rows = a.dim() == 1 ? 1 : static_cast<int64_t>(a.sizes()[0]);
        const int64_t cols = static_cast<int64_t>(a.sizes()[a.dim() - 1]);
        Tensor r = scalar_result();
        cuda_check(ctk_ce_onehot_f32(a.data<float>(), b.data<float>(), rows, cols, r.data<float>(), nullptr, st), who);
        return r;
    }
    if (b.dim() == 1 && a.dim() == 2 && b.sizes()[0] == a.sizes()[0]) {
        Tensor r = scalar_result();
        cuda_check(ctk_ce_index_f32(a.data<float>(), b.data<float>(), static_cast<int64_t>(a.sizes()[0]), static_cast<int64_t>(a.sizes()[1]),
                                    r.data<float>(), nullptr, nullptr, st),
                   who);
        return r;
    }
    Ctorch_Error::log(ErrorLevel::ERROR, ErrorPlatform::kCUDA, ErrorType::DIMENSION, "CUDA CrossEntropy_Kernel: incompatible tensor shapes");
    return Tensor();
}

}  // namespace ctorch
