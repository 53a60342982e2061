// Operator ABI of the scheduler: the two function-pointer types and the CUDA kernels registered on
// DeviceType::kCUDA.  Names and signatures are the ones the reference reserves in
// src/kernels/kernels.h:23,31 (typedefs) and :42-242 (`*_CUDA_kernel` prototypes).
#pragma once
#include "Tensor.h"

namespace ctorch {

typedef Tensor (*BinaryKernelFunc)(const Tensor& a, const Tensor& b);
typedef Tensor (*UnaryKernelFunc)(const Tensor& a);

Tensor Add_CUDA_kernel(const Tensor& a, const Tensor& b);
Tensor Sub_CUDA_kernel(const Tensor& a, const Tensor& b);
Tensor Mul_CUDA_kernel(const Tensor& a, const Tensor& b);
Tensor Div_CUDA_kernel(const Tensor& a, const Tensor& b);
Tensor MatMul_CUDA_kernel(const Tensor& a, const Tensor& b);
Tensor Dot_CUDA_kernel(const Tensor& a, const Tensor& b);
Tensor MSE_CUDA_kernel(const Tensor& a, const Tensor& b);
Tensor CrossEntropy_CUDA_kernel(const Tensor& a, const Tensor& b);
Tensor MAE_CUDA_kernel(const Tensor& a, const Tensor& b);
Tensor Neg_CUDA_kernel(const Tensor& a);
Tensor ReLU_CUDA_kernel(const Tensor& a);
Tensor Cos_CUDA_kernel(const Tensor& a);
Tensor Sin_CUDA_kernel(const Tensor& a);
Tensor Tanh_CUDA_kernel(const Tensor& a);
Tensor Sigmoid_CUDA_kernel(const Tensor& a);
Tensor Softmax_CUDA_kernel(const Tensor& a);

}  // namespace ctorch
