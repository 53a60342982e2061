// Ctorch_Scheduler: singleton op -> device -> kernel table, as the reference's
// include/Ctorch_Scheduler.h (maps :25-27, initKernelMap :30-53, isDeviceAvailable :67-75,
// dispatch :86-166).  The reserved DeviceType::kCUDA slot is filled with the sm_100a kernels and
// reported available when a CUDA device is present.  One deliberate difference: a lookup that finds
// no kernel throws, where the reference logs an error and then calls a null pointer.
#pragma once
#include <mutex>
#include <unordered_map>

#include "Ctorch_Error.h"
#include "Tensor.h"
#include "kernels.h"

namespace ctorch {

class Ctorch_Scheduler {
    Ctorch_Scheduler() = default;
    Ctorch_Scheduler(const Ctorch_Scheduler&) = delete;
    Ctorch_Scheduler& operator=(const Ctorch_Scheduler&) = delete;
    std::mutex mutex_;
    bool inited_ = false;
    struct OpHash { size_t operator()(op o) const { return static_cast<size_t>(o); } };
    struct DevHash { size_t operator()(DeviceType d) const { return static_cast<size_t>(d); } };
    std::unordered_map<op, std::unordered_map<DeviceType, BinaryKernelFunc, DevHash>, OpHash> binary_kernel_map_;
    std::unordered_map<op, std::unordered_map<DeviceType, UnaryKernelFunc, DevHash>, OpHash> unary_kernel_map_;

    void initKernelMap() {
        binary_kernel_map_[op::Add][DeviceType::kCUDA] = Add_CUDA_kernel;
        binary_kernel_map_[op::Sub][DeviceType::kCUDA] = Sub_CUDA_kernel;
        binary_kernel_map_[op::Mul][DeviceType::kCUDA] = Mul_CUDA_kernel;
        binary_kernel_map_[op::Div][DeviceType::kCUDA] = Div_CUDA_kernel;
        binary_kernel_map_[op::MatMul][DeviceType::kCUDA] = MatMul_CUDA_kernel;
        binary_kernel_map_[op::Dot][DeviceType::kCUDA] = Dot_CUDA_kernel;
        binary_kernel_map_[op::MSE][DeviceType::kCUDA] = MSE_CUDA_kernel;
        binary_kernel_map_[op::CE][DeviceType::kCUDA] = CrossEntropy_CUDA_kernel;
        binary_kernel_map_[op::MAE][DeviceType::kCUDA] = MAE_CUDA_kernel;
        unary_kernel_map_[op::Neg][DeviceType::kCUDA] = Neg_CUDA_kernel;
        unary_kernel_map_[op::ReLU][DeviceType::kCUDA] = ReLU_CUDA_kernel;
        unary_kernel_map_[op::Cos][DeviceType::kCUDA] = Cos_CUDA_kernel;
        unary_kernel_map_[op::Sin][DeviceType::kCUDA] = Sin_CUDA_kernel;
        unary_kernel_map_[op::Tanh][DeviceType::kCUDA] = Tanh_CUDA_kernel;
        unary_kernel_map_[op::Sigmoid][DeviceType::kCUDA] = Sigmoid_CUDA_kernel;
        unary_kernel_map_[op::Softmax][DeviceType::kCUDA] = Softmax_CUDA_kernel;
        unary_kernel_map_[op::LReLU];  // key without a function, as in the reference (:52)
    }
    void ensureInit() {
        std::lock_guard<std::mutex> lock(mutex_);
        if (!inited_) {
            initKernelMap();
            inited_ = true;
        }
    }

public:
    static Ctorch_Scheduler& getInstance() {
        static Ctorch_Scheduler instance_;
        return instance_;
    }

    static bool isDeviceAvailable(DeviceType dev_type) {
        switch (dev_type) {
            case DeviceType::kCUDA: {
                int n = 0;
                return ctk_device_count(&n) == 0 && n > 0;
            }
            default: return false;  // this build carries no CPU/MPS/AMX kernels: no fallback
        }
    }

    static DeviceType getTargetDevice(const Tensor& a, const Tensor& b) {
        // A 0-D host tensor (what Tensor(float) makes) combines with a device tensor as an immediate.
        if (a.device() != b.device()) {
            if (a.dim() == 0 && a.device() == DeviceType::kCPU) return b.device();
            if (b.dim() == 0 && b.device() == DeviceType::kCPU) return a.device();
            Ctorch_Error::log(ErrorLevel::ERROR, ErrorPlatform::kGENERAL, ErrorType::DEVICE_COMPAT, "Ctorch_Scheduler: tensors are on different devices");
        }
        return a.device();
    }

    Tensor dispatch(const Tensor& a, const Tensor& b, op op_type) {
        if (a.dtype() != b.dtype())
            Ctorch_Error::log(ErrorLevel::ERROR, ErrorPlatform::kGENERAL, ErrorType::DATATYPE, "Ctorch_Scheduler: tensor dtypes differ");
        if (op_type != op::Add && op_type != op::Mul && op_type != op::Sub && op_type != op::Div && op_type != op::CE &&
            op_type != op::MatMul && a.sizes() != b.sizes())
            Ctorch_Error::log(ErrorLevel::ERROR, ErrorPlatform::kGENERAL, ErrorType::DIMENSION, "Ctorch_Scheduler: tensor shapes differ");
        ensureInit();
        const DeviceType dev = getTargetDevice(a, b);
        BinaryKernelFunc fn = nullptr;
        {
            std::lock_guard<std::mutex> lock(mutex_);
            auto it = binary_kernel_map_.find(op_type);
            if (it != binary_kernel_map_.end()) {
                auto d = it->second.find(dev);
                if (d != it->second.end() && isDeviceAvailable(dev)) fn = d->second;
            }
        }
        if (!fn) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::PLATFORM_API, "Ctorch_Scheduler: no kernel available for this op on this device");
        return fn(a, b);
    }

    Tensor dispatch(const Tensor& a, op op_type) {
        ensureInit();
        const DeviceType dev = a.device();
        UnaryKernelFunc fn = nullptr;
        {
            std::lock_guard<std::mutex> lock(mutex_);
            auto it = unary_kernel_map_.find(op_type);
            if (it != unary_kernel_map_.end()) {
                auto d = it->second.find(dev);
                if (d != it->second.end() && isDeviceAvailable(dev)) fn = d->second;
            }
        }
        if (!fn) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::PLATFORM_API, "Ctorch_Scheduler: no kernel available for this op on this device");
        return fn(a);
    }
};

}  // namespace ctorch
