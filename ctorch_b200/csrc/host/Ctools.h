// Enumerations shared by the front end.  Numeric values match the reference's include/Ctools.h
// (DeviceType :150-157, DType :163-169, op :175-209) so that codes can cross the C ABI unchanged.
#pragma once
#include <cstddef>
#include <cstdint>
#include <stdexcept>

namespace ctorch {

enum class DeviceType { kCPU = 0, kCUDA = 1, kMPS = 2, kAMX = 3, kUNKNOWN = 4, kGENERAL = 5 };

enum class DType { kFloat, kDouble, kInt, kLong, kBool };

enum class op {
    Add, Sub, Neg, Mul, Div, MatMul, Dot, Cos, Sin,
    Conv, Pool,
    ReLU, Tanh, Sigmoid, Softmax,
    LReLU, PReLU,
    MSE, MAE, CE, BCE,
    Sum,
};

enum class ErrorLevel { TRACE = 0, INFO = 1, DEBUG = 2, WARN = 3, ERROR = 4, FATAL = 5 };
enum class ErrorPlatform { kCPU = 0, kCUDA = 1, kMPS = 2, kAMX = 3, kUNKNOWN = 4, kGENERAL = 5, kAutoDiff = 6 };
enum class ErrorType { UNKNOWN = 0, MEMORY = 1, DIMENSION = 2, DEVICE_COMPAT = 3, DATATYPE = 4, KERNEL_LAUNCH = 5, TENSOR_STATE = 6, PLATFORM_API = 7 };
enum class PrintLevel { MINIUM = 0, MEDIUM = 1, FULL = 2 };

struct ShapeTag {};

constexpr size_t dtypeSize(DType d) {
    switch (d) {
        case DType::kFloat: return 4;
        case DType::kDouble: return 8;
        case DType::kInt: return 4;
        case DType::kLong: return 8;
        case DType::kBool: return 1;
    }
    return 0;
}

constexpr const char* dtypeToString(DType d) {
    switch (d) {
        case DType::kFloat: return "float32";
        case DType::kDouble: return "float64";
        case DType::kInt: return "int32";
        case DType::kLong: return "int64";
        case DType::kBool: return "bool";
    }
    return "unknown";
}

inline ErrorPlatform DeviceTypeToErrorPlatform(DeviceType d) { return static_cast<ErrorPlatform>(static_cast<int>(d)); }

}  // namespace ctorch
