// Storage: the typed byte buffer under a Tensor, now device-aware.
//
// Same public surface as the reference's include/Storage.h (ctor :77, copy-in ctor :88-93,
// data<T>() :131-151, clone :175-181, clear/empty), with the DeviceType tag acted on:
//   kCUDA -> memory from the library's stream-ordered device pool (ctk_malloc), host data enters
//            and leaves through page-locked staging buffers;
//   kCPU  -> plain host memory (holds scalars, labels and staging data; no compute runs on it).
// Copies of a Storage share one buffer.  Tensor gives that value semantics by detaching
// (make_unique) before any write, so the reference's deep copies (copy ctor, make_leaf,
// commit_record, t(), get_grad) cost nothing until someone writes.
#pragma once
#include <cstring>
#include <memory>

#include "Ctools.h"
#include "Ctorch_Error.h"
#include "ctorch_b200.h"

namespace ctorch {

void cuda_check(int status, const char* what);  // throws on a non-zero ctk_status

class Storage {
    struct Block {
        void* ptr = nullptr;
        size_t bytes = 0;
        DeviceType device = DeviceType::kCPU;
        Block(size_t b, DeviceType d) : bytes(b), device(d) {
            if (b == 0) return;
            if (d == DeviceType::kCUDA) cuda_check(ctk_malloc(&ptr, b), "Storage: device allocation");
            else ptr = ::operator new(b);
        }
        ~Block() {
            if (!ptr) return;
            if (device == DeviceType::kCUDA) ctk_free(ptr);
            else ::operator delete(ptr);
        }
        Block(const Block&) = delete;
        Block& operator=(const Block&) = delete;
    };

    size_t _size = 0;
    DType _dtype = DType::kFloat;
    DeviceType _device = DeviceType::kCPU;
    std::shared_ptr<Block> _data;

    template <typename T>
    void checkDType() const {
        bool bad = (std::is_same<T, float>::value && _dtype != DType::kFloat) ||
                   (std::is_same<T, double>::value && _dtype != DType::kDouble) ||
                   (std::is_same<T, int32_t>::value && _dtype != DType::kInt) ||
                   (std::is_same<T, int64_t>::value && _dtype != DType::kLong) ||
                   (std::is_same<T, bool>::value && _dtype != DType::kBool);
        if (bad) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DATATYPE, "Storage data type mismatch");
    }

public:
    Storage() = default;
    Storage(size_t size, DType dtype, DeviceType device = DeviceType::kCPU)
        : _size(size), _dtype(dtype), _device(device),
          _data(size > 0 ? std::make_shared<Block>(size * dtypeSize(dtype), device) : nullptr) {}

    // Copy-in from HOST memory (for kCUDA: host -> device).
    template <typename T>
    Storage(const T* host_data, size_t size, DType dtype, DeviceType device = DeviceType::kCPU) : Storage(size, dtype, device) {
        if (size > 0 && _data) copy_from_host(host_data, size * dtypeSize(dtype));
    }

    // Raw typed pointer: a HOST pointer for kCPU, a DEVICE pointer for kCUDA.
    template <typename T>
    T* data() {
        if (_size == 0 || !_data) return nullptr;
        checkDType<T>();
        return static_cast<T*>(_data->ptr);
    }
    template <typename T>
    const T* data() const {
        if (_size == 0 || !_data) return nullptr;
        checkDType<T>();
        return static_cast<const T*>(_data->ptr);
    }
    void* raw() const { return _data ? _data->ptr : nullptr; }

    size_t size() const { return _size; }
    size_t nbytes() const { return _size * dtypeSize(_dtype); }
    DType dtype() const { return _dtype; }
    DeviceType device() const { return _device; }
    bool empty() const { return _size == 0 || !_data; }
    void clear() { _data.reset(); _size = 0; }
    bool unique() const { return !_data || _data.use_count() == 1; }

    // Deep copy on the same device (device-to-device for kCUDA).
    Storage clone() const {
        Storage s(_size, _dtype, _device);
        if (_size > 0 && _data) {
            if (_device == DeviceType::kCUDA) cuda_check(ctk_memcpy_d2d(s._data->ptr, _data->ptr, nbytes(), nullptr), "Storage::clone");
            else std::memcpy(s._data->ptr, _data->ptr, nbytes());
        }
        return s;
    }
    // Detach from other holders of the same buffer before a write.
    void make_unique() {
        if (_data && _data.use_count() > 1) *this = clone();
    }
    // Same contents on another device.
    Storage to(DeviceType device) const {
        if (device == _device) return *this;
        Storage s(_size, _dtype, device);
        if (_size == 0) return s;
        if (device == DeviceType::kCUDA) s.copy_from_host(_data->ptr, nbytes());
        else copy_to_host(s._data->ptr, nbytes());
        return s;
    }
    void copy_from_host(const void* src, size_t bytes);
    void copy_to_host(void* dst, size_t bytes) const;
};

}  // namespace ctorch
