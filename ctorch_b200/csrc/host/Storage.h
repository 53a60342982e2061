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
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <unordered_set>
#include <utility>
#include <vector>

#include "Ctools.h"
#include "Ctorch_Error.h"
#include "ctorch_b200.h"

namespace ctorch {

void cuda_check(int status, const char* what);  // throws on a non-zero ctk_status
void* current_stream();                          // the calling thread's compute stream (Tensor.cpp)

// The hi/lo split of a buffer's contents that the 3xTF32 MatMul made on first use, kept with the
// buffer so that later products of the same values (the same view, or its transpose) reuse it.
// `view` identifies the 2-D view it was made for; `valid` is the flag the kernel library fills in.
// Size-keyed cache of device buffers, the common part of the two caches below.  Freed buffers are
// parked by (rounded) size and handed out again without a call into the CUDA runtime.  Reuse is
// ordered by the compute stream: a parked buffer may still be read by queued kernels, and its next
// owner only touches it with kernels queued after them.
//
// While a training step is being captured into a CUDA graph, every buffer that is handed out or
// given back becomes "pinned" to the graph: the graph's kernels have its address baked in, so until
// the graph is released such a buffer is only ever reused inside the captured sequence (through a
// private free list), never by anyone else.  A miss during capture is remembered -- the capture is
// then abandoned by its owner -- because allocating in the middle of a capture is not allowed.
class SizeKeyedCache {
    // Buffers are parked per (device ordinal, size): a pointer handed out on one GPU is never handed
    // to a tensor on another, however the calling thread switches devices in between.
    using Key = std::pair<int, size_t>;
    std::mutex mu_;
    std::map<Key, std::vector<void*>> free_;         // anyone's
    std::map<Key, std::vector<void*>> pinned_free_;  // the graph's
    std::unordered_set<void*> pinned_;
    size_t parked_bytes_ = 0;
    bool capturing_ = false, missed_ = false;

protected:
    virtual ~SizeKeyedCache() = default;
    virtual size_t rounded(size_t bytes) const = 0;
    virtual size_t max_parked() const = 0;
    virtual void* fresh(size_t bytes) = 0;            // on the current device
    virtual void release(void* p, int device) = 0;
    virtual bool enabled() const { return true; }

public:
    // Ordinal of the calling thread's current device (a subclass used in host-only tests overrides it).
    virtual int current_device() const {
        int dev = 0;
        cuda_check(ctk_get_device(&dev), "current device");
        return dev;
    }
    // A buffer of at least `bytes` on the current device; *device_out receives that device's ordinal,
    // which put() wants back.
    void* get(size_t bytes, int* device_out) {
        bytes = rounded(bytes);
        const int dev = current_device();
        if (device_out) *device_out = dev;
        if (enabled()) {
            std::lock_guard<std::mutex> lock(mu_);
            const Key key(dev, bytes);
            if (capturing_) {
                auto it = pinned_free_.find(key);
                if (it != pinned_free_.end() && !it->second.empty()) {
                    void* p = it->second.back();
                    it->second.pop_back();
                    return p;
                }
            }
            auto it = free_.find(key);
            if (it != free_.end() && !it->second.empty()) {
                void* p = it->second.back();
                it->second.pop_back();
                parked_bytes_ -= bytes;
                if (capturing_) pinned_.insert(p);
                return p;
            }
            if (capturing_) missed_ = true;
        }
        return fresh(bytes);
    }
    void put(void* p, size_t bytes, int device) {
        bytes = rounded(bytes);
        if (enabled()) {
            std::lock_guard<std::mutex> lock(mu_);
            const Key key(device, bytes);
            if (capturing_) pinned_.insert(p);
            if (pinned_.count(p)) {
                pinned_free_[key].push_back(p);
                return;
            }
            if (parked_bytes_ + bytes <= max_parked()) {
                free_[key].push_back(p);
                parked_bytes_ += bytes;
                return;
            }
        }
        release(p, device);
    }
    void begin_capture() {
        std::lock_guard<std::mutex> lock(mu_);
        capturing_ = true;
        missed_ = false;
    }
    // Returns false if a buffer had to be allocated during the capture.
    bool end_capture() {
        std::lock_guard<std::mutex> lock(mu_);
        capturing_ = false;
        return !missed_;
    }
    // The graph is gone: its buffers are anyone's again.
    void release_graph() {
        std::lock_guard<std::mutex> lock(mu_);
        for (auto& kv : pinned_free_)
            for (void* p : kv.second) {
                free_[kv.first].push_back(p);
                parked_bytes_ += kv.first.second;
            }
        pinned_free_.clear();
        pinned_.clear();
    }
};

// Frees on the device a buffer came from, whatever device the calling thread has current.
inline void free_on_device(void* p, int device, bool longlived) {
    int cur = -1;
    const bool switched = ctk_get_device(&cur) == 0 && cur != device && ctk_set_device(device) == 0;
    if (longlived) ctk_free_longlived(p);
    else ctk_free(p);
    if (switched) ctk_set_device(cur);
}

// Split buffers (hi/lo copies of MatMul operands) are large -- twice the operand -- and come and go
// with every activation of every step.  They are plain device allocations, outside the
// stream-ordered pool the tensors live in: mixed in there, their different sizes and lifetimes
// fragment it until it has to map new memory in the middle of a step.
class SplitBufferCache : public SizeKeyedCache {
    size_t rounded(size_t bytes) const override { return (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1); }
    size_t max_parked() const override { return size_t(16) << 30; }
    void* fresh(size_t bytes) override {
        void* p = nullptr;
        cuda_check(ctk_malloc_longlived(&p, bytes), "Storage: split buffer");  // a miss: warm-up only
        return p;
    }
    void release(void* p, int device) override { free_on_device(p, device, true); }

public:
    static SplitBufferCache& instance() {
        static SplitBufferCache* c = new SplitBufferCache();  // never destroyed: outlives every tensor
        return *c;
    }
};

// Device buffers of tensors: every op allocates its result and frees its temporaries, the same sizes
// step after step; a stream-ordered allocate / free pair costs 2-3 us of host time, which is most
// of a small training step.  Misses and overflow go to the device pool.
// CTORCH_BLOCK_CACHE=0 in the environment sends every allocation straight to the pool.
class DeviceBlockCache : public SizeKeyedCache {
    size_t rounded(size_t bytes) const override { return (bytes + 511) & ~size_t(511); }
    size_t max_parked() const override { return size_t(32) << 30; }
    void* fresh(size_t bytes) override {
        void* p = nullptr;
        cuda_check(ctk_malloc(&p, bytes), "Storage: device allocation");
        return p;
    }
    void release(void* p, int device) override { free_on_device(p, device, false); }
    bool enabled() const override {
        static const bool on = [] {
            const char* e = std::getenv("CTORCH_BLOCK_CACHE");
            return !(e && e[0] == '0');
        }();
        return on;
    }

public:
    static DeviceBlockCache& instance() {
        static DeviceBlockCache* c = new DeviceBlockCache();  // never destroyed: outlives every tensor
        return *c;
    }
};

struct KeptSplit {
    void* buf = nullptr;
    size_t bytes = 0;
    int device = 0;  // ordinal of the GPU the buffer lives on
    int valid = 0;
    int64_t view[4] = {0, 0, 0, 0};  // element offset, outer extent, inner (contiguous) extent, outer pitch
    ~KeptSplit() {
        if (buf) SplitBufferCache::instance().put(buf, bytes, device);
    }
};

class Storage {
    struct Block {
        void* ptr = nullptr;
        size_t bytes = 0;
        DeviceType device = DeviceType::kCPU;
        int ordinal = 0;                   // kCUDA: which GPU (the one current when the block was made)
        std::unique_ptr<KeptSplit> split;  // dropped whenever the buffer is about to be written
        Block(size_t b, DeviceType d) : bytes(b), device(d) {
            if (b == 0) return;
            if (d == DeviceType::kCUDA) ptr = DeviceBlockCache::instance().get(b, &ordinal);
            else ptr = ::operator new(b);
        }
        ~Block() {
            if (!ptr) return;
            if (device == DeviceType::kCUDA) DeviceBlockCache::instance().put(ptr, bytes, ordinal);
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
    bool has_split() const { return _data && _data->split; }
    void drop_split() const { if (_data) _data->split.reset(); }
    void clear() { _data.reset(); _size = 0; }
    bool unique() const { return !_data || _data.use_count() == 1; }

    // Deep copy on the same device (device-to-device for kCUDA).
    Storage clone() const {
        Storage s(_size, _dtype, _device);
        if (_size > 0 && _data) {
            if (_device == DeviceType::kCUDA) cuda_check(ctk_memcpy_d2d(s._data->ptr, _data->ptr, nbytes(), current_stream()), "Storage::clone");
            else std::memcpy(s._data->ptr, _data->ptr, nbytes());
        }
        return s;
    }
    // Detach from other holders of the same buffer before a write (every write path of Tensor goes
    // through here, so this is also where a kept split of the old contents is dropped).
    void make_unique() {
        if (!_data) return;
        if (_data.use_count() > 1) *this = clone();
        else _data->split.reset();
    }
    // The kept split of this buffer for the given 2-D view, created (invalid) if there is none or it
    // was made for another view.  Device buffers only.
    KeptSplit* kept_split(int64_t offset, int64_t outer, int64_t inner, int64_t pitch, size_t bytes) const {
        if (!_data || _device != DeviceType::kCUDA) return nullptr;
        KeptSplit* k = _data->split.get();
        if (k && k->view[0] == offset && k->view[1] == outer && k->view[2] == inner && k->view[3] == pitch) return k;
        auto fresh = std::make_unique<KeptSplit>();
        fresh->buf = SplitBufferCache::instance().get(bytes, &fresh->device);
        fresh->bytes = bytes;
        fresh->view[0] = offset; fresh->view[1] = outer; fresh->view[2] = inner; fresh->view[3] = pitch;
        _data->split = std::move(fresh);
        return _data->split.get();
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
