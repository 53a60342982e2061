// Tensor implementation: the op wrappers have the reference's shape (src/Tensor.cpp:482-497 and the
// 15 sibling call sites): check dtype/device, dispatch through Ctorch_Scheduler, defer_record on
// the tape, commit when the result requires grad.  The operations the reference computes with
// host loops outside the scheduler (scalar forms :751-973, sum :638-666, softmax :1645-1803,
// zero/ones :390-455, broadcast_to :289-387, item :154-165) launch device kernels here.
#include <cstdlib>

#include "Tensor.h"

#include <random>

#include <algorithm>
#include <cmath>
#include <limits>
#include <mutex>

#include "Ctorch_Scheduler.h"
#include "ctorch_b200.h"

namespace ctorch {

std::atomic<size_t> Tensor::global_tensor_id(1);

void cuda_check(int status, const char* what) {
    if (status != 0) {
        Ctorch_Error::throwException(ErrorPlatform::kCUDA, status == CTK_ERR_INVALID ? ErrorType::DIMENSION : ErrorType::KERNEL_LAUNCH,
                                     std::string(what) + ": " + ctk_last_error());
    }
}

static thread_local void* t_stream = nullptr;
void* current_stream() { return t_stream; }
void set_current_stream(void* s) { t_stream = s; }

// ---- pinned staging for host <-> device copies --------------------------------------------------
// Two page-locked buffers per thread: while one is in flight on the copy engine the host fills (or
// drains) the other.  The buffers serve every GPU; the events that guard them belong to a device, so
// there is a pair per device ordinal (`ev` points at the pair of the device current at ensure()).
namespace {
struct Staging {
    static constexpr size_t kChunk = 8u << 20;
    void* buf[2] = {nullptr, nullptr};
    void* ev_of[64][2] = {};
    void** ev = ev_of[0];
    void ensure() {
        int dev = 0;
        cuda_check(ctk_get_device(&dev), "current device");
        if (dev < 0 || dev >= 64) Ctorch_Error::throwException(ErrorPlatform::kCUDA, ErrorType::DEVICE_COMPAT, "device ordinal out of range");
        for (int i = 0; i < 2; ++i) {
            if (!buf[i]) cuda_check(ctk_malloc_host(&buf[i], kChunk), "pinned staging allocation");
            if (!ev_of[dev][i]) cuda_check(ctk_event_create(&ev_of[dev][i]), "staging event");
        }
        ev = ev_of[dev];
    }
    ~Staging() {
        for (int i = 0; i < 2; ++i)
            if (buf[i]) ctk_free_host(buf[i]);
        for (auto& pair : ev_of)
            for (void* e : pair)
                if (e) ctk_event_destroy(e);
    }
};
thread_local Staging t_staging;
}  // namespace

void Storage::copy_from_host(const void* src, size_t bytes) {
    if (bytes == 0) return;
    if (bytes > nbytes()) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::MEMORY, "Storage::copy_from_host: too many bytes");
    if (_device != DeviceType::kCUDA) {
        std::memcpy(_data->ptr, src, bytes);
        return;
    }
    Staging& S = t_staging;
    S.ensure();
    const char* s = static_cast<const char*>(src);
    char* d = static_cast<char*>(_data->ptr);
    bool used[2] = {false, false};
    int slot = 0;
    for (size_t off = 0; off < bytes; off += Staging::kChunk, slot ^= 1) {
        const size_t n = std::min(Staging::kChunk, bytes - off);
        if (used[slot]) cuda_check(ctk_event_sync(S.ev[slot]), "staging wait");
        std::memcpy(S.buf[slot], s + off, n);
        cuda_check(ctk_memcpy_h2d(d + off, S.buf[slot], n, t_stream), "host-to-device copy");
        cuda_check(ctk_event_record(S.ev[slot], t_stream), "staging record");
        used[slot] = true;
    }
    for (int i = 0; i < 2; ++i)
        if (used[i]) cuda_check(ctk_event_sync(S.ev[i]), "staging wait");  // the staging buffers are reused by the next call
}

void Storage::copy_to_host(void* dst, size_t bytes) const {
    if (bytes == 0) return;
    if (bytes > nbytes()) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::MEMORY, "Storage::copy_to_host: too many bytes");
    if (_device != DeviceType::kCUDA) {
        std::memcpy(dst, _data->ptr, bytes);
        return;
    }
    Staging& S = t_staging;
    S.ensure();
    char* out = static_cast<char*>(dst);
    const char* s = static_cast<const char*>(_data->ptr);
    size_t pending_off[2] = {0, 0}, pending_n[2] = {0, 0};
    int slot = 0;
    for (size_t off = 0; off < bytes; off += Staging::kChunk, slot ^= 1) {
        const size_t n = std::min(Staging::kChunk, bytes - off);
        if (pending_n[slot]) {
            cuda_check(ctk_event_sync(S.ev[slot]), "staging wait");
            std::memcpy(out + pending_off[slot], S.buf[slot], pending_n[slot]);
        }
        cuda_check(ctk_memcpy_d2h(S.buf[slot], s + off, n, t_stream), "device-to-host copy");
        cuda_check(ctk_event_record(S.ev[slot], t_stream), "staging record");
        pending_off[slot] = off;
        pending_n[slot] = n;
    }
    for (int i = 0; i < 2; ++i) {
        const int sl = slot ^ i;  // older one first
        if (pending_n[sl]) {
            cuda_check(ctk_event_sync(S.ev[sl]), "staging wait");
            std::memcpy(out + pending_off[sl], S.buf[sl], pending_n[sl]);
        }
    }
}

// ---- construction ---------------------------------------------------------------------------------
Tensor::Tensor() : tensor_id_(global_tensor_id++) { computeStrides(); }

Tensor::Tensor(float value) : tensor_id_(global_tensor_id++) {
    _shape = {};
    computeStrides();
    _storage = Storage(&value, 1, _dtype, _device);
}

Tensor::Tensor(std::initializer_list<float> values) : tensor_id_(global_tensor_id++) {
    _shape = {values.size()};
    computeStrides();
    _storage = Storage(values.begin(), values.size(), _dtype, _device);
}

Tensor::Tensor(ShapeTag, const std::vector<size_t>& shape, DType dtype, DeviceType device, bool zero_init)
    : tensor_id_(global_tensor_id++), _device(device), _dtype(dtype) {
    _shape = shape;
    computeStrides();
    _storage = Storage(numel(), _dtype, _device);
    if (zero_init) zero();
}

Tensor::Tensor(size_t size, DType dtype, DeviceType device, bool zero_init) : tensor_id_(global_tensor_id++), _device(device), _dtype(dtype) {
    _shape = {size};
    computeStrides();
    _storage = Storage(size, _dtype, _device);
    if (zero_init) zero();
}

// Copy: a new id and the same value (the reference clones the storage here, include/Tensor.h:320-338;
// sharing until the first write is indistinguishable).
Tensor::Tensor(const Tensor& o)
    : tensor_id_(global_tensor_id++), record_committed_(false), _requires_grad(o._requires_grad), _strides(o._strides),
      _storage_offset(o._storage_offset), _device(o._device), _dtype(o._dtype), _storage(o._storage), _shape(o._shape) {}

Tensor& Tensor::operator=(const Tensor& o) {
    if (this != &o) {
        commit_pending_record();
        tensor_id_ = global_tensor_id++;
        _shape = o._shape;
        _strides = o._strides;
        _storage_offset = o._storage_offset;
        _device = o._device;
        _dtype = o._dtype;
        _storage = o._storage;
        _requires_grad = o._requires_grad;
        record_committed_ = false;
    }
    return *this;
}

// Move keeps the id -- this is what lets `Tensor h = (x.matmul(W) + b).relu();` stay on the tape.
Tensor::Tensor(Tensor&& o) noexcept
    : tensor_id_(o.tensor_id_), record_committed_(o.record_committed_), _requires_grad(o._requires_grad), _strides(std::move(o._strides)),
      _storage_offset(o._storage_offset), _device(o._device), _dtype(o._dtype), _storage(std::move(o._storage)), _shape(std::move(o._shape)) {
    o.tensor_id_ = 0;
    o.record_committed_ = false;
}

Tensor& Tensor::operator=(Tensor&& o) noexcept {
    if (this != &o) {
        tensor_id_ = o.tensor_id_;
        _shape = std::move(o._shape);
        _strides = std::move(o._strides);
        _storage_offset = o._storage_offset;
        _device = o._device;
        _dtype = o._dtype;
        _storage = std::move(o._storage);
        _requires_grad = o._requires_grad;
        record_committed_ = o.record_committed_;
        o.tensor_id_ = 0;
        o.record_committed_ = false;
    }
    return *this;
}

// ---- accessors ------------------------------------------------------------------------------------
void Tensor::requires_grad(bool key) {
    _requires_grad = key;
    if (key && AutoDiffContext::current()) {
        AutoDiffContext::current()->make_leaf(*this, key);
        AutoDiffContext::current()->update_requires_grad(*this, key);
    }
}

size_t Tensor::numel() const {
    size_t n = 1;
    for (size_t s : _shape) n *= s;
    return n;
}

size_t Tensor::size(int d) const {
    if (d < 0) d += static_cast<int>(_shape.size());
    if (d < 0 || d >= static_cast<int>(_shape.size())) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DIMENSION, "invalid dimension");
    return _shape[d];
}

size_t Tensor::stride(int d) const {
    if (d < 0) d += static_cast<int>(_strides.size());
    if (d < 0 || d >= static_cast<int>(_strides.size())) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DIMENSION, "invalid dimension");
    return _strides[d];
}

void Tensor::computeStrides() {
    _strides.resize(_shape.size());
    if (_shape.empty()) return;
    _strides.back() = 1;
    for (int i = static_cast<int>(_shape.size()) - 2; i >= 0; --i) _strides[i] = _strides[i + 1] * _shape[i + 1];
}

bool Tensor::is_contiguous() const {
    size_t expect = 1;
    for (int i = static_cast<int>(_shape.size()) - 1; i >= 0; --i) {
        if (_shape[i] != 1 && _strides[i] != expect) return false;
        expect *= _shape[i];
    }
    return true;
}

template <typename T>
void Tensor::checkDType() const {
    bool ok = (std::is_same<T, float>::value && _dtype == DType::kFloat) || (std::is_same<T, double>::value && _dtype == DType::kDouble) ||
              (std::is_same<T, int32_t>::value && _dtype == DType::kInt) || (std::is_same<T, int64_t>::value && _dtype == DType::kLong) ||
              (std::is_same<T, bool>::value && _dtype == DType::kBool);
    if (!ok) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DATATYPE, std::string("dtype mismatch, tensor is ") + dtypeToString(_dtype));
}

template <typename T>
T* Tensor::data() {
    checkDType<T>();
    _storage.make_unique();
    T* p = _storage.data<T>();
    return p ? p + _storage_offset : nullptr;
}
template <typename T>
const T* Tensor::data() const {
    checkDType<T>();
    const T* p = _storage.data<T>();
    return p ? p + _storage_offset : nullptr;
}
template float* Tensor::data<float>();
template const float* Tensor::data<float>() const;
template int32_t* Tensor::data<int32_t>();
template const int32_t* Tensor::data<int32_t>() const;
template double* Tensor::data<double>();
template const double* Tensor::data<double>() const;
template int64_t* Tensor::data<int64_t>();
template const int64_t* Tensor::data<int64_t>() const;
template bool* Tensor::data<bool>();
template const bool* Tensor::data<bool>() const;

template <typename T>
T Tensor::item() const {
    if (numel() != 1) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::TENSOR_STATE, "item(): tensor is not a scalar");
    const T* p = data<T>();
    if (!p) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::TENSOR_STATE, "item(): tensor has no data");
    if (_device != DeviceType::kCUDA) return *p;
    T v;
    cuda_check(ctk_memcpy_d2h(&v, p, sizeof(T), t_stream), "item()");
    cuda_check(t_stream ? ctk_stream_sync(t_stream) : ctk_device_sync(), "item() sync");
    return v;
}
template float Tensor::item<float>() const;
template int32_t Tensor::item<int32_t>() const;

void Tensor::commit_pending_record() {
    if (AutoDiffContext::current() && has_pending_record()) AutoDiffContext::current()->commit_record(*this);
    record_committed_ = true;
}

// ---- host <-> device ----------------------------------------------------------------------------------
void Tensor::copy_from_host(const float* src, size_t count) {
    if (count != numel() || !is_contiguous()) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DIMENSION, "copy_from_host: size mismatch or non-contiguous tensor");
    if (count == 0) return;
    _storage.make_unique();
    if (_storage_offset == 0) {
        _storage.copy_from_host(src, count * sizeof(float));
    } else if (_device == DeviceType::kCUDA) {
        cuda_check(ctk_memcpy_h2d(data<float>(), src, count * sizeof(float), t_stream), "copy_from_host");
        cuda_check(t_stream ? ctk_stream_sync(t_stream) : ctk_device_sync(), "copy_from_host sync");
    } else {
        std::memcpy(data<float>(), src, count * sizeof(float));
    }
}

void Tensor::copy_to_host(float* dst, size_t count) const {
    if (count != numel()) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DIMENSION, "copy_to_host: size mismatch");
    if (count == 0) return;
    if (!is_contiguous()) {
        contiguous().copy_to_host(dst, count);
        return;
    }
    if (_storage_offset == 0) {
        _storage.copy_to_host(dst, count * sizeof(float));
    } else if (_device == DeviceType::kCUDA) {
        cuda_check(ctk_memcpy_d2h(dst, data<float>(), count * sizeof(float), t_stream), "copy_to_host");
        cuda_check(t_stream ? ctk_stream_sync(t_stream) : ctk_device_sync(), "copy_to_host sync");
    } else {
        std::memcpy(dst, data<float>(), count * sizeof(float));
    }
}

std::vector<float> Tensor::to_vector() const {
    std::vector<float> v(numel());
    copy_to_host(v.data(), v.size());
    return v;
}

Tensor Tensor::to(DeviceType device) const {
    Tensor r(*this);
    if (device == _device) return r;
    if (!is_contiguous() || _storage_offset != 0) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::TENSOR_STATE, "to(device): contiguous tensor expected");
    r._storage = _storage.to(device);
    r._device = device;
    return r;
}

// ---- shape ops --------------------------------------------------------------------------------------------
Tensor Tensor::clone() const {
    Tensor r(*this);
    r._storage = _storage.clone();
    return r;
}

// src/Tensor.cpp:246-261: a copy with two dims and two strides swapped (no data movement here).
Tensor Tensor::transpose(int d0, int d1) const {
    const int rank = static_cast<int>(_shape.size());
    if (d0 < 0 || d0 >= rank || d1 < 0 || d1 >= rank) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DIMENSION, "transpose: dimension out of range");
    Tensor r(*this);
    std::swap(r._shape[d0], r._shape[d1]);
    std::swap(r._strides[d0], r._strides[d1]);
    return r;
}
Tensor Tensor::t() const { return transpose(0, 1); }

Tensor Tensor::narrow_rows(size_t start, size_t count) const {
    if (_shape.empty() || _shape.size() > 2) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DIMENSION, "narrow_rows: 1-D or 2-D tensors only");
    if (start > _shape[0] || count > _shape[0] - start) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DIMENSION, "narrow_rows: range outside the tensor");
    Tensor r(*this);
    r._shape[0] = count;
    r._storage_offset = _storage_offset + start * _strides[0];
    return r;
}

Tensor Tensor::reshape(const std::vector<size_t>& new_shape) const {
    size_t n = 1;
    for (size_t s : new_shape) n *= s;
    if (n != numel()) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DIMENSION, "reshape: element count differs");
    Tensor r(*this);
    r._shape = new_shape;
    r.computeStrides();
    return r;
}

// Materialises a 2-D strided view (what t() makes) into row-major order with one GEMM-free pass:
// out = view * 1 is not needed -- a transposed copy is a MatMul-shaped read, done by the SIMT
// matmul against nothing; here it is only used for host read-back of small views.
Tensor Tensor::contiguous() const {
    if (is_contiguous()) return *this;
    if (_shape.size() != 2) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DIMENSION, "contiguous(): only 2-D views are supported");
    // Read back the underlying buffer and permute on the host (views are small: tests and debugging).
    Tensor base(*this);
    base._shape = {_storage.size()};
    base._strides = {1};
    base._storage_offset = 0;
    std::vector<float> raw = base.to_vector();
    std::vector<float> out(numel());
    for (size_t i = 0; i < _shape[0]; ++i)
        for (size_t j = 0; j < _shape[1]; ++j) out[i * _shape[1] + j] = raw[_storage_offset + i * _strides[0] + j * _strides[1]];
    Tensor r(ShapeTag{}, _shape, _dtype, _device, false);
    r.copy_from_host(out.data(), out.size());
    r._requires_grad = _requires_grad;
    return r;
}

// src/Tensor.cpp:289-387.  NumPy-style broadcast by materialising; on the device the cases the
// training path produces (one element -> any shape, trailing dims equal -> tiled rows) are one
// fill / tile launch.
Tensor Tensor::broadcast_to(const std::vector<size_t>& shape) const {
    if (shape.empty()) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DIMENSION, "broadcast_to: empty target shape");
    std::vector<size_t> cur = _shape, tgt = shape;
    while (cur.size() < tgt.size()) cur.insert(cur.begin(), 1);
    while (tgt.size() < cur.size()) tgt.insert(tgt.begin(), 1);
    for (size_t i = 0; i < cur.size(); ++i)
        if (cur[i] != tgt[i] && cur[i] != 1) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DIMENSION, "broadcast_to: incompatible shapes");
    Tensor result(ShapeTag{}, shape, _dtype, _device, false);
    const size_t n = result.numel(), src_n = numel();
    if (n == 0) return result;
    // trailing-dims broadcast: every broadcast dim is a leading one
    bool trailing = true;
    {
        bool seen_real = false;
        for (size_t i = 0; i < cur.size(); ++i) {
            if (cur[i] == tgt[i] && cur[i] != 1) seen_real = true;
            else if (cur[i] == 1 && tgt[i] != 1 && seen_real) trailing = false;
        }
    }
    if (_device == DeviceType::kCUDA) {
        if (src_n == 1) cuda_check(ctk_fill_f32(result.data<float>(), 0.0f, data<float>(), static_cast<int64_t>(n), t_stream), "broadcast_to");
        else if (trailing) cuda_check(ctk_tile_f32(data<float>(), static_cast<int64_t>(src_n), result.data<float>(), static_cast<int64_t>(n), t_stream), "broadcast_to");
        else Ctorch_Error::throwException(ErrorPlatform::kCUDA, ErrorType::DIMENSION, "broadcast_to: only scalar and trailing-dims broadcasts are implemented on the device");
    } else {
        const float* s = data<float>();
        float* d = result.data<float>();
        if (src_n == 1) std::fill(d, d + n, s[0]);
        else if (trailing) for (size_t i = 0; i < n; ++i) d[i] = s[i % src_n];
        else Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DIMENSION, "broadcast_to: only scalar and trailing-dims broadcasts are implemented");
    }
    return result;
}

void Tensor::fill(float v) {
    const size_t n = numel();
    if (n == 0) return;
    if (_dtype != DType::kFloat) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DATATYPE, "fill: float tensors only");
    if (_device == DeviceType::kCUDA) cuda_check(ctk_fill_f32(data<float>(), v, nullptr, static_cast<int64_t>(n), t_stream), "fill");
    else std::fill(data<float>(), data<float>() + n, v);
}
void Tensor::zero() {
    if (numel() == 0) return;
    if (_dtype == DType::kFloat) { fill(0.0f); return; }
    _storage.make_unique();
    if (_device == DeviceType::kCUDA) cuda_check(ctk_memset(_storage.raw(), 0, _storage.nbytes(), t_stream), "zero");
    else std::memset(_storage.raw(), 0, _storage.nbytes());
}
void Tensor::ones() {
    if (_dtype == DType::kFloat) { fill(1.0f); return; }
    const size_t n = numel();
    if (n == 0) return;
    _storage.make_unique();
    unsigned char* base = static_cast<unsigned char*>(_storage.raw()) + _storage_offset * dtypeSize(_dtype);
    if (_device == DeviceType::kCUDA) {
        cuda_check(ctk_fill_dtype(static_cast<int>(_dtype), base, 1.0, static_cast<int64_t>(n), t_stream), "ones");
        return;
    }
    switch (_dtype) {
        case DType::kDouble: std::fill_n(reinterpret_cast<double*>(base), n, 1.0); break;
        case DType::kInt: std::fill_n(reinterpret_cast<int32_t*>(base), n, 1); break;
        case DType::kLong: std::fill_n(reinterpret_cast<int64_t*>(base), n, int64_t(1)); break;
        default: std::fill_n(reinterpret_cast<bool*>(base), n, true); break;
    }
}

// ---- rand (src/Tensor.cpp:458-479) --------------------------------------------------------------------------
static std::atomic<uint64_t> g_rand_seed{0}, g_rand_offset{0};
static std::atomic<bool> g_rand_seeded{false};
void Tensor::manual_seed(uint64_t seed) {
    g_rand_seed.store(seed);
    g_rand_offset.store(0);
    g_rand_seeded.store(true);
}
void Tensor::rand() {
    const size_t n = numel();
    if (n == 0 || (_dtype != DType::kFloat && _dtype != DType::kDouble)) return;  // other dtypes: untouched, as in the reference
    if (!g_rand_seeded.exchange(true)) {
        std::random_device rd;
        g_rand_seed.store((static_cast<uint64_t>(rd()) << 32) | rd());
    }
    if (_device != DeviceType::kCUDA) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DEVICE_COMPAT, "rand: device tensors only");
    const uint64_t offset = g_rand_offset.fetch_add(n);
    if (_dtype == DType::kFloat) {
        cuda_check(ctk_rand_uniform_f32(data<float>(), static_cast<int64_t>(n), g_rand_seed.load(), offset, t_stream), "rand");
        return;
    }
    // double: the same 24-bit uniforms, widened
    Tensor f(ShapeTag{}, {n}, DType::kFloat, DeviceType::kCUDA, false);
    cuda_check(ctk_rand_uniform_f32(f.data<float>(), static_cast<int64_t>(n), g_rand_seed.load(), offset, t_stream), "rand");
    cuda_check(ctk_cast_f32(CTK_DTYPE_F64, static_cast<const Tensor&>(f).data<float>(), data<double>(), static_cast<int64_t>(n), t_stream), "rand (double)");
}

// ---- to(DType) (src/Tensor.cpp:199-243) ---------------------------------------------------------------------
Tensor Tensor::to(DType dtype) const {
    if (_dtype == dtype) return *this;
    const bool converts = _dtype == DType::kFloat && dtype != DType::kFloat;  // only float sources convert
    Tensor result(ShapeTag{}, _shape, dtype, _device, !converts);
    const size_t n = numel();
    if (!converts || n == 0) return result;
    const float* src = data<float>();
    void* dst = result._storage.raw();
    if (_device == DeviceType::kCUDA) {
        cuda_check(ctk_cast_f32(static_cast<int>(dtype), src, dst, static_cast<int64_t>(n), t_stream), "to(dtype)");
        return result;
    }
    for (size_t i = 0; i < n; ++i) {
        switch (dtype) {
            case DType::kDouble: static_cast<double*>(dst)[i] = static_cast<double>(src[i]); break;
            case DType::kInt: static_cast<int32_t*>(dst)[i] = static_cast<int32_t>(src[i]); break;
            case DType::kLong: static_cast<int64_t*>(dst)[i] = static_cast<int64_t>(src[i]); break;
            default: static_cast<bool*>(dst)[i] = static_cast<bool>(src[i]); break;
        }
    }
    return result;
}

// ---- operator[] (src/Tensor.cpp:175-189) --------------------------------------------------------------------
Tensor Tensor::operator[](size_t index) const {
    if (_shape.size() != 1) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DIMENSION, "operator[]: 1-D tensors only");
    if (index >= _shape[0]) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DIMENSION, "operator[]: index out of range");
    Tensor result(*this);
    result._shape = {1};
    result._strides = {0};
    result._storage_offset += index * _strides[0];
    return result;
}

void Tensor::copy_raw_to_host(void* dst, size_t nbytes) const {
    if (nbytes != numel() * dtypeSize(_dtype)) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DIMENSION, "copy_raw_to_host: size mismatch");
    if (nbytes == 0) return;
    const unsigned char* base = static_cast<const unsigned char*>(_storage.raw()) + _storage_offset * dtypeSize(_dtype);
    if (_device == DeviceType::kCUDA) {
        cuda_check(ctk_memcpy_d2h(dst, base, nbytes, t_stream), "copy_raw_to_host");
        cuda_check(t_stream ? ctk_stream_sync(t_stream) : ctk_device_sync(), "copy_raw_to_host sync");
    } else {
        std::memcpy(dst, base, nbytes);
    }
}

// ---- comparisons (src/Tensor.cpp:985-1309, 1462-1591) -----------------------------------------------------------
template <typename F>
static void host_compare(const float* a, const float* b, float s, int form, bool* out, size_t n, F f) {
    for (size_t i = 0; i < n; ++i) out[i] = form == CTK_CMP_TENSOR ? f(a[i], b[i]) : form == CTK_CMP_SCALAR_RIGHT ? f(a[i], s) : f(s, a[i]);
}
Tensor Tensor::compare(int cmp, int form, const Tensor* other, float s) const {
    Tensor result(ShapeTag{}, _shape, DType::kBool, _device, _dtype != DType::kFloat);
    if (form == CTK_CMP_TENSOR) {
        if (!other) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::TENSOR_STATE, "comparison: missing operand");
        if (_shape != other->shape()) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DIMENSION, "comparison: tensor shapes differ");
        if (_dtype != other->dtype()) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DATATYPE, "comparison: tensor dtypes differ");
        if (_device != other->device()) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DEVICE_COMPAT, "comparison: tensors are on different devices");
    }
    const size_t n = numel();
    if (_dtype != DType::kFloat || n == 0) return result;  // the reference compares float tensors only
    const float* a = data<float>();
    const float* b = form == CTK_CMP_TENSOR ? other->data<float>() : nullptr;
    if (_device == DeviceType::kCUDA) {
        cuda_check(ctk_compare_f32(cmp, form, a, b, s, static_cast<unsigned char*>(result._storage.raw()), static_cast<int64_t>(n), t_stream), "comparison");
        return result;
    }
    bool* out = static_cast<bool*>(result._storage.raw());
    switch (cmp) {
        case CTK_CMP_GT: host_compare(a, b, s, form, out, n, [](float x, float y) { return x > y; }); break;
        case CTK_CMP_LT: host_compare(a, b, s, form, out, n, [](float x, float y) { return x < y; }); break;
        case CTK_CMP_EQ: host_compare(a, b, s, form, out, n, [](float x, float y) { return x == y; }); break;
        case CTK_CMP_GE: host_compare(a, b, s, form, out, n, [](float x, float y) { return x >= y; }); break;
        case CTK_CMP_LE: host_compare(a, b, s, form, out, n, [](float x, float y) { return x <= y; }); break;
        default: host_compare(a, b, s, form, out, n, [](float x, float y) { return x != y; }); break;
    }
    return result;
}
Tensor Tensor::operator>(float s) const { return compare(CTK_CMP_GT, CTK_CMP_SCALAR_RIGHT, nullptr, s); }
Tensor Tensor::operator<(float s) const { return compare(CTK_CMP_LT, CTK_CMP_SCALAR_RIGHT, nullptr, s); }
Tensor Tensor::operator==(float s) const { return compare(CTK_CMP_EQ, CTK_CMP_SCALAR_RIGHT, nullptr, s); }
Tensor Tensor::operator>=(float s) const { return compare(CTK_CMP_GE, CTK_CMP_SCALAR_RIGHT, nullptr, s); }
Tensor Tensor::operator<=(float s) const { return compare(CTK_CMP_LE, CTK_CMP_SCALAR_RIGHT, nullptr, s); }
Tensor Tensor::operator!=(float s) const { return compare(CTK_CMP_NE, CTK_CMP_SCALAR_RIGHT, nullptr, s); }
Tensor Tensor::operator>(const Tensor& o) const { return compare(CTK_CMP_GT, CTK_CMP_TENSOR, &o, 0.0f); }
Tensor Tensor::operator<(const Tensor& o) const { return compare(CTK_CMP_LT, CTK_CMP_TENSOR, &o, 0.0f); }
Tensor Tensor::operator==(const Tensor& o) const { return compare(CTK_CMP_EQ, CTK_CMP_TENSOR, &o, 0.0f); }
Tensor Tensor::operator>=(const Tensor& o) const { return compare(CTK_CMP_GE, CTK_CMP_TENSOR, &o, 0.0f); }
Tensor Tensor::operator<=(const Tensor& o) const { return compare(CTK_CMP_LE, CTK_CMP_TENSOR, &o, 0.0f); }
Tensor Tensor::operator!=(const Tensor& o) const { return compare(CTK_CMP_NE, CTK_CMP_TENSOR, &o, 0.0f); }
Tensor operator>(float s, const Tensor& t) { return t.compare(CTK_CMP_GT, CTK_CMP_SCALAR_LEFT, nullptr, s); }
Tensor operator<(float s, const Tensor& t) { return t.compare(CTK_CMP_LT, CTK_CMP_SCALAR_LEFT, nullptr, s); }
Tensor operator==(float s, const Tensor& t) { return t.compare(CTK_CMP_EQ, CTK_CMP_SCALAR_LEFT, nullptr, s); }
Tensor operator>=(float s, const Tensor& t) { return t.compare(CTK_CMP_GE, CTK_CMP_SCALAR_LEFT, nullptr, s); }
Tensor operator<=(float s, const Tensor& t) { return t.compare(CTK_CMP_LE, CTK_CMP_SCALAR_LEFT, nullptr, s); }
Tensor operator!=(float s, const Tensor& t) { return t.compare(CTK_CMP_NE, CTK_CMP_SCALAR_LEFT, nullptr, s); }

// ---- op wrappers ------------------------------------------------------------------------------------------
void Tensor::record(Tensor& result, op o, std::vector<Tensor*> inputs, bool rg, int op_param) const {
    if (AutoDiffContext::current()) {
        AutoDiffContext::current()->defer_record(result.id(), o, inputs, op_param);
        result._requires_grad = rg;
        if (result._requires_grad) result.commit_pending_record();
    } else {
        result._requires_grad = rg;
    }
}

Tensor Tensor::binary_dispatch(const Tensor& other, op o) const {
    if (_dtype != other.dtype()) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DATATYPE, "tensor dtypes differ");
    const bool scalar_mix = (dim() == 0 && _device == DeviceType::kCPU) || (other.dim() == 0 && other.device() == DeviceType::kCPU);
    if (_device != other.device() && !scalar_mix) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DEVICE_COMPAT, "tensors are on different devices");
    Tensor result = Ctorch_Scheduler::getInstance().dispatch(*this, other, o);
    record(result, o, {const_cast<Tensor*>(this), const_cast<Tensor*>(&other)}, _requires_grad || other.requires_grad());
    return result;
}

Tensor Tensor::unary_dispatch(op o, int op_param) const {
    Tensor result = Ctorch_Scheduler::getInstance().dispatch(*this, o);
    record(result, o, {const_cast<Tensor*>(this)}, _requires_grad, op_param);
    return result;
}

Tensor Tensor::matmul(const Tensor& other) const {
    Tensor result = Ctorch_Scheduler::getInstance().dispatch(*this, other, op::MatMul);
    record(result, op::MatMul, {const_cast<Tensor*>(this), const_cast<Tensor*>(&other)}, _requires_grad || other.requires_grad());
    return result;
}
Tensor Tensor::shape_only(const std::vector<size_t>& shape, DType dtype, DeviceType device) {
    Tensor t;
    t._shape = shape;
    t._dtype = dtype;
    t._device = device;
    t.computeStrides();
    return t;
}

KeptSplit* operand_split(const Tensor& t, int64_t mn, int64_t k, int64_t s_mn, int64_t s_k) {
    int64_t outer, inner, pitch;
    if (s_k == 1 && s_mn >= k) { outer = mn; inner = k; pitch = s_mn; }
    else if (s_mn == 1 && s_k >= mn) { outer = k; inner = mn; pitch = s_k; }
    else return nullptr;
    return t.storage().kept_split(static_cast<int64_t>(t.storage_offset()), outer, inner, pitch, ctk_matmul_split_bytes(mn, k));
}

// y = [relu](A.B + bias) * (mask > 0) in one launch of the 3xTF32 product, operand splits kept with
// their buffers and y's own split written by the epilogue.  False (nothing launched) when the fused
// form does not apply: another device, dtype or mode, operands the tensor cores cannot take.
static bool fused_product(const Tensor& A, const Tensor& B, const Tensor* bias, bool relu, const Tensor* mask, Tensor& y) {
    static const bool fuse = [] {
        const char* e = std::getenv("CTORCH_FUSE_LINEAR");
        return !(e && e[0] == '0');
    }();
    auto plain = [](const Tensor& t, size_t rank) {
        return t.device() == DeviceType::kCUDA && t.dtype() == DType::kFloat && t.shape().size() == rank;
    };
    if (!fuse || !plain(A, 2) || !plain(B, 2) || A.shape()[1] != B.shape()[0] || ctk_get_matmul_mode() != CTK_MATMUL_3XTF32) return false;
    const int64_t m = static_cast<int64_t>(A.shape()[0]), k = static_cast<int64_t>(A.shape()[1]), n = static_cast<int64_t>(B.shape()[1]);
    if (m < 2 || k < 2 || n < 2 || n % 4 != 0) return false;
    if (bias && !(plain(*bias, 1) && static_cast<int64_t>(bias->shape()[0]) == n && bias->is_contiguous())) return false;
    if (mask && !(plain(*mask, 2) && static_cast<int64_t>(mask->shape()[0]) == m && static_cast<int64_t>(mask->shape()[1]) == n && mask->is_contiguous()))
        return false;
    const int64_t sa0 = static_cast<int64_t>(A.strides()[0]), sa1 = static_cast<int64_t>(A.strides()[1]);
    const int64_t sb0 = static_cast<int64_t>(B.strides()[0]), sb1 = static_cast<int64_t>(B.strides()[1]);
    // 0: tensor cores; 2: the short-contraction kernel, which reads the operands as they are (no splits)
    // and has no bias / ReLU form
    const int path = ctk_matmul_path(A.data<float>(), B.data<float>(), m, n, k, sa0, sa1, sb0, sb1, CTK_MATMUL_3XTF32);
    if (path != 0 && !(path == 2 && !bias && !relu)) return false;
    KeptSplit* ka = path == 0 ? operand_split(A, m, k, sa0, sa1) : nullptr;
    KeptSplit* kb = (path != 0 || B.storage().raw() == A.storage().raw()) ? nullptr : operand_split(B, n, k, sb1, sb0);  // one split per buffer
    y = Tensor(ShapeTag{}, {static_cast<size_t>(m), static_cast<size_t>(n)}, A.dtype(), DeviceType::kCUDA, false);
    float* yp = y.data<float>();  // (the mutable pointer first: asking for it drops a kept split)
    // y enters the next product as its K-major A operand and, transposed, a weight-gradient product:
    // its split is written by this kernel's epilogue
    KeptSplit* ky = y.storage().kept_split(0, m, n, n, ctk_matmul_split_bytes(m, n));
    cuda_check(ctk_matmul_3xtf32_fused_f32(A.data<float>(), B.data<float>(), yp, m, n, k, sa0, sa1, sb0, sb1, ka ? ka->buf : nullptr,
                                           ka ? &ka->valid : nullptr, kb ? kb->buf : nullptr, kb ? &kb->valid : nullptr,
                                           bias ? bias->data<float>() : nullptr, relu ? 1 : 0, mask ? mask->data<float>() : nullptr,
                                           ky ? ky->buf : nullptr, nullptr, t_stream),
               "fused MatMul epilogue");
    if (ky) ky->valid = ctk_matmul_split_tag_for(yp, n, n);
    return true;
}

Tensor Tensor::matmul_masked(const Tensor& other, const Tensor& mask) const {
    // (Even a short K, which leaves the product nothing to hide the four-array epilogue behind, comes out
    // ahead: the 10-class layer's g.W^T, K = 10, takes 154 us fused against 117 + 58 us for the product,
    // the ReLU rule and the split of its result.)
    Tensor y;
    if (fused_product(*this, other, nullptr, false, &mask, y)) return y;
    Tensor p = matmul(other);
    Tensor r(ShapeTag{}, p.sizes(), p.dtype(), p.device(), false);
    cuda_check(ctk_unary_backward_f32(CTK_OP_RELU, mask.data<float>(), p.data<float>(), r.data<float>(), static_cast<int64_t>(p.numel()), t_stream),
               "ReLU backward");
    return r;
}

Tensor Tensor::linear(const Tensor& W, const Tensor& bias, bool relu) const {
    Tensor y;
    if (!fused_product(*this, W, &bias, relu, nullptr, y)) {
        // (a returned temporary or moved local keeps its id, which is its key on the tape; a copy would not)
        if (relu) return (matmul(W) + bias).relu();
        return matmul(W) + bias;
    }
    const size_t m = _shape[0], n = W.shape()[1];
    // the tape sees the three operations
    const bool rg = _requires_grad || W.requires_grad() || bias.requires_grad();
    const std::vector<size_t> out_shape = {static_cast<size_t>(m), static_cast<size_t>(n)};
    Tensor mm = shape_only(out_shape, _dtype, DeviceType::kCUDA);
    record(mm, op::MatMul, {const_cast<Tensor*>(this), const_cast<Tensor*>(&W)}, _requires_grad || W.requires_grad());
    if (!relu) {
        record(y, op::Add, {&mm, const_cast<Tensor*>(&bias)}, rg);
        return y;
    }
    Tensor z = shape_only(out_shape, _dtype, DeviceType::kCUDA);
    record(z, op::Add, {&mm, const_cast<Tensor*>(&bias)}, rg);
    record(y, op::ReLU, {&z}, rg);
    return y;
}

Tensor Tensor::dot(const Tensor& other) const {
    Tensor result = Ctorch_Scheduler::getInstance().dispatch(*this, other, op::Dot);
    record(result, op::Dot, {const_cast<Tensor*>(this)}, _requires_grad);
    return result;
}
Tensor Tensor::operator+(const Tensor& o) const { return binary_dispatch(o, op::Add); }
Tensor Tensor::operator-(const Tensor& o) const { return binary_dispatch(o, op::Sub); }
Tensor Tensor::operator*(const Tensor& o) const { return binary_dispatch(o, op::Mul); }
Tensor Tensor::operator/(const Tensor& o) const { return binary_dispatch(o, op::Div); }
Tensor Tensor::operator-() const { return unary_dispatch(op::Neg); }
Tensor Tensor::relu() const { return unary_dispatch(op::ReLU); }
Tensor Tensor::sigmoid() const { return unary_dispatch(op::Sigmoid); }
Tensor Tensor::tanh() const { return unary_dispatch(op::Tanh); }
Tensor Tensor::sin() const { return unary_dispatch(op::Sin); }
Tensor Tensor::cos() const { return unary_dispatch(op::Cos); }

static Tensor loss_dispatch(const Tensor& a, const Tensor& target, op o) { return Ctorch_Scheduler::getInstance().dispatch(a, target, o); }
Tensor Tensor::mse_loss(const Tensor& target) const {
    Tensor r = loss_dispatch(*this, target, op::MSE);
    record(r, op::MSE, {const_cast<Tensor*>(this), const_cast<Tensor*>(&target)}, _requires_grad || target.requires_grad());
    return r;
}
Tensor Tensor::mae_loss(const Tensor& target) const {
    Tensor r = loss_dispatch(*this, target, op::MAE);
    record(r, op::MAE, {const_cast<Tensor*>(this), const_cast<Tensor*>(&target)}, _requires_grad || target.requires_grad());
    return r;
}
Tensor Tensor::cross_entropy(const Tensor& target) const {
    Tensor r = loss_dispatch(*this, target, op::CE);
    record(r, op::CE, {const_cast<Tensor*>(this), const_cast<Tensor*>(&target)}, _requires_grad || target.requires_grad());
    return r;
}

// The reference's Tensor::softmax is inline and throws off the CPU (src/Tensor.cpp:1645-1664); here
// the last-dim case goes to the registered Softmax kernel, which it is bit-identical to.
Tensor Tensor::softmax(int dim) const {
    if (_shape.empty()) Ctorch_Error::throwException(ErrorPlatform::kCPU, ErrorType::DIMENSION, "softmax: scalars are not supported");
    const int rank = static_cast<int>(_shape.size());
    if (dim < 0) dim += rank;
    if (dim < 0 || dim >= rank) Ctorch_Error::throwException(ErrorPlatform::kCPU, ErrorType::DIMENSION, "softmax: dim out of range");
    if (rank > 2) Ctorch_Error::throwException(ErrorPlatform::kCPU, ErrorType::DIMENSION, "softmax: only 1-D and 2-D tensors");
    if (dim != rank - 1) {
        // dim 0 of a 2-D tensor: down the columns (src/Tensor.cpp:1728-1743); like the reference's
        // Tensor::softmax this form is not dispatched through the scheduler
        if (_device != DeviceType::kCUDA) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DEVICE_COMPAT, "softmax: no kernel for this device");
        if (_dtype != DType::kFloat) Ctorch_Error::throwException(ErrorPlatform::kCUDA, ErrorType::DATATYPE, "softmax: float tensors only");
        if (!is_contiguous()) Ctorch_Error::throwException(ErrorPlatform::kCUDA, ErrorType::TENSOR_STATE, "softmax: contiguous tensor expected");
        Tensor result(ShapeTag{}, _shape, _dtype, _device, false);
        cuda_check(ctk_softmax_cols_f32(data<float>(), result.data<float>(), static_cast<int64_t>(_shape[0]), static_cast<int64_t>(_shape[1]), t_stream), "softmax(dim 0)");
        record(result, op::Softmax, {const_cast<Tensor*>(this)}, _requires_grad, dim);
        return result;
    }
    return unary_dispatch(op::Softmax, dim);
}

// src/Tensor.cpp:638-666 (not dispatched in the reference either).
Tensor Tensor::sum() const {
    if (_device != DeviceType::kCUDA) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DEVICE_COMPAT, "sum: no kernel for this device");
    Tensor result(ShapeTag{}, {}, _dtype, _device, false);
    cuda_check(ctk_sum_f32(data<float>(), static_cast<int64_t>(numel()), result.data<float>(), nullptr, t_stream), "sum");
    record(result, op::Sum, {const_cast<Tensor*>(this)}, _requires_grad);
    return result;
}

// src/Tensor.cpp:751-806 (t*s), 855-910 (t+s), 913-973 (t/s): recorded as Mul/Add/Div with a host
// scalar tensor as second input.
Tensor Tensor::scalar_form(int kind, float s, op recorded) const {
    if (_device != DeviceType::kCUDA) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DEVICE_COMPAT, "scalar op: no kernel for this device");
    if (!is_contiguous()) Ctorch_Error::throwException(ErrorPlatform::kCUDA, ErrorType::TENSOR_STATE, "scalar op: contiguous tensor expected");
    Tensor result(ShapeTag{}, _shape, _dtype, _device, false);
    cuda_check(ctk_scalar_f32(kind, data<float>(), s, result.data<float>(), static_cast<int64_t>(numel()), t_stream), "scalar op");
    Tensor scalar_tensor(s);
    record(result, recorded, {const_cast<Tensor*>(this), &scalar_tensor}, _requires_grad);
    return result;
}
Tensor Tensor::operator*(float s) const { return scalar_form(0, s, op::Mul); }
Tensor Tensor::operator+(float s) const { return scalar_form(1, s, op::Add); }
Tensor Tensor::operator/(float s) const {
    if (std::abs(s) < std::numeric_limits<float>::epsilon())
        Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::TENSOR_STATE, "division by zero in tensor / scalar");
    return scalar_form(2, s, op::Div);
}

void Tensor::backward() const {
    if (AutoDiffContext::current()) AutoDiffContext::current()->backward(const_cast<Tensor&>(*this));
}

void Tensor::sgd_update_shared_(const Tensor& g, float lr) {
    if (g.numel() != numel()) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DIMENSION, "sgd_update_shared_: gradient has a different size");
    if (_device != DeviceType::kCUDA || g.device() != DeviceType::kCUDA || _dtype != DType::kFloat)
        Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DEVICE_COMPAT, "sgd_update_shared_: float device tensors expected");
    float* p = static_cast<float*>(_storage.raw()) + _storage_offset;  // no detach: the sharers are meant to see it
    const bool resplit = _storage.has_split() && _shape.size() == 2 && is_contiguous() && g.is_contiguous() && _shape[1] % 4 == 0 &&
                         _storage_offset % 4 == 0 && g.storage_offset() % 4 == 0;
    if (resplit) {
        const int64_t outer = static_cast<int64_t>(_shape[0]), inner = static_cast<int64_t>(_shape[1]);
        KeptSplit* ks = _storage.kept_split(static_cast<int64_t>(_storage_offset), outer, inner, inner, ctk_matmul_split_bytes(inner, outer));
        if (ks) {
            cuda_check(ctk_sgd_update_split_f32(p, g.data<float>(), lr, outer, inner, inner, ks->buf, t_stream), "sgd_update_shared_ (with split)");
            ks->valid = ctk_matmul_split_tag_for(p, inner, inner);
            return;
        }
    }
    _storage.drop_split();  // a split of the old values, if any, is stale now
    cuda_check(ctk_sgd_update_f32(p, g.data<float>(), lr, static_cast<int64_t>(numel()), t_stream), "sgd_update_shared_");
}

void Tensor::sgd_update_(const Tensor& g, float lr) {
    if (g.numel() != numel()) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DIMENSION, "sgd_update_: gradient has a different size");
    if (_device != DeviceType::kCUDA || g.device() != DeviceType::kCUDA)
        Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DEVICE_COMPAT, "sgd_update_: device tensors expected");
    if (!g.is_contiguous()) Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DIMENSION, "sgd_update_: contiguous gradient expected");
    sgd_update_from_(g.data<float>(), lr);
}

void Tensor::sgd_update_from_(const float* g_device, float lr) {
    if (_device != DeviceType::kCUDA || _dtype != DType::kFloat)
        Ctorch_Error::throwException(ErrorPlatform::kGENERAL, ErrorType::DEVICE_COMPAT, "sgd_update_: float device tensor expected");
    // A weight matrix that enters products (its buffer carries a kept hi/lo split) gets the split of
    // its new value from the update kernel itself instead of a separate pass before the next product.
    const bool resplit = _storage.has_split() && _shape.size() == 2 && is_contiguous() && _shape[1] % 4 == 0 && _storage_offset % 4 == 0 &&
                         (reinterpret_cast<uintptr_t>(g_device) & 15u) == 0;
    float* p = data<float>();  // detaches from sharers, drops the split of the old value
    if (resplit) {
        const int64_t outer = static_cast<int64_t>(_shape[0]), inner = static_cast<int64_t>(_shape[1]);
        KeptSplit* ks = _storage.kept_split(static_cast<int64_t>(_storage_offset), outer, inner, inner, ctk_matmul_split_bytes(inner, outer));
        if (ks) {
            cuda_check(ctk_sgd_update_split_f32(p, g_device, lr, outer, inner, inner, ks->buf, t_stream), "sgd_update_ (with split)");
            ks->valid = ctk_matmul_split_tag_for(p, inner, inner);
            return;
        }
    }
    cuda_check(ctk_sgd_update_f32(p, g_device, lr, static_cast<int64_t>(numel()), t_stream), "sgd_update_");
}

// ---- free functions (src/Tensor.cpp:1373-1453) ---------------------------------------------------------------
void backward(Tensor& root) {
    if (AutoDiffContext::current()) AutoDiffContext::current()->backward(root);
}
void backward(Tensor& root, Tensor grad_output) {
    if (AutoDiffContext::current()) AutoDiffContext::current()->backward(root, grad_output);
}
Tensor grad(const Tensor& t) {
    if (AutoDiffContext::current()) return AutoDiffContext::current()->get_grad(&t);
    return Tensor();
}
Tensor matMul(const Tensor& a, const Tensor& b) { return Ctorch_Scheduler::getInstance().dispatch(a, b, op::MatMul); }
Tensor operator+(float s, const Tensor& t) { return t + s; }
Tensor operator*(float s, const Tensor& t) { return t * s; }
Tensor operator-(float s, const Tensor& t) { return Tensor(s) - t; }
Tensor operator/(float s, const Tensor& t) { return Tensor(s) / t; }

}  // namespace ctorch
