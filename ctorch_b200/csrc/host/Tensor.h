// Tensor: value-semantic n-d array with a device tag.  Public API as the reference's
// include/Tensor.h / src/Tensor.cpp for everything on the training path: constructors (:233-313),
// copy = new id + same value (:320-357), move keeps the id (:364-404), accessors, t()/transpose/
// reshape/broadcast_to, zero/ones, the op wrappers that dispatch through Ctorch_Scheduler and
// record on the tape, the float-scalar operators, sum/softmax, the losses, backward/grad.
//
// What is new: DeviceType::kCUDA is real.  data<T>() of a kCUDA tensor is a DEVICE pointer; host
// code moves data with copy_from_host / copy_to_host / to(device) / item().  Copies share storage
// and detach on the first write, which preserves the reference's value semantics without its deep
// copies.
#pragma once
#include <atomic>
#include <initializer_list>
#include <numeric>
#include <string>
#include <vector>

#include "AutoDiff.h"
#include "Ctools.h"
#include "Ctorch_Error.h"
#include "Storage.h"

namespace ctorch {

class Tensor {
    static std::atomic<size_t> global_tensor_id;

    size_t tensor_id_;
    bool record_committed_ = false;
    bool _requires_grad = false;
    std::vector<size_t> _strides;
    size_t _storage_offset = 0;
    DeviceType _device = DeviceType::kCPU;
    DType _dtype = DType::kFloat;
    Storage _storage;
    std::vector<size_t> _shape;

    void computeStrides();
    template <typename T> void checkDType() const;
    Tensor binary_dispatch(const Tensor& other, op o) const;
    Tensor unary_dispatch(op o, int op_param = 0) const;
    Tensor scalar_form(int kind, float s, op recorded) const;
    static Tensor shape_only(const std::vector<size_t>& shape, DType dtype, DeviceType device);  // no storage
    void record(Tensor& result, op o, std::vector<Tensor*> inputs, bool rg, int op_param = 0) const;

public:
    // ---- construction ----
    Tensor();
    Tensor(float value);  // 0-D, always on the host, as in the reference (:239-264)
    Tensor(std::initializer_list<float> values);
    Tensor(ShapeTag, const std::vector<size_t>& shape, DType dtype = DType::kFloat, DeviceType device = DeviceType::kCPU,
           bool zero_init = true);
    Tensor(size_t size, DType dtype = DType::kFloat, DeviceType device = DeviceType::kCPU, bool zero_init = true);
    Tensor(const Tensor& other);
    Tensor& operator=(const Tensor& other);
    Tensor(Tensor&& other) noexcept;
    Tensor& operator=(Tensor&& other) noexcept;
    ~Tensor() = default;

    // ---- accessors ----
    size_t id() const { return tensor_id_; }
    void set_id(size_t id) { tensor_id_ = id; }
    void requires_grad(bool key);
    bool requires_grad() const { return _requires_grad; }
    void set_requires_grad(bool r) { _requires_grad = r; }
    const std::vector<size_t>& shape() const { return _shape; }
    const std::vector<size_t>& sizes() const { return _shape; }
    const std::vector<size_t>& strides() const { return _strides; }
    size_t numel() const;
    int dim() const { return static_cast<int>(_shape.size()); }
    size_t size(int dim) const;
    size_t stride(int dim) const;
    size_t storage_offset() const { return _storage_offset; }
    DeviceType device() const { return _device; }
    DType dtype() const { return _dtype; }
    bool is_contiguous() const;
    bool is_cleared() const { return _storage.empty(); }
    const Storage& storage() const { return _storage; }
    void clear_storage() { _storage.clear(); }
    bool has_pending_record() const { return !record_committed_; }
    void commit_pending_record();

    // Writable pointer (detaches from sharers first) / read-only pointer.  Host pointer for kCPU,
    // device pointer for kCUDA.  Both point at element [storage_offset].
    template <typename T> T* data();
    template <typename T> const T* data() const;
    template <typename T> T item() const;  // kCUDA: synchronising device-to-host read of one element

    // ---- host <-> device ----
    void copy_from_host(const float* src, size_t count);
    void copy_to_host(float* dst, size_t count) const;
    std::vector<float> to_vector() const;
    // numel() * dtypeSize bytes, in memory order from element [storage_offset] (any dtype).
    void copy_raw_to_host(void* dst, size_t nbytes) const;
    Tensor to(DeviceType device) const;
    // Conversion out of float (src/Tensor.cpp:199-243): same dtype -> a copy; float -> double / int /
    // long / bool by static_cast per element; any other source leaves the zero-initialised result.
    Tensor to(DType dtype) const;
    Tensor cuda() const { return to(DeviceType::kCUDA); }
    Tensor cpu() const { return to(DeviceType::kCPU); }

    // ---- shape ops ----
    Tensor clone() const;
    Tensor transpose(int dim0, int dim1) const;
    Tensor t() const;
    // Rows [start, start + count) of a 2-D (or 1-D) tensor as a view of the same buffer: what
    // get_batch of mnist/mnist.cpp:160-188 copies element by element.
    Tensor narrow_rows(size_t start, size_t count) const;
    Tensor reshape(const std::vector<size_t>& new_shape) const;
    Tensor reshape(std::initializer_list<size_t> new_shape) const { return reshape(std::vector<size_t>(new_shape)); }
    Tensor broadcast_to(const std::vector<size_t>& shape) const;
    Tensor contiguous() const;
    void zero();
    void ones();  // every dtype (src/Tensor.cpp:422-450)
    void fill(float v);
    // Uniform [0, 1) for float and double tensors (src/Tensor.cpp:458-479).  The reference seeds a
    // thread-local mt19937 from std::random_device; here a process-wide counter-based generator,
    // seeded the same way unless manual_seed() fixed the seed.
    void rand();
    static void manual_seed(uint64_t seed);
    // Element `index` of a 1-D tensor as a view of shape {1} (src/Tensor.cpp:175-189).
    Tensor operator[](size_t index) const;

    // ---- math (dispatched + recorded) ----
    Tensor matmul(const Tensor& other) const;
    // (this.matmul(W) + bias)[.relu()] as ONE kernel where the device path allows it (2-D float device
    // tensors, 3xTF32 mode, bias of W's column count), recorded on the tape as the same MatMul, Add
    // and ReLU nodes the three calls would record -- the two intermediate results exist there as
    // shapes only, no rule reads their values -- and equal to them bit for bit.  Anything else runs
    // the three calls.  No counterpart in the reference.
    Tensor linear(const Tensor& W, const Tensor& bias, bool relu) const;
    // this.matmul(other) * (mask > 0 ? 1 : 0): a gradient product followed by ReLU's backward rule with
    // mask the ReLU's output, in one kernel where the device path allows it (else the two kernels);
    // not recorded on the tape (backward calls it).  No counterpart in the reference.
    Tensor matmul_masked(const Tensor& other, const Tensor& mask) const;
    Tensor dot(const Tensor& other) const;
    Tensor relu() const;
    Tensor sigmoid() const;
    Tensor tanh() const;
    Tensor sin() const;
    Tensor cos() const;
    Tensor softmax(int dim = -1) const;
    Tensor sum() const;
    Tensor cross_entropy(const Tensor& target) const;
    Tensor mse_loss(const Tensor& target) const;
    Tensor mae_loss(const Tensor& target) const;
    Tensor operator+(const Tensor& other) const;
    Tensor operator-(const Tensor& other) const;
    Tensor operator*(const Tensor& other) const;
    Tensor operator/(const Tensor& other) const;
    Tensor operator-() const;
    Tensor operator+(float s) const;
    Tensor operator*(float s) const;
    Tensor operator/(float s) const;
    // Element-wise comparisons -> kBool tensors of this shape (src/Tensor.cpp:985-1309).  As in the
    // reference the elements are taken in memory order, the two-tensor forms throw on a shape or
    // dtype mismatch, and a non-float tensor compares to all-false.
    Tensor operator>(float s) const;
    Tensor operator<(float s) const;
    Tensor operator==(float s) const;
    Tensor operator>=(float s) const;
    Tensor operator<=(float s) const;
    Tensor operator!=(float s) const;
    Tensor operator>(const Tensor& other) const;
    Tensor operator<(const Tensor& other) const;
    Tensor operator==(const Tensor& other) const;
    Tensor operator>=(const Tensor& other) const;
    Tensor operator<=(const Tensor& other) const;
    Tensor operator!=(const Tensor& other) const;
    // cmp: CTK_CMP_*; form: CTK_CMP_TENSOR (other), CTK_CMP_SCALAR_RIGHT (this cmp s), CTK_CMP_SCALAR_LEFT (s cmp this)
    Tensor compare(int cmp, int form, const Tensor* other, float s) const;
    void backward() const;

    // In-place p -= g*lr on this tensor's device: the SGD loop that user code writes on raw host
    // pointers in the reference (mnist/mnist.cpp:80-92).
    void sgd_update_(const Tensor& g, float lr);
    // The same update with the gradient given as a raw device pointer to numel() contiguous floats
    // (16-byte aligned for the form that also rewrites the kept split): gradients that live in a
    // communicator's registered buffer instead of a Tensor.
    void sgd_update_from_(const float* g_device, float lr);
    // The same update written THROUGH to every tensor that shares this buffer -- in particular the copy
    // the tape took when the parameter was registered, which the reference's backward keeps reading
    // while the live weights move on (src/AutoDiff.cpp:286-290, :1651).  With this form backward sees
    // the updated weights.  Opt-in, no counterpart in the reference.
    void sgd_update_shared_(const Tensor& g, float lr);

    friend class AutoDiff;
};

void backward(Tensor& root);
void backward(Tensor& root, Tensor grad_output);
Tensor grad(const Tensor& t);
Tensor matMul(const Tensor& a, const Tensor& b);
Tensor operator+(float s, const Tensor& t);
Tensor operator-(float s, const Tensor& t);
Tensor operator*(float s, const Tensor& t);
Tensor operator/(float s, const Tensor& t);
// scalar cmp tensor (src/Tensor.cpp:1462-1591)
Tensor operator>(float s, const Tensor& t);
Tensor operator<(float s, const Tensor& t);
Tensor operator==(float s, const Tensor& t);
Tensor operator>=(float s, const Tensor& t);
Tensor operator<=(float s, const Tensor& t);
Tensor operator!=(float s, const Tensor& t);

// The kept hi/lo split of a MatMul operand `t` with extents (mn, k) and strides (s_mn, s_k): the view is
// named by its contiguous ("inner") extent, the other extent and its pitch, so a t() view of the same
// memory finds the same split.  nullptr for an operand without a unit stride (or a host tensor).
KeptSplit* operand_split(const Tensor& t, int64_t mn, int64_t k, int64_t s_mn, int64_t s_k);

// Stream every kernel and copy of this thread's tensors is issued on (NULL = legacy default stream).
void* current_stream();
void set_current_stream(void* stream);

}  // namespace ctorch
