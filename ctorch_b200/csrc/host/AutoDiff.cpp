// AutoDiff implementation.  Graph bookkeeping follows the reference's src/AutoDiff.cpp (make_leaf
// :250-302, defer_record :314-370, commit_record :373-499, zero_grad :502-510,
// update_requires_grad :513-542, backward :547-553 and :1080-1924, get_grad :86-247); the
// behaviours that define the reference's numbers are kept on purpose:
//   - a node owns the VALUE its tensor had when it was registered and never refreshes it, so the
//     MatMul rule multiplies by the weights as they were at first registration (:286-290, :1651);
//   - a gradient sent to a broadcast operand is GATHERED with index 0 on the broadcast dims, not
//     summed: the bias gradient of [B,H] + [H] is row 0 of the upstream gradient (:690-757);
//   - recording is off for the whole of backward (:547-553).
// What differs is where the arithmetic runs: every rule is one or two kernel launches on the
// device that holds the node (fused where the reference chains several single-op kernels, with the
// same intermediate roundings), gradients stay resident on the GPU, and the host scans that only
// feed trace lines (:1268-1279, :1708-1718, :1794-1824) are gone.
#include "AutoDiff.h"

#include <algorithm>

#include "Tensor.h"
#include "ctorch_b200.h"

namespace ctorch {

AutoDiff::Node::Node(size_t id, std::unique_ptr<Tensor> t, bool req_grad, bool leaf)
    : tensor_id(id), tensor(std::move(t)), requires_grad(req_grad), is_leaf(leaf) {}
AutoDiff::Node::~Node() = default;

AutoDiff::AutoDiff() = default;
AutoDiff::~AutoDiff() {
    id_to_node.clear();
    pending_records.clear();
}

AutoDiff::Node* AutoDiff::get_node_by_id(size_t id) {
    std::lock_guard<std::mutex> lock(records_mutex);
    auto it = id_to_node.find(id);
    return it == id_to_node.end() ? nullptr : it->second.get();
}

static std::unique_ptr<Tensor> zeros_like_shape(const std::vector<size_t>& shape, DType dt, DeviceType dev) {
    return std::make_unique<Tensor>(ShapeTag{}, shape, dt, dev, true);
}

void AutoDiff::make_leaf(Tensor& t, bool requires_grad) {
    const size_t id = t.id();
    if (id == 0) return;
    {
        std::lock_guard<std::mutex> lock(records_mutex);
        auto it = id_to_node.find(id);
        if (it != id_to_node.end()) {
            // Already known: only the flag changes.  The stored value is NOT refreshed.
            it->second->requires_grad = requires_grad;
            if (requires_grad && !it->second->grad) it->second->grad = zeros_like_shape(t.sizes(), t.dtype(), t.device());
            return;
        }
    }
    auto copy = std::make_unique<Tensor>(t);  // value snapshot (shares storage until t is written)
    copy->set_id(id);
    auto node = std::make_unique<Node>(id, std::move(copy), requires_grad, true);
    std::lock_guard<std::mutex> lock(records_mutex);
    id_to_node[id] = std::move(node);
}

void AutoDiff::defer_record(size_t output_id, op operation, const std::vector<Tensor*>& inputs, int op_param_i) {
    if (output_id == 0) {
        Ctorch_Error::log(ErrorLevel::WARN, ErrorPlatform::kAutoDiff, ErrorType::TENSOR_STATE, "defer_record: output id is 0");
        return;
    }
    PendingRecord record;
    record.operation = operation;
    record.op_param_i = op_param_i;
    for (Tensor* input : inputs) {
        if (!input || input->id() == 0) continue;
        record.input_ids.push_back(input->id());
        bool needs_registration;
        {
            std::lock_guard<std::mutex> lock(records_mutex);
            needs_registration = id_to_node.find(input->id()) == id_to_node.end();
        }
        if (needs_registration) make_leaf(*input, input->requires_grad());
    }
    std::lock_guard<std::mutex> lock(records_mutex);
    pending_records[output_id] = std::move(record);
}

void AutoDiff::commit_record(Tensor& output) {
    const size_t output_id = output.id();
    if (output_id == 0) return;
    PendingRecord rec;
    {
        std::lock_guard<std::mutex> lock(records_mutex);
        auto it = pending_records.find(output_id);
        if (it == pending_records.end() || it->second.committed) return;
        for (size_t in : it->second.input_ids)
            if (id_to_node.find(in) == id_to_node.end()) {
                pending_records.erase(it);
                return;
            }
        it->second.committed = true;
        rec = it->second;
    }
    bool requires_grad = false;
    for (size_t in : rec.input_ids) {
        Node* n = get_node_by_id(in);
        if (n && n->requires_grad) {
            requires_grad = true;
            break;
        }
    }
    auto node = std::make_unique<Node>(output_id, std::make_unique<Tensor>(output), requires_grad, false);
    node->operation = rec.operation;
    node->op_param_i = rec.op_param_i;
    node->input_ids = rec.input_ids;
    std::lock_guard<std::mutex> lock(records_mutex);
    id_to_node[output_id] = std::move(node);
    pending_records.erase(output_id);
}

void AutoDiff::Node::materialize_grad() {
    if (grad_is_zero && grad) grad->zero();
    grad_is_zero = false;
}

void AutoDiff::zero_grad(Tensor& t) {
    if (t.id() == 0) return;
    std::lock_guard<std::mutex> lock(records_mutex);
    auto it = id_to_node.find(t.id());
    // (:502-510 zero-fills here; the fill is deferred, see Node::grad_is_zero)
    if (it != id_to_node.end() && it->second && it->second->grad) it->second->grad_is_zero = true;
}

void AutoDiff::update_requires_grad(Tensor& t, bool requires_grad) {
    if (t.id() == 0) return;
    std::lock_guard<std::mutex> lock(records_mutex);
    auto it = id_to_node.find(t.id());
    if (it == id_to_node.end() || !it->second) return;
    it->second->requires_grad = requires_grad;
    if (requires_grad && !it->second->grad) it->second->grad = zeros_like_shape(t.sizes(), t.dtype(), t.device());
}

void AutoDiff::set_retain_graph(bool retain) { retain_graph = retain; }

Tensor AutoDiff::get_grad(const Tensor* t) {
    if (!t || t->id() == 0) return Tensor();
    std::lock_guard<std::mutex> lock(records_mutex);
    auto it = id_to_node.find(t->id());
    if (it != id_to_node.end() && it->second && it->second->requires_grad && it->second->grad) {
        it->second->materialize_grad();
        return Tensor(*it->second->grad);
    }
    return Tensor(ShapeTag{}, t->shape(), t->dtype(), t->device(), true);  // no gradient: zeros of the input's shape (:203-246)
}

Tensor* AutoDiff::grad_buffer(const Tensor& t) {
    std::lock_guard<std::mutex> lock(records_mutex);
    auto it = id_to_node.find(t.id());
    if (it == id_to_node.end() || !it->second || !it->second->grad) return nullptr;
    it->second->materialize_grad();
    return it->second->grad.get();
}

void AutoDiff::clear_graph() {
    std::lock_guard<std::mutex> lock(records_mutex);
    id_to_node.clear();
    pending_records.clear();
    retain_graph = false;
}

void AutoDiff::release_step_nodes() {
    std::lock_guard<std::mutex> lock(records_mutex);
    for (auto it = id_to_node.begin(); it != id_to_node.end();) {
        Node* n = it->second.get();
        if (n && n->is_leaf && n->requires_grad) ++it;
        else it = id_to_node.erase(it);
    }
    pending_records.clear();
}

size_t AutoDiff::node_count() {
    std::lock_guard<std::mutex> lock(records_mutex);
    return id_to_node.size();
}

void AutoDiff::dfs_topological_sort(Node* node, std::unordered_set<Node*>& visited, std::vector<Node*>& result) {
    // Iterative post-order (the reference recurses, :1058-1077): deep graphs must not overflow the stack.
    if (!node || visited.count(node)) return;
    std::vector<std::pair<Node*, size_t>> stack;
    stack.push_back({node, 0});
    visited.insert(node);
    while (!stack.empty()) {
        auto& top = stack.back();
        Node* n = top.first;
        if (top.second < n->input_ids.size()) {
            auto it = id_to_node.find(n->input_ids[top.second++]);
            if (it != id_to_node.end() && it->second && !visited.count(it->second.get())) {
                visited.insert(it->second.get());
                stack.push_back({it->second.get(), 0});
            }
        } else {
            result.push_back(n);
            stack.pop_back();
        }
    }
}

void AutoDiff::backward(Tensor& root) {
    AutoDiffContext::Guard guard(nullptr);  // no recording while gradients are computed
    if (root.device() == DeviceType::kCUDA) {
        // the reference's Tensor(1.0f) (:551), made where the root lives: one fill launch instead of an
        // upload through the staging buffers (which waits on the host, and cannot be captured)
        Tensor one(ShapeTag{}, std::vector<size_t>{}, DType::kFloat, DeviceType::kCUDA, false);
        one.fill(1.0f);
        backward(root, one);
        return;
    }
    Tensor grad_output(1.0f);               // a host 0-D tensor, as in the reference (:551)
    backward(root, grad_output);
}

// ---- gradient shape adjustment (src/AutoDiff.cpp:562-1049) ------------------------------------------
static const float* dev_ptr(const Tensor& t) { return t.data<float>(); }

Tensor AutoDiff::check_and_adjust_grad_shape(const Tensor& grad, const std::vector<size_t>& target_shape, DeviceType target_device) {
    if (grad.sizes() == target_shape) return grad;
    const DeviceType dev = grad.device();
    void* st = current_stream();
    // 0-D gradient: fill (:579-627).  A host scalar (the default root gradient Tensor(1.0f)) fills a
    // tensor on the device the gradient is for.
    if (grad.sizes().empty()) {
        Tensor result(ShapeTag{}, target_shape, grad.dtype(), target_device, false);
        if (dev == DeviceType::kCUDA && target_device == DeviceType::kCUDA)
            cuda_check(ctk_fill_f32(result.data<float>(), 0.0f, dev_ptr(grad), static_cast<int64_t>(result.numel()), st), "grad fill");
        else
            result.fill(grad.item<float>());
        return result;
    }
    if (dev != DeviceType::kCUDA) Ctorch_Error::throwException(ErrorPlatform::kAutoDiff, ErrorType::DEVICE_COMPAT, "gradient shape adjustment: device tensor expected");
    const size_t grad_rank = grad.sizes().size(), target_rank = target_shape.size();
    // lower rank: pad with leading ones and tile grad[i % n] (:633-687), then adjust again
    if (grad_rank < target_rank) {
        std::vector<size_t> padded(target_rank, 1);
        for (size_t i = 0; i < grad_rank; ++i) padded[target_rank - grad_rank + i] = grad.sizes()[i];
        Tensor temp(ShapeTag{}, padded, grad.dtype(), dev, false);
        cuda_check(ctk_tile_f32(dev_ptr(grad), static_cast<int64_t>(grad.numel()), temp.data<float>(), static_cast<int64_t>(temp.numel()), st), "grad tile");
        return check_and_adjust_grad_shape(temp, target_shape, target_device);
    }
    // trailing dims compatible: gather, index 0 on every dim the target does not have or has as 1 (:690-890)
    bool can_broadcast = true;
    for (size_t i = 1; i <= target_rank; ++i) {
        const size_t gd = grad.sizes()[grad_rank - i], td = target_shape[target_rank - i];
        if (gd != td && gd != 1 && td != 1) {
            can_broadcast = false;
            break;
        }
    }
    if (!can_broadcast) {
        // Shapes that do not broadcast: the reference folds, result[i] = sum of grad[j] over j = i (mod n),
        // n the target's element count (:910-966; its last-resort branch :971-1048 computes the same sums
        // the slow way).  With grad read as rows of n elements that is a column sum over the whole rows
        // plus the ragged last row added to the first elements.  The reference adds each class of j in
        // ascending order in fp32; the device sums the column in a tree, at least as accurately.
        if (!grad.is_contiguous()) Ctorch_Error::throwException(ErrorPlatform::kAutoDiff, ErrorType::DIMENSION, "gradient shape adjustment: folding needs a contiguous gradient");
        Tensor result(ShapeTag{}, target_shape, grad.dtype(), dev, false);
        const int64_t n = static_cast<int64_t>(result.numel()), total = static_cast<int64_t>(grad.numel());
        if (n == 0) return result;
        const int64_t rows = total / n, rem = total % n;
        if (rows > 0) cuda_check(ctk_colsum_f32(dev_ptr(grad), rows, n, result.data<float>(), st), "grad fold");
        else result.fill(0.0f);
        if (rem > 0) cuda_check(ctk_accumulate_f32(result.data<float>(), dev_ptr(grad) + rows * n, rem, st), "grad fold (last row)");
        return result;
    }
    Tensor result(ShapeTag{}, target_shape, grad.dtype(), dev, false);
    const int64_t n = static_cast<int64_t>(result.numel());
    if (n == 0) return result;
    // Fast case: target == grad's trailing dims -> the leading `n` elements (row 0 for a bias).
    bool prefix = grad.is_contiguous();
    for (size_t i = 1; i <= target_rank && prefix; ++i) prefix = grad.sizes()[grad_rank - i] == target_shape[target_rank - i];
    if (prefix) {
        if (exact_broadcast_grad)  // opt-in: the sum over the broadcast rows instead of row 0
            cuda_check(ctk_colsum_f32(dev_ptr(grad), static_cast<int64_t>(grad.numel()) / n, n, result.data<float>(), st), "grad column sum");
        else
            cuda_check(ctk_memcpy_d2d(result.data<float>(), dev_ptr(grad), static_cast<size_t>(n) * sizeof(float), st), "grad gather");
        return result;
    }
    if (target_rank > 8) Ctorch_Error::throwException(ErrorPlatform::kAutoDiff, ErrorType::DIMENSION, "gradient shape adjustment: rank > 8");
    int64_t dshape[8], sstride[8];
    for (size_t j = 0; j < target_rank; ++j) {
        const size_t gi = grad_rank - target_rank + j;
        dshape[j] = static_cast<int64_t>(target_shape[j]);
        sstride[j] = (grad.sizes()[gi] == 1 || target_shape[j] == 1) ? 0 : static_cast<int64_t>(grad.strides()[gi]);
    }
    cuda_check(ctk_gather_nd_f32(dev_ptr(grad), result.data<float>(), static_cast<int>(target_rank), dshape, sstride, st), "grad gather");
    return result;
}

// ---- per-op rules (src/AutoDiff.cpp:1216-1861) ------------------------------------------------------------
static const float* scalar_arg(const Tensor& g, Tensor& holder) {
    // Upstream 0-D gradient as a device scalar; nullptr means "exactly 1".
    if (g.device() == DeviceType::kCUDA) return g.data<float>();
    const float v = g.item<float>();
    if (v == 1.0f) return nullptr;
    holder = g.to(DeviceType::kCUDA);
    return holder.data<float>();
}

Tensor AutoDiff::rule(Node* node, size_t input_id, Node& input_node, bool& skip) {
    Tensor& node_grad = *node->grad;
    void* st = current_stream();
    const std::vector<size_t>& in_shape = input_node.tensor->sizes();
    auto other_of = [&]() -> Node* {
        if (node->input_ids.size() < 2) return nullptr;
        const size_t oid = (input_id == node->input_ids[0]) ? node->input_ids[1] : node->input_ids[0];
        auto it = id_to_node.find(oid);
        return it == id_to_node.end() ? nullptr : it->second.get();
    };
    auto fused_unary = [&](int opc) {
        Tensor& x = *input_node.tensor;
        Tensor g = check_and_adjust_grad_shape(node_grad, x.sizes(), x.device());
        Tensor dx(ShapeTag{}, x.sizes(), x.dtype(), x.device(), false);
        cuda_check(ctk_unary_backward_f32(opc, x.data<float>(), g.data<float>(), dx.data<float>(), static_cast<int64_t>(x.numel()), st), "unary backward");
        return dx;
    };
    switch (node->operation) {
        case op::Add:
        case op::Sum:
            return check_and_adjust_grad_shape(node_grad, in_shape, input_node.tensor->device());
        case op::Sub: {
            Tensor adj = check_and_adjust_grad_shape(node_grad, in_shape, input_node.tensor->device());
            return input_id == node->input_ids[0] ? adj : -adj;
        }
        case op::Mul: {
            Node* other = other_of();
            if (!other) return node_grad;
            return *other->tensor * node_grad;
        }
        case op::Div: {
            // g / b for the numerator, ((-a) * g) / (b * b) for the denominator.  The reference first
            // scans b on the host and throws on |b| < eps (:1268-1284); that scan would stall the GPU
            // every step and is left out: a zero divisor yields IEEE inf/NaN gradients instead.
            auto a_it = id_to_node.find(node->input_ids[0]);
            auto b_it = id_to_node.find(node->input_ids.size() > 1 ? node->input_ids[1] : 0);
            if (a_it == id_to_node.end() || b_it == id_to_node.end()) { skip = true; return Tensor(); }
            Tensor& a = *a_it->second->tensor;
            Tensor& b = *b_it->second->tensor;
            if (input_id == node->input_ids[0]) return node_grad / b;
            return -a * node_grad / (b * b);
        }
        case op::Neg: return -node_grad;
        case op::ReLU: {
            // g * (x > 0) (:1320-1371).  The mask is taken from the node's OUTPUT y = max(0, x): y > 0
            // exactly when x > 0, and the fused MatMul+bias+ReLU never materialises x.
            const Tensor& y = *node->tensor;
            if (node->grad_premasked) return node_grad;  // g * mask was applied where g was made
            Tensor g = check_and_adjust_grad_shape(node_grad, y.sizes(), y.device());
            Tensor dx(ShapeTag{}, y.sizes(), y.dtype(), y.device(), false);
            cuda_check(ctk_unary_backward_f32(CTK_OP_RELU, y.data<float>(), g.data<float>(), dx.data<float>(), static_cast<int64_t>(y.numel()), st), "ReLU backward");
            return dx;
        }
        case op::Sigmoid: return fused_unary(CTK_OP_SIGMOID);  // (s * (1 - s)) * g      :1372-1383
        case op::Tanh: return fused_unary(CTK_OP_TANH);        // (1 - t*t) * g          :1384-1398
        case op::Sin: return fused_unary(CTK_OP_SIN);          // cos(x) * g             :1399-1407
        case op::Cos: return fused_unary(CTK_OP_COS);          // (-sin(x)) * g          :1408-1416
        case op::Softmax: {
            const Tensor& y = *node->tensor;  // the saved OUTPUT
            const size_t rank = y.sizes().size();
            int dim = node->op_param_i;
            if (dim < 0) dim += static_cast<int>(rank);
            if (rank == 0 || rank > 2 || dim < 0 || dim >= static_cast<int>(rank))
                Ctorch_Error::throwException(ErrorPlatform::kAutoDiff, ErrorType::DIMENSION, "Softmax backward: 1-D and 2-D tensors, dim 0 or 1");
            const int64_t rows = rank == 1 ? 1 : static_cast<int64_t>(y.sizes()[0]);
            const int64_t cols = static_cast<int64_t>(y.sizes()[rank - 1]);
            Tensor g = check_and_adjust_grad_shape(node_grad, y.sizes(), y.device());
            Tensor dx(ShapeTag{}, y.sizes(), y.dtype(), y.device(), false);
            if (dim == static_cast<int>(rank) - 1)   // along the rows (:1461-1472)
                cuda_check(ctk_softmax_backward_rows_f32(y.data<float>(), g.data<float>(), dx.data<float>(), rows, cols, st), "softmax backward");
            else                                     // down the columns (:1473-1484)
                cuda_check(ctk_softmax_backward_cols_f32(y.data<float>(), g.data<float>(), dx.data<float>(), rows, cols, st), "softmax backward (dim 0)");
            return dx;
        }
        case op::MSE:
        case op::MAE: {
            Node* target = other_of();
            if (!target) { skip = true; return Tensor(); }
            Tensor& p = *input_node.tensor;
            Tensor& t = *target->tensor;
            Tensor holder;
            const float* g = scalar_arg(node_grad, holder);
            Tensor dp(ShapeTag{}, p.sizes(), p.dtype(), p.device(), false);
            if (node->operation == op::MSE)
                cuda_check(ctk_mse_backward_f32(p.data<float>(), t.data<float>(), g, dp.data<float>(), static_cast<int64_t>(p.numel()), st), "mse backward");
            else
                cuda_check(ctk_mae_backward_f32(p.data<float>(), t.data<float>(), g, dp.data<float>(), static_cast<int64_t>(p.numel()), st), "mae backward");
            return dp;
        }
        case op::CE: {
            Node* target = other_of();
            if (!target) { skip = true; return Tensor(); }
            Tensor& logits = *input_node.tensor;
            Tensor& t = *target->tensor;
            const size_t rank = logits.sizes().size();
            if (rank != 1 && rank != 2) Ctorch_Error::throwException(ErrorPlatform::kAutoDiff, ErrorType::DIMENSION, "CrossEntropy backward: only 1-D/2-D logits");
            // softmax(logits) - target needs a target of the logits' shape; with index labels the
            // reference's Sub cannot broadcast and throws (:1569) -- same here.
            if (t.sizes() != logits.sizes())
                Ctorch_Error::throwException(ErrorPlatform::kAutoDiff, ErrorType::DIMENSION, "CrossEntropy backward: target must have the logits' shape (one-hot); index labels cannot be back-propagated");
            const int64_t rows = rank == 1 ? 1 : static_cast<int64_t>(logits.sizes()[0]);
            const int64_t cols = static_cast<int64_t>(logits.sizes()[rank - 1]);
            Tensor holder;
            const float* g = scalar_arg(node_grad, holder);
            Tensor d(ShapeTag{}, logits.sizes(), logits.dtype(), logits.device(), false);
            cuda_check(ctk_ce_backward_f32(logits.data<float>(), t.data<float>(), g, d.data<float>(), rows, cols, st), "cross entropy backward");
            return d;
        }
        case op::MatMul: {
            Node* other = other_of();
            if (!other) {
                Tensor z(ShapeTag{}, in_shape, node_grad.dtype(), input_node.tensor->device(), true);
                return z;
            }
            Tensor& other_tensor = *other->tensor;
            const bool first = (input_id == node->input_ids[0]);
            if (node_grad.sizes().empty()) {
                return other_tensor.t() * node_grad.item<float>();
            }
            if (node_grad.sizes().size() != 2)
                Ctorch_Error::throwException(ErrorPlatform::kAutoDiff, ErrorType::DIMENSION, "MatMul gradient must be a 2-D tensor or a scalar");
            // dA = g . B^T ; dB = A^T . g -- the transposes are stride-swapped views, the kernel reads them in place.
            if (first) {
                // the operand is a ReLU's output that only this product reads: its gradient goes through
                // the ReLU's rule next and nowhere else, so the product applies that rule itself
                auto cons = consumers.find(input_id);
                if (fuse_relu_backward && input_node.operation == op::ReLU && !input_node.is_leaf && cons != consumers.end() &&
                    cons->second == 1 && (!input_node.grad || input_node.grad_is_zero) && node_grad.device() == DeviceType::kCUDA &&
                    input_node.tensor->device() == DeviceType::kCUDA && input_node.tensor->sizes() == in_shape && input_node.tensor->is_contiguous()) {
                    input_node.grad_premasked = true;
                    return node_grad.matmul_masked(other_tensor.t(), *input_node.tensor);
                }
                return node_grad.matmul(other_tensor.t());
            }
            return other_tensor.t().matmul(node_grad);
        }
        default:
            skip = true;
            return Tensor();
    }
}

void AutoDiff::backward(Tensor& root, Tensor grad_output) {
    AutoDiffContext::Guard guard(nullptr);
    if (root.id() == 0) Ctorch_Error::throwException(ErrorPlatform::kAutoDiff, ErrorType::TENSOR_STATE, "backward: invalid root tensor (id 0)");
    std::lock_guard<std::mutex> lock(records_mutex);
    auto rit = id_to_node.find(root.id());
    if (rit == id_to_node.end() || !rit->second) return;
    Node* root_node = rit->second.get();
    if (!root_node->requires_grad) return;
    {
        // The root gradient lives where the root lives (the default Tensor(1.0f) is a host tensor).
        Tensor g0 = check_and_adjust_grad_shape(grad_output, root.sizes(), root.device());
        root_node->grad = std::make_unique<Tensor>(g0.device() == root.device() ? g0 : g0.to(root.device()));
        root_node->grad_is_zero = false;
    }

    std::unordered_set<Node*> visited;
    std::vector<Node*> order;
    dfs_topological_sort(root_node, visited, order);
    std::reverse(order.begin(), order.end());
    consumers.clear();
    for (Node* node : order) {
        node->grad_premasked = false;
        for (size_t input_id : node->input_ids) ++consumers[input_id];
    }

    // A leaf's gradient is handed to on_leaf_grad once, after the LAST contribution of this pass: a
    // leaf that enters several nodes (a shared weight, a bias used twice) is still being added to until
    // every edge that ends in it has been walked.  `remaining` counts those edges down; the order is
    // topological, so by the time a node is visited all of its own consumers have been.
    std::unordered_map<size_t, int> remaining = consumers;
    std::unordered_set<size_t> contributed;
    auto edge_done = [&](size_t input_id) {
        auto r = remaining.find(input_id);
        if (r == remaining.end() || --r->second > 0) return;
        if (!on_leaf_grad || !contributed.count(input_id)) return;
        auto it = id_to_node.find(input_id);
        if (it != id_to_node.end() && it->second && it->second->is_leaf && it->second->grad) on_leaf_grad(input_id, *it->second->grad);
    };

    for (Node* node : order) {
        if (!node->requires_grad || !node->grad) {
            for (size_t input_id : node->input_ids) edge_done(input_id);
            continue;
        }
        node->materialize_grad();  // an upstream gradient that was only flagged zero is read as zeros
        // The reference visits the inputs in recorded order (:1189).  The contributions of one node do
        // not depend on one another, so a product's second operand -- the weights, a leaf whose
        // gradient a data-parallel driver starts reducing the moment it exists -- goes first: its
        // all-reduce then overlaps the product for the first operand as well.
        std::vector<size_t> visit(node->input_ids);
        if (node->operation == op::MatMul && visit.size() == 2 && visit[0] != visit[1]) std::swap(visit[0], visit[1]);
        for (size_t input_id : visit) {
            auto in_it = id_to_node.find(input_id);
            if (in_it == id_to_node.end() || !in_it->second || !in_it->second->requires_grad) {
                edge_done(input_id);
                continue;
            }
            Node& input_node = *in_it->second;
            // The contribution, alone in its scope so that no temporary still shares its buffer when
            // it becomes the gradient (a hook that reduces the gradient in place would otherwise
            // have to detach it with a full copy).
            std::unique_ptr<Tensor> contribution;
            {
                bool skip = false;
                Tensor val = rule(node, input_id, input_node, skip);
                if (skip) {
                    edge_done(input_id);
                    continue;
                }
                Tensor adjusted = check_and_adjust_grad_shape(val, input_node.tensor->sizes(), input_node.tensor->device());
                if (adjusted.device() != input_node.tensor->device()) adjusted = adjusted.to(input_node.tensor->device());
                contribution = std::make_unique<Tensor>(std::move(adjusted));
            }
            if (!input_node.grad || input_node.grad_is_zero) {
                // First contribution to a gradient that does not exist yet or was zeroed: the
                // reference allocates / keeps zeros and adds (:1202-1208, :1868-1907); 0 + x is x, so
                // the value is adopted as is and a zero-fill + read-modify-write pass is saved.
                input_node.grad = std::move(contribution);
                input_node.grad_is_zero = false;
            } else if (input_node.grad->device() == DeviceType::kCUDA) {
                Tensor& acc = *input_node.grad;
                const Tensor& add = *contribution;
                cuda_check(ctk_accumulate_f32(acc.data<float>(), add.data<float>(), static_cast<int64_t>(acc.numel()), current_stream()), "gradient accumulate");
            } else {
                // host gradients only exist for host 0-D operands (Tensor(float) inputs)
                Tensor& acc = *input_node.grad;
                const Tensor& add = *contribution;
                float* gp = acc.data<float>();
                const float* ap = add.data<float>();
                for (size_t i = 0; i < acc.numel(); ++i) gp[i] += ap[i];
            }
            contributed.insert(input_id);
            edge_done(input_id);
        }
    }
}

Tensor create_empty_tensor() { return Tensor(ShapeTag{}, std::vector<size_t>{}, DType::kFloat, DeviceType::kCPU); }

}  // namespace ctorch
