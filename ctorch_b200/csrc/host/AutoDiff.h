// AutoDiff: the tape.  Same interface and graph semantics as the reference's include/AutoDiff.h
// and src/AutoDiff.cpp (thread-local context + RAII Guard :35-66; Node owns a copy of the tensor
// and of its gradient :79-102; deferred record / commit; DFS topological order; per-op rules),
// with gradients and saved tensors resident on the device and every rule a kernel launch.
#pragma once
#include <functional>
#include <memory>
#include <mutex>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "Ctools.h"

namespace ctorch {

class Tensor;
class AutoDiff;

class AutoDiffContext {
public:
    static AutoDiff*& current() {
        static thread_local AutoDiff* ctx = nullptr;
        return ctx;
    }
    class Guard {
    public:
        explicit Guard(AutoDiff* new_ctx) : prev_ctx(current()) { current() = new_ctx; }
        ~Guard() { current() = prev_ctx; }
        Guard(const Guard&) = delete;
        Guard& operator=(const Guard&) = delete;

    private:
        AutoDiff* prev_ctx;
    };
};

class AutoDiff {
    struct Node {
        size_t tensor_id;
        std::unique_ptr<Tensor> tensor;  // value at registration time (shares storage until someone writes)
        std::unique_ptr<Tensor> grad;
        // zero_grad() only raises this flag: the zeros are written when someone reads the gradient
        // before backward has replaced it (backward adopts its first contribution instead of adding
        // it to zeros: 0 + x is x).
        bool grad_is_zero = false;
        // the gradient of this ReLU node already went through the node's own backward rule (in the
        // epilogue of the product that made it): the rule passes it on
        bool grad_premasked = false;
        void materialize_grad();
        std::vector<size_t> input_ids;
        op operation = op::Add;
        int op_param_i = 0;
        bool requires_grad;
        bool is_leaf;
        Node(size_t id, std::unique_ptr<Tensor> t, bool req_grad, bool leaf);
        ~Node();
    };
    struct PendingRecord {
        op operation;
        std::vector<size_t> input_ids;
        int op_param_i = 0;
        bool committed = false;
    };

    std::unordered_map<size_t, std::unique_ptr<Node>> id_to_node;
    std::unordered_map<size_t, PendingRecord> pending_records;
    std::mutex records_mutex;
    bool retain_graph = false;
    bool fuse_relu_backward = false;
    bool exact_broadcast_grad = false;
    std::unordered_map<size_t, int> consumers;  // per tensor id, within the backward pass that is running

    Node* get_node_by_id(size_t id);
    void dfs_topological_sort(Node* node, std::unordered_set<Node*>& visited, std::vector<Node*>& result);
    Tensor check_and_adjust_grad_shape(const Tensor& grad, const std::vector<size_t>& target_shape, DeviceType target_device);
    Tensor rule(Node* node, size_t input_id, Node& input_node, bool& skip);

public:
    AutoDiff();
    ~AutoDiff();

    Tensor get_grad(const Tensor* t);
    void make_leaf(Tensor& t, bool requires_grad);
    void zero_grad(Tensor& t);
    void defer_record(size_t output_id, op operation, const std::vector<Tensor*>& inputs, int op_param_i = 0);
    void commit_record(Tensor& output);
    void update_requires_grad(Tensor& t, bool requires_grad);
    void set_retain_graph(bool retain);
    void backward(Tensor& root);
    void backward(Tensor& root, Tensor grad_output);
    void clear_graph();

    // ---- additions (no counterpart in the reference) ----
    // Called during backward once per leaf, right after that leaf's gradient received its LAST
    // contribution of the pass (a leaf that enters several nodes is complete only then); a data-parallel
    // driver uses it to start that gradient's all-reduce while the rest of backward still runs.
    std::function<void(size_t tensor_id, Tensor& grad)> on_leaf_grad;
    // Drops every node that a future root can no longer reach: all non-leaf nodes and all leaves that
    // do not require grad (each step's inputs and activations, which the reference keeps forever).
    // Leaves that require grad -- the parameters, including the snapshot taken when they were first
    // registered, which backward keeps using -- stay, so results do not change.
    void release_step_nodes();
    // When a ReLU's output enters exactly one MatMul (as its first operand) and nothing else, let the
    // product g.W^T that computes the output's gradient apply the ReLU's backward rule in its epilogue.
    // The gradients of everything upstream are bit for bit the same; what get_grad returns for that
    // ReLU output itself is then the masked gradient (the reference: the unmasked one), which is why
    // this is off unless asked for.
    void set_fuse_relu_backward(bool on) { fuse_relu_backward = on; }
    // The gradient of an operand that was broadcast over leading dimensions ([H] in [N,H] + [H]) is, in
    // the reference, the FIRST row of the upstream gradient (:690-757).  on: the sum over the broadcast
    // rows, which is the derivative.  Off by default: it changes results away from the reference's.
    void set_exact_broadcast_grad(bool on) { exact_broadcast_grad = on; }
    size_t node_count();
    // In-place access to a leaf's gradient buffer (nullptr if none).
    Tensor* grad_buffer(const Tensor& t);
};

Tensor create_empty_tensor();

}  // namespace ctorch
