// C ABI over the C++ front end (Tensor / AutoDiff / Ctorch_Scheduler on DeviceType::kCUDA), so that
// a host written in another language -- here the Python tests and the benchmark -- can drive exactly
// the path user C++ code takes: op wrappers -> scheduler dispatch -> `*_CUDA_kernel` -> kernels,
// with the tape recording and back-propagating on the device.
//
// Also holds MlpTrainer: the training step of the reference's mnist/mnist.cpp:44-92 written against
// this front end for any layer list, with an optional NCCL gradient all-reduce that overlaps
// backward (data-parallel replicas; the reference is single-process).
#include <cstring>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include <cstdio>

#include "AutoDiff.h"
#include "Ctorch_Error.h"
#include "Ctorch_Scheduler.h"
#include "Tensor.h"
#include "mnist_loader.h"
#include "ctorch_b200.h"
#include "ctorch_b200_frontend.h"

using namespace ctorch;

namespace {

thread_local std::string t_err;

template <typename F>
int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const std::exception& e) {
        t_err = e.what();
        return 1;
    } catch (...) {
        t_err = "unknown exception";
        return 1;
    }
}

Tensor* T(void* h) { return static_cast<Tensor*>(h); }

std::unordered_map<AutoDiff*, std::shared_ptr<std::unordered_map<size_t, uint64_t>>>& g_leaf_counts() {
    static std::unordered_map<AutoDiff*, std::shared_ptr<std::unordered_map<size_t, uint64_t>>> m;
    return m;
}

// ---------------------------------------------------------------------------------------------------
// MlpTrainer: x -> (matmul W + b -> relu)* -> matmul W + b -> cross_entropy(one-hot) -> backward -> SGD
// ---------------------------------------------------------------------------------------------------
class MlpTrainer {
public:
    std::vector<int64_t> dims;
    std::vector<Tensor> W, b;
    AutoDiff ctx;
    float lr;
    void* comm = nullptr;         // ctk communicator (not owned)
    void* comm_stream = nullptr;  // non-blocking stream for the gradient all-reduce
    void* ev_grad = nullptr;      // compute -> comm: "this gradient is final"
    void* ev_comm = nullptr;      // comm -> compute: "all gradients are reduced"
    std::vector<void*> ev_param;  // comm -> compute, per parameter (W0, b0, W1, b1, ...): "this gradient is reduced"
    std::vector<int> reduced_order;  // parameters in the order their all-reduces were issued this step
    // How the gradients cross the ranks (cth_mlp_set_dp_mode):
    //   DP_INPLACE  each gradient is all-reduced where backward left it, the moment it is complete;
    //   DP_ARENA    gradients are copied into one buffer registered with the communicator (so NCCL can
    //               reduce in the switch straight out of it with few CTAs) and all-reduced there, one
    //               call per layer (weights and bias together), under backward;
    //   DP_SERIAL   the same buffer, ONE all-reduce after backward: nothing shares the SMs with the
    //               products, the exchange is fully exposed;
    //   DP_SHARDED  reduce-scatter per parameter under backward, SGD on the shard this rank owns,
    //               all-gather of the updated weights (parameters whose size is not a multiple of
    //               4 * world -- the 10-class bias -- stay on the all-reduce path).
    enum DpMode { DP_INPLACE = 0, DP_ARENA = 1, DP_SERIAL = 2, DP_SHARDED = 3 };
    int dp_mode = DP_INPLACE;
    int comm_world = 1, comm_rank = 0;
    float* arena = nullptr;             // registered gradient buffer (modes 1-3), slots in parameter order
    std::vector<int64_t> slot_off;      // per parameter (W0, b0, W1, ...): offset of its slot in floats
    std::vector<int64_t> slot_len;      // ... and the slot's padded length (a multiple of 4 * world)
    std::vector<void*> ev_upd, ev_ag;   // sharded: shard updated (compute -> comm), weights gathered (comm -> compute)
    std::vector<char> in_arena;         // this step: the parameter's gradient has been copied to its slot
    void* ev_done = nullptr;            // compute: end of the step
    void* ev_loss = nullptr;            // compute: the step's loss has reached the page-locked slot (what a step waits for)
    int comm_timeout_ms = 30000;        // a step that has not completed by then has lost a peer
    bool comm_failed = false;
    void* pinned_loss = nullptr;  // page-locked slot the loss is copied into
    void* pinned_x = nullptr;     // page-locked staging for host inputs
    size_t pinned_x_bytes = 0;
    Tensor last_logits;
    bool keep_logits = false;
    bool fresh_weights = false;  // corrected mode: backward reads the updated weights
    // Deferred losses: a step does not wait for the device.  Its loss is still copied to page-locked
    // memory by the step itself (slot steps_done % kLossSlots); the host reads the slots in sync_losses().
    bool deferred_loss = false;
    static constexpr int kLossSlots = 16;
    uint64_t steps_done = 0;
    uint64_t deferred_since = 0;
    // Input staging: up to two uploaded batches wait on the device, each with an event that says
    // its copy has landed, so the upload of batch k+1 (on its own stream) overlaps step k.
    struct Staged {
        Tensor x, labels;
        void* ready = nullptr;     // copy stream: the upload has landed
        void* consumed = nullptr;  // compute stream: the step that read this batch is done with it
        int64_t batch = -1;
    };
    Staged staged[2];
    uint64_t n_staged = 0, n_consumed = 0;
    void* copy_stream = nullptr;

    MlpTrainer(int n_layers, const int64_t* d, const float* params, float lr_) : dims(d, d + n_layers + 1), lr(lr_) {
        // hidden activations are read by the next layer's product only, and nobody asks for their
        // gradients: their ReLU's backward rule runs in the epilogue of the product g.W^T
        const char* frb = std::getenv("CTORCH_FUSE_RELU_BACKWARD");
        ctx.set_fuse_relu_backward(!(frb && frb[0] == '0'));
        const float* p = params;
        for (int l = 0; l < n_layers; ++l) {
            const size_t in = static_cast<size_t>(dims[l]), out = static_cast<size_t>(dims[l + 1]);
            Tensor w(ShapeTag{}, {in, out}, DType::kFloat, DeviceType::kCUDA, false);
            w.copy_from_host(p, in * out);
            p += in * out;
            Tensor bias(ShapeTag{}, {out}, DType::kFloat, DeviceType::kCUDA, false);
            bias.copy_from_host(p, out);
            p += out;
            W.push_back(std::move(w));
            b.push_back(std::move(bias));
        }
        cuda_check(ctk_malloc_host(&pinned_loss, 64), "pinned loss slot");
    }

    ~MlpTrainer() {
        finish_exchange();
        ctk_device_sync();
        release_graph();
        if (graph.stream) ctk_stream_destroy(graph.stream);
        if (comm_stream) ctk_stream_destroy(comm_stream);
        if (ev_grad) ctk_event_destroy(ev_grad);
        if (ev_comm) ctk_event_destroy(ev_comm);
        for (auto* v : {&ev_param, &ev_upd, &ev_ag})
            for (void* e : *v)
                if (e) ctk_event_destroy(e);
        if (ev_done) ctk_event_destroy(ev_done);
        if (ev_loss) ctk_event_destroy(ev_loss);
        if (arena && comm) ctk_comm_free(comm, arena);
        if (pinned_loss) ctk_free_host(pinned_loss);
        if (pinned_x) ctk_free_host(pinned_x);
        for (Staged& s : staged) {
            if (s.ready) ctk_event_destroy(s.ready);
            if (s.consumed) ctk_event_destroy(s.consumed);
        }
        if (copy_stream) ctk_stream_destroy(copy_stream);
    }

    // Opt-in departure from the reference's arithmetic (no counterpart there): bias gradients summed over
    // the batch instead of taken from row 0, and backward products against the current weights instead
    // of the copy the tape took at registration.  Switching fresh_weights on forgets the tape, so that the
    // next step registers the parameters again and their copies share the live buffers from then on.
    void set_corrected(bool exact_bias_grad, bool fresh) {
        release_graph();
        ctx.set_exact_broadcast_grad(exact_bias_grad);
        if (fresh != fresh_weights) {
            cuda_check(ctk_device_sync(), "set_corrected sync");
            ctx.clear_graph();
            fresh_weights = fresh;
        }
    }

    int64_t n_params() const {
        int64_t n = 0;
        for (size_t l = 0; l + 1 < dims.size(); ++l) n += dims[l] * dims[l + 1] + dims[l + 1];
        return n;
    }

    Tensor& param(int p) { return p % 2 ? b[p / 2] : W[p / 2]; }
    int param_index(size_t id) const {
        for (size_t l = 0; l < W.size(); ++l) {
            if (id == W[l].id()) return static_cast<int>(2 * l);
            if (id == b[l].id()) return static_cast<int>(2 * l + 1);
        }
        return -1;
    }
    bool sharded_param(int p) { return dp_mode == DP_SHARDED && static_cast<int64_t>(param(p).numel()) % (4 * comm_world) == 0; }
    void* event_in(std::vector<void*>& v, int p) {
        if (v.size() < 2 * W.size()) v.resize(2 * W.size(), nullptr);
        if (!v[p]) cuda_check(ctk_event_create(&v[p]), "event");
        return v[p];
    }

    void set_dp_mode(int mode) {
        if (mode < DP_INPLACE || mode > DP_SHARDED) throw std::runtime_error("cth_mlp_set_dp_mode: 0 in place, 1 registered buffer, 2 one all-reduce after backward, 3 sharded update");
        if (comm) throw std::runtime_error("cth_mlp_set_dp_mode: choose the mode before cth_mlp_set_comm");
        dp_mode = mode;
    }

    // Waits, bounded, for the last step's exchange (a step itself returns at its loss): a peer that dropped
    // out of it is found here instead of in a device synchronisation that would never return.
    void finish_exchange() {
        if (!comm || comm_failed || !ev_done || steps_done == 0) return;
        if (ctk_comm_wait(comm, ev_done, comm_timeout_ms)) comm_failed = true;   // (the communicator has been aborted: its kernels end)
    }

    void set_comm(void* c) {
        if (!c && comm) {
            finish_exchange();
            cuda_check(ctk_device_sync(), "set_comm sync");
            if (arena) { ctk_comm_free(comm, arena); arena = nullptr; }
        }
        comm = c;
        comm_failed = false;
        if (c && !comm_stream) {
            // Highest priority: the MatMul kernels are persistent and hold every SM until they end, so
            // an all-reduce gets SMs only at a product's boundary -- and only if its blocks are placed
            // before the next product's (CTORCH_COMM_PRIORITY=0: default priority).
            const char* cp = std::getenv("CTORCH_COMM_PRIORITY");
            cuda_check(ctk_stream_create_priority(&comm_stream, 1, (cp && cp[0] == '0') ? 0 : 1), "comm stream");
            cuda_check(ctk_event_create(&ev_grad), "event");
            cuda_check(ctk_event_create(&ev_comm), "event");
        }
        if (c && !ev_done) cuda_check(ctk_event_create(&ev_done), "event");
        if (!c) {
            ctx.on_leaf_grad = nullptr;
            return;
        }
        cuda_check(ctk_comm_info(c, &comm_world, &comm_rank, nullptr), "communicator info");
        if (dp_mode != DP_INPLACE) {
            // one slot per parameter, in parameter order, each padded to a multiple of 4 * world floats so
            // that every rank's shard of it starts on a 16-byte boundary
            slot_off.assign(2 * W.size(), 0);
            slot_len.assign(2 * W.size(), 0);
            int64_t total = 0;
            const int64_t q = 4 * static_cast<int64_t>(comm_world);
            for (size_t p = 0; p < 2 * W.size(); ++p) {
                slot_off[p] = total;
                slot_len[p] = (static_cast<int64_t>(param(static_cast<int>(p)).numel()) + q - 1) / q * q;
                total += slot_len[p];
            }
            void* buf = nullptr;
            const char* sym = std::getenv("CTORCH_DP_SYMMETRIC");
            cuda_check(ctk_comm_alloc(c, static_cast<size_t>(total) * sizeof(float), (sym && sym[0] == '1') ? 1 : 0, &buf), "gradient buffer");
            arena = static_cast<float*>(buf);
            cuda_check(ctk_memset(arena, 0, static_cast<size_t>(total) * sizeof(float), nullptr), "gradient buffer clear");  // the pads stay zero for good
            cuda_check(ctk_device_sync(), "gradient buffer clear");
        }
        ctx.on_leaf_grad = [this](size_t id, Tensor& g) {
            // The gradient of this leaf is complete: exchange it on the communication stream while
            // backward carries on.
            const int p = param_index(id);
            if (p < 0) return;
            void* compute = current_stream();
            cuda_check(ctk_event_record(ev_grad, compute), "record");
            cuda_check(ctk_stream_wait_event(comm_stream, ev_grad), "wait");
            const Tensor& gc = g;
            const int64_t n = static_cast<int64_t>(g.numel());
            if (dp_mode == DP_INPLACE) {
                cuda_check(ctk_allreduce_sum_f32(comm, g.data<float>(), n, comm_stream), "gradient all-reduce");
            } else {
                float* slot = arena + slot_off[p];
                cuda_check(ctk_memcpy_d2d(slot, gc.data<float>(), static_cast<size_t>(n) * sizeof(float), comm_stream), "gradient copy");
                in_arena[p] = 1;
                if (dp_mode == DP_SERIAL) return;  // one all-reduce of the whole buffer after backward
                if (sharded_param(p)) {
                    const int64_t chunk = slot_len[p] / comm_world;
                    cuda_check(ctk_reduce_scatter_sum_f32(comm, slot, slot + comm_rank * chunk, chunk, comm_stream), "gradient reduce-scatter");
                } else if (dp_mode == DP_ARENA && p % 2 == 0 && in_arena[p + 1]) {
                    // the layer's bias (visited just before its weights) sits in the next slot: one call for both
                    cuda_check(ctk_allreduce_sum_f32(comm, slot, slot_len[p] + slot_len[p + 1], comm_stream), "gradient all-reduce");
                    cuda_check(ctk_event_record(event_in(ev_param, p + 1), comm_stream), "record");
                    reduced_order.push_back(p + 1);
                } else if (dp_mode == DP_ARENA && p % 2 == 1) {
                    return;  // a bias: travels with its layer's weights (or, failing that, after backward)
                } else {
                    cuda_check(ctk_allreduce_sum_f32(comm, slot, slot_len[p], comm_stream), "gradient all-reduce");
                }
            }
            // an event of its own: this parameter's update waits for its own exchange only, so the
            // updates of the other layers run under the last exchange
            cuda_check(ctk_event_record(event_in(ev_param, p), comm_stream), "record");
            reduced_order.push_back(p);
        };
    }

    Tensor forward(const Tensor& x) {
        Tensor h = x;
        const size_t L = W.size();
        // (h.matmul(W) + b).relu() of the reference step; linear() runs the three as one kernel where it
        // can and records the same three tape nodes
        for (size_t l = 0; l < L; ++l) h = h.linear(W[l], b[l], l + 1 < L);
        return h;
    }

    // One training step on device-resident inputs; returns the loss read back from the device.
    // Live device memory of one step, estimated generously: per layer the product, the biased sum,
    // the activation and their three gradients, [batch, width] each, plus parameters, gradients and the
    // tape's snapshot.  The pool is grown to that once, before the first step of a batch size.
    int64_t reserved_batch = -1;
    void reserve_for(int64_t batch) {
        if (batch == reserved_batch) return;
        reserved_batch = batch;
        size_t widths = 0;
        for (int64_t d : dims) widths += static_cast<size_t>(d);
        const size_t bytes = static_cast<size_t>(batch) * widths * sizeof(float) * 8 + static_cast<size_t>(n_params()) * sizeof(float) * 4;
        cuda_check(ctk_pool_reserve(bytes), "pool reservation");
    }

    // capturing: the step is being recorded into a graph -- nothing may wait on the device, and the
    // loss is read by whoever launches the graph.
    float step(const Tensor& x, const Tensor& y_one_hot, bool capturing = false) {
        AutoDiffContext::Guard guard(&ctx);
        void* st = current_stream();
        if (!capturing) {
            if (graph.exec && st != graph.stream) release_graph();  // an eager step changes what the graph's buffers hold
            reserve_for(static_cast<int64_t>(x.sizes()[0]));
        }
        if (comm_failed) throw std::runtime_error("the communicator of this trainer was aborted after a peer failed to take part; detach it (cth_mlp_set_comm(NULL)) or attach a new one");
        in_arena.assign(2 * W.size(), 0);
        for (size_t l = 0; l < W.size(); ++l) {
            ctx.make_leaf(W[l], true);
            ctx.make_leaf(b[l], true);
        }
        for (size_t l = 0; l < W.size(); ++l) {
            W[l].requires_grad(true);
            b[l].requires_grad(true);
        }
        for (size_t l = 0; l < W.size(); ++l) {
            ctx.zero_grad(W[l]);
            ctx.zero_grad(b[l]);
        }
        Tensor logits = forward(x);
        Tensor loss = logits.cross_entropy(y_one_hot);
        // loss.item() of the reference step, without stalling the GPU between forward and backward:
        // the value is copied to a page-locked slot now and read once the step has been issued.
        {
            const Tensor& loss_value = loss;  // read-only access: the tape shares this buffer, a writable pointer would copy it
            float* slot = static_cast<float*>(pinned_loss) + (deferred_loss ? steps_done % kLossSlots : 0);
            cuda_check(ctk_memcpy_d2h(slot, loss_value.data<float>(), sizeof(float), st), "loss read-back");
            if (!capturing) {
                if (!ev_loss) cuda_check(ctk_event_create(&ev_loss), "event");
                cuda_check(ctk_event_record(ev_loss, st), "record");
            }
        }
        backward(loss);
        auto update = [&](int p) {
            Tensor& t = param(p);
            if (comm && dp_mode != DP_INPLACE && in_arena[p]) {
                float* slot = arena + slot_off[p];
                if (sharded_param(p)) {
                    // SGD on the shard this rank owns (the same single fused multiply-add per element), then
                    // every rank's shard travels to everyone.  The weights' kept split is dropped by the
                    // write access; the next product that reads them makes it again.
                    const int64_t chunk = slot_len[p] / comm_world, first = comm_rank * chunk;
                    float* w = t.data<float>();
                    cuda_check(ctk_sgd_update_f32(w + first, slot + first, lr, chunk, st), "sharded update");
                    cuda_check(ctk_event_record(event_in(ev_upd, p), st), "record");
                    cuda_check(ctk_stream_wait_event(comm_stream, ev_upd[p]), "wait");
                    cuda_check(ctk_allgather_f32(comm, w + first, w, chunk, comm_stream), "weight all-gather");
                    cuda_check(ctk_event_record(event_in(ev_ag, p), comm_stream), "record");
                    return;
                }
                t.sgd_update_from_(slot, lr);
                return;
            }
            if (fresh_weights) t.sgd_update_shared_(grad(t), lr);
            else t.sgd_update_(grad(t), lr);
        };
        std::vector<char> updated(2 * W.size(), 0);
        if (comm) {
            if (dp_mode == DP_SERIAL) {
                // everything backward produced is in the buffer: one all-reduce, then the updates
                cuda_check(ctk_event_record(ev_grad, st), "record");
                cuda_check(ctk_stream_wait_event(comm_stream, ev_grad), "wait");
                cuda_check(ctk_allreduce_sum_f32(comm, arena, slot_off.back() + slot_len.back(), comm_stream), "gradient all-reduce");
                cuda_check(ctk_event_record(ev_comm, comm_stream), "record");
                cuda_check(ctk_stream_wait_event(st, ev_comm), "wait");
            } else {
                // a gradient that is in the buffer but was not exchanged under backward (a bias whose
                // weights produced no gradient) goes now
                for (int p = 0; dp_mode == DP_ARENA && p < static_cast<int>(2 * W.size()); ++p) {
                    bool sent = false;
                    for (int q : reduced_order) sent = sent || q == p;
                    if (!in_arena[p] || sent) continue;
                    cuda_check(ctk_event_record(ev_grad, st), "record");
                    cuda_check(ctk_stream_wait_event(comm_stream, ev_grad), "wait");
                    cuda_check(ctk_allreduce_sum_f32(comm, arena + slot_off[p], slot_len[p], comm_stream), "gradient all-reduce");
                    cuda_check(ctk_event_record(event_in(ev_param, p), comm_stream), "record");
                    reduced_order.push_back(p);
                }
                // in the order the exchanges were issued, each update behind its own
                for (int p : reduced_order) {
                    if (updated[p]) continue;
                    cuda_check(ctk_stream_wait_event(st, ev_param[p]), "wait");
                    update(p);
                    updated[p] = 1;
                }
            }
            reduced_order.clear();
        }
        for (int p = 0; p < static_cast<int>(2 * W.size()); ++p)
            if (!updated[p]) update(p);
        if (comm) {
            // the step ends when the communication stream has nothing left (sharded: the gathered weights)
            cuda_check(ctk_event_record(ev_comm, comm_stream), "record");
            cuda_check(ctk_stream_wait_event(st, ev_comm), "wait");
        }
        if (keep_logits) last_logits = logits;
        // A step returns its loss -- which the forward pass has produced -- not the end of its backward pass
        // and updates: those stay queued on the stream, the next step's kernels line up behind them, and the
        // GPU never waits for the host between two steps.  Whatever reads the trainer's state afterwards is
        // ordered on the same stream.  The host is never more than one step ahead: the next loss needs this
        // step's updates.
        const bool wait = !capturing && !deferred_loss;
        if (wait && comm) {
            // Bounded: a peer that died or never joined leaves a collective spinning on the GPU -- the one of
            // the step BEFORE this one keeps this step's forward pass, hence its loss, from ever arriving; the
            // wait polls the loss event and the communicator's health and gives up at the deadline (the
            // communicator is aborted, which ends its kernels; the context stays usable).  ev_done marks the
            // end of this step for finish().
            cuda_check(ctk_event_record(ev_done, st), "record");
            const int rc = ctk_comm_wait(comm, ev_loss, comm_timeout_ms);
            if (rc) {
                comm_failed = true;
                ctx.release_step_nodes();
                throw std::runtime_error(std::string("data-parallel step: ") + ctk_last_error());
            }
        } else if (wait) {
            cuda_check(ctk_event_sync(ev_loss), "step: wait for the loss");
        }
        ctx.release_step_nodes();
        ++steps_done;
        return wait ? *static_cast<float*>(pinned_loss) : 0.0f;
    }

    // Waits for every step issued so far and hands out the losses of the last min(cap, 16, steps since
    // the mode was switched on) steps, oldest first.
    int sync_losses(float* out, int cap) {
        void* st = current_stream();
        cuda_check(st ? ctk_stream_sync(st) : ctk_device_sync(), "sync_losses");
        const uint64_t have = steps_done - deferred_since;
        int n = static_cast<int>(have < static_cast<uint64_t>(kLossSlots) ? have : kLossSlots);
        if (n > cap) n = cap;
        for (int i = 0; i < n; ++i) out[i] = static_cast<float*>(pinned_loss)[(steps_done - n + i) % kLossSlots];
        return n;
    }
    void set_deferred_loss(bool on) {
        void* st = current_stream();
        cuda_check(st ? ctk_stream_sync(st) : ctk_device_sync(), "set_deferred_loss");
        release_graph();
        deferred_loss = on;
        deferred_since = steps_done;
    }

    // ---- the step as a CUDA graph -------------------------------------------------------------------
    // For steps that are bound by launch latency (small layers, small batches): the third step of a
    // batch size is recorded -- ~20 kernels, their buffers and tensor maps -- and every later step
    // replays it with one launch.  The first two run eagerly: they set up everything that may not
    // happen during a capture (kernel attributes, scratch, the caches' buffers).  Inputs enter through two
    // fixed device tensors.  The recorded kernels have their buffers' addresses baked in, so those
    // buffers stay pinned to the graph in the caches until the graph is released (a different batch
    // size, an eager step, the trainer's end).  Not available with a communicator.
    struct GraphStep {
        void* exec = nullptr;
        void* stream = nullptr;
        Tensor x, labels;
        int64_t batch = -1;
        int warm_steps = 0;
        int kernels = 0;
        bool first_launch = false;
    } graph;
    // The caches keep one set of graph-pinned buffers per process: one trainer at a time owns it.
    static MlpTrainer*& graph_owner() {
        static MlpTrainer* owner = nullptr;
        return owner;
    }

    void release_graph() {
        if (!graph.exec) return;
        ctk_device_sync();
        ctk_graph_destroy(graph.exec);
        graph.exec = nullptr;
        graph.warm_steps = 0;
        DeviceBlockCache::instance().release_graph();
        SplitBufferCache::instance().release_graph();
        if (graph_owner() == this) graph_owner() = nullptr;
    }

    // Uploads (or copies, for device sources) one batch into the graph's input tensors.
    void graph_inputs(const float* x_src, const float* labels_src, int64_t batch, bool src_on_device) {
        const size_t in = static_cast<size_t>(dims.front());
        if (graph.batch != batch) {
            release_graph();
            graph.x = Tensor(ShapeTag{}, {static_cast<size_t>(batch), in}, DType::kFloat, DeviceType::kCUDA, false);
            graph.labels = Tensor(ShapeTag{}, {static_cast<size_t>(batch)}, DType::kFloat, DeviceType::kCUDA, false);
            graph.batch = batch;
            graph.warm_steps = 0;
            cuda_check(ctk_device_sync(), "graph input allocation");
        }
        const size_t xb = static_cast<size_t>(batch) * in * sizeof(float), lb = static_cast<size_t>(batch) * sizeof(float);
        if (src_on_device) {
            cuda_check(ctk_memcpy_d2d(graph.x.data<float>(), x_src, xb, graph.stream), "batch copy");
            cuda_check(ctk_memcpy_d2d(graph.labels.data<float>(), labels_src, lb, graph.stream), "label copy");
            return;
        }
        int px = 0, pl = 0;
        ctk_host_is_pinned(x_src, &px);
        ctk_host_is_pinned(labels_src, &pl);
        if (px) cuda_check(ctk_memcpy_h2d(graph.x.data<float>(), x_src, xb, graph.stream), "input upload");
        else graph.x.copy_from_host(x_src, static_cast<size_t>(batch) * in);
        if (pl) cuda_check(ctk_memcpy_h2d(graph.labels.data<float>(), labels_src, lb, graph.stream), "label upload");
        else graph.labels.copy_from_host(labels_src, static_cast<size_t>(batch));
    }

    // One step on the batch that graph_inputs put in place: eager (first), capture + launch (second),
    // launch (from then on).
    float graph_step() {
        const size_t classes = static_cast<size_t>(dims.back());
        auto eager = [&](bool capturing) {
            Tensor y(ShapeTag{}, {static_cast<size_t>(graph.batch), classes}, DType::kFloat, DeviceType::kCUDA, false);
            const Tensor& labels = graph.labels;
            cuda_check(ctk_onehot_f32(labels.data<float>(), graph.batch, static_cast<int64_t>(classes), y.data<float>(), graph.stream), "one-hot");
            return step(graph.x, y, capturing);
        };
        // two eager steps first: the very first step of a trainer allocates things no later step does
        // (gradient buffers, the split of the weight snapshot), so only from the second step on does a
        // step take from the caches exactly what the previous one gave back
        if (!graph.exec && graph.warm_steps < 2) {
            ++graph.warm_steps;
            return eager(false);
        }
        if (!graph.exec) {
            if (graph_owner() && graph_owner() != this)
                throw std::runtime_error("cth_mlp_step_graph_*: another trainer of this process holds a recorded step; destroy it or run an eager step on it first");
            graph_owner() = this;
            const uint64_t launches0 = ctk_launch_count();
            DeviceBlockCache::instance().begin_capture();
            SplitBufferCache::instance().begin_capture();
            int rc = ctk_stream_begin_capture(graph.stream);
            bool threw = false;
            std::string what;
            if (!rc) {
                try {
                    eager(true);
                } catch (const std::exception& e) {
                    threw = true;
                    what = e.what();
                }
                void* exec = nullptr;
                rc = ctk_stream_end_capture(graph.stream, &exec);
                graph.exec = exec;
            }
            const bool hit_a = DeviceBlockCache::instance().end_capture();
            const bool hit_b = SplitBufferCache::instance().end_capture();
            graph.kernels = static_cast<int>(ctk_launch_count() - launches0);
            if (rc || threw || !hit_a || !hit_b || !graph.exec) {
                if (graph.exec) { ctk_graph_destroy(graph.exec); graph.exec = nullptr; }
                DeviceBlockCache::instance().release_graph();
                SplitBufferCache::instance().release_graph();
                graph_owner() = nullptr;
                // (the recorded step never ran: this trainer's weights and gradients are no longer defined)
                throw std::runtime_error("the training step could not be captured into a graph: " +
                                         (threw ? what : rc ? std::string(ctk_last_error()) : std::string("a buffer had to be allocated during the capture")));
            }
            graph.first_launch = true;  // its kernels were already counted while they were recorded
        }
        cuda_check(ctk_graph_launch(graph.exec, graph.stream, graph.first_launch ? 0 : graph.kernels), "graph launch");
        graph.first_launch = false;
        cuda_check(ctk_stream_sync(graph.stream), "step sync");
        return *static_cast<float*>(pinned_loss);
    }

    float step_graph(const float* x_src, const float* labels_src, int64_t batch, bool src_on_device) {
        if (comm) throw std::runtime_error("cth_mlp_step_graph_*: not available with a communicator");
        if (!graph.stream) cuda_check(ctk_stream_create_ex(&graph.stream, 0), "graph stream");
        void* saved = current_stream();
        set_current_stream(graph.stream);
        try {
            graph_inputs(x_src, labels_src, batch, src_on_device);
            const float loss = graph_step();
            set_current_stream(saved);
            return loss;
        } catch (...) {
            set_current_stream(saved);
            throw;
        }
    }

    // The same step from HOST inputs: pixels and integer labels (as floats) in caller memory.  The
    // one-hot matrix of mnist/mnist.cpp:67-72 is built on the device from the uploaded labels (same
    // 0/1 values).  Page-locked caller buffers are copied straight from where they are, without
    // blocking; pageable ones go through the staging buffers.
    float step_host(const float* x_host, const float* labels_host, int64_t batch) {
        const size_t in = static_cast<size_t>(dims.front()), classes = static_cast<size_t>(dims.back());
        void* st = current_stream();
        Tensor x(ShapeTag{}, {static_cast<size_t>(batch), in}, DType::kFloat, DeviceType::kCUDA, false);
        Tensor labels(ShapeTag{}, {static_cast<size_t>(batch)}, DType::kFloat, DeviceType::kCUDA, false);
        int px = 0, pl = 0;
        ctk_host_is_pinned(x_host, &px);
        ctk_host_is_pinned(labels_host, &pl);
        if (px) cuda_check(ctk_memcpy_h2d(x.data<float>(), x_host, static_cast<size_t>(batch) * in * sizeof(float), st), "input upload");
        else x.copy_from_host(x_host, static_cast<size_t>(batch) * in);
        if (pl) cuda_check(ctk_memcpy_h2d(labels.data<float>(), labels_host, static_cast<size_t>(batch) * sizeof(float), st), "label upload");
        else labels.copy_from_host(labels_host, static_cast<size_t>(batch));
        Tensor y(ShapeTag{}, {static_cast<size_t>(batch), classes}, DType::kFloat, DeviceType::kCUDA, false);
        cuda_check(ctk_onehot_f32(labels.data<float>(), batch, static_cast<int64_t>(classes), y.data<float>(), st), "one-hot");
        return step(x, y);  // ends with a stream synchronisation: the caller's buffers are free again
    }

    // Starts the upload of one batch (HOST pixels and labels) on the copy stream and returns at once
    // when the buffers are page-locked; the caller keeps them unchanged until the step that consumes
    // the batch has returned.  Pageable buffers are copied through the staging buffers before returning.
    void stage_host(const float* x_host, const float* labels_host, int64_t batch) {
        if (n_staged - n_consumed >= 2) throw std::runtime_error("cth_mlp_stage_host: two batches are already staged; run a step first");
        const size_t in = static_cast<size_t>(dims.front());
        Staged& s = staged[n_staged % 2];
        if (!copy_stream) cuda_check(ctk_stream_create_ex(&copy_stream, 1), "copy stream");
        if (!s.ready) cuda_check(ctk_event_create(&s.ready), "event");
        if (!s.consumed) cuda_check(ctk_event_create(&s.consumed), "event");
        else cuda_check(ctk_stream_wait_event(copy_stream, s.consumed), "wait for the slot's last reader");  // (deferred losses: no host wait did it)
        if (s.batch != batch) {
            s.x = Tensor(ShapeTag{}, {static_cast<size_t>(batch), in}, DType::kFloat, DeviceType::kCUDA, false);
            s.labels = Tensor(ShapeTag{}, {static_cast<size_t>(batch)}, DType::kFloat, DeviceType::kCUDA, false);
            s.batch = batch;
            cuda_check(ctk_device_sync(), "staging allocation");  // the allocation is ordered on another stream than the copies
        }
        int px = 0, pl = 0;
        ctk_host_is_pinned(x_host, &px);
        ctk_host_is_pinned(labels_host, &pl);
        void* saved = current_stream();
        set_current_stream(copy_stream);
        try {
            if (px) cuda_check(ctk_memcpy_h2d(s.x.data<float>(), x_host, static_cast<size_t>(batch) * in * sizeof(float), copy_stream), "input upload");
            else s.x.copy_from_host(x_host, static_cast<size_t>(batch) * in);
            if (pl) cuda_check(ctk_memcpy_h2d(s.labels.data<float>(), labels_host, static_cast<size_t>(batch) * sizeof(float), copy_stream), "label upload");
            else s.labels.copy_from_host(labels_host, static_cast<size_t>(batch));
        } catch (...) {
            set_current_stream(saved);
            throw;
        }
        set_current_stream(saved);
        cuda_check(ctk_event_record(s.ready, copy_stream), "record");
        ++n_staged;
    }

    // The training step on the oldest staged batch.
    float step_staged() {
        if (n_consumed == n_staged) throw std::runtime_error("cth_mlp_step_staged: no batch is staged");
        Staged& s = staged[n_consumed % 2];
        ++n_consumed;
        const size_t classes = static_cast<size_t>(dims.back());
        void* st = current_stream();
        cuda_check(ctk_stream_wait_event(st, s.ready), "wait for the upload");
        Tensor y(ShapeTag{}, {static_cast<size_t>(s.batch), classes}, DType::kFloat, DeviceType::kCUDA, false);
        const Tensor& labels = s.labels;
        cuda_check(ctk_onehot_f32(labels.data<float>(), s.batch, static_cast<int64_t>(classes), y.data<float>(), st), "one-hot");
        const float loss = step(s.x, y);
        cuda_check(ctk_event_record(s.consumed, st), "record");
        return loss;
    }

    // Class probabilities of a batch without recording anything: NeuralNetwork::predict of
    // mnist/mnist.cpp:94-131 (forward, then a row softmax).
    Tensor predict(const Tensor& x) {
        AutoDiffContext::Guard guard(nullptr);
        Tensor logits = forward(x);
        return logits.softmax(1);
    }

    // calculate_accuracy of mnist/mnist.cpp:134-158: per row the first class whose probability exceeds
    // -1 and every earlier one, compared with (int)label; correct / total in float.  Runs on the
    // device; one float comes back.
    float accuracy(const Tensor& x, const Tensor& labels) {
        const Tensor probs = predict(x);
        const int64_t rows = static_cast<int64_t>(probs.sizes()[0]), classes = static_cast<int64_t>(probs.sizes()[1]);
        if (static_cast<int64_t>(labels.numel()) != rows) throw std::runtime_error("accuracy: one label per row expected");
        void* st = current_stream();
        Tensor pred(ShapeTag{}, {static_cast<size_t>(rows)}, DType::kFloat, DeviceType::kCUDA, false);
        Tensor count(ShapeTag{}, std::vector<size_t>{}, DType::kFloat, DeviceType::kCUDA, false);
        cuda_check(ctk_argmax_rows_f32(probs.data<float>(), rows, classes, -1.0f, pred.data<float>(), st), "argmax");
        const Tensor& pred_c = pred;
        cuda_check(ctk_count_matches_f32(pred_c.data<float>(), labels.data<float>(), rows, count.data<float>(), nullptr, st), "count matches");
        const int correct = static_cast<int>(count.item<float>());
        return static_cast<float>(correct) / static_cast<float>(rows);
    }

    // One pass over a device-resident data set in batches of `batch_size` rows, in order, as the
    // epoch loop of mnist/mnist.cpp:246-262 (the remainder that does not fill a batch is skipped, as
    // there).  Batches are views of the data set, not copies.  Returns the mean of the step losses.
    float train_epoch(const Tensor& images, const Tensor& labels, int64_t batch_size, bool use_graph = false) {
        if (batch_size <= 0) throw std::runtime_error("train_epoch: batch size must be positive");
        if (deferred_loss) throw std::runtime_error("train_epoch adds up every step's loss: switch deferred losses off first");
        if (use_graph) {
            const int64_t n = static_cast<int64_t>(images.sizes()[0]);
            const int64_t num_batches = n / batch_size;
            const size_t in = static_cast<size_t>(dims.front());
            float epoch_loss = 0.0f;
            for (int64_t bi = 0; bi < num_batches; ++bi)
                epoch_loss += step_graph(images.data<float>() + static_cast<size_t>(bi * batch_size) * in, labels.data<float>() + bi * batch_size, batch_size, true);
            return num_batches ? epoch_loss / static_cast<float>(num_batches) : 0.0f;
        }
        const int64_t n = static_cast<int64_t>(images.sizes()[0]);
        const int64_t num_batches = n / batch_size;
        const size_t classes = static_cast<size_t>(dims.back());
        float epoch_loss = 0.0f;
        for (int64_t bi = 0; bi < num_batches; ++bi) {
            const Tensor xb = images.narrow_rows(static_cast<size_t>(bi * batch_size), static_cast<size_t>(batch_size));
            const Tensor lb = labels.narrow_rows(static_cast<size_t>(bi * batch_size), static_cast<size_t>(batch_size));
            Tensor y(ShapeTag{}, {static_cast<size_t>(batch_size), classes}, DType::kFloat, DeviceType::kCUDA, false);
            cuda_check(ctk_onehot_f32(lb.data<float>(), batch_size, static_cast<int64_t>(classes), y.data<float>(), current_stream()), "one-hot");
            epoch_loss += step(xb, y);
        }
        return num_batches ? epoch_loss / static_cast<float>(num_batches) : 0.0f;
    }

    void get_params(float* out) {
        finish_exchange();
        for (size_t l = 0; l < W.size(); ++l) {
            W[l].copy_to_host(out, W[l].numel());
            out += W[l].numel();
            b[l].copy_to_host(out, b[l].numel());
            out += b[l].numel();
        }
    }
    // The gradients the last step applied (data parallel: summed over the ranks).  Sharded mode: only
    // this rank's shard of a sharded parameter is the sum; the rest of its slot holds local values.
    void get_grads(float* out) {
        AutoDiffContext::Guard guard(&ctx);
        for (int p = 0; p < static_cast<int>(2 * W.size()); ++p) {
            Tensor& t = param(p);
            if (comm && dp_mode != DP_INPLACE && arena) {
                finish_exchange();
                cuda_check(ctk_device_sync(), "get_grads sync");
                cuda_check(ctk_memcpy_d2h(out, arena + slot_off[p], t.numel() * sizeof(float), nullptr), "gradient read-back");
                cuda_check(ctk_device_sync(), "get_grads sync");
            } else {
                Tensor g = grad(t);
                g.copy_to_host(out, g.numel());
            }
            out += t.numel();
        }
    }
};

}  // namespace

extern "C" {

const char* cth_last_error(void) { return t_err.c_str(); }
void cth_set_quiet(int q) { Ctorch_Error::setQuiet(q != 0); }
uint64_t cth_error_count(void) { return Ctorch_Error::errorCount(); }
int cth_cuda_available(void) { return Ctorch_Scheduler::isDeviceAvailable(DeviceType::kCUDA) ? 1 : 0; }

// Host-only self-test of the buffer caches' keying (needs no GPU): a cache with a fake allocator and a
// fake "current device" must never hand a buffer parked on one device to a request made on another,
// must give a parked buffer back to a request on its own device, and must release overflow with the
// device the buffer came from.  *failed receives the number of checks that did not hold.
int cth_selftest_cache_keying(int* failed) {
    return guarded([&] {
        struct Fake : SizeKeyedCache {
            int dev = 0, made = 0;
            std::vector<std::pair<void*, int>> released;
            size_t rounded(size_t b) const override { return (b + 511) & ~size_t(511); }
            size_t max_parked() const override { return 2048; }
            void* fresh(size_t) override { return reinterpret_cast<void*>(static_cast<uintptr_t>(dev + 1) * 0x10000000u + 0x1000u * static_cast<uintptr_t>(++made)); }
            void release(void* p, int d) override { released.emplace_back(p, d); }
            int current_device() const override { return dev; }
        } c;
        int bad = 0, d = -1;
        c.dev = 0;
        void* p0 = c.get(1000, &d);
        bad += d != 0;
        c.put(p0, 1000, d);
        c.dev = 1;
        void* q = c.get(1000, &d);            // same size, other device: must not be p0
        bad += (q == p0) + (d != 1) + (c.made != 2);
        c.put(q, 1000, d);
        void* q2 = c.get(1000, &d);           // device 1's own buffer comes back
        bad += q2 != q;
        c.dev = 0;
        void* p1 = c.get(1000, &d);           // and device 0's
        bad += (p1 != p0) + (d != 0);
        c.put(p1, 1000, 0);                   // parked: 1024 bytes
        c.put(q2, 1000, 1);                   // parked: 2048 bytes = the limit
        void* extra = c.get(3000, &d);        // another size: a miss
        bad += c.made != 3;
        c.put(extra, 3000, 0);                // over the limit: released, with its device
        bad += !(c.released.size() == 1 && c.released[0].first == extra && c.released[0].second == 0);
        // a captured sequence pins what it touches to the graph; after release_graph it is anyone's (of that device)
        c.begin_capture();
        void* g0 = c.get(1000, &d);
        c.put(g0, 1000, 0);
        void* g1 = c.get(1000, &d);
        bad += (g0 != p0) + (g1 != g0);
        c.put(g1, 1000, 0);
        bad += !c.end_capture();
        c.dev = 1;
        c.begin_capture();
        void* h = c.get(1000, &d);            // device 1 must not see device 0's pinned buffer
        bad += h != q;
        c.put(h, 1000, 1);
        c.end_capture();
        c.release_graph();
        *failed = bad;
    });
}

// ---- tensors ----
int cth_tensor_from_host(const float* data, const int64_t* shape, int rank, int device, void** out) {
    return guarded([&] {
        std::vector<size_t> s(shape, shape + rank);
        auto t = std::make_unique<Tensor>(ShapeTag{}, s, DType::kFloat, static_cast<DeviceType>(device), data == nullptr);
        if (data) t->copy_from_host(data, t->numel());
        *out = t.release();
    });
}
int cth_tensor_scalar(float v, void** out) {
    return guarded([&] { *out = new Tensor(v); });
}
int cth_tensor_free(void* t) {
    return guarded([&] { delete T(t); });
}
int cth_tensor_info(void* t, int64_t* shape_out8, int* rank, int* device, int* requires_grad, uint64_t* id) {
    return guarded([&] {
        const Tensor& x = *T(t);
        if (rank) *rank = x.dim();
        if (shape_out8) for (int i = 0; i < x.dim() && i < 8; ++i) shape_out8[i] = static_cast<int64_t>(x.sizes()[i]);
        if (device) *device = static_cast<int>(x.device());
        if (requires_grad) *requires_grad = x.requires_grad() ? 1 : 0;
        if (id) *id = x.id();
    });
}
int cth_tensor_to_host(void* t, float* out) {
    return guarded([&] { T(t)->copy_to_host(out, T(t)->numel()); });
}
int cth_tensor_item(void* t, float* out) {
    return guarded([&] { *out = T(t)->item<float>(); });
}
int cth_tensor_requires_grad(void* t, int flag) {
    return guarded([&] { T(t)->requires_grad(flag != 0); });
}
int cth_tensor_to_device(void* t, int device, void** out) {
    return guarded([&] { *out = new Tensor(T(t)->to(static_cast<DeviceType>(device))); });
}
int cth_tensor_copy(void* t, void** out) {  // copy constructor: new id, same value
    return guarded([&] { *out = new Tensor(*T(t)); });
}
int cth_tensor_fill(void* t, float v) {
    return guarded([&] { T(t)->fill(v); });
}

// ---- dtype-aware additions: comparisons, to(DType), ones, rand, operator[] ----
int cth_tensor_empty(const int64_t* shape, int rank, int dtype, int device, void** out) {
    return guarded([&] {
        std::vector<size_t> s(shape, shape + rank);
        *out = new Tensor(ShapeTag{}, s, static_cast<DType>(dtype), static_cast<DeviceType>(device), true);
    });
}
int cth_tensor_dtype(void* t, int* dtype) {
    return guarded([&] { *dtype = static_cast<int>(T(t)->dtype()); });
}
int cth_tensor_read_raw(void* t, void* dst, uint64_t nbytes) {
    return guarded([&] { T(t)->copy_raw_to_host(dst, static_cast<size_t>(nbytes)); });
}
int cth_tensor_compare(void* a, void* b_or_null, float scalar, int cmp, int form, void** out) {
    return guarded([&] { *out = new Tensor(T(a)->compare(cmp, form, b_or_null ? T(b_or_null) : nullptr, scalar)); });
}
int cth_tensor_to_dtype(void* t, int dtype, void** out) {
    return guarded([&] { *out = new Tensor(T(t)->to(static_cast<DType>(dtype))); });
}
int cth_tensor_ones(void* t) {
    return guarded([&] { T(t)->ones(); });
}
int cth_tensor_rand(void* t) {
    return guarded([&] { T(t)->rand(); });
}
int cth_manual_seed(uint64_t seed) {
    return guarded([&] { Tensor::manual_seed(seed); });
}
int cth_tensor_index(void* t, uint64_t index, void** out) {
    return guarded([&] { *out = new Tensor((*T(t))[static_cast<size_t>(index)]); });
}

// ---- ops (the reference's Tensor methods / operators) ----
// op codes: values of `enum class op`; Sum = 21, Softmax = 14 (param = dim), Neg = 2.
int cth_unary(void* t, int opc, int param, void** out) {
    return guarded([&] {
        const Tensor& x = *T(t);
        Tensor r;
        switch (static_cast<op>(opc)) {
            case op::Neg: r = -x; break;
            case op::ReLU: r = x.relu(); break;
            case op::Sigmoid: r = x.sigmoid(); break;
            case op::Tanh: r = x.tanh(); break;
            case op::Sin: r = x.sin(); break;
            case op::Cos: r = x.cos(); break;
            case op::Softmax: r = x.softmax(param); break;
            case op::Sum: r = x.sum(); break;
            default: throw std::runtime_error("cth_unary: unsupported op");
        }
        *out = new Tensor(std::move(r));
    });
}
int cth_binary(void* a, void* b, int opc, void** out) {
    return guarded([&] {
        const Tensor &x = *T(a), &y = *T(b);
        Tensor r;
        switch (static_cast<op>(opc)) {
            case op::Add: r = x + y; break;
            case op::Sub: r = x - y; break;
            case op::Mul: r = x * y; break;
            case op::Div: r = x / y; break;
            case op::MatMul: r = x.matmul(y); break;
            case op::Dot: r = x.dot(y); break;
            case op::MSE: r = x.mse_loss(y); break;
            case op::MAE: r = x.mae_loss(y); break;
            case op::CE: r = x.cross_entropy(y); break;
            default: throw std::runtime_error("cth_binary: unsupported op");
        }
        *out = new Tensor(std::move(r));
    });
}
// kind: 0 t*s, 1 t+s, 2 t/s, 3 s-t, 4 s/t, 5 s*t, 6 s+t
int cth_scalar(void* t, float s, int kind, void** out) {
    return guarded([&] {
        const Tensor& x = *T(t);
        Tensor r;
        switch (kind) {
            case 0: r = x * s; break;
            case 1: r = x + s; break;
            case 2: r = x / s; break;
            case 3: r = s - x; break;
            case 4: r = s / x; break;
            case 5: r = s * x; break;
            case 6: r = s + x; break;
            default: throw std::runtime_error("cth_scalar: bad kind");
        }
        *out = new Tensor(std::move(r));
    });
}
int cth_transpose(void* t, void** out) {
    return guarded([&] { *out = new Tensor(T(t)->t()); });
}

// ---- tape ----
int cth_ctx_create(void** out) {
    return guarded([&] { *out = new AutoDiff(); });
}
int cth_ctx_destroy(void* c) {
    return guarded([&] {
        if (AutoDiffContext::current() == c) AutoDiffContext::current() = nullptr;
        g_leaf_counts().erase(static_cast<AutoDiff*>(c));
        delete static_cast<AutoDiff*>(c);
    });
}
int cth_ctx_set_current(void* c) {  // NULL switches recording off
    return guarded([&] { AutoDiffContext::current() = static_cast<AutoDiff*>(c); });
}
int cth_ctx_node_count(void* c, uint64_t* n) {
    return guarded([&] { *n = static_cast<AutoDiff*>(c)->node_count(); });
}
int cth_ctx_clear(void* c) {
    return guarded([&] { static_cast<AutoDiff*>(c)->clear_graph(); });
}
int cth_ctx_release_step_nodes(void* c) {
    return guarded([&] { static_cast<AutoDiff*>(c)->release_step_nodes(); });
}
int cth_ctx_set_fuse_relu_backward(void* c, int on) {
    return guarded([&] { static_cast<AutoDiff*>(c)->set_fuse_relu_backward(on != 0); });
}
// Installs a hook that only counts: how often on_leaf_grad fired, per tensor id (a debugging aid, and
// what the test of "once per leaf, after its last contribution" reads).  on = 0 removes it.
int cth_ctx_count_leaf_grads(void* c, int on) {
    return guarded([&] {
        auto* ctx = static_cast<AutoDiff*>(c);
        if (!on) { ctx->on_leaf_grad = nullptr; return; }
        auto counts = std::make_shared<std::unordered_map<size_t, uint64_t>>();
        g_leaf_counts()[ctx] = counts;
        ctx->on_leaf_grad = [counts](size_t id, Tensor&) { ++(*counts)[id]; };
    });
}
int cth_ctx_leaf_grad_count(void* c, void* t, uint64_t* n) {
    return guarded([&] {
        auto it = g_leaf_counts().find(static_cast<AutoDiff*>(c));
        *n = 0;
        if (it == g_leaf_counts().end()) return;
        auto f = it->second->find(T(t)->id());
        if (f != it->second->end()) *n = f->second;
    });
}
int cth_ctx_make_leaf(void* c, void* t, int requires_grad) {
    return guarded([&] { static_cast<AutoDiff*>(c)->make_leaf(*T(t), requires_grad != 0); });
}
int cth_ctx_zero_grad(void* c, void* t) {
    return guarded([&] { static_cast<AutoDiff*>(c)->zero_grad(*T(t)); });
}
int cth_backward(void* root, void* grad_or_null) {
    return guarded([&] {
        if (grad_or_null) backward(*T(root), *T(grad_or_null));
        else backward(*T(root));
    });
}
int cth_grad(void* t, void** out) {
    return guarded([&] { *out = new Tensor(grad(*T(t))); });
}
int cth_linear(void* x, void* w, void* bias, int relu, void** out) {
    return guarded([&] { *out = new Tensor(T(x)->linear(*T(w), *T(bias), relu != 0)); });
}
int cth_sgd_update(void* p, void* g, float lr) {
    return guarded([&] { T(p)->sgd_update_(*T(g), lr); });
}

// ---- MLP trainer ----
int cth_mlp_create(int n_layers, const int64_t* dims, const float* params, float lr, void** out) {
    return guarded([&] {
        if (n_layers < 1) throw std::runtime_error("cth_mlp_create: need at least one layer");
        *out = new MlpTrainer(n_layers, dims, params, lr);
    });
}
int cth_mlp_destroy(void* m) {
    return guarded([&] { delete static_cast<MlpTrainer*>(m); });
}
int cth_mlp_set_comm(void* m, void* comm) {
    return guarded([&] { static_cast<MlpTrainer*>(m)->set_comm(comm); });
}
int cth_mlp_set_dp_mode(void* m, int mode) {
    return guarded([&] { static_cast<MlpTrainer*>(m)->set_dp_mode(mode); });
}
int cth_mlp_set_comm_timeout_ms(void* m, int timeout_ms) {
    return guarded([&] {
        if (timeout_ms <= 0) throw std::runtime_error("cth_mlp_set_comm_timeout_ms: a positive number of milliseconds");
        static_cast<MlpTrainer*>(m)->comm_timeout_ms = timeout_ms;
    });
}
int cth_mlp_set_corrected(void* m, int exact_bias_grad, int fresh_weights) {
    return guarded([&] { static_cast<MlpTrainer*>(m)->set_corrected(exact_bias_grad != 0, fresh_weights != 0); });
}
int cth_mlp_set_deferred_loss(void* m, int on) {
    return guarded([&] { static_cast<MlpTrainer*>(m)->set_deferred_loss(on != 0); });
}
int cth_mlp_sync_losses(void* m, float* out, int cap, int* n) {
    return guarded([&] { *n = static_cast<MlpTrainer*>(m)->sync_losses(out, cap); });
}
int cth_mlp_keep_logits(void* m, int keep) {
    return guarded([&] { static_cast<MlpTrainer*>(m)->keep_logits = keep != 0; });
}
int cth_mlp_step_host(void* m, const float* x_host, const float* labels_host, int64_t batch, float* loss) {
    return guarded([&] { *loss = static_cast<MlpTrainer*>(m)->step_host(x_host, labels_host, batch); });
}
int cth_mlp_stage_host(void* m, const float* x_host, const float* labels_host, int64_t batch) {
    return guarded([&] { static_cast<MlpTrainer*>(m)->stage_host(x_host, labels_host, batch); });
}
int cth_mlp_step_staged(void* m, float* loss) {
    return guarded([&] { *loss = static_cast<MlpTrainer*>(m)->step_staged(); });
}
int cth_mlp_step_graph_host(void* m, const float* x_host, const float* labels_host, int64_t batch, float* loss) {
    return guarded([&] { *loss = static_cast<MlpTrainer*>(m)->step_graph(x_host, labels_host, batch, false); });
}
int cth_mlp_train_epoch_graph(void* m, void* images, void* labels, int64_t batch_size, float* mean_loss) {
    return guarded([&] { *mean_loss = static_cast<MlpTrainer*>(m)->train_epoch(*T(images), *T(labels), batch_size, true); });
}
int cth_mlp_step_device(void* m, void* x, void* onehot, float* loss) {
    return guarded([&] { *loss = static_cast<MlpTrainer*>(m)->step(*T(x), *T(onehot)); });
}
int cth_mlp_predict(void* m, void* x, void** probs) {
    return guarded([&] { *probs = new Tensor(static_cast<MlpTrainer*>(m)->predict(*T(x))); });
}
int cth_mlp_accuracy(void* m, void* x, void* labels, float* acc) {
    return guarded([&] { *acc = static_cast<MlpTrainer*>(m)->accuracy(*T(x), *T(labels)); });
}
int cth_mlp_train_epoch(void* m, void* images, void* labels, int64_t batch_size, float* mean_loss) {
    return guarded([&] { *mean_loss = static_cast<MlpTrainer*>(m)->train_epoch(*T(images), *T(labels), batch_size); });
}
int cth_mnist_load(const char* dir, const char* image_file, const char* label_file, int device, void** images, void** labels) {
    return guarded([&] {
        MNISTLoader loader(dir, static_cast<DeviceType>(device));
        auto im = std::make_unique<Tensor>();
        auto lb = std::make_unique<Tensor>();
        if (image_file && label_file) loader.load(image_file, label_file, *im, *lb);
        else if (image_file && std::string(image_file) == "test") loader.load_test_data(*im, *lb);
        else loader.load_training_data(*im, *lb);
        *images = im.release();
        *labels = lb.release();
    });
}
int cth_tensor_narrow_rows(void* t, int64_t start, int64_t count, void** out) {
    return guarded([&] {
        if (start < 0 || count < 0) throw std::runtime_error("cth_tensor_narrow_rows: negative range");
        *out = new Tensor(T(t)->narrow_rows(static_cast<size_t>(start), static_cast<size_t>(count)));
    });
}
int cth_mlp_get_params(void* m, float* out) {
    return guarded([&] { static_cast<MlpTrainer*>(m)->get_params(out); });
}
int cth_mlp_get_grads(void* m, float* out) {
    return guarded([&] { static_cast<MlpTrainer*>(m)->get_grads(out); });
}
int cth_mlp_get_logits(void* m, float* out) {
    return guarded([&] {
        auto* t = static_cast<MlpTrainer*>(m);
        t->last_logits.copy_to_host(out, t->last_logits.numel());
    });
}
int cth_mlp_n_params(void* m, int64_t* n) {
    return guarded([&] { *n = static_cast<MlpTrainer*>(m)->n_params(); });
}
int cth_mlp_node_count(void* m, uint64_t* n) {
    return guarded([&] { *n = static_cast<MlpTrainer*>(m)->ctx.node_count(); });
}

}  // extern "C"
