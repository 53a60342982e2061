/*
 * ctorch_b200_frontend -- C ABI over the C++ front end (Tensor / AutoDiff / Ctorch_Scheduler with
 * DeviceType::kCUDA filled in), for hosts that are not C++.
 *
 * Every call goes through the same path as user C++ code written against the reference's API:
 * Tensor op wrapper (src/Tensor.cpp:482-497 and its 15 siblings) -> Ctorch_Scheduler::dispatch
 * (include/Ctorch_Scheduler.h:86-166) -> `*_CUDA_kernel` (src/kernels/kernels.h:42-242) -> the
 * kernels of ctorch_b200.h, recording on the current AutoDiff tape (include/AutoDiff.h:156-219).
 *
 * Handles are opaque pointers (tensor: a heap-allocated Tensor; ctx: an AutoDiff; mlp: a trainer).
 * Every function returns 0 on success, 1 if the front end threw; cth_last_error() has the message.
 * Operator codes are the numeric values of the reference's `enum class op` (include/Ctools.h:175-209);
 * device codes those of DeviceType (0 = kCPU, 1 = kCUDA).
 */
#ifndef CTORCH_B200_FRONTEND_H
#define CTORCH_B200_FRONTEND_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

const char* cth_last_error(void);
void cth_set_quiet(int quiet);          /* silence Ctorch_Error::log printing (errors are still counted) */
uint64_t cth_error_count(void);         /* number of log(ERROR) calls so far */
int cth_cuda_available(void);           /* Ctorch_Scheduler::isDeviceAvailable(kCUDA), include/Ctorch_Scheduler.h:67-75 */

/* ---- Tensor (include/Tensor.h) ---- */
/* Tensor(ShapeTag, shape, kFloat, device); data == NULL leaves it zero-filled. */
int cth_tensor_from_host(const float* data, const int64_t* shape, int rank, int device, void** tensor);
int cth_tensor_scalar(float value, void** tensor);   /* Tensor(float): 0-D, on the host (include/Tensor.h:239-264) */
int cth_tensor_free(void* tensor);
int cth_tensor_info(void* tensor, int64_t* shape_out8, int* rank, int* device, int* requires_grad, uint64_t* id);
int cth_tensor_to_host(void* tensor, float* out);     /* row-major values, also of a strided view */
int cth_tensor_item(void* tensor, float* out);        /* Tensor::item<float>, src/Tensor.cpp:154-165 */
int cth_tensor_requires_grad(void* tensor, int flag); /* Tensor::requires_grad(bool), src/Tensor.cpp:28-39 */
int cth_tensor_to_device(void* tensor, int device, void** out);
int cth_tensor_copy(void* tensor, void** out);        /* copy constructor: new id, same value */
int cth_tensor_fill(void* tensor, float value);
int cth_transpose(void* tensor, void** out);          /* Tensor::t(), src/Tensor.cpp:246-261 */

/* ---- operators ---- */
/* relu/sigmoid/tanh/sin/cos/unary minus/softmax(param = dim)/sum */
int cth_unary(void* tensor, int op, int param, void** out);
/* + - * / matmul dot mse_loss mae_loss cross_entropy */
int cth_binary(void* a, void* b, int op, void** out);
/* kind: 0 t*s, 1 t+s, 2 t/s, 3 s-t, 4 s/t, 5 s*t, 6 s+t (src/Tensor.cpp:751-973, 1416-1453) */
int cth_scalar(void* tensor, float s, int kind, void** out);

/* ---- AutoDiff (include/AutoDiff.h) ---- */
/* Dtype-aware part of the Tensor API.  dtype: the values of `enum class DType` (include/Ctools.h:163-169:
 * 0 float, 1 double, 2 int32, 3 int64, 4 bool). */
int cth_tensor_empty(const int64_t* shape, int rank, int dtype, int device, void** out); /* zero-initialised, Tensor(ShapeTag, ...) include/Tensor.h:280-296 */
int cth_tensor_dtype(void* tensor, int* dtype);
int cth_tensor_read_raw(void* tensor, void* dst, uint64_t nbytes);   /* numel * sizeof(dtype) bytes in memory order */
/* Tensor::operator>, <, ==, >=, <=, != (src/Tensor.cpp:985-1309) and the scalar-on-the-left free
 * operators (:1462-1591): cmp = CTK_CMP_*, form = CTK_CMP_TENSOR (b given), CTK_CMP_SCALAR_RIGHT
 * (a cmp scalar) or CTK_CMP_SCALAR_LEFT (scalar cmp a); the result is a kBool tensor. */
int cth_tensor_compare(void* a, void* b_or_null, float scalar, int cmp, int form, void** out);
int cth_tensor_to_dtype(void* tensor, int dtype, void** out);        /* Tensor::to(DType), src/Tensor.cpp:199-243 */
int cth_tensor_ones(void* tensor);                                   /* Tensor::ones, src/Tensor.cpp:422-450 */
int cth_tensor_rand(void* tensor);                                   /* Tensor::rand, src/Tensor.cpp:458-479 */
int cth_manual_seed(uint64_t seed);                                  /* no counterpart: fixes rand's seed and restarts its counter */
int cth_tensor_index(void* tensor, uint64_t index, void** out);      /* Tensor::operator[], src/Tensor.cpp:175-189 */

/* Host-only self-test (no GPU needed, no counterpart in the reference): the caches that recycle     */
/* device buffers are keyed by (device ordinal, size); *failed = number of checks that did not hold. */
int cth_selftest_cache_keying(int* failed);

int cth_ctx_create(void** ctx);
int cth_ctx_destroy(void* ctx);
int cth_ctx_set_current(void* ctx_or_null);           /* AutoDiffContext::current() of the calling thread */
int cth_ctx_make_leaf(void* ctx, void* tensor, int requires_grad);
int cth_ctx_zero_grad(void* ctx, void* tensor);
int cth_ctx_clear(void* ctx);                         /* AutoDiff::clear_graph */
int cth_ctx_release_step_nodes(void* ctx);            /* drop nodes no future root can reach (no counterpart) */
int cth_ctx_node_count(void* ctx, uint64_t* n);
/* AutoDiff::on_leaf_grad (no counterpart in the reference) fires once per leaf and backward pass,   */
/* after the leaf's last contribution.  count_leaf_grads(1) installs a hook that only counts the     */
/* calls per tensor, leaf_grad_count reads the count for one tensor.                                  */
int cth_ctx_count_leaf_grads(void* ctx, int on);
int cth_ctx_leaf_grad_count(void* ctx, void* tensor, uint64_t* n);
/* No counterpart.  on != 0: a ReLU output that exactly one MatMul reads (as its first operand) gets its
 * backward rule (src/AutoDiff.cpp:1320-1371) applied in the epilogue of the product g.W^T that computes
 * its gradient.  Every gradient upstream is bit for bit the same; cth_grad of that ReLU output itself
 * then returns the masked gradient.  Off by default; the MLP trainer switches it on for its own tape. */
int cth_ctx_set_fuse_relu_backward(void* ctx, int on);
int cth_backward(void* root, void* grad_output_or_null); /* free backward(root[, grad]), src/Tensor.cpp:1373-1384 */
int cth_grad(void* tensor, void** out);                /* free grad(t), src/Tensor.cpp:1387-1392 */
/* (x.matmul(w) + bias)[.relu()] as one kernel where possible, recorded as the same MatMul, Add and
 * ReLU nodes and equal to the three calls bit for bit (Tensor::linear). */
int cth_linear(void* x, void* w, void* bias, int relu, void** out);
int cth_sgd_update(void* param, void* grad, float lr); /* p -= g*lr on the device (mnist/mnist.cpp:80-92) */

/* ---- the MLP training step of mnist/mnist.cpp:44-92 for any layer list ----
 * dims[0..n_layers]; params packed W1,b1,W2,b2,... (W row-major [in,out]).  A step is
 * make_leaf/requires_grad/zero_grad, forward (matmul + bias, ReLU between layers), one-hot
 * cross entropy (summed over the batch), backward, SGD; it returns the loss. */
int cth_mlp_create(int n_layers, const int64_t* dims, const float* params, float lr, void** mlp);
int cth_mlp_destroy(void* mlp);
/* Data parallel: all-reduce (sum) every parameter gradient over `comm` (a ctk_comm_init_rank
 * communicator), started per gradient while backward is still running.  NULL switches it off. */
int cth_mlp_set_comm(void* mlp, void* comm);
/* How the gradients cross the ranks; choose before cth_mlp_set_comm.  0 (default): each gradient is
 * all-reduced in place the moment backward has completed it.  1: gradients are copied into one buffer
 * registered with the communicator and all-reduced there, one call per layer, under backward.  2: the
 * same buffer, one all-reduce after backward (nothing shares the SMs with the products; fully exposed).
 * 3: reduce-scatter per parameter under backward, SGD on the shard this rank owns, all-gather of the
 * updated weights -- the replicated update of mnist/mnist.cpp:80-92 done once per shard.  Every mode
 * applies the same sums; they differ in the order NCCL adds the ranks' values. */
int cth_mlp_set_dp_mode(void* mlp, int mode);
/* A data-parallel step waits for its end with a deadline (default 30000 ms) and watches the
 * communicator's health meanwhile; a step that runs out reports an error and the communicator is
 * aborted (ctk_comm_wait). */
int cth_mlp_set_comm_timeout_ms(void* mlp, int timeout_ms);
int cth_mlp_keep_logits(void* mlp, int keep);
/* Deferred losses (no counterpart: the reference's loop reads loss.item() every step, mnist/mnist.cpp:255).
 * on: the step calls return without waiting for the device and report 0; each step still copies its
 * loss to page-locked memory, and cth_mlp_sync_losses waits for everything issued and returns the
 * losses of the last n <= min(cap, 16) steps, oldest first.  Host buffers given to cth_mlp_stage_host
 * must then stay unchanged until cth_mlp_sync_losses has returned.  The numbers do not change. */
int cth_mlp_set_deferred_loss(void* mlp, int on);
int cth_mlp_sync_losses(void* mlp, float* out, int cap, int* n);
/* No counterpart: an opt-in mode that leaves the reference's arithmetic on purpose.  exact_bias_grad: the
 * gradient of a bias is the sum of the upstream gradient over the batch (the reference: its first row,
 * src/AutoDiff.cpp:690-757).  fresh_weights: backward multiplies by the current weights (the reference: by
 * the copy taken when the parameter was first registered, src/AutoDiff.cpp:286-290).  Both 0 by default;
 * every parity test runs with both 0. */
int cth_mlp_set_corrected(void* mlp, int exact_bias_grad, int fresh_weights);
/* x_host [batch, dims[0]] and labels_host [batch] (class indices as floats) in HOST memory.
 * Every eager step call returns once the step's loss has arrived on the host (the forward pass is over and
 * the host buffers have been read); its backward pass and updates may still be queued on the stream, in
 * front of whatever is issued next -- cth_mlp_get_params / get_grads / predict and the next step are ordered
 * behind them.  With a communicator set the wait is bounded (cth_mlp_set_comm_timeout_ms): a peer that
 * never takes part in the previous step's exchange keeps this step's loss from arriving. */
int cth_mlp_step_host(void* mlp, const float* x_host, const float* labels_host, int64_t batch, float* loss);
/* The same step with the upload taken off the critical path, as an input pipeline would run it:
 * cth_mlp_stage_host starts the host-to-device copy of one batch on a copy stream and returns (page-locked
 * buffers; pageable ones are copied before it returns); cth_mlp_step_staged runs the step on the
 * oldest staged batch once its copy has landed.  Up to two batches may be staged, so calling
 * stage(k+1) before step_staged() of batch k overlaps the upload of k+1 with the compute of k.
 * A staged host buffer must stay unchanged until the step that consumes it has returned. */
int cth_mlp_stage_host(void* mlp, const float* x_host, const float* labels_host, int64_t batch);
int cth_mlp_step_staged(void* mlp, float* loss);
/* The same step replayed as a CUDA graph, for steps bound by launch latency: the first two calls of a
 * batch size run eagerly, the third records the step (its ~20 kernels, buffers and tensor maps) and every
 * later call replays it with one launch; inputs pass through two fixed device tensors.  Results are
 * the eager step's, bit for bit.  An eager step, another batch size or the trainer's end release
 * the graph.  Not available while a communicator is set.  cth_mlp_train_epoch_graph is
 * cth_mlp_train_epoch with every step taken this way (batches copied device-to-device). */
int cth_mlp_step_graph_host(void* mlp, const float* x_host, const float* labels_host, int64_t batch, float* loss);
int cth_mlp_train_epoch_graph(void* mlp, void* images, void* labels, int64_t batch_size, float* mean_loss);
/* x and onehot are device tensors ([batch, dims[0]] and [batch, classes]). */
int cth_mlp_step_device(void* mlp, void* x, void* onehot, float* loss);
/* NeuralNetwork::predict (mnist/mnist.cpp:94-131): class probabilities [batch, classes] of a device
 * batch, nothing recorded on the tape.  calculate_accuracy (:134-158): first-maximum class per row
 * against (int)label, correct / total; computed on the device.  The epoch loop (:246-262): batches
 * of `batch_size` consecutive rows of a device-resident data set (views, no copies; a trailing
 * partial batch is skipped as there), one training step each; returns the mean step loss. */
int cth_mlp_predict(void* mlp, void* x, void** probs);
int cth_mlp_accuracy(void* mlp, void* x, void* labels, float* accuracy);
int cth_mlp_train_epoch(void* mlp, void* images, void* labels, int64_t batch_size, float* mean_loss);
/* MNISTLoader (mnist/mnist_loader.h): reads an IDX image file (magic 2051) and label file (magic
 * 2049) of directory `dir` into an [n, rows*cols] tensor of pixel/255 and an [n] tensor of labels
 * as floats, on `device` (0 host, 1 CUDA: the bytes are uploaded and converted on the device).
 * image_file / label_file NULL: the training pair "train-images-idx3-ubyte" /
 * "train-labels-idx1-ubyte"; image_file "test" with label_file NULL: the "t10k-..." pair.
 * Fails (message in cth_last_error) if a file cannot be opened, has the wrong magic number or is
 * shorter than its header says. */
int cth_mnist_load(const char* dir, const char* image_file, const char* label_file, int device, void** images, void** labels);
/* Rows [start, start+count) as a view of the same buffer (the batch of get_batch, :160-188, without its copy). */
int cth_tensor_narrow_rows(void* tensor, int64_t start, int64_t count, void** out);
int cth_mlp_n_params(void* mlp, int64_t* n);
int cth_mlp_get_params(void* mlp, float* out);
int cth_mlp_get_grads(void* mlp, float* out);         /* gradients of the last step (after the all-reduce) */
int cth_mlp_get_logits(void* mlp, float* out);        /* logits of the last step, if kept */
int cth_mlp_node_count(void* mlp, uint64_t* n);

#ifdef __cplusplus
}
#endif
#endif /* CTORCH_B200_FRONTEND_H */
