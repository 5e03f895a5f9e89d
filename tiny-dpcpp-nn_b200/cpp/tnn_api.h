// Header-only C++ layer over the C ABI of libtnn_b200 with the class names of the reference
// (include/tnn_api.h, include/network/Network.h, include/network/SwiftNetMLP.h, include/encodings/encoding.h,
// include/losses/l2.h, include/optimizers/optimizer.h, include/trainer.h).  Where the reference passes
// DeviceMatrixView<T> and a sycl::queue, these methods take raw device pointers, a batch size and a cudaStream_t
// (as void*).  Failures throw std::runtime_error carrying tnn_last_error(), like the reference's
// std::invalid_argument / std::runtime_error paths.  The element type T is a tag: tnn::bf16 or tnn::half.
#pragma once
#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>

#include "../../include/tnn_b200.h"

namespace tnn {

enum class Activation { ReLU = 0, LeakyReLU, Exponential, Sine, Sigmoid, Squareplus, Softplus, Tanh, None };

// Element-type tags standing where the reference uses sycl::ext::oneapi::bfloat16 and sycl::half.
struct bf16 {
    static constexpr int dtype = TNN_DTYPE_BF16;
};
struct half {
    static constexpr int dtype = TNN_DTYPE_FP16;
};

inline void check(int rc) {
    if (rc != 0) throw std::runtime_error(tnn_last_error());
}

// tnn::NetworkModule<T, WIDTH> (include/tnn_api.h:491-697) / Network<T> (include/network/Network.h:59-323);
// WIDTH is a run-time argument.
template <typename T = bf16> class Network {
  public:
    Network(int input_width, int output_width, int n_hidden_layers, Activation activation, Activation output_activation,
            int width, bool use_bias, uint64_t seed = 0, void *stream = nullptr) {
        check(tnn_network_create(input_width, output_width, n_hidden_layers, (int)activation, (int)output_activation,
                                 width, T::dtype, use_bias ? 1 : 0, &h_));
        check(tnn_network_initialize_params(h_, seed, stream));
    }
    ~Network() { tnn_network_destroy(h_); }
    Network(const Network &) = delete;
    Network &operator=(const Network &) = delete;

    size_t n_params() const { return tnn_network_n_params(h_); }           // tnn_api.h:631-633
    size_t n_output_dims() const { return tnn_network_n_output_dims(h_); } // tnn_api.h:634
    int get_network_width() const { return tnn_network_width(h_); }
    int get_n_hidden_layers() const { return tnn_network_n_hidden_layers(h_); }
    // bytes of workspace the unfused training path needs (the reference's modules grow theirs silently)
    size_t workspace_bytes(size_t batch) const { return tnn_network_workspace_bytes(h_, batch); }
    void set_workspace(void *workspace, size_t bytes) { check(tnn_network_set_workspace(h_, workspace, bytes)); }

    void set_params(const void *params, int dtype, bool weights_are_packed, void *stream) { // tnn_api.h:637-641
        check(tnn_network_set_params(h_, params, dtype, weights_are_packed ? 1 : 0, stream));
    }
    void get_params(void *out, void *stream) const { check(tnn_network_get_params(h_, out, stream)); }
    void inference(const void *x, void *y, size_t batch, void *stream) { // tnn_api.h:512-530
        check(tnn_network_inference(h_, x, y, batch, stream));
    }
    void forward_pass(const void *x, void *interm_fwd, size_t batch, void *stream, void *y = nullptr) { // 532-552
        check(tnn_network_forward(h_, x, y, interm_fwd, batch, stream));
    }
    void backward_pass(const void *grad_output, const void *interm_fwd, void *grads, int grads_dtype,
                       bool pack_transpose_gradient, void *dl_dinput, void *interm_bwd, size_t batch,
                       void *stream) { // tnn_api.h:561-620
        check(tnn_network_backward(h_, grad_output, interm_fwd, grads, grads_dtype, pack_transpose_gradient ? 1 : 0,
                                   dl_dinput, interm_bwd, batch, stream));
    }
    // backward_pass from the input of the forward pass instead of stored activations (recomputed on chip by one fused
    // kernel); supported where the network fits the fused training kernel
    bool backward_from_input_supported() const { return tnn_network_backward_from_input_supported(h_) != 0; }
    void backward_pass_from_input(const void *x, const void *grad_output, void *grads, int grads_dtype,
                                  bool pack_transpose_gradient, void *dl_dinput, size_t batch, void *stream) {
        check(tnn_network_backward_from_input(h_, x, grad_output, grads, grads_dtype, pack_transpose_gradient ? 1 : 0,
                                              dl_dinput, batch, stream));
    }
    int sync_status(void *stream) { // non-zero: a bounded device-side wait gave up, results are invalid
        int st = 0;
        check(tnn_network_sync_status(h_, &st, stream));
        return st;
    }
    tnn_network *handle() { return h_; }

  private:
    tnn_network *h_ = nullptr;
};
using NetworkModule = Network<bf16>;
// SwiftNetMLP<T, WIDTH> (include/network/SwiftNetMLP.h:75-248): the same object under the reference's model name.
template <typename T = bf16> using SwiftNetMLP = Network<T>;

// Encoding<T> (include/encodings/encoding.h:75-160) / tnn::EncodingModule<float> (include/tnn_api.h:306-488).
class Encoding {
  public:
    Encoding(const std::string &json_config, int padded_output_width = 0, uint64_t seed = 0, void *stream = nullptr) {
        check(tnn_encoding_create(json_config.c_str(), padded_output_width, &h_));
        check(tnn_encoding_initialize_params(h_, seed, stream));
    }
    ~Encoding() { tnn_encoding_destroy(h_); }
    Encoding(const Encoding &) = delete;
    Encoding &operator=(const Encoding &) = delete;

    size_t n_params() const { return tnn_encoding_n_params(h_); }
    size_t n_output_dims() const { return tnn_encoding_n_output_dims(h_); }
    size_t n_input_dims() const { return tnn_encoding_n_input_dims(h_); }
    void set_params(const float *params, void *stream) { check(tnn_encoding_set_params(h_, params, stream)); }
    void get_params(float *out, void *stream) const { check(tnn_encoding_get_params(h_, out, stream)); }
    void forward_pass(const float *input, void *output, int out_dtype, size_t batch, void *stream) { // 332-356
        check(tnn_encoding_forward(h_, input, output, out_dtype, batch, stream));
    }
    // parameter gradients (tnn_api.h:368-416) and, optionally, dL/dinput (encoding.h:120-135)
    void backward_pass(const float *input_from_fwd, const void *grad_output, int grad_dtype, float *grads,
                       size_t batch, void *stream, bool deterministic = false, float *dl_dinput = nullptr) {
        if (n_params())
            check(tnn_encoding_backward(h_, input_from_fwd, grad_output, grad_dtype, grads, batch, deterministic ? 1 : 0,
                                        stream));
        if (dl_dinput) check(tnn_encoding_backward_input(h_, input_from_fwd, grad_output, grad_dtype, dl_dinput, batch, stream));
    }
    tnn_encoding *handle() { return h_; }

  private:
    tnn_encoding *h_ = nullptr;
};
using EncodingModule = Encoding;

// Loss<T> / L2Loss<T>::evaluate (include/losses/loss.h:19-25, include/losses/l2.h:29-40).
template <typename T = bf16> struct L2Loss {
    static void evaluate(void *stream, float loss_scale, const void *predictions, const float *targets, int n_targets,
                         float *values, void *gradients, size_t batch, int stride, float *loss_sum = nullptr) {
        check(tnn_l2_loss_dtype(predictions, T::dtype, targets, n_targets, values, gradients, batch, stride, loss_scale,
                                loss_sum, stream));
    }
};
template <typename T = bf16> using Loss = L2Loss<T>;

// Optimizer::step (include/optimizers/optimizer.h) with the arithmetic of torch.optim.Adam, the optimiser every
// runnable training path of the reference uses.
struct Optimizer {
    float lr = 1e-3f, beta1 = 0.9f, beta2 = 0.99f, eps = 1e-15f;
    void step(float *params, float *m, float *v, const float *grads, size_t n, int step_count, void *stream,
              float grad_scale = 1.0f) const {
        check(tnn_adam_step(params, m, v, grads, n, grad_scale, step_count, lr, beta1, beta2, eps, stream));
    }
};

// One process per GPU: the communicator over which a Trainer averages its gradients.  On one host whose GPUs can map
// each other's memory it also carries peer windows, through which the optimiser kernel exchanges the weight gradient
// itself; otherwise the exchange is one ncclAllReduce per step.
class DataParallel {
  public:
    static void unique_id(void *id128) { check(tnn_dp_get_unique_id(id128)); }
    // collective over all `world` ranks, each with its own device current
    DataParallel(const void *id128, int rank, int world) { check(tnn_dp_comm_create(id128, rank, world, &c_)); }
    // wraps an existing ncclComm_t
    explicit DataParallel(void *nccl_comm) { check(tnn_dp_init(nccl_comm, &c_)); }
    ~DataParallel() { tnn_dp_comm_destroy(c_); }
    DataParallel(const DataParallel &) = delete;
    DataParallel &operator=(const DataParallel &) = delete;
    int rank() const { return tnn_dp_rank(c_); }
    int world_size() const { return tnn_dp_world_size(c_); }
    bool peer_window() const { return tnn_dp_peer_window(c_) != 0; }
    void set_peer_window(bool on) { check(tnn_dp_set_peer_window(c_, on ? 1 : 0)); } // alike on every rank
    void allreduce_sum(float *buf, size_t n, void *stream) { check(tnn_dp_allreduce_sum(c_, buf, n, stream)); }
    tnn_dp_comm *handle() { return c_; }

  private:
    tnn_dp_comm *c_ = nullptr;
};

// Trainer<T> (include/trainer.h:16-52): training_step = forward_pass -> backward_pass, here with the L2 loss in
// between and the Adam update after it, all on the device; with an Encoding the inputs are fp32 positions
// (NetworkWithInputEncoding); with a DataParallel the gradients are averaged over its ranks.
template <typename T = bf16> class Trainer {
  public:
    explicit Trainer(Network<T> &network, Encoding *encoding = nullptr, const Optimizer &opt = Optimizer(),
                     float loss_scale = 1.0f) {
        check(tnn_trainer_create(network.handle(), encoding ? encoding->handle() : nullptr, opt.lr, opt.beta1, opt.beta2,
                                 opt.eps, loss_scale, &h_));
    }
    ~Trainer() { tnn_trainer_destroy(h_); }
    Trainer(const Trainer &) = delete;
    Trainer &operator=(const Trainer &) = delete;

    void set_data_parallel(DataParallel *dp) { check(tnn_trainer_set_dp(h_, dp ? dp->handle() : nullptr)); }
    void set_master_params(const float *packed_fp32, void *stream) { check(tnn_trainer_set_master_params(h_, packed_fp32, stream)); }
    // forward + loss + backward + optimiser step; the loss sum of the pass is at loss() afterwards (device memory)
    void training_step(const void *x, const float *targets, int n_targets, size_t batch, void *stream) {
        check(tnn_trainer_training_step(h_, x, targets, n_targets, batch, stream));
    }
    void forward_backward(const void *x, const float *targets, int n_targets, size_t batch, void *stream) {
        check(tnn_trainer_forward_backward(h_, x, targets, n_targets, batch, stream));
        check(tnn_trainer_reduce(h_, stream));
    }
    void optimizer_step(void *stream) { check(tnn_trainer_optimizer_step(h_, stream)); }
    const float *loss() const { return tnn_trainer_loss(h_); }
    const float *grads() const { return tnn_trainer_grads(h_); }
    float *master_params() { return tnn_trainer_master_params(h_); }
    int step_count() const { return tnn_trainer_step_count(h_); }

  private:
    tnn_trainer *h_ = nullptr;
};

} // namespace tnn
