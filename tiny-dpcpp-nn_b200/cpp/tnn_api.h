// Header-only C++ layer over the C ABI of libtnn_b200 with the class names of the reference
// (include/tnn_api.h, include/network/SwiftNetMLP.h, include/encodings/encoding.h, include/losses/l2.h,
// include/trainer.h).  Where the reference passes DeviceMatrixView<T> and a sycl::queue, these methods
// take raw device pointers, a batch size and a cudaStream_t (as void*).  Failures throw
// std::runtime_error carrying tnn_last_error(), like the reference's std::invalid_argument /
// std::runtime_error paths.
#pragma once
#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>

#include "../../include/tnn_b200.h"

namespace tnn {

enum class Activation { ReLU = 0, LeakyReLU, Exponential, Sine, Sigmoid, Squareplus, Softplus, Tanh, None };

inline void check(int rc) {
    if (rc != 0) throw std::runtime_error(tnn_last_error());
}

// tnn::NetworkModule<T, WIDTH> (include/tnn_api.h:491-697); T is bf16, WIDTH is a run-time argument.
class NetworkModule {
  public:
    NetworkModule(int input_width, int output_width, int n_hidden_layers, Activation activation,
                  Activation output_activation, int width, bool use_bias, uint64_t seed = 0, void *stream = nullptr) {
        check(tnn_network_create(input_width, output_width, n_hidden_layers, (int)activation, (int)output_activation,
                                 width, TNN_DTYPE_BF16, use_bias ? 1 : 0, &h_));
        check(tnn_network_initialize_params(h_, seed, stream));
    }
    ~NetworkModule() { tnn_network_destroy(h_); }
    NetworkModule(const NetworkModule &) = delete;
    NetworkModule &operator=(const NetworkModule &) = delete;

    size_t n_params() const { return tnn_network_n_params(h_); }        // tnn_api.h:631-633
    size_t n_output_dims() const { return tnn_network_n_output_dims(h_); } // tnn_api.h:634
    int get_network_width() const { return tnn_network_width(h_); }
    int get_n_hidden_layers() const { return tnn_network_n_hidden_layers(h_); }

    void set_params(const void *params, int dtype, bool weights_are_packed, void *stream) { // tnn_api.h:637-641
        check(tnn_network_set_params(h_, params, dtype, weights_are_packed ? 1 : 0, stream));
    }
    void get_params(void *out_bf16, void *stream) const { check(tnn_network_get_params(h_, out_bf16, stream)); }
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
    tnn_network *handle() { return h_; }

  private:
    tnn_network *h_ = nullptr;
};

// SwiftNetMLP<T, WIDTH> (include/network/SwiftNetMLP.h:75-248): the same object under the reference's model name.
using SwiftNetMLP = NetworkModule;

// tnn::EncodingModule<float> (include/tnn_api.h:306-488).
class EncodingModule {
  public:
    EncodingModule(const std::string &json_config, int padded_output_width = 0, uint64_t seed = 0,
                   void *stream = nullptr) {
        check(tnn_encoding_create(json_config.c_str(), padded_output_width, &h_));
        check(tnn_encoding_initialize_params(h_, seed, stream));
    }
    ~EncodingModule() { tnn_encoding_destroy(h_); }
    EncodingModule(const EncodingModule &) = delete;
    EncodingModule &operator=(const EncodingModule &) = delete;

    size_t n_params() const { return tnn_encoding_n_params(h_); }
    size_t n_output_dims() const { return tnn_encoding_n_output_dims(h_); }
    void set_params(const float *params, void *stream) { check(tnn_encoding_set_params(h_, params, stream)); }
    void get_params(float *out, void *stream) const { check(tnn_encoding_get_params(h_, out, stream)); }
    void forward_pass(const float *input, void *output, int out_dtype, size_t batch, void *stream) { // 332-356
        check(tnn_encoding_forward(h_, input, output, out_dtype, batch, stream));
    }
    void backward_pass(const float *input_from_fwd, const void *grad_output, int grad_dtype, float *grads,
                       size_t batch, void *stream, bool deterministic = true) { // tnn_api.h:368-416
        check(tnn_encoding_backward(h_, input_from_fwd, grad_output, grad_dtype, grads, batch, deterministic ? 1 : 0,
                                    stream));
    }
    tnn_encoding *handle() { return h_; }

  private:
    tnn_encoding *h_ = nullptr;
};

// L2Loss<T>::evaluate (include/losses/l2.h:29-40, include/losses/loss.h:19-25).
struct L2Loss {
    static void evaluate(void *stream, float loss_scale, const void *predictions, const float *targets, int n_targets,
                         float *values, void *gradients, size_t batch, int stride, float *loss_sum = nullptr) {
        check(tnn_l2_loss(predictions, targets, n_targets, values, gradients, batch, stride, loss_scale, loss_sum,
                          stream));
    }
};

// Trainer<T> (include/trainer.h:23-46): training_step = forward_pass -> backward_pass; here with the L2
// loss in between and, optionally, the Adam update, all on the device.
class Trainer {
  public:
    explicit Trainer(NetworkModule &network) : net_(network) {}
    void training_step(const void *x, const float *targets, int n_targets, size_t batch, float *grads_fp32,
                       float *loss_sum, void *stream, float loss_scale = 1.0f) {
        check(tnn_network_train_step(net_.handle(), x, targets, n_targets, batch, loss_scale, grads_fp32,
                                     TNN_DTYPE_FP32, 1, loss_sum, stream));
    }
    void optimizer_step(float *master, float *m, float *v, const float *grads, int step, void *stream,
                        float lr = 1e-3f, float beta1 = 0.9f, float beta2 = 0.99f, float eps = 1e-15f,
                        float grad_scale = 1.0f) {
        check(tnn_network_adam_step(net_.handle(), master, m, v, grads, grad_scale, step, lr, beta1, beta2, eps,
                                    stream));
    }

  private:
    NetworkModule &net_;
};

} // namespace tnn
