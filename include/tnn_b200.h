/* C ABI of libtnn_b200: the B200 (sm_100a) implementation of tiny-dpcpp-nn's fully fused MLP
 * ("SwiftNet") and multi-resolution hash-grid encoding, with L2 loss and Adam.
 *
 * Conventions
 *   - Every function returns 0 on success and a non-zero code otherwise; the message of the last
 *     failure on the calling thread is available from tnn_last_error().  Nothing throws across
 *     this boundary.
 *   - All data pointers are DEVICE pointers owned by the caller unless stated otherwise.  Matrices
 *     are row-major, batch x width.  Network activations are bf16, encodings take fp32 inputs.
 *   - `stream` is a cudaStream_t passed as void*; calls only enqueue work on it and never
 *     synchronise, except where a function says so.
 *   - Handles are not thread-safe; use one handle per host thread or lock around it.
 *   - There is no CPU fallback: without a CUDA device of compute capability 10.x the create
 *     functions fail.
 *
 * Each entry point names the reference interface (intel/tiny-dpcpp-nn, path:line) it stands in for.
 */
#ifndef TNN_B200_H
#define TNN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct tnn_network tnn_network;
typedef struct tnn_encoding tnn_encoding;

/* Activation codes: same enumerator order as `enum class Activation`, include/common/common.h:28-38.
 * Only ReLU, Sigmoid and None are accepted, as in include/network/SwiftNetMLP.h:281-288. */
enum { TNN_ACT_RELU = 0, TNN_ACT_SIGMOID = 4, TNN_ACT_NONE = 8 };
/* Element types of caller buffers. */
enum { TNN_DTYPE_BF16 = 0, TNN_DTYPE_FP16 = 1, TNN_DTYPE_FP32 = 2 };

/* Message of the last error raised on this thread ("" if none). */
const char *tnn_last_error(void);
/* Library version string. */
const char *tnn_version(void);

/* ------------------------------------------------------------------------------------------
 * Network: replaces tnn::NetworkModule<T, WIDTH> (include/tnn_api.h:491-697) and the
 * create_network factory (dpcpp_bindings/tiny_dpcpp_nn/pybind_module.cpp:90-139).
 * ------------------------------------------------------------------------------------------ */

/* create_network(input_width, output_width, n_hidden_layers, activation, output_activation, width,
 * dtype, use_bias) - pybind_module.cpp:90-139; checks of include/network/Network.h:129-167.
 * width in {16, 32, 64, 128}; input/output widths are padded up to `width`.  dtype must be
 * TNN_DTYPE_BF16.  Weights start as zeros; call tnn_network_initialize_params or
 * tnn_network_set_params. */
int tnn_network_create(int input_width, int output_width, int n_hidden_layers, int activation,
                       int output_activation, int width, int dtype, int use_bias, tnn_network **out);
/* ~NetworkModule - include/tnn_api.h:510. */
int tnn_network_destroy(tnn_network *net);
/* Module::n_params - include/tnn_api.h:631-633: (n_hidden_layers + 1) * width^2. */
size_t tnn_network_n_params(const tnn_network *net);
/* Module::n_output_dims - include/tnn_api.h:634: the padded output width (= width). */
int tnn_network_n_output_dims(const tnn_network *net);
int tnn_network_width(const tnn_network *net);
int tnn_network_n_hidden_layers(const tnn_network *net);

/* Network::initialize_xavier_normal - include/network/Network.h:271-295: uniform(+-sqrt(6 / fan)),
 * fan of first and last matrix = pad16(input_width) + width.  The reference seeds from
 * std::random_device; here the seed is explicit (std::mt19937). */
int tnn_network_initialize_params(tnn_network *net, uint64_t seed, void *stream);
/* Module::set_params(tensor, weights_are_packed) - include/tnn_api.h:637-641 and
 * Network::set_weights_matrices, include/network/Network.h:90-112.  `params` holds n_params values
 * of `dtype` (bf16 or fp32) on the device, either in the packed layout of
 * source/common/common.cpp:33-42 or unpacked (matrix l = in x out, row-major).  Padding rows /
 * columns are zeroed as in Network.h:171-233.  Device-to-device; no host round trip. */
int tnn_network_set_params(tnn_network *net, const void *params, int dtype, int weights_are_packed,
                           void *stream);
/* Module::get_params - include/tnn_api.h:622-624: n_params bf16 values in the packed layout. */
int tnn_network_get_params(const tnn_network *net, void *params_out_bf16, void *stream);

/* Module::inference - include/tnn_api.h:512-530 (EsimdKernels::inference_impl,
 * include/network/kernel_esimd.h:242-247).  x, y: batch x width bf16; batch % 8 == 0 as in
 * include/network/SwiftNetMLP.h:293-346. */
int tnn_network_inference(tnn_network *net, const void *x, void *y, size_t batch, void *stream);
/* Module::forward_pass - include/tnn_api.h:532-552 (forward_impl, kernel_esimd.h:153-158).
 * y (optional) receives the output; interm_fwd (optional) receives the n_hidden_layers + 2 matrices
 * batch x width the backward pass needs: matrix 0 = input copy, matrix l+1 = activation of layer l. */
int tnn_network_forward(tnn_network *net, const void *x, void *y, void *interm_fwd, size_t batch,
                        void *stream);
/* Module::backward_pass(grad_output, pack_transpose_gradient, get_dl_dinput) -
 * include/tnn_api.h:561-620 (backward_impl + gemm_batch, kernel_esimd.h:160-240).
 * dy: batch x width bf16 = dL/d(output); interm_fwd: what tnn_network_forward stored.
 * grads: n_params values of grads_dtype (bf16 like the reference, or fp32), matrix l as (out x in)
 * row-major, or transposed and packed like the weights when pack_transpose != 0.
 * dx (optional): batch x width bf16 = dL/d(input).  interm_bwd (optional): n_hidden_layers + 1
 * matrices batch x width bf16, matrix l = dL/d(pre-activation of layer l). */
int tnn_network_backward(tnn_network *net, const void *dy, const void *interm_fwd, void *grads,
                         int grads_dtype, int pack_transpose, void *dx, void *interm_bwd,
                         size_t batch, void *stream);
/* Trainer<T>::training_step - include/trainer.h:23-46 (forward_pass then backward_pass), with the L2
 * loss of include/losses/l2.h:19-41 evaluated in between as the reference's training loops do:
 * forward, loss, backward and the weight-gradient reduction in one pass.  x: batch x width bf16;
 * targets: batch x n_targets fp32 (output columns >= n_targets compare against 0); the loss is
 * normalised by batch * width.  grads as in tnn_network_backward; loss_sum (optional): one fp32.
 * Where width and depth allow (all activations of a 128-row tile resident on the SM) this is a single
 * kernel; otherwise the forward, loss and backward kernels run one after another on a workspace
 * owned by the handle. */
int tnn_network_train_step(tnn_network *net, const void *x, const float *targets, int n_targets,
                           size_t batch, float loss_scale, void *grads, int grads_dtype,
                           int pack_transpose, float *loss_sum, void *stream);
/* Waits for `stream` and returns the kernels' status word in *status (0 = fine; non-zero = a
 * bounded device-side wait gave up, results are invalid).  No reference counterpart: the
 * reference kernels have no device-side waits. */
int tnn_network_sync_status(tnn_network *net, int *status, void *stream);
/* Selects a kernel variant for tuning experiments.  Default 0 (the fastest measured choice everywhere).
 *   1    inference keeps hidden activations in shared memory instead of tensor memory
 *   2    MN-major weight operand in the forward / backward kernels
 *   4    fewer tiles in flight in the forward kernel        8    three tiles in flight (inference)
 *   16   training through the forward / loss / backward kernels instead of a fused kernel
 *   32   the pipelined training kernel prints event time stamps of one tile (tuning build)
 *   64   single-tile instead of pipelined fused training kernel
 *   256  stream the weights through per-slot rings even if they would fit on chip
 * No reference counterpart. */
int tnn_network_set_variant(tnn_network *net, int variant);

/* ------------------------------------------------------------------------------------------
 * Encoding: replaces tnn::EncodingModule<float> (include/tnn_api.h:306-488) and create_encoding
 * (pybind_module.cpp:141-147, include/encodings/encoding_factory.h:109-176).
 * ------------------------------------------------------------------------------------------ */

/* `json_config`: flat JSON object with the reference's keys (include/encodings/encoding.h:28-52):
 * otype ("HashGrid" | "Identity"), n_dims_to_encode, type, n_levels | n_features,
 * n_features_per_level, log2_hashmap_size, base_resolution, per_level_scale, hash, interpolation,
 * scale, offset.  Defaults as in include/encodings/grid.h:1010-1047.  Enum values may be strings
 * or integers.  padded_output_width 0 = natural width. */
int tnn_encoding_create(const char *json_config, int padded_output_width, tnn_encoding **out);
int tnn_encoding_destroy(tnn_encoding *enc);
/* Encoding::get_n_params - include/encodings/encoding.h:147. */
size_t tnn_encoding_n_params(const tnn_encoding *enc);
/* Module::n_output_dims - include/tnn_api.h:441-443: padded output width. */
int tnn_encoding_n_output_dims(const tnn_encoding *enc);
int tnn_encoding_n_input_dims(const tnn_encoding *enc);
/* Level l of a grid: first table entry and number of entries (GridEncoding::level_params_offset /
 * level_n_params, include/encodings/grid_interface.h:38-39), in entries of n_features_per_level floats. */
int tnn_encoding_level_info(const tnn_encoding *enc, int level, uint32_t *offset, uint32_t *size,
                            float *scale, uint32_t *resolution);
/* DeviceMatrix::fill_random(-1e-4, 1e-4) - include/encodings/grid.h:650.  The reference draws from
 * oneMKL philox (seed 777); only the distribution is reproduced, from an explicit seed. */
int tnn_encoding_initialize_params(tnn_encoding *enc, uint64_t seed, void *stream);
/* EncodingModule::set_params / get_params - include/tnn_api.h:424-439: n_params fp32, never packed. */
int tnn_encoding_set_params(tnn_encoding *enc, const float *params, void *stream);
int tnn_encoding_get_params(const tnn_encoding *enc, float *params_out, void *stream);
/* Device pointer of the fp32 table the handle currently uses (for in-place optimiser steps). */
float *tnn_encoding_params_ptr(tnn_encoding *enc);
/* Makes the handle read its n_params fp32 parameters from caller-owned device memory (16-byte aligned) instead of
 * its own table, so that a framework's parameter tensor is used in place; NULL returns to the owned table.  The
 * memory must stay valid while it is bound.  No reference counterpart: the reference copies the parameter tensor
 * into the module before every forward pass (dpcpp_bindings/tiny_dpcpp_nn/modules.py:236). */
int tnn_encoding_bind_params(tnn_encoding *enc, float *params);
/* EncodingModule::forward_pass - include/tnn_api.h:332-356 (kernel_grid, grid.h:37-135; identity,
 * identity.h:63-77).  x: batch x n_input_dims fp32.  out: batch x n_output_dims of out_dtype
 * (fp32 like the reference, or bf16 to feed a network directly). */
int tnn_encoding_forward(tnn_encoding *enc, const float *x, void *out, int out_dtype, size_t batch,
                         void *stream);
/* EncodingModule::backward_pass(grad_output, input_from_fwd, false, false) - include/tnn_api.h:368-416
 * (kernel_grid_backward, grid.h:137-245).  grads: n_params fp32, overwritten.  deterministic == 0: fp32
 * reductions in memory like the reference (summation order not fixed); otherwise 64-bit fixed-point integer
 * reductions, whose result does not depend on the order and repeats bit for bit. */
int tnn_encoding_backward(tnn_encoding *enc, const float *x, const void *dy, int dy_dtype, float *grads,
                          size_t batch, int deterministic, void *stream);

/* ------------------------------------------------------------------------------------------
 * Loss and optimiser
 * ------------------------------------------------------------------------------------------ */

/* L2Loss::evaluate - include/losses/l2.h:19-41, include/losses/loss.h:19-25.
 * pred: batch x stride bf16; target: batch x n_targets fp32 (columns >= n_targets compare with 0);
 * values (optional): batch x stride fp32; grads (optional): batch x stride bf16;
 * loss_sum (optional): one fp32 = sum of values. */
int tnn_l2_loss(const void *pred, const float *target, int n_targets, float *values, void *grads,
                size_t batch, int stride, float loss_scale, float *loss_sum, void *stream);
/* No counterpart in the reference.  Same computation and arguments as tnn_l2_loss for callers that must
 * not allocate device memory - e.g. a plug-in inside a host application whose allocator already owns all
 * free device memory, or a latency-critical loop that cannot afford the device-wide synchronisation an
 * allocation implies.  It calls no cudaMalloc / cudaFree and no allocating library routine: the per-block
 * partial sums live in a fixed 16 KiB array inside the library image (present on every GPU that loads
 * the library until the process exits).  Limits and rules that follow from that:
 *   - batch * stride must not exceed 2^27 elements (4096 partial sums x 32768 elements); larger inputs
 *     are rejected with an error, use tnn_l2_loss or split the batch;
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
 *     device current); make that first call before any stream capture;
 *   - all calls on a device share the array: calls that overlap on the GPU (different streams) race on it.
 *     The array keeps the previous call's contents, which is harmless - every slot a call reads is first
 *     overwritten by that call. */
int tnn_l2_loss_static(const void *pred, const float *target, int n_targets, float *values, void *grads,
                       size_t batch, int stride, float loss_scale, float *loss_sum, void *stream);
/* Optimizer::step - include/optimizers/optimizer.h; arithmetic is torch.optim.Adam's (the optimiser
 * every runnable reference path uses: test/python/test_compare_torch_dpcpp.py:37), not the vestigial
 * source/optimizers/adam.cpp.  `step` counts from 1.  grads are multiplied by grad_scale first. */
int tnn_adam_step(float *params, float *m, float *v, const float *grads, size_t n, float grad_scale,
                  int step, float lr, float beta1, float beta2, float eps, void *stream);
/* Adam on a network's fp32 master copy (packed layout, as exposed to the optimiser by
 * dpcpp_bindings/tiny_dpcpp_nn/modules.py:169-175) followed by the refresh of the bf16 weights the
 * kernels read - the device-side equivalent of optimizer.step() + Module.set_params(). */
int tnn_network_adam_step(tnn_network *net, float *master, float *m, float *v, const float *grads,
                          float grad_scale, int step, float lr, float beta1, float beta2, float eps,
                          void *stream);

#ifdef __cplusplus
}
#endif
#endif /* TNN_B200_H */
