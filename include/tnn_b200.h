/* C ABI of libtnn_b200: the B200 (sm_100a) implementation of tiny-dpcpp-nn's fully fused MLP
 * ("SwiftNet") and multi-resolution hash-grid encoding, with L2 loss and Adam.
 *
 * Conventions
 *   - Every function returns 0 on success and a non-zero code otherwise; the message of the last
 *     failure on the calling thread is available from tnn_last_error().  Nothing throws across
 *     this boundary.
 *   - All data pointers are DEVICE pointers owned by the caller unless stated otherwise.  Matrices
 *     are row-major, batch x width.  Network activations have the network's 16-bit type (bf16 or fp16; "bf16"
 *     in the comments below stands for either), encodings take fp32 inputs.
 *   - `stream` is a cudaStream_t passed as void*; calls only enqueue work on it and never
 *     synchronise or allocate, except where a function says so (workspace growth, parameter initialisation).
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
typedef struct tnn_trainer tnn_trainer;
typedef struct tnn_dp_comm tnn_dp_comm;

/* Activation codes: same enumerator order as `enum class Activation`, include/common/common.h:28-38.
 * Only ReLU, Sigmoid and None are accepted, as in include/network/SwiftNetMLP.h:281-288. */
enum { TNN_ACT_RELU = 0, TNN_ACT_SIGMOID = 4, TNN_ACT_NONE = 8 };
/* Element types of caller buffers. */
enum { TNN_DTYPE_BF16 = 0, TNN_DTYPE_FP16 = 1, TNN_DTYPE_FP32 = 2 };

/* Message of the last error raised on this thread ("" if none). */
const char *tnn_last_error(void);
/* Library version string. */
const char *tnn_version(void);
/* Number of kernels of this library that the process has launched so far, on all streams and devices (library
 * routines such as memset, memcpy and NCCL collectives are not counted).  No reference counterpart. */
unsigned long long tnn_launch_count(void);

/* ------------------------------------------------------------------------------------------
 * Network: replaces tnn::NetworkModule<T, WIDTH> (include/tnn_api.h:491-697) and the
 * create_network factory (dpcpp_bindings/tiny_dpcpp_nn/pybind_module.cpp:90-139).
 * ------------------------------------------------------------------------------------------ */

/* create_network(input_width, output_width, n_hidden_layers, activation, output_activation, width,
 * dtype, use_bias) - pybind_module.cpp:90-139; checks of include/network/Network.h:129-167.
 * width in {16, 32, 64, 128}; input/output widths are padded up to `width`.  dtype: TNN_DTYPE_BF16 or
 * TNN_DTYPE_FP16 (the reference's sycl::half instantiations, include/network/kernel_esimd.h:643-721) - the type of
 * weights, activations and of every "16-bit" buffer of this network below.  Weights start as zeros; call tnn_network_initialize_params or
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
 * std::random_device; here the seed is explicit (std::mt19937).  Draws on the host, copies, and waits for
 * `stream`. */
int tnn_network_initialize_params(tnn_network *net, uint64_t seed, void *stream);
/* Module::set_params(tensor, weights_are_packed) - include/tnn_api.h:637-641 and
 * Network::set_weights_matrices, include/network/Network.h:90-112.  `params` holds n_params values
 * of `dtype` (bf16, fp16 or fp32) on the device, either in the packed layout of
 * source/common/common.cpp:33-42 or unpacked (matrix l = in x out, row-major).  Padding rows /
 * columns are zeroed as in Network.h:171-233.  Device-to-device; no host round trip. */
int tnn_network_set_params(tnn_network *net, const void *params, int dtype, int weights_are_packed,
                           void *stream);
/* Module::get_params - include/tnn_api.h:622-624: n_params values of the network's 16-bit type, packed layout. */
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
 * grads: n_params values of grads_dtype (bf16 / fp16 like the reference's T, or fp32), matrix l as (out x in)
 * row-major, or transposed and packed like the weights when pack_transpose != 0.
 * dx (optional): batch x width bf16 = dL/d(input).  interm_bwd (optional): n_hidden_layers + 1
 * matrices batch x width bf16, matrix l = dL/d(pre-activation of layer l). */
int tnn_network_backward(tnn_network *net, const void *dy, const void *interm_fwd, void *grads,
                         int grads_dtype, int pack_transpose, void *dx, void *interm_bwd,
                         size_t batch, void *stream);
/* The same backward pass without stored activations: Module::backward_pass (include/tnn_api.h:561-620) given the
 * input x of the forward pass instead of interm_fwd.  One fused kernel recomputes the activations tile by tile on
 * chip (they never reach HBM), applies dy and runs the delta chain and the weight-gradient reduction: a training
 * loop then needs tnn_network_inference for its forward pass, not tnn_network_forward with its
 * (n_hidden_layers + 2) x batch x width store.  x, dy: batch x width of the network's type; grads, pack_transpose,
 * dl_dinput (optional, batch x width of the network's type) as in tnn_network_backward; 16-byte aligned pointers.
 * Supported where the network fits the fused training kernel (widths 16 / 32 / 64, e.g. up to 5 hidden layers at
 * width 64): ask tnn_network_backward_from_input_supported first (1 / 0). */
int tnn_network_backward_from_input_supported(const tnn_network *net);
int tnn_network_backward_from_input(tnn_network *net, const void *x, const void *dy, void *grads, int grads_dtype,
                                    int pack_transpose, void *dl_dinput, size_t batch, void *stream);
/* Trainer<T>::training_step - include/trainer.h:23-46 (forward_pass then backward_pass), with the L2
 * loss of include/losses/l2.h:19-41 evaluated in between as the reference's training loops do:
 * forward, loss, backward and the weight-gradient reduction in one pass.  x: batch x width bf16;
 * targets: batch x n_targets fp32 (output columns >= n_targets compare against 0); the loss is
 * normalised by batch * width.  grads as in tnn_network_backward; loss_sum (optional): one fp32.
 * Where width and depth allow (all activations of a 128-row tile resident on the SM) this is a single
 * kernel that needs no workspace; otherwise the forward, loss and backward kernels run one after another on a
 * workspace of tnn_network_workspace_bytes(batch) bytes.  Unless the caller has lent one with
 * tnn_network_set_workspace, the handle allocates it at the first such call and re-allocates it when a larger
 * batch arrives; that (re-)allocation synchronises `stream` - the one place where this call is not purely
 * asynchronous.  targets: 4-byte aligned; 16-byte aligned targets are staged by bulk copies (faster). */
int tnn_network_train_step(tnn_network *net, const void *x, const float *targets, int n_targets,
                           size_t batch, float loss_scale, void *grads, int grads_dtype,
                           int pack_transpose, float *loss_sum, void *stream);
/* Bytes of workspace tnn_network_train_step needs for `batch` rows when the network does not fit a fused
 * kernel (n_hidden_layers + 3 matrices batch x width bf16).  No reference counterpart: the reference's modules
 * grow their workspaces silently (include/tnn_api.h:649-684). */
size_t tnn_network_workspace_bytes(const tnn_network *net, size_t batch);
/* Lends the handle a caller-owned workspace (256-byte aligned device memory) so that no call allocates or
 * synchronises; a call that needs more than `bytes` fails with a message instead of allocating.  NULL returns to
 * the library-owned, growing workspace.  The memory must stay valid while it is lent. */
int tnn_network_set_workspace(tnn_network *net, void *workspace, size_t bytes);
/* Waits for `stream` and returns the kernels' status word in *status (0 = fine; non-zero = a
 * bounded device-side wait gave up, results are invalid).  No reference counterpart: the
 * reference kernels have no device-side waits. */
int tnn_network_sync_status(tnn_network *net, int *status, void *stream);
/* Forces a kernel path that the library would not pick by itself, so that tests can cover every path on
 * small networks.  Default 0 (the fastest measured choice everywhere).
 *   16   training through the forward / loss / backward kernels instead of a fused kernel
 *   64   single-tile instead of pipelined fused training kernel
 *   128  tnn_network_with_encoding_*: gather a HashGrid encoding inside the network's forward kernel (extra warps
 *        write the features straight into the input tile) instead of running the encoding kernel first; slower
 *        than the two kernels at the sizes measured, kept for grids small enough to live in L1
 *   256  stream the weights through per-slot rings even if they would fit on chip
 * No reference counterpart. */
int tnn_network_set_variant(tnn_network *net, int variant);

/* ------------------------------------------------------------------------------------------
 * Encoding: replaces tnn::EncodingModule<float> (include/tnn_api.h:306-488) and create_encoding
 * (pybind_module.cpp:141-147, include/encodings/encoding_factory.h:109-176).
 * ------------------------------------------------------------------------------------------ */

/* `json_config`: flat JSON object with the reference's keys (include/encodings/encoding.h:28-52):
 * otype ("HashGrid" | "Identity" | "Frequency" | "SphericalHarmonics"), n_dims_to_encode, n_frequencies, degree, type, n_levels | n_features,
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
 * (fp32 like the reference, or bf16 / fp16 to feed a network directly). */
int tnn_encoding_forward(tnn_encoding *enc, const float *x, void *out, int out_dtype, size_t batch,
                         void *stream);
/* EncodingModule::backward_pass(grad_output, input_from_fwd, false, false) - include/tnn_api.h:368-416
 * (kernel_grid_backward, grid.h:137-245).  grads: n_params fp32, overwritten.  deterministic == 0: fp32
 * reductions in memory like the reference (summation order not fixed); 1: 64-bit fixed-point integer
 * reductions, whose result does not depend on the order and repeats bit for bit (an inf or NaN in dy then makes
 * every gradient of the call NaN); 2: no atomics at all - the contributions are written out sorted by table
 * bucket and summed as a segmented reduction in a fixed order (bit-reproducible too, plain fp32 sums, about three
 * times slower than 1 at the benchmark grid).  grads must be 16-byte aligned.  Modes 1 and 2 keep scratch in the
 * handle (8 bytes per parameter; for 2 up to 1 GiB of records), allocated - with a synchronisation of `stream` -
 * at first use and when a larger batch needs more. */
int tnn_encoding_backward(tnn_encoding *enc, const float *x, const void *dy, int dy_dtype, float *grads,
                          size_t batch, int deterministic, void *stream);

/* dL/dinput of an encoding - the `dL_dinput` output of Encoding::backward_impl (include/encodings/encoding.h:120-135):
 * dx: batch x n_input_dims fp32, overwritten.  Identity: dL/dy * scale (identity.h:91-97); Frequency:
 * include/encodings/frequency.h:91-131; HashGrid: the product of kernel_grid_backward_input
 * (include/encodings/grid.h:247-268) with the derivative taken directly from the interpolation formula (the reference's
 * forward pass never fills the dy/dx context that kernel reads, grid.h:669-670); SphericalHarmonics: fails with the
 * reference's message (spherical_harmonics.h:66-71).  The reference's Python layer never asks for it
 * (include/tnn_api.h:380-382). */
int tnn_encoding_backward_input(tnn_encoding *enc, const float *x, const void *dy, int dy_dtype, float *dx,
                                size_t batch, void *stream);

/* ------------------------------------------------------------------------------------------
 * Network with input encoding: replaces NetworkWithInputEncoding
 * (dpcpp_bindings/tiny_dpcpp_nn/modules.py:357-421, a torch.nn.Sequential of the two modules) without the
 * batch x width matrix between them where a kernel can produce the network's input tile itself.  The
 * encoding's padded output width must equal the network width.  x: batch x n_input_dims fp32.
 *   Identity (up to 16 inputs): folded into the first-layer load of the network kernels - the encoded matrix
 *     never exists (include/encodings/identity.h:63-77 + include/network/kernel_esimd.h:565-640 in one kernel).
 *   Other encodings: encoding kernel, then network kernels, through the network handle's workspace
 *     (tnn_network_with_encoding_workspace_bytes; same allocation rule as tnn_network_train_step).  For a 2-D / 3-D
 *     HashGrid with two features per level a forward kernel that gathers the grid itself exists as well
 *     (tnn_network_set_variant bit 128).
 * ------------------------------------------------------------------------------------------ */
size_t tnn_network_with_encoding_workspace_bytes(const tnn_network *net, size_t batch);
/* Sequential(encoding, network) in eval mode: y = network(encoding(x)), batch x width bf16. */
int tnn_network_with_encoding_inference(tnn_network *net, tnn_encoding *enc, const float *x, void *y,
                                        size_t batch, void *stream);
/* Sequential(encoding, network) forward in training mode: like tnn_network_forward; matrix 0 of interm_fwd
 * receives the encoded input. */
int tnn_network_with_encoding_forward(tnn_network *net, tnn_encoding *enc, const float *x, void *y,
                                      void *interm_fwd, size_t batch, void *stream);
/* One training pass of the pair: forward, L2 loss, backward, network weight gradients (as
 * tnn_network_train_step) and - for an encoding with parameters, when encoding_grads is given - the
 * encoding's parameter gradient (n_params fp32, as tnn_encoding_backward with `deterministic`). */
int tnn_network_with_encoding_train_step(tnn_network *net, tnn_encoding *enc, const float *x,
                                         const float *targets, int n_targets, size_t batch, float loss_scale,
                                         void *grads, int grads_dtype, int pack_transpose,
                                         float *encoding_grads, int deterministic, float *loss_sum,
                                         void *stream);

/* ------------------------------------------------------------------------------------------
 * Loss and optimiser
 * ------------------------------------------------------------------------------------------ */

/* L2Loss::evaluate - include/losses/l2.h:19-41, include/losses/loss.h:19-25.
 * pred: batch x stride bf16; target: batch x n_targets fp32 (columns >= n_targets compare with 0);
 * values (optional): batch x stride fp32; grads (optional): batch x stride bf16;
 * loss_sum (optional): one fp32 = sum of values.  pred, values and grads must be 16-byte aligned, target 4-byte
 * (16-byte when n_targets == stride).  The per-block partial sums behind loss_sum live in one buffer per device
 * that the library allocates at the first call on that device and keeps: calls that overlap on one device (two
 * streams) race on it. */
int tnn_l2_loss(const void *pred, const float *target, int n_targets, float *values, void *grads,
                size_t batch, int stride, float loss_scale, float *loss_sum, void *stream);
/* The same loss for predictions of either 16-bit type: dtype = TNN_DTYPE_BF16 or TNN_DTYPE_FP16 (pred and grads
 * share it) - Loss<T> with T = sycl::half, include/losses/loss.h:19-25. */
int tnn_l2_loss_dtype(const void *pred, int dtype, const float *target, int n_targets, float *values, void *grads,
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

/* ------------------------------------------------------------------------------------------
 * Data parallelism.  No reference counterpart: the reference's multi-GPU benchmarks are independent MPI replicas
 * without any exchange (benchmarks/common_benchmarks.h:53-54).  One process per GPU; the only exchange of a
 * training step is the sum of the (n_hidden_layers + 1) * width^2 fp32 weight-gradient buffer over the ranks
 * (plus reduce-scatter / all-gather of a trainable encoding's table).  NCCL is loaded with dlopen("libnccl.so.2")
 * at the first of these calls - the copy the process already uses, if it has one.
 *
 * Peer windows: when all ranks (at most 8) run on one host and can map each other's memory (CUDA IPC over NVLink),
 * making a communicator also gives every rank a window in every other rank's address space, and the optimiser
 * kernel of a trainer exchanges the weight gradient itself: it sums the per-CTA slabs, stores every value together
 * with the number of the exchange - one 8-byte store per element, no fence, no separate flag - into every peer's
 * window, polls its own window until the elements of all ranks carry that number (bounded: TNN_DP_WAIT_MS, default
 * 30 000, after which tnn_network_sync_status reports 2 and the step is invalid), adds the ranks' contributions in
 * rank order - every rank computes bit-identical parameters - and applies Adam.  Otherwise (several hosts, no peer
 * access, more than 262 144 parameters, or TNN_DP_PEER_WINDOW=0 in the environment of every rank) the exchange is
 * one ncclAllReduce(sum) between a reduction kernel and the Adam kernel.  Windows cost 4 MiB per rank pair.
 * ------------------------------------------------------------------------------------------ */
/* ncclGetUniqueId into 128 caller bytes (rank 0 calls this and sends the bytes to the other ranks). */
int tnn_dp_get_unique_id(void *id128);
/* ncclCommInitRank on the current device, then the peer windows: collective over all `world` ranks;
 * allocates and synchronises the device. */
int tnn_dp_comm_create(const void *id128, int rank, int world, tnn_dp_comm **out);
/* Wraps a communicator the application already has (an ncclComm_t passed as void*); not destroyed by
 * tnn_dp_comm_destroy.  Collective like tnn_dp_comm_create (the peer windows are set up over it). */
int tnn_dp_init(void *nccl_comm, tnn_dp_comm **out);
int tnn_dp_comm_destroy(tnn_dp_comm *comm);
int tnn_dp_rank(const tnn_dp_comm *comm);
int tnn_dp_world_size(const tnn_dp_comm *comm);
/* 1 when trainers on this communicator exchange gradients through peer windows, 0 when through ncclAllReduce. */
int tnn_dp_peer_window(const tnn_dp_comm *comm);
/* Turns the windowed exchange off (0) or back on (1); to be called alike on every rank, between steps. */
int tnn_dp_set_peer_window(tnn_dp_comm *comm, int enable);
/* In-place sum of n fp32 values over the ranks, enqueued on `stream` (comm == NULL: single process, no-op). */
int tnn_dp_allreduce_sum(tnn_dp_comm *comm, float *buf, size_t n, void *stream);

/* ------------------------------------------------------------------------------------------
 * Trainer: replaces Trainer<T> (include/trainer.h:16-52) together with the loss and optimiser the reference's
 * training loops wrap around it (L2Loss, include/losses/l2.h:19-41; torch.optim.Adam on the fp32 master copy of
 * the packed parameters, dpcpp_bindings/tiny_dpcpp_nn/modules.py:169-175).  Owns master parameters, Adam moments,
 * the fp32 gradient and the loss sum on the device.  With `enc` the input is batch x n_input_dims fp32 and the
 * pair trains like NetworkWithInputEncoding; a trainable encoding (HashGrid) gets its own Adam state (sharded
 * over the ranks when a communicator is set: reduce-scatter, Adam on this rank's slice, all-gather).
 * ------------------------------------------------------------------------------------------ */
int tnn_trainer_create(tnn_network *net, tnn_encoding *enc_or_null, float lr, float beta1, float beta2, float eps,
                       float loss_scale, tnn_trainer **out);
int tnn_trainer_destroy(tnn_trainer *trainer);
/* Gradients are averaged over the ranks of `comm` (NULL: single GPU).  Set before the first step. */
int tnn_trainer_set_dp(tnn_trainer *trainer, tnn_dp_comm *comm);
/* Table gradient of a trainable encoding by order-independent fixed-point sums (see tnn_encoding_backward). */
int tnn_trainer_set_deterministic_encoding(tnn_trainer *trainer, int deterministic);
/* n_params fp32 in the packed layout -> master copy and the network's working weights. */
int tnn_trainer_set_master_params(tnn_trainer *trainer, const float *packed_fp32, void *stream);
/* Device pointers into the trainer's state (valid until tnn_trainer_destroy): master parameters and gradient
 * (n_params fp32, packed layout), table gradient of a trainable encoding, loss sum of the last pass (one fp32). */
float *tnn_trainer_master_params(tnn_trainer *trainer);
float *tnn_trainer_grads(tnn_trainer *trainer);
float *tnn_trainer_encoding_grads(tnn_trainer *trainer);
float *tnn_trainer_loss(tnn_trainer *trainer);
int tnn_trainer_step_count(const tnn_trainer *trainer);
/* Trainer::training_step - include/trainer.h:23-46: forward_pass + backward_pass (with the L2 loss between them).
 * x: batch x width bf16 (no encoding) or batch x n_input_dims fp32 (with encoding). */
int tnn_trainer_forward_backward(tnn_trainer *trainer, const void *x, const float *targets, int n_targets,
                                 size_t batch, void *stream);
/* Finishes the sums of the last forward_backward into tnn_trainer_grads / tnn_trainer_loss without an optimiser
 * step (tnn_trainer_optimizer_step does this itself). */
int tnn_trainer_reduce(tnn_trainer *trainer, void *stream);
/* optimizer.step() + Module.set_params(): gradient sum over the ranks when a communicator is set (inside the
 * optimiser kernel with peer windows, else ncclAllReduce), Adam on the master copy, refresh of the 16-bit weights
 * the kernels read.  A single-GPU trainer without a trainable encoding counts its steps on the device: its
 * training step (both calls, or tnn_trainer_training_step) can be captured into a CUDA graph and replayed, every
 * replay being one more optimiser step (tnn_trainer_step_count counts calls, not replays).  With a communicator or
 * a trainable encoding the call is refused (error code) on a capturing stream: the exchange number and the step
 * count of the encoding's Adam kernel are host state passed as kernel arguments. */
int tnn_trainer_optimizer_step(tnn_trainer *trainer, void *stream);
/* forward_backward + optimizer_step: one call enqueues the whole loop body. */
int tnn_trainer_training_step(tnn_trainer *trainer, const void *x, const float *targets, int n_targets,
                              size_t batch, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* TNN_B200_H */
