// Launchers of the small memory-bound kernels (parameter layout, identity encoding, loss, Adam).
#pragma once
#include <cstddef>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace tnn {

// Counts kernel launches of this library (tnn_launch_count): every launcher reports the kernels it enqueued.
void count_launch(int n = 1);

// Element-type codes of buffers (the values of TNN_DTYPE_* in the C ABI).  The 16-bit network type is bf16 or fp16;
// buffers of that type are passed as __nv_bfloat16* whatever the 16 bits mean, with an `fp16` flag beside them.
enum DType : int { DT_BF16 = 0, DT_FP16 = 1, DT_FP32 = 2 };

// src: n_mat * width^2 values of src_dtype; net_fp16: the network computes in fp16 (else bf16)
cudaError_t launch_set_params(int width, const void *src, int src_dtype, int src_packed, int n_mat, int one_padded_in,
                              int unpadded_out, int net_fp16, __nv_bfloat16 *packed_out, float *master_out,
                              __nv_bfloat16 *wimg, __nv_bfloat16 *wimg_t, cudaStream_t stream);
// loss_out (optional): also receives the sum of the n_loss loss partials of the same pass
cudaError_t launch_reduce_dw(const float *slabs, int n_slabs, int n_mat, int width, int pack_transpose, float scale,
                             float *out_f32, __nv_bfloat16 *out_16, int out_fp16, cudaStream_t stream,
                             const float *loss_partials = nullptr, int n_loss = 0, float *loss_out = nullptr);
cudaError_t launch_identity_fwd(const float *x, void *out, int out_dtype, size_t batch, int n_in, int padded,
                                float scale, float offset, cudaStream_t stream);
cudaError_t launch_frequency_fwd(const float *x, void *out, int out_dtype, size_t batch, int n_in, int n_freq, int padded,
                                 cudaStream_t stream);
cudaError_t launch_identity_bwd_input(const void *dy, int dy_dtype, float *dx, size_t batch, int n_in, int padded,
                                      float scale, cudaStream_t stream);
// dL/dinput of the frequency encoding: dx[batch][n_in] fp32 from dy[batch][padded] of dy_dtype
cudaError_t launch_frequency_bwd_input(const float *x, const void *dy, int dy_dtype, float *dx, size_t batch, int n_in,
                                       int n_freq, int padded, cudaStream_t stream);
// spherical harmonics of 2 x - 1 (x: batch x 3), degree in [1, 8]
cudaError_t launch_spherical_harmonics_fwd(const float *x, void *out, int out_dtype, size_t batch, int degree, int padded,
                                           cudaStream_t stream);
// pred and grads: 16-bit values, fp16 when `fp16` (else bf16)
cudaError_t launch_l2_loss(const __nv_bfloat16 *pred, int fp16, const float *target, int n_targets, float *values,
                           __nv_bfloat16 *grads, size_t batch, int stride, float loss_scale, float *loss_partials,
                           int n_partials, float *loss_sum, cudaStream_t stream);
cudaError_t launch_sum_partials(const float *partials, int n, float *out, cudaStream_t stream);
cudaError_t launch_adam(float *p, float *m, float *v, const float *g, size_t n, float grad_scale, int step, float lr,
                        float b1, float b2, float eps, __nv_bfloat16 *p_bf16, cudaStream_t stream);
cudaError_t launch_f32_to_bf16(const float *a, __nv_bfloat16 *b, size_t n, cudaStream_t s);
cudaError_t launch_bf16_to_f32(const __nv_bfloat16 *a, float *b, size_t n, cudaStream_t s);
cudaError_t launch_fp16_to_f32(const void *a, float *b, size_t n, cudaStream_t s);

} // namespace tnn
