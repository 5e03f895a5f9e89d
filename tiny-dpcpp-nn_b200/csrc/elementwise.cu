// Small memory-bound kernels around the fused MLP: parameter layout conversion, identity
// encoding, L2 loss, Adam, and the deterministic reduction of per-CTA weight-gradient slabs.
#include "elementwise.h"
#include "mlp_common.cuh"
#include "slab_sum.cuh"

#include <cmath>
#include <cuda_fp16.h>

namespace tnn {

// Packed ("VNNI") coordinate of element (i, j) of a rows x cols matrix: consecutive row pairs
// are interleaved element-wise (reference source/common/common.cpp:33-42).
__host__ __device__ inline int packed_coord(int i, int j, int cols) {
    return (i & 1) == 0 ? i * cols + 2 * j : (i - 1) * cols + 2 * j + 1;
}

// 16-bit storage of a value in the network's element type
__device__ __forceinline__ __nv_bfloat16 to_net16(float v, int fp16) {
    if (!fp16) return __float2bfloat16_rn(v);
    const unsigned short h = __half_as_ushort(__float2half_rn(v));
    return __ushort_as_bfloat16(h); // the bits of the fp16 value, carried in the 16-bit slot
}

template <int W>
__global__ void set_params_kernel(const void *__restrict__ src, int src_dtype, int src_packed, int n_mat,
                                  int one_padded_in, int unpadded_out, int net_fp16,
                                  __nv_bfloat16 *__restrict__ packed_out, float *__restrict__ master_out,
                                  __nv_bfloat16 *__restrict__ wimg, __nv_bfloat16 *__restrict__ wimg_t) {
    using T = Tile<W>;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_mat * W * W) return;
    const int l = idx / (W * W);
    const int k = (idx / W) % W; // input feature (row of the in x out matrix)
    const int n = idx % W;       // output feature
    const int pk = l * W * W + packed_coord(k, n, W);
    const int si = src_packed ? pk : idx;
    float v = src_dtype == DT_FP32   ? reinterpret_cast<const float *>(src)[si]
              : src_dtype == DT_FP16 ? __half2float(reinterpret_cast<const __half *>(src)[si])
                                     : __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(src)[si]);
    // rows of the first matrix beyond the (ones-padded) input and columns of the last matrix
    // beyond the real output carry no signal: force them to zero (Network.h:171-233).
    if (l == 0 && k >= one_padded_in) v = 0.0f;
    if (l == n_mat - 1 && n >= unpadded_out) v = 0.0f;
    const __nv_bfloat16 b = to_net16(v, net_fp16);
    packed_out[pk] = b;
    if (master_out) master_out[pk] = v;
    uint8_t *wi = reinterpret_cast<uint8_t *>(wimg) + (size_t)l * T::WGT_BYTES;
    uint8_t *wt = reinterpret_cast<uint8_t *>(wimg_t) + (size_t)l * T::WGT_BYTES;
    *reinterpret_cast<__nv_bfloat16 *>(wi + T::elem_off(k, n, T::WGT_ATOM_BYTES)) = b;
    *reinterpret_cast<__nv_bfloat16 *>(wt + T::elem_off(n, k, T::WGT_ATOM_BYTES)) = b;
}

cudaError_t launch_set_params(int width, const void *src, int src_dtype, int src_packed, int n_mat, int one_padded_in,
                              int unpadded_out, int net_fp16, __nv_bfloat16 *packed_out, float *master_out,
                              __nv_bfloat16 *wimg, __nv_bfloat16 *wimg_t, cudaStream_t stream) {
    const int n = n_mat * width * width;
    const int blocks = (n + 255) / 256;
    count_launch();
#define TNN_CASE(WW)                                                                                                    \
    case WW:                                                                                                            \
        set_params_kernel<WW><<<blocks, 256, 0, stream>>>(src, src_dtype, src_packed, n_mat, one_padded_in, unpadded_out, \
                                                          net_fp16, packed_out, master_out, wimg, wimg_t);             \
        break;
    switch (width) {
        TNN_CASE(16) TNN_CASE(32) TNN_CASE(64) TNN_CASE(128)
    default: return cudaErrorInvalidValue;
    }
#undef TNN_CASE
    return cudaGetLastError();
}

// Sum the per-CTA fp32 slabs [n_slabs][n_mat][W(out)][W(in)] in a fixed order (slab_sum: deterministic) and emit
// the gradient in the requested layout: (out x in) row-major as the reference's gemm_batch leaves it
// (kernel_esimd.h:234-239), or transposed to (in x out) and packed like the weights
// (DeviceMatrix.h:469-488 PackAndTranspose).
__global__ void __launch_bounds__(kSlabBlock *kSlabWays)
reduce_dw_kernel(const float *__restrict__ slabs, int n_slabs, int n_mat, int W, int pack_transpose, float scale,
                 float *__restrict__ out_f32, __nv_bfloat16 *__restrict__ out_16, int out_fp16,
                 const float *__restrict__ loss_partials, int n_loss, float *__restrict__ loss_out) {
    __shared__ float part[kSlabWays][kSlabBlock];
    const int idx = blockIdx.x * kSlabBlock + threadIdx.x;
    const int per = n_mat * W * W;
    if (loss_out && blockIdx.x == 0) { // the loss partials of the same pass, summed in a fixed order by block 0
        float *red = part[0];
        if (threadIdx.y == 0) {
            float local = 0.0f;
            for (int i = threadIdx.x; i < n_loss; i += kSlabBlock) local += loss_partials[i];
            red[threadIdx.x] = local;
        }
        __syncthreads();
        for (int s = kSlabBlock / 2; s > 0; s >>= 1) {
            if (threadIdx.y == 0 && (int)threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
            __syncthreads();
        }
        if (threadIdx.y == 0 && threadIdx.x == 0) *loss_out = red[0];
        __syncthreads();
    }
    float acc = slab_sum(slabs, n_slabs, per, idx, part);
    if (threadIdx.y != 0 || idx >= per) return;
    acc *= scale;
    const int l = idx / (W * W);
    const int o = (idx / W) % W; // output feature
    const int i = idx % W;       // input feature
    const int dst = pack_transpose ? l * W * W + packed_coord(i, o, W) : idx;
    if (out_f32) out_f32[dst] = acc;
    if (out_16) out_16[dst] = to_net16(acc, out_fp16);
}

cudaError_t launch_reduce_dw(const float *slabs, int n_slabs, int n_mat, int width, int pack_transpose, float scale,
                             float *out_f32, __nv_bfloat16 *out_16, int out_fp16, cudaStream_t stream,
                             const float *loss_partials, int n_loss, float *loss_out) {
    const int n = n_mat * width * width;
    count_launch();
    reduce_dw_kernel<<<(n + kSlabBlock - 1) / kSlabBlock, dim3(kSlabBlock, kSlabWays), 0, stream>>>(
        slabs, n_slabs, n_mat, width, pack_transpose, scale, out_f32, out_16, out_fp16, loss_partials, n_loss, loss_out);
    return cudaGetLastError();
}

// Identity encoding (include/encodings/identity.h:63-77): out[i, j] = j < n_in ? x * scale + offset : 1.
template <typename OutT>
__global__ void identity_fwd_kernel(const float *__restrict__ x, OutT *__restrict__ out, size_t batch, int n_in,
                                    int padded, float scale, float offset) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= batch * (size_t)padded) return;
    const size_t row = idx / padded;
    const int col = (int)(idx % padded);
    const float v = col < n_in ? __fadd_rn(__fmul_rn(x[row * n_in + col], scale), offset) : 1.0f;
    out[idx] = (OutT)v; // round-to-nearest conversions of the 16-bit types
}

// Same values, eight bf16 columns (one 16-byte store) per thread: the layout a network input uses.
__global__ void __launch_bounds__(256) identity_fwd_bf16x8_kernel(const float *__restrict__ x, uint4 *__restrict__ out,
                                                                   size_t batch, int n_in, int padded, float scale,
                                                                   float offset, int fp16) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int groups = padded / 8;
    if (idx >= batch * (size_t)groups) return;
    const size_t row = idx / groups;
    const int col0 = (int)(idx % groups) * 8;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
        v[j] = (col0 + j < n_in) ? __fadd_rn(__fmul_rn(x[row * n_in + col0 + j], scale), offset) : 1.0f;
    out[idx] = fp16 ? make_uint4(ptx::pack_f16x2(v[0], v[1]), ptx::pack_f16x2(v[2], v[3]), ptx::pack_f16x2(v[4], v[5]),
                                 ptx::pack_f16x2(v[6], v[7]))
                    : make_uint4(ptx::pack_bf16x2(v[0], v[1]), ptx::pack_bf16x2(v[2], v[3]), ptx::pack_bf16x2(v[4], v[5]),
                                 ptx::pack_bf16x2(v[6], v[7]));
}

cudaError_t launch_identity_fwd(const float *x, void *out, int out_dtype, size_t batch, int n_in, int padded,
                                float scale, float offset, cudaStream_t stream) {
    const size_t n = batch * (size_t)padded;
    if (n == 0) return cudaSuccess;
    count_launch();
    if (out_dtype != DT_FP32 && padded % 8 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0) {
        const size_t n8 = n / 8;
        identity_fwd_bf16x8_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, stream>>>(x, (uint4 *)out, batch, n_in, padded,
                                                                                 scale, offset, out_dtype == DT_FP16);
        return cudaGetLastError();
    }
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (out_dtype == DT_BF16)
        identity_fwd_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(x, (__nv_bfloat16 *)out, batch, n_in, padded,
                                                                       scale, offset);
    else if (out_dtype == DT_FP16)
        identity_fwd_kernel<__half><<<blocks, 256, 0, stream>>>(x, (__half *)out, batch, n_in, padded, scale, offset);
    else
        identity_fwd_kernel<float><<<blocks, 256, 0, stream>>>(x, (float *)out, batch, n_in, padded, scale, offset);
    return cudaGetLastError();
}

// dL/dinput of the identity encoding: dL/dx[i, j] = dL/dy[i, j] * scale (include/encodings/identity.h:91-97).
template <typename DyT>
__global__ void identity_bwd_input_kernel(const DyT *__restrict__ dy, float *__restrict__ dx, size_t batch, int n_in,
                                          int padded, float scale) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= batch * (size_t)n_in) return;
    dx[idx] = (float)dy[(idx / n_in) * padded + idx % n_in] * scale;
}

cudaError_t launch_identity_bwd_input(const void *dy, int dy_dtype, float *dx, size_t batch, int n_in, int padded,
                                      float scale, cudaStream_t stream) {
    const size_t n = batch * (size_t)n_in;
    if (n == 0) return cudaSuccess;
    count_launch();
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (dy_dtype == DT_BF16)
        identity_bwd_input_kernel<<<blocks, 256, 0, stream>>>((const __nv_bfloat16 *)dy, dx, batch, n_in, padded, scale);
    else if (dy_dtype == DT_FP16)
        identity_bwd_input_kernel<<<blocks, 256, 0, stream>>>((const __half *)dy, dx, batch, n_in, padded, scale);
    else
        identity_bwd_input_kernel<<<blocks, 256, 0, stream>>>((const float *)dy, dx, batch, n_in, padded, scale);
    return cudaGetLastError();
}

// Frequency encoding (include/encodings/frequency.h:63-80): column j of input feature j / (2 F) holds
// sin(x * 2^((j / 2) % F) * pi + (j % 2) * pi / 2), i.e. sin / cos pairs of F octaves; padding columns are 1.
// The argument is formed in double precision and rounded to fp32 before the sine, as the reference's
// expression does (its pi is a double constant).
template <typename OutT>
__global__ void frequency_fwd_kernel(const float *__restrict__ x, OutT *__restrict__ out, size_t batch, int n_in,
                                     int n_freq, int padded) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= batch * (size_t)padded) return;
    const size_t row = idx / padded;
    const int col = (int)(idx % padded);
    float v = 1.0f;
    if (col < n_in * n_freq * 2) {
        const int feature = col / (n_freq * 2);
        const int log2_frequency = (col / 2) % n_freq;
        const float phase_shift = (float)((col % 2) * (3.14159265358979323846 / 2.0));
        const float scaled = x[row * n_in + feature] * (float)((size_t)1 << log2_frequency);
        const float arg = (float)__dadd_rn(__dmul_rn((double)scaled, 3.14159265358979323846), (double)phase_shift);
        v = sinf(arg);
    }
    out[idx] = (OutT)v;
}

cudaError_t launch_frequency_fwd(const float *x, void *out, int out_dtype, size_t batch, int n_in, int n_freq, int padded,
                                 cudaStream_t stream) {
    const size_t n = batch * (size_t)padded;
    if (n == 0) return cudaSuccess;
    count_launch();
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (out_dtype == DT_BF16)
        frequency_fwd_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(x, (__nv_bfloat16 *)out, batch, n_in, n_freq, padded);
    else if (out_dtype == DT_FP16)
        frequency_fwd_kernel<__half><<<blocks, 256, 0, stream>>>(x, (__half *)out, batch, n_in, n_freq, padded);
    else
        frequency_fwd_kernel<float><<<blocks, 256, 0, stream>>>(x, (float *)out, batch, n_in, n_freq, padded);
    return cudaGetLastError();
}

// dL/dinput of the frequency encoding (include/encodings/frequency.h:91-131): the reference keeps
// dy/dx = 2^f pi cos(arg) from the forward pass; here it is recomputed from the input, with the same argument
// arithmetic as the forward kernel.  One thread per (row, input feature), sum over its 2 F outputs in column order.
template <typename DyT>
__global__ void frequency_bwd_input_kernel(const float *__restrict__ x, const DyT *__restrict__ dy, float *__restrict__ dx,
                                           size_t batch, int n_in, int n_freq, int padded) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= batch * (size_t)n_in) return;
    const size_t row = idx / n_in;
    const int feature = (int)(idx % n_in);
    const float xv = x[idx];
    float result = 0.0f;
    for (int k = 0; k < 2 * n_freq; ++k) {
        const int col = feature * 2 * n_freq + k;
        const int log2_frequency = (col / 2) % n_freq;
        const float phase_shift = (float)((col % 2) * (3.14159265358979323846 / 2.0));
        const float f = (float)((size_t)1 << log2_frequency);
        const float arg = (float)__dadd_rn(__dmul_rn((double)(xv * f), 3.14159265358979323846), (double)phase_shift);
        const float dy_dx = (float)__dmul_rn((double)f, 3.14159265358979323846) * cosf(arg);
        result += (float)dy[row * padded + col] * dy_dx;
    }
    dx[idx] = result;
}

cudaError_t launch_frequency_bwd_input(const float *x, const void *dy, int dy_dtype, float *dx, size_t batch, int n_in,
                                       int n_freq, int padded, cudaStream_t stream) {
    const size_t n = batch * (size_t)n_in;
    if (n == 0) return cudaSuccess;
    count_launch();
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (dy_dtype == DT_BF16)
        frequency_bwd_input_kernel<<<blocks, 256, 0, stream>>>(x, (const __nv_bfloat16 *)dy, dx, batch, n_in, n_freq, padded);
    else if (dy_dtype == DT_FP16)
        frequency_bwd_input_kernel<<<blocks, 256, 0, stream>>>(x, (const __half *)dy, dx, batch, n_in, n_freq, padded);
    else
        frequency_bwd_input_kernel<<<blocks, 256, 0, stream>>>(x, (const float *)dy, dx, batch, n_in, n_freq, padded);
    return cudaGetLastError();
}

// Spherical-harmonics encoding (include/encodings/spherical_harmonics.h:28-64): the degree^2 real spherical harmonics
// Y_l^m, l < degree, of the direction 2 x - 1, in the order l (l + 1) + m, padded with ones.  The reference evaluates a
// generated table of polynomials (include/common/common_device.h:33-206); the same functions are evaluated here from
// their definition by the recurrences of Sloan, "Stupid Spherical Harmonics Tricks", appendix A1:
//     Y_l^m  = sqrt(2) K_l^m (-1)^m Q_l^m(z) Re (x + i y)^m        m > 0
//     Y_l^-m = sqrt(2) K_l^m (-1)^m Q_l^m(z) Im (x + i y)^m        m > 0
//     Y_l^0  = K_l^0 Q_l^0(z)
// with K_l^m = sqrt((2 l + 1) (l - m)! / (4 pi (l + m)!)) and Q_l^m = d^m P_l / dz^m (Legendre polynomial P_l), built by
//     Q_m^m = (2 m - 1)!!,   Q_(m+1)^m = (2 m + 1) z Q_m^m,   (l - m) Q_l^m = (2 l - 1) z Q_(l-1)^m - (l + m - 1) Q_(l-2)^m.
// Like the reference's polynomials these are functions of z times the real / imaginary part of (x + i y)^m, so the two
// agree for inputs off the unit sphere as well.
constexpr int kMaxShDegree = 8;
struct ShNorm {
    float k[kMaxShDegree][kMaxShDegree]; // k[l][m]: sqrt(2) K_l^m (-1)^m for m > 0, K_l^0 for m = 0
};

static ShNorm make_sh_norm() {
    ShNorm n{};
    for (int l = 0; l < kMaxShDegree; ++l)
        for (int m = 0; m <= l; ++m) {
            double ratio = 1.0; // (l - m)! / (l + m)!
            for (int i = l - m + 1; i <= l + m; ++i) ratio /= (double)i;
            double k = std::sqrt((2.0 * l + 1.0) / (4.0 * 3.14159265358979323846) * ratio);
            if (m > 0) k *= std::sqrt(2.0) * ((m & 1) ? -1.0 : 1.0);
            n.k[l][m] = (float)k;
        }
    return n;
}

template <typename OutT>
__global__ void spherical_harmonics_fwd_kernel(const float *__restrict__ in, OutT *__restrict__ out, size_t batch, int degree,
                                               int padded, const ShNorm norm) {
    const size_t row = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= batch) return;
    const float x = in[row * 3 + 0] * 2.0f - 1.0f, y = in[row * 3 + 1] * 2.0f - 1.0f, z = in[row * 3 + 2] * 2.0f - 1.0f;
    OutT *o = out + row * padded;
    for (int j = degree * degree; j < padded; ++j) o[j] = (OutT)1.0f;
    float c = 1.0f, s = 0.0f; // real and imaginary part of (x + i y)^m
    float qmm = 1.0f;         // Q_m^m = (2 m - 1)!!
#pragma unroll
    for (int m = 0; m < kMaxShDegree; ++m) {
        if (m >= degree) break;
        if (m > 0) {
            const float cn = c * x - s * y;
            s = c * y + s * x;
            c = cn;
            qmm *= (float)(2 * m - 1);
        }
        float q2 = 0.0f, q1 = 0.0f; // Q_(l-2)^m, Q_(l-1)^m
#pragma unroll
        for (int l = m; l < kMaxShDegree; ++l) {
            if (l >= degree) break;
            float q;
            if (l == m)
                q = qmm;
            else if (l == m + 1)
                q = (float)(2 * m + 1) * z * q1;
            else
                q = ((float)(2 * l - 1) * z * q1 - (float)(l + m - 1) * q2) / (float)(l - m);
            q2 = q1;
            q1 = q;
            const float base = norm.k[l][m] * q;
            if (m == 0) {
                o[l * (l + 1)] = (OutT)base;
            } else {
                o[l * (l + 1) + m] = (OutT)(base * c);
                o[l * (l + 1) - m] = (OutT)(base * s);
            }
        }
    }
}

cudaError_t launch_spherical_harmonics_fwd(const float *x, void *out, int out_dtype, size_t batch, int degree, int padded,
                                           cudaStream_t stream) {
    if (batch == 0) return cudaSuccess;
    if (degree < 1 || degree > kMaxShDegree) return cudaErrorInvalidValue;
    static const ShNorm norm = make_sh_norm();
    count_launch();
    const unsigned blocks = (unsigned)((batch + 127) / 128);
    if (out_dtype == DT_BF16)
        spherical_harmonics_fwd_kernel<<<blocks, 128, 0, stream>>>(x, (__nv_bfloat16 *)out, batch, degree, padded, norm);
    else if (out_dtype == DT_FP16)
        spherical_harmonics_fwd_kernel<<<blocks, 128, 0, stream>>>(x, (__half *)out, batch, degree, padded, norm);
    else
        spherical_harmonics_fwd_kernel<<<blocks, 128, 0, stream>>>(x, (float *)out, batch, degree, padded, norm);
    return cudaGetLastError();
}

// L2 loss (include/losses/l2.h:19-41): value = (p - t)^2 / n, grad = scale * 2 (p - t) / n with
// n = batch * stride.  Targets are [batch][n_targets]; prediction columns >= n_targets are padding and
// compare against 0.  Per-block partial sums of the loss values go to `loss_partials` (fixed order).
template <bool H>
__global__ void __launch_bounds__(256)
l2_loss_kernel(const __nv_bfloat16 *__restrict__ pred, const float *__restrict__ target, int n_targets,
               float *__restrict__ values, __nv_bfloat16 *__restrict__ grads, size_t batch, int stride,
               float loss_scale, float *__restrict__ loss_partials) {
    // one thread handles 8 consecutive columns of one row (16 bytes of bf16); stride is a multiple of 16
    const size_t n_el = batch * (size_t)stride;
    const size_t n_vec = n_el / 8;
    const float inv_n = 1.0f / (float)n_el;
    const bool full_targets = n_targets == stride;
    float local = 0.0f;
    for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < n_vec; v += (size_t)gridDim.x * blockDim.x) {
        const size_t idx = v * 8;
        const size_t row = idx / stride;
        const int col = (int)(idx % stride);
        const uint4 p4 = *reinterpret_cast<const uint4 *>(pred + idx);
        const uint32_t pw[4] = {p4.x, p4.y, p4.z, p4.w};
        float t[8];
        if (full_targets) {
            const float4 a = *reinterpret_cast<const float4 *>(target + idx);
            const float4 b = *reinterpret_cast<const float4 *>(target + idx + 4);
            t[0] = a.x, t[1] = a.y, t[2] = a.z, t[3] = a.w, t[4] = b.x, t[5] = b.y, t[6] = b.z, t[7] = b.w;
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) t[j] = (col + j) < n_targets ? target[row * n_targets + col + j] : 0.0f;
        }
        float g[8], val[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float p = (j & 1) ? ptx::hi_f32<H>(pw[j >> 1]) : ptx::lo_f32<H>(pw[j >> 1]);
            const float d = p - t[j];
            val[j] = d * d * inv_n;
            g[j] = loss_scale * 2.0f * d * inv_n;
            local += val[j];
        }
        if (values) {
            *reinterpret_cast<float4 *>(values + idx) = make_float4(val[0], val[1], val[2], val[3]);
            *reinterpret_cast<float4 *>(values + idx + 4) = make_float4(val[4], val[5], val[6], val[7]);
        }
        if (grads)
            *reinterpret_cast<uint4 *>(grads + idx) =
                make_uint4(ptx::pack2<H>(g[0], g[1]), ptx::pack2<H>(g[2], g[3]), ptx::pack2<H>(g[4], g[5]),
                           ptx::pack2<H>(g[6], g[7]));
    }
    __shared__ float red[256];
    red[threadIdx.x] = local;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if ((int)threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0 && loss_partials) loss_partials[blockIdx.x] = red[0];
}

__global__ void sum_partials_kernel(const float *__restrict__ partials, int n, float *__restrict__ out) {
    __shared__ float red[256];
    float local = 0.0f;
    for (int i = threadIdx.x; i < n; i += 256) local += partials[i];
    red[threadIdx.x] = local;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if ((int)threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0) *out = red[0];
}

cudaError_t launch_sum_partials(const float *partials, int n, float *out, cudaStream_t stream) {
    count_launch();
    sum_partials_kernel<<<1, 256, 0, stream>>>(partials, n, out);
    return cudaGetLastError();
}

cudaError_t launch_l2_loss(const __nv_bfloat16 *pred, int fp16, const float *target, int n_targets, float *values,
                           __nv_bfloat16 *grads, size_t batch, int stride, float loss_scale, float *loss_partials,
                           int n_partials, float *loss_sum, cudaStream_t stream) {
    if (batch == 0) return cudaSuccess;
    count_launch(loss_sum && loss_partials ? 2 : 1);
    if (fp16)
        l2_loss_kernel<true><<<n_partials, 256, 0, stream>>>(pred, target, n_targets, values, grads, batch, stride,
                                                             loss_scale, loss_partials);
    else
        l2_loss_kernel<false><<<n_partials, 256, 0, stream>>>(pred, target, n_targets, values, grads, batch, stride,
                                                              loss_scale, loss_partials);
    if (loss_sum && loss_partials) sum_partials_kernel<<<1, 256, 0, stream>>>(loss_partials, n_partials, loss_sum);
    return cudaGetLastError();
}

// Adam with torch.optim.Adam semantics (no weight decay, no amsgrad):
//   m = b1 m + (1-b1) g;  v = b2 v + (1-b2) g^2;  p -= lr * (m / (1-b1^t)) / (sqrt(v / (1-b2^t)) + eps)
// torch evaluates the update as  p -= (lr / bc1) * m / (sqrt(v) / sqrt(bc2) + eps); the same grouping is
// used here.  Optionally refreshes the bf16 working copy in the same pass.
__global__ void adam_kernel(float *__restrict__ p, float *__restrict__ m, float *__restrict__ v,
                            const float *__restrict__ g, size_t n, float grad_scale, float lr, float b1, float b2,
                            float eps, float bc1, float bc2_sqrt, __nv_bfloat16 *__restrict__ p_bf16) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float gi = g[i] * grad_scale;
    const float mi = b1 * m[i] + (1.0f - b1) * gi;
    const float vi = b2 * v[i] + (1.0f - b2) * gi * gi;
    m[i] = mi;
    v[i] = vi;
    const float denom = sqrtf(vi) / bc2_sqrt + eps;
    const float pi = p[i] - (lr / bc1) * (mi / denom);
    p[i] = pi;
    if (p_bf16) p_bf16[i] = __float2bfloat16_rn(pi);
}

// Same update, four parameters per thread with 16-byte accesses (large tables: the step is a pure HBM stream of
// 28 bytes per parameter).  Same per-element arithmetic as adam_kernel.
__global__ void __launch_bounds__(256) adam_vec4_kernel(float4 *__restrict__ p, float4 *__restrict__ m,
                                                        float4 *__restrict__ v, const float4 *__restrict__ g, size_t n4,
                                                        float grad_scale, float lr, float b1, float b2, float eps,
                                                        float bc1, float bc2_sqrt) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n4) return;
    const float4 g4 = g[i];
    float4 m4 = m[i], v4 = v[i], p4 = p[i];
    auto one = [&](float gi, float &mi, float &vi, float &pi) {
        gi *= grad_scale;
        mi = b1 * mi + (1.0f - b1) * gi;
        vi = b2 * vi + (1.0f - b2) * gi * gi;
        const float denom = sqrtf(vi) / bc2_sqrt + eps;
        pi = pi - (lr / bc1) * (mi / denom);
    };
    one(g4.x, m4.x, v4.x, p4.x);
    one(g4.y, m4.y, v4.y, p4.y);
    one(g4.z, m4.z, v4.z, p4.z);
    one(g4.w, m4.w, v4.w, p4.w);
    m[i] = m4;
    v[i] = v4;
    p[i] = p4;
}

cudaError_t launch_adam(float *p, float *m, float *v, const float *g, size_t n, float grad_scale, int step, float lr,
                        float b1, float b2, float eps, __nv_bfloat16 *p_bf16, cudaStream_t stream) {
    if (n == 0) return cudaSuccess;
    const float bc1 = 1.0f - powf(b1, (float)step);
    const float bc2_sqrt = sqrtf(1.0f - powf(b2, (float)step));
    auto aligned16 = [](const void *q) { return reinterpret_cast<uintptr_t>(q) % 16 == 0; };
    size_t done = 0;
    if (!p_bf16 && n >= (1u << 16) && aligned16(p) && aligned16(m) && aligned16(v) && aligned16(g)) {
        const size_t n4 = n / 4;
        count_launch();
        adam_vec4_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, stream>>>(
            reinterpret_cast<float4 *>(p), reinterpret_cast<float4 *>(m), reinterpret_cast<float4 *>(v),
            reinterpret_cast<const float4 *>(g), n4, grad_scale, lr, b1, b2, eps, bc1, bc2_sqrt);
        done = n4 * 4;
    }
    if (done < n) {
        count_launch();
        adam_kernel<<<(unsigned)((n - done + 255) / 256), 256, 0, stream>>>(p + done, m + done, v + done, g + done, n - done,
                                                                        grad_scale, lr, b1, b2, eps, bc1, bc2_sqrt,
                                                                        p_bf16 ? p_bf16 + done : nullptr);
    }
    return cudaGetLastError();
}

template <typename A, typename B> __global__ void convert_kernel(const A *__restrict__ a, B *__restrict__ b, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) b[i] = (B)(float)a[i];
}
cudaError_t launch_f32_to_bf16(const float *a, __nv_bfloat16 *b, size_t n, cudaStream_t s) {
    count_launch(n ? 1 : 0);
    if (n) convert_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(a, b, n);
    return cudaGetLastError();
}
cudaError_t launch_bf16_to_f32(const __nv_bfloat16 *a, float *b, size_t n, cudaStream_t s) {
    count_launch(n ? 1 : 0);
    if (n) convert_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(a, b, n);
    return cudaGetLastError();
}
cudaError_t launch_fp16_to_f32(const void *a, float *b, size_t n, cudaStream_t s) {
    count_launch(n ? 1 : 0);
    if (n) convert_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(reinterpret_cast<const __half *>(a), b, n);
    return cudaGetLastError();
}

} // namespace tnn
