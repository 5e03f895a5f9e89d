// Deterministic hash-grid backward (parameter gradients): the reference's scatter with exact accumulation.
//
// The reference adds w_c * dL/dy into the gradient table with fp32 atomics (include/encodings/grid.h:137-245), so
// the rounding of every sum depends on the order in which the additions happen to arrive.  Integer addition has no
// such dependence: here every contribution is converted to 64-bit fixed point with one power-of-two scale for the
// whole call and added with 64-bit integer reductions in memory; the finished sums are converted back to fp32.
// Two runs on the same inputs therefore give identical bits, whatever the scheduling.
//
// The scale is chosen from the largest |dL/dy| of the call so that even a table entry hit by every contribution of
// the batch cannot overflow: with a = max |dy| < 2^e and n = batch * 2^D <= 2^b contributions per level, the scale
// 2^(61 - e - b) keeps every sum below 2^61.  An entry that receives k contributions of typical size loses at
// most k / 2 units of 2^-(61 - e - b), i.e. a relative error far below fp32 rounding.
#include "grid.h"
#include "elementwise.h"
#include "grid_device.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace tnn {

namespace {

struct FixedHeader {
    uint32_t absmax_bits; // max |dy| over the real feature columns, as float bits (non-negative floats order like integers)
    uint32_t non_finite;  // set when dy holds an inf or a NaN: every gradient of the call is then reported as NaN
    uint32_t pad[62];
};

template <typename DyT>
__global__ void __launch_bounds__(256) grid_absmax_kernel(const DyT *__restrict__ dy, size_t batch, uint32_t n_features,
                                                          uint32_t padded, FixedHeader *hdr) {
    float m = 0.0f;
    bool bad = false;
    const size_t n = batch * (size_t)n_features;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / n_features;
        const uint32_t c = (uint32_t)(i % n_features);
        const float v = fabsf((float)dy[r * padded + c]);
        if (v <= 3.0e38f)
            m = fmaxf(m, v); // non-finite values do not take part in choosing the scale
        else
            bad = true;
    }
    // The reference's float atomics (and the default path here) propagate inf / NaN into the gradient; integer
    // accumulation cannot represent them, so the call is flagged and the finalize kernel reports NaN instead of
    // finite garbage (a loss-scale overflow check on the gradients then still fires).
    if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) atomicOr(&hdr->non_finite, 1u);
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0 && m > 0.0f) atomicMax(&hdr->absmax_bits, __float_as_uint(m));
}

// exponent E of the scale 2^E (see the file comment); clamped to what fp32 can represent
__device__ __forceinline__ int fixed_exponent(uint32_t absmax_bits, size_t contributions) {
    const float a = __uint_as_float(absmax_bits);
    if (!(a > 0.0f)) return 0;
    int e;
    frexpf(a, &e); // a = f * 2^e with 0.5 <= f < 1
    const int b = contributions > 1 ? 64 - __clzll((unsigned long long)(contributions - 1)) : 0;
    int E = 61 - e - b;
    return E > 126 ? 126 : (E < -126 ? -126 : E);
}

template <int D, int F, typename DyT>
__global__ void __launch_bounds__(256) grid_bwd_fixed_kernel(const GridParams p, const float *__restrict__ x,
                                                              const DyT *__restrict__ dy, const FixedHeader *hdr,
                                                              unsigned long long *__restrict__ acc, size_t batch,
                                                              uint32_t first_level) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t NL = p.n_levels - first_level; // levels [first_level, n_levels): the coarser ones are privatised
    const size_t i = idx / NL;
    const uint32_t level = first_level + (uint32_t)(idx % NL);
    if (i >= batch) return;
    const float max_level = (p.max_level * (float)p.n_features) / (float)F;
    if ((float)level >= max_level + 1e-3f) return;
    const float scale = ldexpf(1.0f, fixed_exponent(hdr->absmax_bits, batch << D));

    unsigned long long *al = acc + (size_t)p.offsets[level] * F;
    const uint32_t hsize = p.offsets[level + 1] - p.offsets[level];
    const uint32_t res = p.resolution[level];
    float w[D], xin[D];
    uint32_t g[D];
#pragma unroll
    for (int d = 0; d < D; ++d) xin[d] = __ldg(x + i * D + d);
    grid_pos<D>(xin, p.scale[level], p.interpolation, w, g);
    float gr[F];
#pragma unroll
    for (int f = 0; f < F; ++f) gr[f] = (float)dy[i * p.padded_width + level * F + f];

    auto add = [&](uint32_t e, float weight) {
#pragma unroll
        for (int f = 0; f < F; ++f) {
            // the product is rounded to fp32 like the reference's, the scaling by a power of two is exact
            const float prod = __fmul_rn(__fmul_rn(weight, gr[f]), scale);
            const long long q = fabsf(prod) <= 3.0e38f ? __float2ll_rn(prod) : 0ll; // flagged by grid_absmax_kernel
            if (q != 0) atomicAdd(al + (size_t)e * F + f, (unsigned long long)q);
        }
    };
    if (p.interpolation == INTERP_NEAREST) {
        add(grid_index<D>(p.grid_type, p.hash_type, hsize, res, g), 1.0f);
        return;
    }
    uint32_t ent[1 << D];
    float wt[1 << D];
#pragma unroll
    for (int c = 0; c < (1 << D); ++c) {
        float weight = 1.0f;
        uint32_t gc[D];
#pragma unroll
        for (int d = 0; d < D; ++d) {
            if ((c & (1 << d)) == 0) {
                weight = __fmul_rn(weight, __fsub_rn(1.0f, w[d]));
                gc[d] = g[d];
            } else {
                weight = __fmul_rn(weight, w[d]);
                gc[d] = g[d] + 1u;
            }
        }
        wt[c] = weight;
        ent[c] = grid_index_raw<D>(p.grid_type, p.hash_type, hsize, res, gc);
    }
    grid_wrap<(1 << D)>(ent, hsize);
#pragma unroll
    for (int c = 0; c < (1 << D); ++c) add(ent[c], wt[c]);
}

// Levels [0, n_coarse): the same fixed-point sums in per-CTA shared-memory accumulators (see grid_coarse_levels),
// added to the global accumulators once per CTA.  Integer sums: still independent of every order.
template <int D, int F, typename DyT>
__global__ void __launch_bounds__(kGridCoarseThreads) grid_bwd_fixed_coarse_kernel(const GridParams p, const float *__restrict__ x,
                                                                      const DyT *__restrict__ dy, const FixedHeader *hdr,
                                                                      unsigned long long *__restrict__ acc, size_t batch,
                                                                      uint32_t n_coarse) {
    extern __shared__ unsigned long long coarse_fixed[]; // [offsets[n_coarse] * F]
    const uint32_t n_acc = p.offsets[n_coarse] * F;
    for (uint32_t k = threadIdx.x; k < n_acc; k += blockDim.x) coarse_fixed[k] = 0ull;
    __syncthreads();
    const float max_level = (p.max_level * (float)p.n_features) / (float)F;
    const float scale = ldexpf(1.0f, fixed_exponent(hdr->absmax_bits, batch << D));
    const size_t total = batch * n_coarse;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t i = idx / n_coarse;
        const uint32_t level = (uint32_t)(idx % n_coarse);
        if ((float)level >= max_level + 1e-3f) continue;
        uint32_t ent[1 << D];
        float wt[1 << D];
        const int n = grid_corner_entries<D>(p, level, x + i * D, ent, wt);
        float gr[F];
#pragma unroll
        for (int f = 0; f < F; ++f) gr[f] = (float)dy[i * p.padded_width + level * F + f];
        unsigned long long *al = coarse_fixed + (size_t)p.offsets[level] * F;
#pragma unroll
        for (int c = 0; c < (1 << D); ++c) {
            if (c < n) {
#pragma unroll
                for (int f = 0; f < F; ++f) {
                    const float prod = __fmul_rn(__fmul_rn(wt[c], gr[f]), scale);
                    const long long q = fabsf(prod) <= 3.0e38f ? __float2ll_rn(prod) : 0ll;
                    if (q != 0) atomicAdd(al + ent[c] * F + f, (unsigned long long)q);
                }
            }
        }
    }
    __syncthreads();
    for (uint32_t k = threadIdx.x; k < n_acc; k += blockDim.x)
        if (coarse_fixed[k] != 0ull) atomicAdd(acc + k, coarse_fixed[k]);
}

template <int D, int F, typename DyT>
cudaError_t run_fixed_t(const GridParams &p, const float *x, const DyT *dy, FixedHeader *hdr, unsigned long long *acc,
                        size_t batch, unsigned red_blocks, cudaStream_t stream) {
    grid_absmax_kernel<DyT><<<red_blocks ? red_blocks : 1, 256, 0, stream>>>(dy, batch, p.n_features, p.padded_width, hdr);
    count_launch();
    int grid = 0;
    const uint32_t n_coarse = grid_coarse_levels(p, batch, sizeof(unsigned long long), &grid);
    cudaError_t e;
    if (n_coarse > 0) {
        const size_t smem = (size_t)p.offsets[n_coarse] * F * sizeof(unsigned long long);
        auto kern = grid_bwd_fixed_coarse_kernel<D, F, DyT>;
        if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return e;
        count_launch();
        kern<<<grid, kGridCoarseThreads, smem, stream>>>(p, x, dy, hdr, acc, batch, n_coarse);
    }
    if (n_coarse < p.n_levels) {
        const size_t n = batch * (p.n_levels - n_coarse);
        count_launch();
        grid_bwd_fixed_kernel<D, F, DyT><<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(p, x, dy, hdr, acc, batch, n_coarse);
    }
    return cudaGetLastError();
}

__global__ void __launch_bounds__(256) grid_fixed_finalize_kernel(const unsigned long long *__restrict__ acc,
                                                                   const FixedHeader *hdr, float *__restrict__ grads,
                                                                   size_t n, size_t contributions) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const double inv_scale = ldexp(1.0, -fixed_exponent(hdr->absmax_bits, contributions));
    grads[i] = hdr->non_finite ? __int_as_float(0x7FC00000) : (float)((double)(long long)acc[i] * inv_scale);
}

template <int D, int F>
cudaError_t run_fixed(const GridParams &p, const float *x, const void *dy, int dy_dtype, float *grads, size_t batch,
                      void *scratch, size_t scratch_bytes, cudaStream_t stream) {
    const size_t n_params = (size_t)p.offsets[p.n_levels] * F;
    if (scratch_bytes < sizeof(FixedHeader) + n_params * sizeof(unsigned long long)) return cudaErrorInvalidValue;
    FixedHeader *hdr = reinterpret_cast<FixedHeader *>(scratch);
    unsigned long long *acc = reinterpret_cast<unsigned long long *>(hdr + 1);
    cudaError_t e = cudaMemsetAsync(scratch, 0, sizeof(FixedHeader) + n_params * sizeof(unsigned long long), stream);
    if (e != cudaSuccess) return e;
    const size_t n_dy = batch * (size_t)p.n_features;
    const unsigned red_blocks = (unsigned)((n_dy + 256 * 8 - 1) / (256 * 8) < 148 * 8 ? (n_dy + 256 * 8 - 1) / (256 * 8) : 148 * 8);
    if (dy_dtype == 0)
        e = run_fixed_t<D, F>(p, x, (const __nv_bfloat16 *)dy, hdr, acc, batch, red_blocks, stream);
    else if (dy_dtype == 1)
        e = run_fixed_t<D, F>(p, x, (const __half *)dy, hdr, acc, batch, red_blocks, stream);
    else
        e = run_fixed_t<D, F>(p, x, (const float *)dy, hdr, acc, batch, red_blocks, stream);
    if (e != cudaSuccess) return e;
    count_launch();
    grid_fixed_finalize_kernel<<<(unsigned)((n_params + 255) / 256), 256, 0, stream>>>(acc, hdr, grads, n_params,
                                                                                      batch << D);
    return cudaGetLastError();
}

} // namespace

size_t grid_bwd_segmented_scratch_bytes(const GridParams &p, size_t batch);

size_t grid_bwd_scratch_bytes(const GridParams &p, size_t batch, int mode) {
    if (mode == GRID_BWD_ATOMIC) return 0;
    if (mode == GRID_BWD_SEGMENTED) return grid_bwd_segmented_scratch_bytes(p, batch);
    return sizeof(FixedHeader) + (size_t)p.offsets[p.n_levels] * p.features_per_level * sizeof(unsigned long long);
}

cudaError_t launch_grid_bwd_det(const GridParams &p, const float *x, const void *dy, int dy_dtype, float *grads,
                                size_t batch, void *scratch, size_t scratch_bytes, cudaStream_t stream) {
    const int key = (int)p.n_dims * 16 + (int)p.features_per_level;
    switch (key) {
    case 2 * 16 + 1: return run_fixed<2, 1>(p, x, dy, dy_dtype, grads, batch, scratch, scratch_bytes, stream);
    case 2 * 16 + 2: return run_fixed<2, 2>(p, x, dy, dy_dtype, grads, batch, scratch, scratch_bytes, stream);
    case 2 * 16 + 4: return run_fixed<2, 4>(p, x, dy, dy_dtype, grads, batch, scratch, scratch_bytes, stream);
    case 2 * 16 + 8: return run_fixed<2, 8>(p, x, dy, dy_dtype, grads, batch, scratch, scratch_bytes, stream);
    case 3 * 16 + 1: return run_fixed<3, 1>(p, x, dy, dy_dtype, grads, batch, scratch, scratch_bytes, stream);
    case 3 * 16 + 2: return run_fixed<3, 2>(p, x, dy, dy_dtype, grads, batch, scratch, scratch_bytes, stream);
    case 3 * 16 + 4: return run_fixed<3, 4>(p, x, dy, dy_dtype, grads, batch, scratch, scratch_bytes, stream);
    case 3 * 16 + 8: return run_fixed<3, 8>(p, x, dy, dy_dtype, grads, batch, scratch, scratch_bytes, stream);
    default: return cudaErrorInvalidValue;
    }
}

} // namespace tnn
