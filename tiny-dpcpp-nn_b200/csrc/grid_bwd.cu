// Hash-grid parameter-gradient backward (reference kernel_grid_backward, include/encodings/grid.h:137-245).
//
// Two implementations of the same sum  grad[l][index(g + c)][f] += w_c * dL/dy[i, l F + f]:
//   * an atomic scatter with the reference's structure (fp32 atomics, summation order not fixed), and
//   * the same scatter with 64-bit fixed-point integer reductions (grid_bwd_fixed.cu): order-independent, so two runs
//     give identical bits; chosen with `deterministic` in the C ABI.
#include "grid.h"
#include "elementwise.h"
#include "grid_device.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace tnn {

// grad[0..F) += v[0..F) at one table entry.  sm_90+ has vector reductions: one `red` per 2 or 4 features instead
// of one per feature (each element is still added atomically on its own; entries are F * 4 bytes apart, so the
// vector forms are naturally aligned).
template <int F> __device__ __forceinline__ void red_add_entry(float *dst, const float (&v)[F]) {
    if constexpr (F % 4 == 0) {
#pragma unroll
        for (int f = 0; f < F; f += 4)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + f), "f"(v[f]), "f"(v[f + 1]),
                         "f"(v[f + 2]), "f"(v[f + 3])
                         : "memory");
    } else if constexpr (F % 2 == 0) {
#pragma unroll
        for (int f = 0; f < F; f += 2)
            asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(dst + f), "f"(v[f]), "f"(v[f + 1]) : "memory");
    } else {
#pragma unroll
        for (int f = 0; f < F; ++f) atomicAdd(dst + f, v[f]);
    }
}

template <int D, int F, typename DyT>
__global__ void __launch_bounds__(256) grid_bwd_atomic_kernel(const GridParams p, const float *__restrict__ x,
                                                               const DyT *__restrict__ dy, float *__restrict__ grads,
                                                               size_t batch, uint32_t first_level) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t NL = p.n_levels - first_level; // levels [first_level, n_levels): the coarser ones are privatised
    const size_t i = idx / NL;
    const uint32_t level = first_level + (uint32_t)(idx % NL);
    if (i >= batch) return;
    const float max_level = (p.max_level * (float)p.n_features) / (float)F;
    if ((float)level >= max_level + 1e-3f) return;

    float *gl = grads + (size_t)p.offsets[level] * F;
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

    if (p.interpolation == INTERP_NEAREST) {
        const uint32_t e = grid_index<D>(p.grid_type, p.hash_type, hsize, res, g);
        red_add_entry<F>(gl + (size_t)e * F, gr);
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
    for (int c = 0; c < (1 << D); ++c) {
        const uint32_t e = ent[c];
        float contrib[F];
#pragma unroll
        for (int f = 0; f < F; ++f) contrib[f] = __fmul_rn(wt[c], gr[f]);
        if constexpr (F == 2) {
            // corners c and c + 1 (c even) are often the two entries of one aligned 16-byte pair: one reduction for both
            if ((c & 1) == 0) {
                const uint32_t e1 = ent[c + 1];
                const float n0 = __fmul_rn(wt[c + 1], gr[0]), n1 = __fmul_rn(wt[c + 1], gr[1]);
                if ((e ^ e1) == 1u) {
                    const bool odd = e & 1u;
                    const float both[4] = {odd ? n0 : contrib[0], odd ? n1 : contrib[1], odd ? contrib[0] : n0,
                                           odd ? contrib[1] : n1};
                    red_add_entry<4>(gl + (size_t)(e & ~1u) * 2, both);
                } else {
                    const float next[2] = {n0, n1};
                    red_add_entry<2>(gl + (size_t)e * 2, contrib);
                    red_add_entry<2>(gl + (size_t)e1 * 2, next);
                }
            }
        } else {
            red_add_entry<F>(gl + (size_t)e * F, contrib);
        }
    }
}

// Levels [0, n_coarse): per-CTA accumulators in shared memory (see grid_coarse_levels), added to the table gradient
// once per CTA.  One CTA per SM walks over (sample, level) pairs.
template <int D, int F, typename DyT>
__global__ void __launch_bounds__(kGridCoarseThreads) grid_bwd_coarse_kernel(const GridParams p, const float *__restrict__ x,
                                                                const DyT *__restrict__ dy, float *__restrict__ grads,
                                                                size_t batch, uint32_t n_coarse) {
    extern __shared__ float coarse_acc[]; // [offsets[n_coarse] * F]
    const uint32_t n_acc = p.offsets[n_coarse] * F;
    for (uint32_t k = threadIdx.x; k < n_acc; k += blockDim.x) coarse_acc[k] = 0.0f;
    __syncthreads();
    const float max_level = (p.max_level * (float)p.n_features) / (float)F;
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
        float *al = coarse_acc + (size_t)p.offsets[level] * F;
#pragma unroll
        for (int c = 0; c < (1 << D); ++c) {
            if (c < n) {
#pragma unroll
                for (int f = 0; f < F; ++f) atomicAdd(al + ent[c] * F + f, __fmul_rn(wt[c], gr[f]));
            }
        }
    }
    __syncthreads();
    // (offsets[0] = 0: the coarse levels are the first n_acc floats of the gradient)
    if constexpr (F % 2 == 0) {
        for (uint32_t k = threadIdx.x; k < n_acc / 2; k += blockDim.x) {
            const float v[2] = {coarse_acc[2 * k], coarse_acc[2 * k + 1]};
            if (v[0] != 0.0f || v[1] != 0.0f) red_add_entry<2>(grads + 2 * (size_t)k, v);
        }
    } else {
        for (uint32_t k = threadIdx.x; k < n_acc; k += blockDim.x)
            if (coarse_acc[k] != 0.0f) atomicAdd(grads + k, coarse_acc[k]);
    }
}

template <int D, int F, typename DyT>
static cudaError_t launch_bwd_atomic_t(const GridParams &p, const float *x, const DyT *dy, float *grads, size_t batch,
                                       cudaStream_t stream) {
    int grid = 0;
    const uint32_t n_coarse = grid_coarse_levels(p, batch, sizeof(float), &grid);
    cudaError_t e;
    if (n_coarse > 0) {
        const size_t smem = (size_t)p.offsets[n_coarse] * F * sizeof(float);
        auto kern = grid_bwd_coarse_kernel<D, F, DyT>;
        if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return e;
        count_launch();
        kern<<<grid, kGridCoarseThreads, smem, stream>>>(p, x, dy, grads, batch, n_coarse);
    }
    if (n_coarse < p.n_levels) {
        const size_t n = batch * (p.n_levels - n_coarse);
        count_launch();
        grid_bwd_atomic_kernel<D, F, DyT><<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(p, x, dy, grads, batch, n_coarse);
    }
    return cudaGetLastError();
}

template <int D, int F>
static cudaError_t launch_bwd_atomic_df(const GridParams &p, const float *x, const void *dy, int dy_dtype, float *grads,
                                        size_t batch, cudaStream_t stream) {
    const size_t n_params = (size_t)p.offsets[p.n_levels] * F;
    cudaError_t e = cudaMemsetAsync(grads, 0, n_params * sizeof(float), stream); // grid.h:758-762
    if (e != cudaSuccess) return e;
    if (batch == 0) return cudaSuccess;
    if (dy_dtype == 0) return launch_bwd_atomic_t<D, F>(p, x, (const __nv_bfloat16 *)dy, grads, batch, stream);
    if (dy_dtype == 1) return launch_bwd_atomic_t<D, F>(p, x, (const __half *)dy, grads, batch, stream);
    return launch_bwd_atomic_t<D, F>(p, x, (const float *)dy, grads, batch, stream);
}

cudaError_t launch_grid_bwd_det(const GridParams &p, const float *x, const void *dy, int dy_dtype, float *grads,
                                size_t batch, void *scratch, size_t scratch_bytes, cudaStream_t stream);

cudaError_t launch_grid_bwd_segmented(const GridParams &p, const float *x, const void *dy, int dy_dtype, float *grads,
                                      size_t batch, void *scratch, size_t scratch_bytes, cudaStream_t stream);

cudaError_t launch_grid_bwd(const GridParams &p, const float *x, const void *dy, int dy_dtype, float *grads,
                            size_t batch, void *scratch, size_t scratch_bytes, cudaStream_t stream, int mode) {
    if (scratch && mode == GRID_BWD_SEGMENTED)
        return launch_grid_bwd_segmented(p, x, dy, dy_dtype, grads, batch, scratch, scratch_bytes, stream);
    if (scratch) return launch_grid_bwd_det(p, x, dy, dy_dtype, grads, batch, scratch, scratch_bytes, stream);
    const int key = (int)p.n_dims * 16 + (int)p.features_per_level;
    switch (key) {
    case 2 * 16 + 1: return launch_bwd_atomic_df<2, 1>(p, x, dy, dy_dtype, grads, batch, stream);
    case 2 * 16 + 2: return launch_bwd_atomic_df<2, 2>(p, x, dy, dy_dtype, grads, batch, stream);
    case 2 * 16 + 4: return launch_bwd_atomic_df<2, 4>(p, x, dy, dy_dtype, grads, batch, stream);
    case 2 * 16 + 8: return launch_bwd_atomic_df<2, 8>(p, x, dy, dy_dtype, grads, batch, stream);
    case 3 * 16 + 1: return launch_bwd_atomic_df<3, 1>(p, x, dy, dy_dtype, grads, batch, stream);
    case 3 * 16 + 2: return launch_bwd_atomic_df<3, 2>(p, x, dy, dy_dtype, grads, batch, stream);
    case 3 * 16 + 4: return launch_bwd_atomic_df<3, 4>(p, x, dy, dy_dtype, grads, batch, stream);
    case 3 * 16 + 8: return launch_bwd_atomic_df<3, 8>(p, x, dy, dy_dtype, grads, batch, stream);
    default: return cudaErrorInvalidValue;
    }
}

} // namespace tnn
