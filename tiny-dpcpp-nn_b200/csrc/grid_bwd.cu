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
                                                               size_t batch) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t NL = p.n_levels;
    const size_t i = idx / NL;
    const uint32_t level = (uint32_t)(idx % NL);
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

template <int D, int F>
static cudaError_t launch_bwd_atomic_df(const GridParams &p, const float *x, const void *dy, int dy_dtype, float *grads,
                                        size_t batch, cudaStream_t stream) {
    const size_t n_params = (size_t)p.offsets[p.n_levels] * F;
    cudaError_t e = cudaMemsetAsync(grads, 0, n_params * sizeof(float), stream); // grid.h:758-762
    if (e != cudaSuccess) return e;
    const size_t n = batch * p.n_levels;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    count_launch();
    if (dy_dtype == 0)
        grid_bwd_atomic_kernel<D, F, __nv_bfloat16><<<blocks, 256, 0, stream>>>(p, x, (const __nv_bfloat16 *)dy, grads, batch);
    else if (dy_dtype == 1)
        grid_bwd_atomic_kernel<D, F, __half><<<blocks, 256, 0, stream>>>(p, x, (const __half *)dy, grads, batch);
    else
        grid_bwd_atomic_kernel<D, F, float><<<blocks, 256, 0, stream>>>(p, x, (const float *)dy, grads, batch);
    return cudaGetLastError();
}

cudaError_t launch_grid_bwd_det(const GridParams &p, const float *x, const void *dy, int dy_dtype, float *grads,
                                size_t batch, void *scratch, size_t scratch_bytes, cudaStream_t stream);

cudaError_t launch_grid_bwd(const GridParams &p, const float *x, const void *dy, int dy_dtype, float *grads,
                            size_t batch, void *scratch, size_t scratch_bytes, cudaStream_t stream) {
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
