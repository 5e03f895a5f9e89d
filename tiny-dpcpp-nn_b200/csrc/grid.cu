// Multi-resolution hash-grid encoding for sm_100a: forward gather + interpolation and the
// parameter-gradient backward.
//
// Follows the arithmetic of the reference kernels (include/encodings/grid.h:37-245,
// include/common/common_device.h:700-775) operation by operation: fp32 throughout, the same
// fma order over the 2^D corners, and 32-bit unsigned index arithmetic *with wrap-around* -
// on fine levels the dense stride overflows to 0, the hash branch is then not taken and the
// index degenerates; the reference's known-answer vector depends on exactly that.
//
// Thread mapping (forward): consecutive lanes take consecutive *levels* of the same sample,
// so the F features of all levels of one sample are written as one contiguous segment and
// the only uncoalesced traffic is the unavoidable random gather from the tables.
#include "grid.h"
#include "elementwise.h"
#include "grid_device.cuh"

#include <cmath>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <limits>
#include <type_traits>

namespace tnn {

// ------------------------------------------------------------------ level table (host)
static uint32_t powi_u32(uint32_t base, uint32_t e) {
    uint32_t r = 1;
    for (uint32_t i = 0; i < e; ++i) r *= base; // wraps like the reference (common.h:58-65)
    return r;
}

uint32_t grid_build_level_table(GridParams &p, uint32_t log2_hashmap_size) {
    uint32_t offset = 0;
    for (uint32_t l = 0; l < p.n_levels; ++l) {
        const float scale = std::exp2((float)l * p.log2_per_level_scale) * (float)p.base_resolution - 1.0f;
        const uint32_t res = (uint32_t)std::ceil(scale) + 1u;
        p.scale[l] = scale;
        p.resolution[l] = res;
        const uint32_t max_params = std::numeric_limits<uint32_t>::max() / 2;
        uint32_t n = std::pow((float)res, (float)p.n_dims) > (float)max_params ? max_params : powi_u32(res, p.n_dims);
        n = (n + 7u) / 8u * 8u;
        if (p.grid_type == GRID_TILED)
            n = std::min(n, powi_u32(p.base_resolution, p.n_dims));
        else if (p.grid_type == GRID_HASH)
            n = std::min(n, 1u << log2_hashmap_size);
        p.offsets[l] = offset;
        offset += n;
    }
    p.offsets[p.n_levels] = offset;
    return offset;
}

// ------------------------------------------------------------------ forward
template <int D, int F, typename OutT>
__global__ void __launch_bounds__(256) grid_fwd_kernel(const GridParams p, const float *__restrict__ x,
                                                        const float *__restrict__ table, OutT *__restrict__ out,
                                                        size_t batch) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t NL = p.n_levels;
    const size_t i = idx / NL;
    const uint32_t level = (uint32_t)(idx % NL);
    if (i >= batch) return;
    OutT *orow = out + i * p.padded_width;

    // zero the padding columns, spread over the levels of the sample (grid.h:683-694)
    for (uint32_t c = p.n_features + level * F; c < p.padded_width; c += NL * F)
#pragma unroll
        for (int f = 0; f < F; ++f)
            if (c + f < p.padded_width) orow[c + f] = (OutT)0.0f;

    float res_v[F];
#pragma unroll
    for (int f = 0; f < F; ++f) res_v[f] = 0.0f;

    const float max_level = (p.max_level * (float)p.n_features) / (float)F;
    if (!((float)level >= max_level + 1e-3f)) {
        const float *tl = table + (size_t)p.offsets[level] * F;
        const uint32_t hsize = p.offsets[level + 1] - p.offsets[level];
        const uint32_t res = p.resolution[level];
        float w[D];
        uint32_t g[D];
        float xin[D];
#pragma unroll
        for (int d = 0; d < D; ++d) xin[d] = __ldg(x + i * D + d);
        grid_pos<D>(xin, p.scale[level], p.interpolation, w, g);

        if (p.interpolation == INTERP_NEAREST) {
            const uint32_t e = grid_index<D>(p.grid_type, p.hash_type, hsize, res, g);
#pragma unroll
            for (int f = 0; f < F; ++f) res_v[f] = __ldg(tl + (size_t)e * F + f);
        } else {
            // issue all 2^D gathers first, then combine in corner order 0..2^D-1 (grid.h:114-129)
            float vals[1 << D][F];
            float wt[1 << D];
            uint32_t ent[1 << D];
#pragma unroll
            for (int c = 0; c < (1 << D); ++c) {
                float weight = 1.0f;
                uint32_t gl[D];
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    if ((c & (1 << d)) == 0) {
                        weight = __fmul_rn(weight, __fsub_rn(1.0f, w[d]));
                        gl[d] = g[d];
                    } else {
                        weight = __fmul_rn(weight, w[d]);
                        gl[d] = g[d] + 1u;
                    }
                }
                wt[c] = weight;
                ent[c] = grid_index_raw<D>(p.grid_type, p.hash_type, hsize, res, gl);
            }
            grid_wrap<(1 << D)>(ent, hsize);
#pragma unroll
            for (int c = 0; c < (1 << D); ++c) {
                const uint32_t e = ent[c];
                if constexpr (F == 2) {
                    const float2 v = __ldg(reinterpret_cast<const float2 *>(tl) + e);
                    vals[c][0] = v.x;
                    vals[c][1] = v.y;
                } else if constexpr (F == 4) {
                    const float4 v = __ldg(reinterpret_cast<const float4 *>(tl) + e);
                    vals[c][0] = v.x, vals[c][1] = v.y, vals[c][2] = v.z, vals[c][3] = v.w;
                } else {
#pragma unroll
                    for (int f = 0; f < F; ++f) vals[c][f] = __ldg(tl + (size_t)e * F + f);
                }
            }
#pragma unroll
            for (int c = 0; c < (1 << D); ++c)
#pragma unroll
                for (int f = 0; f < F; ++f) res_v[f] = fmaf(wt[c], vals[c][f], res_v[f]);
        }
    }
    // A level's two features go out as one vector store when every row starts on a vector boundary: an even padded
    // width and a base pointer aligned to two elements (uniform over the launch).  Odd widths use scalar stores.
    const bool vec2 = F == 2 && (p.padded_width & 1u) == 0u && (reinterpret_cast<uintptr_t>(out) % (2 * sizeof(OutT))) == 0;
    if (vec2) {
        if constexpr (std::is_same<OutT, __nv_bfloat16>::value)
            *reinterpret_cast<__nv_bfloat162 *>(orow + level * F) = __floats2bfloat162_rn(res_v[0], res_v[1]);
        else if constexpr (std::is_same<OutT, __half>::value)
            *reinterpret_cast<__half2 *>(orow + level * F) = __floats2half2_rn(res_v[0], res_v[F > 1 ? 1 : 0]);
        else
            *reinterpret_cast<float2 *>(orow + level * F) = make_float2(res_v[0], res_v[F > 1 ? 1 : 0]);
    } else {
#pragma unroll
        for (int f = 0; f < F; ++f) orow[level * F + f] = (OutT)res_v[f];
    }
}

// ------------------------------------------------------------------ forward, tiled
// Same values as grid_fwd_kernel with a mapping that keeps every table parameter warp-uniform: a block owns a tile of
// 128 consecutive samples; a warp takes 32 of them at ONE level at a time (two warps share a 32-sample group and split
// its levels), so offsets / scale / resolution come out of the constant bank with a single address per warp and the
// only divergent traffic is the gather itself.  The features go to a shared-memory image of the tile's output rows
// (row stride padded to an odd number of words: the 32 lanes of a warp write 32 different rows) and leave as one
// contiguous, fully coalesced copy.  (Measured at the benchmark grid, batch 2^20: 40 registers, six blocks per SM.
// Forcing eight blocks per SM with a 32-register bound was 5 - 10 % slower.)
constexpr int kGridTileRows = 128;
__host__ __device__ inline uint32_t grid_tile_row_words(uint32_t padded_width, uint32_t elem_bytes) {
    return ((padded_width * elem_bytes + 3u) / 4u) | 1u;
}

template <int D, int F, typename OutT>
__global__ void __launch_bounds__(256) grid_fwd_tile_kernel(const GridParams p, const float *__restrict__ x,
                                                             const float *__restrict__ table, OutT *__restrict__ out,
                                                             size_t batch) {
    extern __shared__ uint32_t stage_words[];
    const uint32_t row_words = grid_tile_row_words(p.padded_width, sizeof(OutT));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = (warp & 3) * 32 + lane;
    const size_t tile0 = (size_t)blockIdx.x * kGridTileRows;
    const size_t i = tile0 + row;
    OutT *srow = reinterpret_cast<OutT *>(stage_words + (size_t)row * row_words);
    // padding columns of the tile are zero (grid.h:683-694)
    const uint32_t n_pad = p.padded_width - p.n_features;
    for (uint32_t k = threadIdx.x; k < kGridTileRows * n_pad; k += blockDim.x)
        reinterpret_cast<OutT *>(stage_words + (size_t)(k / n_pad) * row_words)[p.n_features + k % n_pad] = (OutT)0.0f;
    if (i < batch) {
        float xin[D];
#pragma unroll
        for (int d = 0; d < D; ++d) xin[d] = __ldg(x + i * D + d);
        const GridCommon gc = grid_common(p);
#pragma unroll 2
        for (uint32_t level = (uint32_t)(warp >> 2); level < p.n_levels; level += 2) {
            float res_v[F];
            grid_level_features<D, F>(gc, grid_level_info(p, level), level, table, xin, res_v);
            if constexpr (F == 2 && sizeof(OutT) == 2) {
                uint32_t packed;
                if constexpr (std::is_same<OutT, __half>::value) {
                    const __half2 h = __floats2half2_rn(res_v[0], res_v[1]);
                    memcpy(&packed, &h, 4);
                } else {
                    const __nv_bfloat162 h = __floats2bfloat162_rn(res_v[0], res_v[1]);
                    memcpy(&packed, &h, 4);
                }
                reinterpret_cast<uint32_t *>(srow)[level] = packed;
            } else {
#pragma unroll
                for (int f = 0; f < F; ++f) srow[level * F + f] = (OutT)res_v[f];
            }
        }
    }
    __syncthreads();
    // copy-out: the tile's rows are contiguous in the output
    const size_t rows_here = batch - tile0 < (size_t)kGridTileRows ? batch - tile0 : (size_t)kGridTileRows;
    const uint32_t row_bytes = p.padded_width * (uint32_t)sizeof(OutT);
    OutT *gout = out + tile0 * p.padded_width;
    if ((row_bytes & 3u) == 0u && (reinterpret_cast<uintptr_t>(out) & 3u) == 0u) {
        const uint32_t wpr = row_bytes >> 2;
        uint32_t *gw = reinterpret_cast<uint32_t *>(gout);
        for (uint32_t k = threadIdx.x; k < (uint32_t)rows_here * wpr; k += blockDim.x)
            gw[k] = stage_words[(size_t)(k / wpr) * row_words + k % wpr];
    } else {
        for (uint32_t k = threadIdx.x; k < (uint32_t)rows_here * p.padded_width; k += blockDim.x)
            gout[k] = reinterpret_cast<const OutT *>(stage_words + (size_t)(k / p.padded_width) * row_words)[k % p.padded_width];
    }
}

// ------------------------------------------------------------------ dL/dinput
// Gradient of the encoding with respect to the input positions (the product the reference's kernel_grid_backward_input
// forms from a stored dy/dx, include/encodings/grid.h:247-268; its forward pass never fills that context - grid.h:669-670
// - so the derivative is taken here directly from the interpolation formula):
//     dL/dx_d = sum_l scale_l sum_f dL/dy[l F + f] sum_c (d w_c / d pos_d) table_l[index(g + c)][f],
//     d w_c / d pos_d = (c_d ? +1 : -1) prod_(e != d) (c_e ? w_e : 1 - w_e)   (times 6 p (1 - p) with smoothstep).
// One thread per sample walks the levels in order (fixed summation order).  Nearest interpolation has no gradient.
template <int D, int F, typename DyT>
__global__ void __launch_bounds__(256) grid_bwd_input_kernel(const GridParams p, const float *__restrict__ x,
                                                              const float *__restrict__ table, const DyT *__restrict__ dy,
                                                              float *__restrict__ dx, size_t batch) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= batch) return;
    float xin[D], acc[D];
#pragma unroll
    for (int d = 0; d < D; ++d) {
        xin[d] = __ldg(x + i * D + d);
        acc[d] = 0.0f;
    }
    const float max_level = (p.max_level * (float)p.n_features) / (float)F;
    if (p.interpolation != INTERP_NEAREST) {
        for (uint32_t level = 0; level < p.n_levels; ++level) {
            if ((float)level >= max_level + 1e-3f) break;
            const float *tl = table + (size_t)p.offsets[level] * F;
            const uint32_t hsize = p.offsets[level + 1] - p.offsets[level];
            const uint32_t res = p.resolution[level];
            const float scale = p.scale[level];
            float w[D], dw[D];
            uint32_t g[D];
#pragma unroll
            for (int d = 0; d < D; ++d) {
                float pos = fmaf(scale, xin[d], 0.5f);
                const float fl = floorf(pos);
                g[d] = (uint32_t)(int)fl;
                pos -= fl;
                if (p.interpolation == INTERP_SMOOTHSTEP) {
                    dw[d] = 6.0f * pos * (1.0f - pos);
                    pos = pos * pos * (3.0f - 2.0f * pos);
                } else {
                    dw[d] = 1.0f;
                }
                w[d] = pos;
            }
            float gr[F];
#pragma unroll
            for (int f = 0; f < F; ++f) gr[f] = (float)dy[i * p.padded_width + level * F + f];
            uint32_t ent[1 << D];
#pragma unroll
            for (int c = 0; c < (1 << D); ++c) {
                uint32_t gl[D];
#pragma unroll
                for (int d = 0; d < D; ++d) gl[d] = g[d] + ((c >> d) & 1u);
                ent[c] = grid_index_raw<D>(p.grid_type, p.hash_type, hsize, res, gl);
            }
            grid_wrap<(1 << D)>(ent, hsize);
#pragma unroll
            for (int c = 0; c < (1 << D); ++c) {
                float v = 0.0f; // dL/dy . table entry
#pragma unroll
                for (int f = 0; f < F; ++f) v = fmaf(gr[f], __ldg(tl + (size_t)ent[c] * F + f), v);
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    float wd = ((c >> d) & 1) ? dw[d] : -dw[d];
#pragma unroll
                    for (int e = 0; e < D; ++e)
                        if (e != d) wd *= ((c >> e) & 1) ? w[e] : 1.0f - w[e];
                    acc[d] = fmaf(scale * wd, v, acc[d]);
                }
            }
        }
    }
#pragma unroll
    for (int d = 0; d < D; ++d) dx[i * D + d] = acc[d];
}

template <int D, int F>
static cudaError_t launch_bwd_input_df(const GridParams &p, const float *x, const float *table, const void *dy,
                                       int dy_dtype, float *dx, size_t batch, cudaStream_t stream) {
    const unsigned blocks = (unsigned)((batch + 255) / 256);
    count_launch();
    if (dy_dtype == 0)
        grid_bwd_input_kernel<D, F, __nv_bfloat16><<<blocks, 256, 0, stream>>>(p, x, table, (const __nv_bfloat16 *)dy, dx, batch);
    else if (dy_dtype == 1)
        grid_bwd_input_kernel<D, F, __half><<<blocks, 256, 0, stream>>>(p, x, table, (const __half *)dy, dx, batch);
    else
        grid_bwd_input_kernel<D, F, float><<<blocks, 256, 0, stream>>>(p, x, table, (const float *)dy, dx, batch);
    return cudaGetLastError();
}

template <int D, int F>
static cudaError_t launch_fwd_df(const GridParams &p, const float *x, const float *table, void *out, int out_dtype,
                                 size_t batch, cudaStream_t stream) {
    count_launch();
    const uint32_t elem = out_dtype == 2 ? 4u : 2u;
    const size_t stage_bytes = (size_t)kGridTileRows * grid_tile_row_words(p.padded_width, elem) * 4;
    if (stage_bytes <= 48 * 1024 && p.n_levels >= 2) {
        const unsigned blocks = (unsigned)((batch + kGridTileRows - 1) / kGridTileRows);
        if (out_dtype == 0)
            grid_fwd_tile_kernel<D, F, __nv_bfloat16><<<blocks, 256, stage_bytes, stream>>>(p, x, table, (__nv_bfloat16 *)out, batch);
        else if (out_dtype == 1)
            grid_fwd_tile_kernel<D, F, __half><<<blocks, 256, stage_bytes, stream>>>(p, x, table, (__half *)out, batch);
        else
            grid_fwd_tile_kernel<D, F, float><<<blocks, 256, stage_bytes, stream>>>(p, x, table, (float *)out, batch);
        return cudaGetLastError();
    }
    // very wide outputs (or a single level): one thread per (sample, level), stores straight to global memory
    const size_t n = batch * p.n_levels;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (out_dtype == 0)
        grid_fwd_kernel<D, F, __nv_bfloat16><<<blocks, 256, 0, stream>>>(p, x, table, (__nv_bfloat16 *)out, batch);
    else if (out_dtype == 1)
        grid_fwd_kernel<D, F, __half><<<blocks, 256, 0, stream>>>(p, x, table, (__half *)out, batch);
    else
        grid_fwd_kernel<D, F, float><<<blocks, 256, 0, stream>>>(p, x, table, (float *)out, batch);
    return cudaGetLastError();
}

#define TNN_GRID_DISPATCH(FN, ...)                                                                                     \
    do {                                                                                                               \
        const int key = (int)p.n_dims * 16 + (int)p.features_per_level;                                                \
        switch (key) {                                                                                                 \
        case 2 * 16 + 1: return FN<2, 1>(__VA_ARGS__);                                                                 \
        case 2 * 16 + 2: return FN<2, 2>(__VA_ARGS__);                                                                 \
        case 2 * 16 + 4: return FN<2, 4>(__VA_ARGS__);                                                                 \
        case 2 * 16 + 8: return FN<2, 8>(__VA_ARGS__);                                                                 \
        case 3 * 16 + 1: return FN<3, 1>(__VA_ARGS__);                                                                 \
        case 3 * 16 + 2: return FN<3, 2>(__VA_ARGS__);                                                                 \
        case 3 * 16 + 4: return FN<3, 4>(__VA_ARGS__);                                                                 \
        case 3 * 16 + 8: return FN<3, 8>(__VA_ARGS__);                                                                 \
        default: return cudaErrorInvalidValue;                                                                         \
        }                                                                                                              \
    } while (0)

cudaError_t launch_grid_bwd_input(const GridParams &p, const float *x, const float *table, const void *dy, int dy_dtype,
                                  float *dx, size_t batch, cudaStream_t stream);

cudaError_t launch_grid_fwd(const GridParams &p, const float *x, const float *table, void *out, int out_dtype,
                            size_t batch, cudaStream_t stream) {
    if (batch == 0) return cudaSuccess;
    TNN_GRID_DISPATCH(launch_fwd_df, p, x, table, out, out_dtype, batch, stream);
}

cudaError_t launch_grid_bwd_input(const GridParams &p, const float *x, const float *table, const void *dy, int dy_dtype,
                                  float *dx, size_t batch, cudaStream_t stream) {
    if (batch == 0) return cudaSuccess;
    TNN_GRID_DISPATCH(launch_bwd_input_df, p, x, table, dy, dy_dtype, dx, batch, stream);
}

uint32_t grid_coarse_levels(const GridParams &p, size_t batch, size_t acc_bytes, int *grid_out) {
    static int sm_count[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    if (sm_count[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 0;
        sm_count[dev] = n;
    }
    const int grid = sm_count[dev];
    *grid_out = grid;
    const size_t smem_budget = 160 * 1024;
    const size_t contributions = batch << p.n_dims; // per level
    uint32_t n = 0;
    while (n < p.n_levels) {
        const size_t entries_upto = p.offsets[n + 1];
        const size_t entries_here = p.offsets[n + 1] - p.offsets[n];
        if (entries_upto * p.features_per_level * acc_bytes > smem_budget) break;
        if (contributions < 8 * (size_t)grid * entries_here) break;
        ++n;
    }
    return n;
}

} // namespace tnn
