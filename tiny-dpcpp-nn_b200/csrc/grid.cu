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
#include <limits>

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
        if constexpr (sizeof(OutT) == 2)
            *reinterpret_cast<__nv_bfloat162 *>(orow + level * F) = __floats2bfloat162_rn(res_v[0], res_v[1]);
        else
            *reinterpret_cast<float2 *>(orow + level * F) = make_float2(res_v[0], res_v[F > 1 ? 1 : 0]);
    } else {
#pragma unroll
        for (int f = 0; f < F; ++f) orow[level * F + f] = (OutT)res_v[f];
    }
}

template <int D, int F>
static cudaError_t launch_fwd_df(const GridParams &p, const float *x, const float *table, void *out, int out_bf16,
                                 size_t batch, cudaStream_t stream) {
    const size_t n = batch * p.n_levels;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    count_launch();
    if (out_bf16)
        grid_fwd_kernel<D, F, __nv_bfloat16><<<blocks, 256, 0, stream>>>(p, x, table, (__nv_bfloat16 *)out, batch);
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

cudaError_t launch_grid_fwd(const GridParams &p, const float *x, const float *table, void *out, int out_bf16,
                            size_t batch, cudaStream_t stream) {
    if (batch == 0) return cudaSuccess;
    TNN_GRID_DISPATCH(launch_fwd_df, p, x, table, out, out_bf16, batch, stream);
}

} // namespace tnn
