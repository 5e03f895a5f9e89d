// Device-side index arithmetic shared by the grid forward and backward kernels.
#pragma once
#include "grid.h"

namespace tnn {

// ------------------------------------------------------------------ device helpers
template <int D> __device__ __forceinline__ uint32_t grid_hash(int hash_type, const uint32_t (&g)[D]) {
    // factor tables of common_device.h:712-735
    constexpr uint32_t prime[7] = {1958374283u, 2654435761u, 805459861u, 3674653429u,
                                   2097192037u, 1434869437u, 2165219737u};
    constexpr uint32_t coherent[7] = {1u,          2654435761u, 805459861u, 3674653429u,
                                      2097192037u, 1434869437u, 2165219737u};
    constexpr uint32_t reversed[7] = {2165219737u, 1434869437u, 2097192037u, 3674653429u,
                                      805459861u,  2654435761u, 1958374283u};
    uint32_t r = 0;
    if (hash_type == HASH_COHERENT_PRIME) {
#pragma unroll
        for (int d = 0; d < D; ++d) r ^= g[d] * coherent[d];
    } else if (hash_type == HASH_PRIME) {
#pragma unroll
        for (int d = 0; d < D; ++d) r ^= g[d] * prime[d];
    } else if (hash_type == HASH_REVERSED_PRIME) {
#pragma unroll
        for (int d = 0; d < D; ++d) r ^= g[d] * reversed[d];
    }
    return r; // HASH_RNG hashes everything to 0, as in the reference
}

// index before the reduction modulo the level's table size
template <int D>
__device__ __forceinline__ uint32_t grid_index_raw(int grid_type, int hash_type, uint32_t hashmap_size, uint32_t res,
                                                   const uint32_t (&g)[D]) {
    // Written with selects instead of branches: lanes work on different levels, so every condition on the level's
    // table size or resolution would split the warp (the branch unit was the busiest pipe of the forward kernel).
    uint32_t stride = 1, index = 0;
#pragma unroll
    for (int d = 0; d < D; ++d) {
        const bool in = stride <= hashmap_size;
        index += in ? g[d] * stride : 0u;
        stride = in ? stride * res : stride;
    }
    if (grid_type == GRID_HASH) { // same for every thread of the launch
        const uint32_t h = grid_hash<D>(hash_type, g);
        index = (hashmap_size < stride) ? h : index;
    }
    return index;
}

// indices of all N corners modulo the table size, with one branch for the lot (table sizes are powers of two on all
// but the coarsest levels, where the general remainder is taken)
template <int N> __device__ __forceinline__ void grid_wrap(uint32_t (&idx)[N], uint32_t hashmap_size) {
    if ((hashmap_size & (hashmap_size - 1u)) == 0u) {
#pragma unroll
        for (int c = 0; c < N; ++c) idx[c] &= hashmap_size - 1u;
    } else {
#pragma unroll
        for (int c = 0; c < N; ++c) idx[c] %= hashmap_size;
    }
}

template <int D>
__device__ __forceinline__ uint32_t grid_index(int grid_type, int hash_type, uint32_t hashmap_size, uint32_t res,
                                               const uint32_t (&g)[D]) {
    uint32_t idx[1] = {grid_index_raw<D>(grid_type, hash_type, hashmap_size, res, g)};
    grid_wrap<1>(idx, hashmap_size);
    return idx[0];
}

// fractional position and base vertex of sample x at one level
template <int D>
__device__ __forceinline__ void grid_pos(const float *__restrict__ x, float scale, int interpolation, float (&w)[D],
                                         uint32_t (&g)[D]) {
#pragma unroll
    for (int d = 0; d < D; ++d) {
        float p = fmaf(scale, x[d], 0.5f);
        const float fl = floorf(p);
        g[d] = (uint32_t)(int)fl;
        p -= fl;
        if (interpolation == INTERP_SMOOTHSTEP) p = p * p * (3.0f - 2.0f * p);
        w[d] = p;
    }
}


// What a kernel needs to know about one level, and about the grid as a whole.
struct GridLevelInfo {
    uint32_t offset; // first table entry
    uint32_t hsize;  // entries
    uint32_t res;
    float scale;
};
struct GridCommon {
    int interpolation, grid_type, hash_type;
    float max_level_f; // levels >= this produce zeros (grid.h:56-63)
};
__host__ __device__ inline GridLevelInfo grid_level_info(const GridParams &p, uint32_t level) {
    return GridLevelInfo{p.offsets[level], p.offsets[level + 1] - p.offsets[level], p.resolution[level], p.scale[level]};
}
__host__ __device__ inline GridCommon grid_common(const GridParams &p) {
    return GridCommon{p.interpolation, p.grid_type, p.hash_type,
                      (p.max_level * (float)p.n_features) / (float)p.features_per_level + 1e-3f};
}

// The F interpolated features of one sample at one level (reference kernel_grid, include/encodings/grid.h:64-133):
// fp32 throughout, all 2^D gathers issued first, then combined with fma in corner order 0..2^D-1.  `level` should be
// uniform over the warp: its table parameters are then read with one address per warp (a per-lane level serialises
// those reads in the constant bank, which was the busiest pipe of an earlier forward kernel).
template <int D, int F>
__device__ __forceinline__ void grid_level_features(const GridCommon &gc, const GridLevelInfo &lv, uint32_t level,
                                                    const float *__restrict__ table, const float (&xin)[D],
                                                    float (&res_v)[F]) {
#pragma unroll
    for (int f = 0; f < F; ++f) res_v[f] = 0.0f;
    if ((float)level >= gc.max_level_f) return;
    const float *tl = table + (size_t)lv.offset * F;
    const uint32_t hsize = lv.hsize;
    const uint32_t res = lv.res;
    struct {
        int interpolation, grid_type, hash_type;
    } p{gc.interpolation, gc.grid_type, gc.hash_type};
    float w[D];
    uint32_t g[D];
    grid_pos<D>(xin, lv.scale, p.interpolation, w, g);
    if (p.interpolation == INTERP_NEAREST) {
        const uint32_t e = grid_index<D>(p.grid_type, p.hash_type, hsize, res, g);
#pragma unroll
        for (int f = 0; f < F; ++f) res_v[f] = __ldg(tl + (size_t)e * F + f);
        return;
    }
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

// The table entries one sample touches at one level and their interpolation weights, in the corner order of the
// reference's kernels (include/encodings/grid.h:137-245): n = 2^D, or 1 with nearest-neighbour interpolation.
template <int D>
__device__ __forceinline__ int grid_corner_entries(const GridParams &p, uint32_t level, const float *__restrict__ xrow,
                                                   uint32_t (&ent)[1 << D], float (&wt)[1 << D]) {
    const uint32_t hsize = p.offsets[level + 1] - p.offsets[level];
    const uint32_t res = p.resolution[level];
    float w[D], xin[D];
    uint32_t g[D];
#pragma unroll
    for (int d = 0; d < D; ++d) xin[d] = __ldg(xrow + d);
    grid_pos<D>(xin, p.scale[level], p.interpolation, w, g);
    if (p.interpolation == INTERP_NEAREST) {
        ent[0] = grid_index<D>(p.grid_type, p.hash_type, hsize, res, g);
        wt[0] = 1.0f;
        return 1;
    }
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
    return 1 << D;
}

} // namespace tnn
