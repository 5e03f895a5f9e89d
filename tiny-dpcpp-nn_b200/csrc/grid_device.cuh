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


} // namespace tnn
