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

template <int D>
__device__ __forceinline__ uint32_t grid_index(int grid_type, int hash_type, uint32_t hashmap_size, uint32_t res,
                                               const uint32_t (&g)[D]) {
    uint32_t stride = 1, index = 0;
#pragma unroll
    for (int d = 0; d < D; ++d) {
        if (stride <= hashmap_size) {
            index += g[d] * stride;
            stride *= res;
        }
    }
    if (grid_type == GRID_HASH && hashmap_size < stride) index = grid_hash<D>(hash_type, g);
    // same value as index % hashmap_size; table sizes are powers of two on all but the coarsest levels
    if ((hashmap_size & (hashmap_size - 1u)) == 0u) return index & (hashmap_size - 1u);
    return index % hashmap_size;
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
