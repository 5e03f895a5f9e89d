// Sum of the per-CTA weight-gradient slabs a training kernel leaves behind, shared by the kernels that finish a
// training pass (reduce_dw_kernel, adam_refresh_kernel, dp_adam_refresh_kernel).
#pragma once
#include <cstddef>

namespace tnn {

constexpr int kSlabBlock = 128; // weights per block (threadIdx.x)
constexpr int kSlabWays = 8;    // threads per weight (threadIdx.y)

// Blocks of (kSlabBlock, kSlabWays) threads.  Thread (x, y) adds the entries of weight `idx` in the slabs y, y + 8,
// y + 16, ... in that order; the eight partial sums are then added in the order of y by the thread with y == 0, which
// gets the result (the others get 0).  The order is fixed, so the sum is bit-reproducible, and the loads of one weight
// are spread over eight threads: with up to 148 slabs a single thread per weight spends its time on load latency.
// Every thread of the block must call this (it holds a __syncthreads).
__device__ __forceinline__ float slab_sum(const float *__restrict__ slabs, int n_slabs, int per, int idx,
                                          float (*part)[kSlabBlock]) {
    float g = 0.0f;
    if (idx < per) {
        // eight loads in flight per thread; the additions keep the slab order (absent slabs add an exact zero)
        for (int s0 = threadIdx.y; s0 < n_slabs; s0 += 8 * kSlabWays) {
            float t[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int s = s0 + k * kSlabWays;
                t[k] = s < n_slabs ? __ldcg(slabs + (size_t)s * per + idx) : 0.0f;
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) g += t[k];
        }
    }
    part[threadIdx.y][threadIdx.x] = g;
    __syncthreads();
    g = 0.0f;
    if (threadIdx.y == 0) {
#pragma unroll
        for (int y = 0; y < kSlabWays; ++y) g += part[y][threadIdx.x];
    }
    return g;
}

} // namespace tnn
