// Multi-resolution hash-grid encoding: level table and kernel launchers.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cuda_runtime.h>

namespace tnn {

constexpr int kMaxGridLevels = 128; // same cap as the reference (grid_interface.h:24)

enum GridType : int { GRID_HASH = 0, GRID_DENSE = 1, GRID_TILED = 2 };
enum HashType : int { HASH_PRIME = 0, HASH_COHERENT_PRIME = 1, HASH_REVERSED_PRIME = 2, HASH_RNG = 3 };
enum InterpolationType : int { INTERP_NEAREST = 0, INTERP_LINEAR = 1, INTERP_SMOOTHSTEP = 2 };

// Everything a grid kernel needs, passed by value.
struct GridParams {
    uint32_t n_levels;
    uint32_t n_features; // n_levels * features_per_level
    uint32_t features_per_level;
    uint32_t n_dims;
    uint32_t padded_width;
    uint32_t base_resolution;
    float log2_per_level_scale;
    float max_level;
    int interpolation;
    int grid_type;
    int hash_type;
    uint32_t offsets[kMaxGridLevels + 1]; // first table entry of each level (in entries, not floats)
    float scale[kMaxGridLevels];          // exp2(l * log2_per_level_scale) * base_resolution - 1
    uint32_t resolution[kMaxGridLevels];  // ceil(scale) + 1
};

// Fills offsets / scale / resolution from the scalar fields (reference grid.h:588-659,
// common_device.h:767-775).  Returns the total number of table entries.
uint32_t grid_build_level_table(GridParams &p, uint32_t log2_hashmap_size);

// out_dtype / dy_dtype: 0 = bf16, 1 = fp16, 2 = fp32 (the TNN_DTYPE_* codes)
cudaError_t launch_grid_fwd(const GridParams &p, const float *x, const float *table, void *out, int out_dtype,
                            size_t batch, cudaStream_t stream);

// dL/dinput: dx[batch][n_dims] fp32 from dy[batch][padded_width] of dy_dtype
cudaError_t launch_grid_bwd_input(const GridParams &p, const float *x, const float *table, const void *dy, int dy_dtype,
                                  float *dx, size_t batch, cudaStream_t stream);

// Coarse levels of a backward pass: the first levels of a grid have few entries, each hit by thousands of samples, and
// reductions into so few addresses queue up in L2.  The backward kernels therefore add the contributions of levels
// [0, n) in shared-memory accumulators (one copy per CTA, one CTA per SM) and add each copy to the table gradient
// once.  (Run beside the kernel of the other levels on a second stream the pair was slower than one after the other:
// 0.55 against 0.50 ms at the benchmark grid, batch 2^20.)  Returns n: the leading levels whose accumulators (acc_bytes per table float) fit into shared memory together
// and receive at least 8 contributions per accumulator copy and entry; *grid_out = CTAs to launch.
constexpr int kGridCoarseThreads = 1024; // CTA of the coarse-level kernels (one per SM)
uint32_t grid_coarse_levels(const GridParams &p, size_t batch, size_t acc_bytes, int *grid_out);

// Backward modes: reductions in memory with fp32 atomics (the reference's structure, order not fixed), with 64-bit
// fixed-point integer atomics (order-independent: deterministic), or an atomic-free segmented reduction
// (deterministic; see grid_bwd_segmented.cu).
enum GridBackwardMode : int { GRID_BWD_ATOMIC = 0, GRID_BWD_FIXED = 1, GRID_BWD_SEGMENTED = 2 };
// Scratch (bytes) a backward pass of `mode` needs for `batch` samples (0 for GRID_BWD_ATOMIC).
size_t grid_bwd_scratch_bytes(const GridParams &p, size_t batch, int mode = GRID_BWD_FIXED);
cudaError_t launch_grid_bwd(const GridParams &p, const float *x, const void *dy, int dy_dtype, float *grads,
                            size_t batch, void *scratch, size_t scratch_bytes, cudaStream_t stream,
                            int mode = GRID_BWD_FIXED /* ignored (atomic) when scratch is null */);

} // namespace tnn
