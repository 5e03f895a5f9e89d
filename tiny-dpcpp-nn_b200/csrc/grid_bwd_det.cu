// Placeholder translation unit replaced below by the deterministic pipeline.
#include "grid.h"
namespace tnn {
size_t grid_bwd_scratch_bytes(const GridParams &, size_t) { return 0; }
cudaError_t launch_grid_bwd_det(const GridParams &, const float *, const void *, int, float *, size_t, void *, size_t,
                                cudaStream_t) {
    return cudaErrorNotSupported;
}
} // namespace tnn
