// Host-visible launch descriptors of the fused-MLP kernels (plain structs, no torch types).
#pragma once
#include <cstddef>
#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace tnn {

// Identity encoding folded into a kernel's first-layer load (include/encodings/identity.h:63-77).
struct EncodedInput {
    const float *x; // [batch][n_in] fp32; nullptr = the input is a bf16 matrix fetched by TMA
    int n_in;       // 1..kMaxFoldedInputs
    float scale, offset;
};
constexpr int kMaxFoldedInputs = 16;

struct FwdLaunch {
    CUtensorMap tm_x;      // [batch][W] bf16 input, box 128 x min(W, 64)
    CUtensorMap tm_y;      // [batch][W] bf16 output
    CUtensorMap tm_interm; // [L+2][batch][W] bf16 activations (only read when store_all)
    const __nv_bfloat16 *wimg;   // (L+1) swizzled tiles, rows = input feature, cols = output feature
    const __nv_bfloat16 *wimg_t; // (L+1) swizzled tiles, rows = output feature, cols = input feature
    size_t batch;
    int width;
    int n_mat; // number of weight matrices = n_hidden_layers + 1
    int act, out_act;
    int fp16; // operands and activations are fp16 instead of bf16
    int store_all;
    int write_y;
    int live8; // inference: output columns from the 9th on are exactly zero (<= 8 real outputs, act_out(0) = 0)
    EncodedInput enc; // enc.x != nullptr: the input tile is produced in the kernel from fp32 coordinates
    // grid_params != nullptr: the input tile is the hash-grid encoding (2-D or 3-D, 2 features per level, at most
    // `width` features) of the fp32 positions grid_x, gathered from grid_table by extra warps of the kernel
    const struct GridParams *grid_params; // device copy
    const float *grid_table;
    const float *grid_x;
    int variant;
    int n_sm;
    int *status;
    cudaStream_t stream;
};
cudaError_t launch_mlp_fwd(const FwdLaunch &p);

struct BwdLaunch {
    CUtensorMap tm_dy;      // [batch][W] bf16 dL/dy (after loss)
    CUtensorMap tm_interm;  // [L+2][batch][W] bf16 forward activations (matrix 0 = input)
    CUtensorMap tm_a0;      // [batch][W] bf16 network input: matrix 0 of the workspace, or the caller's x itself
    CUtensorMap tm_ibwd;    // [L+1][batch][W] bf16 deltas (written when store_bwd)
    CUtensorMap tm_dx;      // [batch][W] bf16 dL/dx (written when want_dx)
    const __nv_bfloat16 *wimg;
    const __nv_bfloat16 *wimg_t;
    float *dw_partials; // [grid][L+1][W][W] fp32, layout (out, in)
    size_t batch;
    int width;
    int n_mat;
    int act, out_act;
    int fp16; // operands and activations are fp16 instead of bf16
    int store_bwd;
    int want_dx;
    int variant;
    int n_sm;
    int *status;
    cudaStream_t stream;
    int grid_out; // number of partial slabs written (set by the launcher)
};
cudaError_t launch_mlp_bwd(BwdLaunch &p);

struct TrainLaunch {
    CUtensorMap tm_x;       // [batch][W] bf16 input
    const __nv_bfloat16 *wimg;
    const float *targets;   // [batch][n_targets] fp32
    int n_targets;
    CUtensorMap tm_tgt;     // the same targets as a tiled map, box 128 x 32 fp32 (valid when tgt_mode == 1)
    // how the pipelined kernel fetches targets: 0 = per-thread loads, 1 = TMA boxes (n_targets == width),
    // 2 = one bulk copy of the tile's 128 * n_targets contiguous floats (n_targets < width); 1 and 2 need
    // 16-byte aligned targets.  4 = 2 for a network whose output columns from the 9th on are exactly zero (they are
    // weight padding, have no target, and act_out(0) = 0): only the first 8 columns take part in the loss.  3 = no targets and no loss: tm_tgt maps the upstream gradient dL/dy ([batch][W] of the
    // network's type, like tm_x) and the pass is the backward pass of the network with its forward recomputed on chip
    int tgt_mode;
    EncodedInput enc;       // enc.x != nullptr: the input tile is produced in the kernel from fp32 coordinates
    int want_dx;            // also compute dL/dinput (batch x width, the network's type) and store it through tm_dx
    CUtensorMap tm_dx;      // (pipelined kernel only; the single-tile kernel reports cudaErrorInvalidConfiguration)
    float *dw_partials;     // [grid][L+1][W][W] fp32, layout (out, in)
    int max_slabs;          // slabs dw_partials has room for: the launcher never starts more CTAs than that
    float *loss_partials;   // [grid] fp32
    size_t batch;
    int width;
    int n_mat;
    int act, out_act;
    int fp16; // operands and activations are fp16 instead of bf16
    float loss_scale;
    int n_sm;
    int *status;
    cudaStream_t stream;
    int grid_out;
};
// cudaErrorInvalidConfiguration when the network does not fit the on-chip budget of the fused kernel.
cudaError_t launch_mlp_train(TrainLaunch &p);
// Same pass with the forward stage of one tile overlapped with the backward stage of the previous one.
cudaError_t launch_mlp_train_pipe(TrainLaunch &p);
// Whether that kernel takes a network of this shape (tgt_mode as in TrainLaunch).
bool mlp_train_pipe_fits(int width, int n_mat, int tgt_mode);

} // namespace tnn
