// The objects behind the opaque handles of the C ABI (include/tnn_b200.h), shared by the translation units that
// implement entry points.
#pragma once
#include "grid.h"
#include "mlp_launch.h"

#include <cstddef>
#include <cuda_bf16.h>
#include <string>

namespace tnn {
// records the message behind tnn_last_error() and returns `code`
int api_fail(const std::string &msg, int code = 1);
} // namespace tnn

struct tnn_network {
    int input_width = 0, output_width = 0; // as requested (unpadded)
    int width = 0, n_hidden = 0, n_mat = 0;
    int act = 0, out_act = 0, use_bias = 1;
    int fp16 = 0; // element type of operands and activations: bf16 (0) or fp16 (1)
    int variant = 0;
    int n_sm = 0;
    int max_slabs = 0; // capacity of dw_slabs in slabs (CTAs of a training kernel)
    size_t n_params = 0;
    // (16-bit buffers are typed __nv_bfloat16 whatever the element type; see fp16)
    __nv_bfloat16 *packed = nullptr; // packed-layout 16-bit weights (what get_params returns)
    __nv_bfloat16 *wimg = nullptr;   // swizzled operand images, rows = input feature
    __nv_bfloat16 *wimg_t = nullptr; // swizzled operand images, rows = output feature
    float *dw_slabs = nullptr;       // per-CTA weight-gradient partial sums
    float *loss_partials = nullptr;  // per-CTA loss partial sums of the fused training kernel
    int *status = nullptr;
    // workspace of the unfused training path (grown on demand, like the reference's module workspaces)
    // (one block: [n_mat + 1] activation matrices, then dL/dy; either grown by the library or lent by the caller)
    void *ws = nullptr;
    size_t ws_bytes = 0;
    bool ws_owned = false;

    int one_padded_input() const {
        // rows of the first matrix that can carry signal: the real inputs, plus (with bias) the
        // ones-padding up to the next multiple of 16 (Network.h:188-200)
        if (!use_bias) return input_width;
        if (input_width % 16 == 0) return width;
        return (input_width / 16 + 1) * 16;
    }
};


struct tnn_encoding {
    bool is_grid = false;
    int n_in = 0;
    int n_out = 0;    // natural output width
    int padded = 0;   // padded output width
    float scale = 1.0f, offset = 0.0f; // identity
    int n_frequencies = 0;             // > 0: frequency encoding
    int sh_degree = 0;                 // > 0: spherical-harmonics encoding
    tnn::GridParams gp{};
    tnn::GridParams *gp_dev = nullptr; // device copy, read by kernels that keep the level table in shared memory
    size_t n_params = 0;
    float *table = nullptr;    // owned storage
    float *bound = nullptr;    // caller-owned storage used instead, when set (tnn_encoding_bind_params)
    float *params() const { return bound ? bound : table; }
    void *scratch = nullptr;
    size_t scratch_bytes = 0;
};

