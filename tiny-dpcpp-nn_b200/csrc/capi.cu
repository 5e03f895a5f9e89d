// Host side of libtnn_b200: the Network / Encoding classes behind the C ABI declared in
// include/tnn_b200.h.  Argument checks mirror the reference's host classes
// (include/network/Network.h:129-167, include/network/SwiftNetMLP.h:277-346,
// include/encodings/grid.h:588-659, include/encodings/encoding_factory.h:109-176).
#include "../../include/tnn_b200.h"

#include "elementwise.h"
#include "grid.h"
#include "handles.h"
#include "json_min.h"
#include "mlp_common.cuh"
#include "mlp_launch.h"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstring>
#include <memory>
#include <mutex>
#include <random>
#include <stdexcept>
#include <string>
#include <vector>

namespace {

thread_local std::string g_last_error;

int fail(const std::string &msg, int code = 1) {
    g_last_error = msg;
    return code;
}
#define TNN_CUDA(expr)                                                                                                 \
    do {                                                                                                               \
        cudaError_t e_ = (expr);                                                                                       \
        if (e_ != cudaSuccess) return fail(std::string(#expr) + ": " + cudaGetErrorString(e_), 2);                     \
    } while (0)
#define TNN_GUARD_BEGIN try {
#define TNN_GUARD_END                                                                                                  \
    }                                                                                                                  \
    catch (const std::exception &ex) { return fail(ex.what()); }                                                      \
    catch (...) { return fail("unknown C++ exception"); }

// cuTensorMapEncodeTiled is fetched through the runtime so the library does not link libcuda.
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess || !p)
            throw std::runtime_error("cuTensorMapEncodeTiled is not available from this driver");
        fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

CUtensorMapSwizzle swizzle_for(int width) {
    return width >= 64 ? CU_TENSOR_MAP_SWIZZLE_128B : width == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
}

// [n_mat][rows][width] bf16 (n_mat == 1: plain 2-D), box = 128 rows x min(width, 64) columns.
void make_act_tmap(CUtensorMap *m, const void *base, size_t rows, int width, int n_mat) {
    if (reinterpret_cast<uintptr_t>(base) % 16 != 0) throw std::invalid_argument("device buffer must be 16-byte aligned");
    const cuuint32_t box_cols = width < 64 ? width : 64;
    cuuint64_t dims[3] = {(cuuint64_t)width, (cuuint64_t)rows, (cuuint64_t)n_mat};
    cuuint64_t strides[2] = {(cuuint64_t)width * 2, (cuuint64_t)width * 2 * rows};
    cuuint32_t box[3] = {box_cols, 128, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    const cuuint32_t rank = n_mat > 1 ? 3 : 2;
    CUresult r = get_encode_fn()(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void *>(base), dims, strides, box,
                                 estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_for(width),
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
}

// fp32 targets [rows][width] as 128-row boxes of 32 columns (128 bytes, the swizzle span)
void make_tgt_tmap(CUtensorMap *m, const float *base, size_t rows, int width) {
    cuuint64_t dims[2] = {(cuuint64_t)width, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)width * sizeof(float)};
    cuuint32_t box[2] = {32, 128};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = get_encode_fn()(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), dims, strides, box, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
}

int device_checks() {
    int dev = 0;
    TNN_CUDA(cudaGetDevice(&dev));
    int major = 0;
    TNN_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    if (major != 10)
        return fail("libtnn_b200 needs a compute-capability 10.x device (B200); found major " + std::to_string(major));
    return 0;
}

// The L2 kernel moves 16 bytes at a time: eight bf16 predictions / gradients, four fp32 values, and - when the
// targets are as wide as the predictions - four fp32 targets.
int check_l2_alignment(const void *pred, const float *target, int n_targets, const float *values, const void *grads,
                       int stride) {
    auto mis = [](const void *q, uintptr_t a) { return q && reinterpret_cast<uintptr_t>(q) % a != 0; };
    if (mis(pred, 16) || mis(values, 16) || mis(grads, 16)) return fail("pred, values and grads must be 16-byte aligned");
    if (mis(target, n_targets == stride ? 16 : 4))
        return fail("target must be 16-byte aligned when n_targets == stride (4-byte aligned otherwise)");
    return 0;
}

bool act_supported(int a) { return a == tnn::ACT_RELU || a == tnn::ACT_SIGMOID || a == tnn::ACT_NONE; }

} // namespace

namespace tnn {
// error recording for translation units that implement further entry points
int api_fail(const std::string &msg, int code) { return fail(msg, code); }

static std::atomic<unsigned long long> g_launches{0};
void count_launch(int n) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }
} // namespace tnn

// ======================================================================== network
extern "C" {

const char *tnn_last_error(void) { return g_last_error.c_str(); }
const char *tnn_version(void) { return "tnn_b200 0.2 (sm_100a)"; }
unsigned long long tnn_launch_count(void) { return tnn::g_launches.load(std::memory_order_relaxed); }

int tnn_network_create(int input_width, int output_width, int n_hidden_layers, int activation, int output_activation,
                       int width, int dtype, int use_bias, tnn_network **out) {
    TNN_GUARD_BEGIN
    if (!out) return fail("out is null");
    *out = nullptr;
    if (dtype != TNN_DTYPE_BF16 && dtype != TNN_DTYPE_FP16) return fail("Unsupported dtype. Only fp16 and bf16 are supported");
    if (width != 16 && width != 32 && width != 64 && width != 128)
        return fail("Network width has to be a power of 2 between 16 and 128.");
    if (input_width <= 0) return fail("Input width of " + std::to_string(input_width) + " is not supported. Value must be larger than 0.");
    if (output_width <= 0) return fail("Output width of " + std::to_string(output_width) + " is not supported. Value must be larger than 0.");
    if (input_width > width) return fail("Input width of " + std::to_string(input_width) + " is not supported. Value must be <= network width (" + std::to_string(width) + ").");
    if (output_width > width) return fail("Output width of " + std::to_string(output_width) + " is not supported. Value must be <= network width (" + std::to_string(width) + ").");
    if (n_hidden_layers <= 0) return fail("N hidden layers must be >= 1, i.e., 1 hidden layer and 1 output layer.");
    if (!act_supported(activation)) return fail("activation must be ReLU, Sigmoid or None");
    if (!act_supported(output_activation)) return fail("output activation must be ReLU, Sigmoid or None");
    if (int rc = device_checks()) return rc;

    auto *n = new tnn_network();
    n->input_width = input_width;
    n->output_width = output_width;
    n->width = width;
    n->n_hidden = n_hidden_layers;
    n->n_mat = n_hidden_layers + 1;
    n->act = activation;
    n->out_act = output_activation;
    n->use_bias = use_bias ? 1 : 0;
    n->fp16 = dtype == TNN_DTYPE_FP16 ? 1 : 0;
    n->n_params = (size_t)n->n_mat * width * width;
    if (n->one_padded_input() > width) {
        delete n;
        return fail("one_padded_input_width > padded_input_width, the input width is too small.");
    }
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n->n_sm, cudaDevAttrMultiProcessorCount, dev);
    const size_t bytes = n->n_params * sizeof(__nv_bfloat16);
    cudaError_t e = cudaMalloc(&n->packed, bytes);
    if (e == cudaSuccess) e = cudaMalloc(&n->wimg, bytes);
    if (e == cudaSuccess) e = cudaMalloc(&n->wimg_t, bytes);
    // one weight-gradient slab per CTA of the training kernels: up to two CTAs per SM at widths 16 and 32
    n->max_slabs = n->n_sm * (width <= 32 ? 2 : 1);
    if (e == cudaSuccess) e = cudaMalloc(&n->dw_slabs, (size_t)n->max_slabs * n->n_params * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&n->loss_partials, 1024 * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&n->status, sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(n->packed, 0, bytes);
    if (e == cudaSuccess) e = cudaMemset(n->wimg, 0, bytes);
    if (e == cudaSuccess) e = cudaMemset(n->wimg_t, 0, bytes);
    if (e == cudaSuccess) e = cudaMemset(n->status, 0, sizeof(int));
    if (e != cudaSuccess) {
        tnn_network_destroy(n);
        return fail(std::string("device allocation failed: ") + cudaGetErrorString(e), 2);
    }
    *out = n;
    return 0;
    TNN_GUARD_END
}

int tnn_network_destroy(tnn_network *n) {
    if (!n) return 0;
    cudaFree(n->packed);
    cudaFree(n->wimg);
    cudaFree(n->wimg_t);
    cudaFree(n->dw_slabs);
    cudaFree(n->loss_partials);
    if (n->ws_owned) cudaFree(n->ws);
    cudaFree(n->status);
    delete n;
    return 0;
}

size_t tnn_network_n_params(const tnn_network *n) { return n ? n->n_params : 0; }
int tnn_network_n_output_dims(const tnn_network *n) { return n ? n->width : 0; }
int tnn_network_width(const tnn_network *n) { return n ? n->width : 0; }
int tnn_network_n_hidden_layers(const tnn_network *n) { return n ? n->n_hidden : 0; }

int tnn_network_set_variant(tnn_network *n, int variant) {
    if (!n) return fail("network is null");
    n->variant = variant;
    return 0;
}

int tnn_network_set_params(tnn_network *n, const void *params, int dtype, int packed, void *stream) {
    TNN_GUARD_BEGIN
    if (!n || !params) return fail("null argument");
    if (dtype != TNN_DTYPE_BF16 && dtype != TNN_DTYPE_FP16 && dtype != TNN_DTYPE_FP32)
        return fail("params must be bf16, fp16 or fp32");
    TNN_CUDA(tnn::launch_set_params(n->width, params, dtype, packed, n->n_mat, n->one_padded_input(), n->output_width,
                                    n->fp16, n->packed, nullptr, n->wimg, n->wimg_t, (cudaStream_t)stream));
    return 0;
    TNN_GUARD_END
}

int tnn_network_initialize_params(tnn_network *n, uint64_t seed, void *stream) {
    TNN_GUARD_BEGIN
    if (!n) return fail("network is null");
    std::mt19937 gen((uint32_t)seed);
    std::vector<float> w(n->n_params);
    size_t pos = 0;
    const int W = n->width;
    for (int l = 0; l < n->n_mat; ++l) {
        int fan = W + W;
        if (l == 0 || l + 1 == n->n_mat) fan = (n->input_width + 15) / 16 * 16 + W; // Network.h:278-286
        const double bound = std::sqrt(6.0 / fan);
        std::uniform_real_distribution<> dis(-bound, bound);
        for (int i = 0; i < W * W; ++i, ++pos) w[pos] = (float)dis(gen);
    }
    float *tmp = nullptr;
    TNN_CUDA(cudaMalloc(&tmp, w.size() * sizeof(float)));
    cudaError_t e = cudaMemcpyAsync(tmp, w.data(), w.size() * sizeof(float), cudaMemcpyHostToDevice, (cudaStream_t)stream);
    // the reference fills the matrices in their stored (packed) order
    if (e == cudaSuccess)
        e = tnn::launch_set_params(W, tmp, TNN_DTYPE_FP32, 1, n->n_mat, n->one_padded_input(), n->output_width, n->fp16,
                                   n->packed, nullptr, n->wimg, n->wimg_t, (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    cudaFree(tmp);
    TNN_CUDA(e);
    return 0;
    TNN_GUARD_END
}

int tnn_network_get_params(const tnn_network *n, void *out, void *stream) {
    if (!n || !out) return fail("null argument");
    TNN_CUDA(cudaMemcpyAsync(out, n->packed, n->n_params * sizeof(__nv_bfloat16), cudaMemcpyDeviceToDevice,
                             (cudaStream_t)stream));
    return 0;
}

// copy_input: matrix 0 of the workspace becomes a copy of x, as callers of the C ABI expect; the training path of
// this library reads x itself in its backward pass and skips the copy.
// enc: when set, the kernel produces its input tiles from fp32 coordinates (folded identity encoding) and x is unused
// grid / grid_x: when set, extra warps of the kernel gather the hash-grid encoding of the fp32 positions grid_x
static int run_forward(tnn_network *n, const void *x, void *y, void *interm, size_t batch, void *stream,
                       bool copy_input = true, const tnn::EncodedInput *enc = nullptr, const tnn_encoding *grid = nullptr,
                       const float *grid_x = nullptr) {
    TNN_GUARD_BEGIN
    if (!n) return fail("network is null");
    if (batch == 0) return 0;
    if (!x && !enc && !grid) return fail("input is null");
    if (batch % 8 != 0) return fail("Batch size is not divisible by 8."); // SwiftNetMLP.h:293-302
    if (batch > (size_t)1 << 30) return fail("batch too large");
    if (!y && !interm) return fail("forward needs y or interm_fwd");
    tnn::FwdLaunch p{};
    if (y) make_act_tmap(&p.tm_y, y, batch, n->width, 1);
    if (interm) make_act_tmap(&p.tm_interm, interm, batch, n->width, n->n_mat + 1);
    if (grid) {
        p.grid_params = grid->gp_dev;
        p.grid_table = grid->params();
        p.grid_x = grid_x;
    } else if (enc) {
        p.enc = *enc;
    } else {
        make_act_tmap(&p.tm_x, x, batch, n->width, 1);
    }
    // (maps that a launch does not use are never dereferenced; give them a valid value all the same)
    const CUtensorMap &any = y ? p.tm_y : p.tm_interm;
    if (enc || grid) p.tm_x = any;
    if (!y) p.tm_y = any;
    if (!interm) p.tm_interm = any;
    p.wimg = n->wimg;
    p.wimg_t = n->wimg_t;
    p.batch = batch;
    p.width = n->width;
    p.n_mat = n->n_mat;
    p.act = n->act;
    p.out_act = n->out_act;
    p.fp16 = n->fp16;
    p.store_all = interm ? 1 : 0;
    p.write_y = y ? 1 : 0;
    p.live8 = (!interm && n->output_width <= 8 && (n->out_act == tnn::ACT_NONE || n->out_act == tnn::ACT_RELU)) ? 1 : 0;
    p.variant = n->variant;
    p.n_sm = n->n_sm;
    p.status = n->status;
    p.stream = (cudaStream_t)stream;
    if (interm && copy_input && !enc && !grid) // matrix 0 of the forward workspace is a copy of the input (kernel_esimd.h:601-605)
        TNN_CUDA(cudaMemcpyAsync(interm, x, batch * n->width * sizeof(__nv_bfloat16), cudaMemcpyDeviceToDevice, p.stream));
    cudaError_t e = tnn::launch_mlp_fwd(p);
    if (e == cudaErrorInvalidConfiguration && grid) {
        cudaGetLastError();
        return -1; // the caller falls back to the two-kernel path
    }
    if (e == cudaErrorInvalidConfiguration)
        return fail("this width / depth does not fit the on-chip weight staging of the forward kernel");
    TNN_CUDA(e);
    return 0;
    TNN_GUARD_END
}

int tnn_network_inference(tnn_network *n, const void *x, void *y, size_t batch, void *stream) {
    if (!y && batch) return fail("output is null");
    return run_forward(n, x, y, nullptr, batch, stream);
}

int tnn_network_forward(tnn_network *n, const void *x, void *y, void *interm_fwd, size_t batch, void *stream) {
    return run_forward(n, x, y, interm_fwd, batch, stream);
}

// x_override: where the network input lives when it is not matrix 0 of interm_fwd
// n_slabs_out: when set, the per-CTA weight-gradient slabs are left unreduced in n->dw_slabs and their number is
// returned (the trainer sums them in its optimiser kernel); grads is then unused
static int run_backward(tnn_network *n, const void *dy, const void *interm_fwd, const void *x_override, void *grads,
                        int grads_dtype, int pack_transpose, void *dx, void *interm_bwd, size_t batch, void *stream,
                        int *n_slabs_out = nullptr) {
    TNN_GUARD_BEGIN
    if (!n) return fail("network is null");
    if (!grads && !n_slabs_out) return fail("grads is null");
    if (grads_dtype != TNN_DTYPE_BF16 && grads_dtype != TNN_DTYPE_FP16 && grads_dtype != TNN_DTYPE_FP32)
        return fail("grads must be bf16, fp16 or fp32");
    cudaStream_t s = (cudaStream_t)stream;
    if (batch == 0) {
        const size_t esz = grads_dtype == TNN_DTYPE_FP32 ? 4 : 2;
        TNN_CUDA(cudaMemsetAsync(grads, 0, n->n_params * esz, s));
        return 0;
    }
    if (!dy || !interm_fwd) return fail("dy and interm_fwd are required");
    if (batch % 8 != 0) return fail("Batch size is not divisible by 8.");
    tnn::BwdLaunch p{};
    make_act_tmap(&p.tm_dy, dy, batch, n->width, 1);
    make_act_tmap(&p.tm_interm, interm_fwd, batch, n->width, n->n_mat + 1);
    make_act_tmap(&p.tm_a0, x_override ? x_override : interm_fwd, batch, n->width, 1);
    if (interm_bwd)
        make_act_tmap(&p.tm_ibwd, interm_bwd, batch, n->width, n->n_mat);
    else
        p.tm_ibwd = p.tm_dy;
    if (dx)
        make_act_tmap(&p.tm_dx, dx, batch, n->width, 1);
    else
        p.tm_dx = p.tm_dy;
    p.wimg = n->wimg;
    p.wimg_t = n->wimg_t;
    p.dw_partials = n->dw_slabs;
    p.batch = batch;
    p.width = n->width;
    p.n_mat = n->n_mat;
    p.act = n->act;
    p.out_act = n->out_act;
    p.fp16 = n->fp16;
    p.store_bwd = interm_bwd ? 1 : 0;
    p.want_dx = dx ? 1 : 0;
    p.variant = n->variant;
    p.n_sm = n->n_sm;
    p.status = n->status;
    p.stream = s;
    cudaError_t e = tnn::launch_mlp_bwd(p);
    if (e == cudaErrorInvalidConfiguration)
        return fail("this width / depth does not fit the on-chip staging of the backward kernel");
    TNN_CUDA(e);
    if (n_slabs_out) {
        *n_slabs_out = p.grid_out;
        return 0;
    }
    TNN_CUDA(tnn::launch_reduce_dw(n->dw_slabs, p.grid_out, n->n_mat, n->width, pack_transpose, 1.0f,
                                   grads_dtype == TNN_DTYPE_FP32 ? (float *)grads : nullptr,
                                   grads_dtype != TNN_DTYPE_FP32 ? (__nv_bfloat16 *)grads : nullptr,
                                   grads_dtype == TNN_DTYPE_FP16, s));
    return 0;
    TNN_GUARD_END
}

int tnn_network_backward(tnn_network *n, const void *dy, const void *interm_fwd, void *grads, int grads_dtype,
                         int pack_transpose, void *dx, void *interm_bwd, size_t batch, void *stream) {
    return run_backward(n, dy, interm_fwd, nullptr, grads, grads_dtype, pack_transpose, dx, interm_bwd, batch, stream);
}

// Bytes of the workspace the three-kernel training path (forward with stored activations, L2 loss, backward)
// needs for `batch` rows: n_mat + 1 activation matrices and dL/dy.
static size_t unfused_workspace_bytes(const tnn_network *n, size_t batch) {
    return (size_t)(n->n_mat + 2) * batch * n->width * sizeof(__nv_bfloat16);
}

// Makes n->ws hold at least `need` bytes.  A workspace lent by the caller is never replaced; one owned by the
// library grows (synchronising the stream first, since earlier launches may still use the old block).
static int ensure_workspace(tnn_network *n, size_t need, cudaStream_t s) {
    if (need <= n->ws_bytes) return 0;
    if (n->ws && !n->ws_owned)
        return fail("the workspace set with tnn_network_set_workspace is too small: " + std::to_string(n->ws_bytes) +
                    " bytes, " + std::to_string(need) + " needed (see tnn_network_workspace_bytes)");
    TNN_CUDA(cudaStreamSynchronize(s));
    cudaFree(n->ws);
    n->ws = nullptr;
    n->ws_bytes = 0;
    TNN_CUDA(cudaMalloc(&n->ws, need));
    n->ws_bytes = need;
    n->ws_owned = true;
    return 0;
}

// One training pass.  Input: x (batch x width bf16) or, when enc is set, fp32 coordinates the kernels encode
// themselves.  dx (optional): dL/dinput, batch x width bf16 - only the three-kernel path produces it.
// raw (optional, two ints): leave the per-CTA slabs and loss partials unreduced in the network's buffers and return
// their counts in raw[0] (slabs) and raw[1] (loss partials); grads and loss_sum are then unused.
static int train_step_impl(tnn_network *n, const void *x, const tnn::EncodedInput *enc, const float *targets,
                           int n_targets, size_t batch, float loss_scale, void *grads, int grads_dtype,
                           int pack_transpose, void *dx, float *loss_sum, void *stream, int *raw = nullptr) {
    TNN_GUARD_BEGIN
    if (!n) return fail("network is null");
    if (!grads && !raw) return fail("grads is null");
    if (grads_dtype != TNN_DTYPE_BF16 && grads_dtype != TNN_DTYPE_FP16 && grads_dtype != TNN_DTYPE_FP32)
        return fail("grads must be bf16, fp16 or fp32");
    if (batch == 0) return fail("batch_size == 0");
    if ((!x && !enc) || !targets) return fail("x and targets are required");
    if (batch % 8 != 0) return fail("Batch size is not divisible by 8.");
    if (n_targets <= 0 || n_targets > n->width) return fail("n_targets must be in [1, width]");
    if (loss_scale == 0.0f) return fail("loss_scale must not be 0");
    if (reinterpret_cast<uintptr_t>(targets) % 4 != 0) return fail("targets must be 4-byte aligned");
    cudaStream_t s = (cudaStream_t)stream;
    float *gf = grads_dtype == TNN_DTYPE_FP32 ? (float *)grads : nullptr;
    __nv_bfloat16 *gb = grads_dtype != TNN_DTYPE_FP32 ? (__nv_bfloat16 *)grads : nullptr;

    if (!(n->variant & 16)) { // fused single-kernel path
        tnn::TrainLaunch p{};
        if (enc)
            p.enc = *enc;
        else
            make_act_tmap(&p.tm_x, x, batch, n->width, 1);
        p.wimg = n->wimg;
        p.targets = targets;
        p.n_targets = n_targets;
        const bool aligned = reinterpret_cast<uintptr_t>(targets) % 16 == 0;
        p.tgt_mode = (!aligned || n->width < 32) ? 0 : (n_targets == n->width ? 1 : 2);
        // output columns past the targets and past the network's real outputs hold act_out(0) under zero weights:
        // exactly zero for a linear or ReLU output, so they carry neither loss nor gradient
        const int live_out = n_targets > n->output_width ? n_targets : n->output_width;
        if (p.tgt_mode == 2 && live_out <= 8 && (n->out_act == tnn::ACT_NONE || n->out_act == tnn::ACT_RELU))
            p.tgt_mode = 4;
        if (p.tgt_mode == 1) make_tgt_tmap(&p.tm_tgt, targets, batch, n->width);
        if (dx) {
            p.want_dx = 1;
            make_act_tmap(&p.tm_dx, dx, batch, n->width, 1);
        }
        p.dw_partials = n->dw_slabs;
        p.max_slabs = n->max_slabs;
        p.loss_partials = n->loss_partials;
        p.batch = batch;
        p.width = n->width;
        p.n_mat = n->n_mat;
        p.act = n->act;
        p.out_act = n->out_act;
        p.fp16 = n->fp16;
    p.fp16 = n->fp16;
        p.loss_scale = loss_scale;
        p.n_sm = n->n_sm;
        p.status = n->status;
        p.stream = s;
        // widest-overlap kernel first; the single-tile kernel covers deeper networks
        cudaError_t e = (n->variant & 64) ? cudaErrorInvalidConfiguration : tnn::launch_mlp_train_pipe(p);
        if (e == cudaErrorInvalidConfiguration) {
            cudaGetLastError();
            e = tnn::launch_mlp_train(p);
        }
        if (e == cudaSuccess && raw) {
            raw[0] = raw[1] = p.grid_out;
            return 0;
        }
        if (e == cudaSuccess) {
            TNN_CUDA(tnn::launch_reduce_dw(n->dw_slabs, p.grid_out, n->n_mat, n->width, pack_transpose, 1.0f, gf, gb,
                                           grads_dtype == TNN_DTYPE_FP16, s, n->loss_partials, p.grid_out, loss_sum));
            return 0;
        }
        if (e != cudaErrorInvalidConfiguration) TNN_CUDA(e);
        cudaGetLastError(); // the fused kernel does not cover this width / depth: use the three-kernel path
    }
    if (int rc = ensure_workspace(n, unfused_workspace_bytes(n, batch), s)) return rc;
    __nv_bfloat16 *interm = reinterpret_cast<__nv_bfloat16 *>(n->ws);
    __nv_bfloat16 *ws_dy = interm + (size_t)(n->n_mat + 1) * batch * n->width;
    // (with an encoded input the forward kernel stores the encoded tile as matrix 0, which the backward pass reads)
    if (int rc = run_forward(n, x, nullptr, interm, batch, stream, /*copy_input=*/false, enc)) return rc;
    const __nv_bfloat16 *pred = interm + (size_t)n->n_mat * batch * n->width;
    TNN_CUDA(tnn::launch_l2_loss(pred, n->fp16, targets, n_targets, nullptr, ws_dy, batch, n->width, loss_scale,
                                 (loss_sum || raw) ? n->loss_partials : nullptr, 1024, raw ? nullptr : loss_sum, s));
    if (raw) raw[1] = 1024;
    return run_backward(n, ws_dy, interm, enc ? nullptr : x, grads, grads_dtype, pack_transpose, dx, nullptr, batch, stream,
                        raw ? &raw[0] : nullptr);
    TNN_GUARD_END
}

int tnn_network_train_step(tnn_network *n, const void *x, const float *targets, int n_targets, size_t batch,
                           float loss_scale, void *grads, int grads_dtype, int pack_transpose, float *loss_sum,
                           void *stream) {
    if (!x) return fail("x and targets are required");
    return train_step_impl(n, x, nullptr, targets, n_targets, batch, loss_scale, grads, grads_dtype, pack_transpose,
                           nullptr, loss_sum, stream);
}

int tnn_network_backward_from_input_supported(const tnn_network *n) {
    return (n && !(n->variant & (16 | 64)) && tnn::mlp_train_pipe_fits(n->width, n->n_mat, 3)) ? 1 : 0;
}

int tnn_network_backward_from_input(tnn_network *n, const void *x, const void *dy, void *grads, int grads_dtype,
                                    int pack_transpose, void *dl_dinput, size_t batch, void *stream) {
    TNN_GUARD_BEGIN
    if (!n) return fail("network is null");
    if (!x || !dy || !grads) return fail("x, dy and grads are required");
    if (grads_dtype != TNN_DTYPE_BF16 && grads_dtype != TNN_DTYPE_FP16 && grads_dtype != TNN_DTYPE_FP32)
        return fail("grads must be bf16, fp16 or fp32");
    if (batch == 0) return fail("batch_size == 0");
    if (batch % 8 != 0) return fail("Batch size is not divisible by 8.");
    if (!tnn_network_backward_from_input_supported(n))
        return fail("this network does not fit the fused kernel: use tnn_network_forward + tnn_network_backward");
    for (const void *ptr : {x, dy, (const void *)dl_dinput})
        if (reinterpret_cast<uintptr_t>(ptr) % 16 != 0) return fail("x, dy and dl_dinput must be 16-byte aligned");
    cudaStream_t s = (cudaStream_t)stream;
    tnn::TrainLaunch p{};
    make_act_tmap(&p.tm_x, x, batch, n->width, 1);
    make_act_tmap(&p.tm_tgt, dy, batch, n->width, 1);
    p.tgt_mode = 3;
    p.wimg = n->wimg;
    p.n_targets = n->width;
    if (dl_dinput) {
        p.want_dx = 1;
        make_act_tmap(&p.tm_dx, dl_dinput, batch, n->width, 1);
    }
    p.dw_partials = n->dw_slabs;
    p.max_slabs = n->max_slabs;
    p.loss_partials = nullptr;
    p.batch = batch;
    p.width = n->width;
    p.n_mat = n->n_mat;
    p.act = n->act;
    p.out_act = n->out_act;
    p.fp16 = n->fp16;
    p.loss_scale = 1.0f;
    p.n_sm = n->n_sm;
    p.status = n->status;
    p.stream = s;
    TNN_CUDA(tnn::launch_mlp_train_pipe(p));
    float *gf = grads_dtype == TNN_DTYPE_FP32 ? (float *)grads : nullptr;
    __nv_bfloat16 *gb = grads_dtype != TNN_DTYPE_FP32 ? (__nv_bfloat16 *)grads : nullptr;
    TNN_CUDA(tnn::launch_reduce_dw(n->dw_slabs, p.grid_out, n->n_mat, n->width, pack_transpose, 1.0f, gf, gb,
                                   grads_dtype == TNN_DTYPE_FP16, s, nullptr, 0, nullptr));
    return 0;
    TNN_GUARD_END
}

size_t tnn_network_workspace_bytes(const tnn_network *n, size_t batch) { return n ? unfused_workspace_bytes(n, batch) : 0; }

int tnn_network_set_workspace(tnn_network *n, void *workspace, size_t bytes) {
    if (!n) return fail("network is null");
    if (workspace && reinterpret_cast<uintptr_t>(workspace) % 256 != 0) return fail("workspace must be 256-byte aligned");
    if (n->ws_owned) {
        // a launch may still be using the library's own block
        TNN_CUDA(cudaDeviceSynchronize());
        cudaFree(n->ws);
    }
    n->ws = workspace;
    n->ws_bytes = workspace ? bytes : 0;
    n->ws_owned = false;
    return 0;
}

int tnn_network_sync_status(tnn_network *n, int *status, void *stream) {
    if (!n || !status) return fail("null argument");
    TNN_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    TNN_CUDA(cudaMemcpy(status, n->status, sizeof(int), cudaMemcpyDeviceToHost));
    if (*status != 0) TNN_CUDA(cudaMemset(n->status, 0, sizeof(int)));
    return 0;
}

int tnn_network_adam_step(tnn_network *n, float *master, float *m, float *v, const float *grads, float grad_scale,
                          int step, float lr, float beta1, float beta2, float eps, void *stream) {
    TNN_GUARD_BEGIN
    if (!n || !master || !m || !v || !grads) return fail("null argument");
    if (step < 1) return fail("step counts from 1");
    cudaStream_t s = (cudaStream_t)stream;
    TNN_CUDA(tnn::launch_adam(master, m, v, grads, n->n_params, grad_scale, step, lr, beta1, beta2, eps, nullptr, s));
    TNN_CUDA(tnn::launch_set_params(n->width, master, TNN_DTYPE_FP32, 1, n->n_mat, n->one_padded_input(), n->output_width,
                                    n->fp16, n->packed, nullptr, n->wimg, n->wimg_t, s));
    return 0;
    TNN_GUARD_END
}

int tnn_l2_loss(const void *pred, const float *target, int n_targets, float *values, void *grads, size_t batch,
                int stride, float loss_scale, float *loss_sum, void *stream) {
    return tnn_l2_loss_dtype(pred, TNN_DTYPE_BF16, target, n_targets, values, grads, batch, stride, loss_scale, loss_sum,
                             stream);
}

int tnn_l2_loss_dtype(const void *pred, int dtype, const float *target, int n_targets, float *values, void *grads,
                      size_t batch, int stride, float loss_scale, float *loss_sum, void *stream) {
    TNN_GUARD_BEGIN
    if (dtype != TNN_DTYPE_BF16 && dtype != TNN_DTYPE_FP16) return fail("pred must be bf16 or fp16");
    if (batch == 0) return 0;
    if (!pred || !target) return fail("null argument");
    if (n_targets <= 0 || n_targets > stride) return fail("n_targets must be in [1, stride]");
    if (loss_scale == 0.0f) return fail("loss_scale must not be 0");
    if (stride % 16 != 0) return fail("stride must be a multiple of 16 (network widths are)");
    if (int rc = check_l2_alignment(pred, target, n_targets, values, grads, stride)) return rc;
    // Per-block partial sums of the loss: one buffer per device, allocated at the first call on that device that
    // asks for the sum and kept until the process exits.  Calls on one device share it, like tnn_l2_loss_static.
    constexpr int kPartials = 1024;
    constexpr int kMaxDevices = 64;
    static float *partials[kMaxDevices] = {};
    static std::mutex mu;
    float *buf = nullptr;
    if (loss_sum) {
        int dev = 0;
        TNN_CUDA(cudaGetDevice(&dev));
        if (dev < 0 || dev >= kMaxDevices) return fail("device ordinal out of range");
        std::lock_guard<std::mutex> lock(mu);
        if (!partials[dev]) TNN_CUDA(cudaMalloc(&partials[dev], kPartials * sizeof(float)));
        buf = partials[dev];
    }
    TNN_CUDA(tnn::launch_l2_loss((const __nv_bfloat16 *)pred, dtype == TNN_DTYPE_FP16, target, n_targets, values,
                                 (__nv_bfloat16 *)grads, batch, stride, loss_scale, buf, kPartials, loss_sum,
                                 (cudaStream_t)stream));
    return 0;
    TNN_GUARD_END
}

int tnn_adam_step(float *params, float *m, float *v, const float *grads, size_t n, float grad_scale, int step, float lr,
                  float beta1, float beta2, float eps, void *stream) {
    if (!params || !m || !v || !grads) return fail("null argument");
    if (step < 1) return fail("step counts from 1");
    TNN_CUDA(tnn::launch_adam(params, m, v, grads, n, grad_scale, step, lr, beta1, beta2, eps, nullptr,
                              (cudaStream_t)stream));
    return 0;
}

} // extern "C"

// ======================================================================== encoding
namespace {

int enum_value(const tnn::JsonObject &cfg, const char *key, const std::vector<const char *> &names, int dflt) {
    if (!cfg.has(key)) return dflt;
    const tnn::JsonValue &v = cfg.at(key);
    if (v.is_string) {
        for (size_t i = 0; i < names.size(); ++i)
            if (v.str == names[i]) return (int)i;
        throw std::runtime_error("Invalid enum value");
    }
    return (int)v.num;
}

} // namespace

extern "C" {

int tnn_encoding_create(const char *json_config, int padded_output_width, tnn_encoding **out) {
    TNN_GUARD_BEGIN
    if (!out || !json_config) return fail("null argument");
    *out = nullptr;
    tnn::JsonObject cfg = tnn::parse_json_object(json_config);
    if (!cfg.has("otype")) return fail("Config needs to contain encoding, key otype");
    const std::string name = cfg.at("otype").str;
    auto enc = std::make_unique<tnn_encoding>();
    if (name == "Identity") {
        if (!cfg.has("offset")) return fail("Config misses offset");
        if (!cfg.has("scale")) return fail("Config misses scale");
        if (!cfg.has("n_dims_to_encode")) return fail("Config misses n_dims_to_encode");
        enc->n_in = (int)cfg.at("n_dims_to_encode").num;
        enc->n_out = enc->n_in;
        enc->scale = (float)cfg.at("scale").num;
        enc->offset = (float)cfg.at("offset").num;
    } else if (name == "HashGrid") {
        enc->is_grid = true;
        tnn::GridParams &g = enc->gp;
        const uint32_t log2_hashmap = (uint32_t)cfg.number("log2_hashmap_size", 19);
        g.n_dims = (uint32_t)cfg.number("n_dims_to_encode", 2);
        g.features_per_level = (uint32_t)cfg.number("n_features_per_level", 2);
        const uint32_t F = g.features_per_level;
        if (F != 1 && F != 2 && F != 4 && F != 8) return fail("GridEncoding: n_features_per_level must be 1, 2, 4, or 8.");
        if (cfg.has("n_features")) {
            if (cfg.has("n_levels"))
                return fail("GridEncoding: may not specify n_features and n_levels simultaneously (one determines the other)");
            g.n_features = (uint32_t)cfg.at("n_features").num;
        } else {
            g.n_features = F * (uint32_t)cfg.number("n_levels", 16);
        }
        if (g.n_features % F != 0) return fail("GridEncoding: n_features must be a multiple of n_features_per_level");
        g.n_levels = g.n_features / F;
        if (g.n_levels == 0) return fail("Output width cannot be zero");
        if (g.n_levels > tnn::kMaxGridLevels) return fail("GridEncoding: n_levels must be at most 128");
        if (g.n_dims != 2 && g.n_dims != 3) return fail("GridEncoding: number of input dims must be 2 or 3.");
        g.grid_type = enum_value(cfg, "type", {"Hash", "Dense", "Tiled"}, tnn::GRID_HASH);
        g.hash_type = enum_value(cfg, "hash", {"Prime", "CoherentPrime", "ReversedPrime", "Rng"}, tnn::HASH_COHERENT_PRIME);
        g.interpolation = enum_value(cfg, "interpolation", {"Nearest", "Linear", "Smoothstep"}, tnn::INTERP_LINEAR);
        if (cfg.has("stochastic_interpolation") && cfg.at("stochastic_interpolation").truthy())
            return fail("stochastic_interpolation is not implemented");
        g.base_resolution = (uint32_t)cfg.number("base_resolution", 16);
        float per_level_scale = 2.0f;
        if (g.grid_type == tnn::GRID_DENSE && g.n_levels > 1)
            per_level_scale = std::exp(std::log(256.0f / (float)g.base_resolution) / (float)(g.n_levels - 1));
        per_level_scale = (float)cfg.number("per_level_scale", per_level_scale);
        g.log2_per_level_scale = std::log2(per_level_scale);
        g.max_level = 1000.0f;
        const uint32_t entries = tnn::grid_build_level_table(g, log2_hashmap);
        enc->n_params = (size_t)entries * F;
        enc->n_in = (int)g.n_dims;
        enc->n_out = (int)g.n_features;
    } else if (name == "Frequency") {
        // encoding_factory.h:88-107
        if (!cfg.has("n_frequencies")) return fail("Config misses n_frequencies");
        if (!cfg.has("n_dims_to_encode")) return fail("Config misses n_dims_to_encode");
        const double nf = cfg.at("n_frequencies").num;
        const double nd = cfg.at("n_dims_to_encode").num;
        if (nf < 1.0 || nf > 32.0) return fail("n_frequencies must be in [1, 32]");
        if (nd < 1.0 || nd * nf * 2.0 > 2147483647.0) return fail("n_frequencies * 2 * n_dims_to_encode out of range");
        enc->n_frequencies = (int)nf;
        enc->n_in = (int)nd;
        enc->n_out = enc->n_in * enc->n_frequencies * 2;
    } else if (name == "SphericalHarmonics") {
        // encoding_factory.h:55-72, spherical_harmonics.h:18-26
        if (!cfg.has("degree")) return fail("Config misses degree");
        if (!cfg.has("n_dims_to_encode")) return fail("Config misses n_dims_to_encode");
        const double degree = cfg.at("degree").num;
        if ((int)cfg.at("n_dims_to_encode").num != 3) return fail("Can only encode 3D directions in spherical harmonics.");
        if (degree < 1.0 || degree > 8.0) return fail("Spherical harmonics degree > 0 and <= 8.");
        enc->sh_degree = (int)degree;
        enc->n_in = 3;
        enc->n_out = enc->sh_degree * enc->sh_degree;
    } else {
        return fail("Unknown encoding type: " + name);
    }
    enc->padded = padded_output_width > 0 ? padded_output_width : enc->n_out;
    if (enc->n_in <= 0) return fail("Input width cannot be zero");
    if (enc->padded < enc->n_out) return fail("Padded output width cannot be less than output width");
    if (int rc = device_checks()) return rc; // configuration errors above are reported even without a device
    if (enc->is_grid) {
        enc->gp.padded_width = (uint32_t)enc->padded;
        TNN_CUDA(cudaMalloc(&enc->table, enc->n_params * sizeof(float)));
        TNN_CUDA(cudaMemset(enc->table, 0, enc->n_params * sizeof(float)));
        TNN_CUDA(cudaMalloc(&enc->gp_dev, sizeof(tnn::GridParams)));
        TNN_CUDA(cudaMemcpy(enc->gp_dev, &enc->gp, sizeof(tnn::GridParams), cudaMemcpyHostToDevice));
    }
    *out = enc.release();
    return 0;
    TNN_GUARD_END
}

int tnn_encoding_destroy(tnn_encoding *e) {
    if (!e) return 0;
    cudaFree(e->table);
    cudaFree(e->gp_dev);
    cudaFree(e->scratch);
    delete e;
    return 0;
}

size_t tnn_encoding_n_params(const tnn_encoding *e) { return e ? e->n_params : 0; }
int tnn_encoding_n_output_dims(const tnn_encoding *e) { return e ? e->padded : 0; }
int tnn_encoding_n_input_dims(const tnn_encoding *e) { return e ? e->n_in : 0; }
float *tnn_encoding_params_ptr(tnn_encoding *e) { return e ? e->params() : nullptr; }

int tnn_encoding_bind_params(tnn_encoding *e, float *params) {
    if (!e) return fail("encoding is null");
    if (params && reinterpret_cast<uintptr_t>(params) % 16 != 0) return fail("parameter storage must be 16-byte aligned");
    e->bound = params;
    return 0;
}

int tnn_encoding_level_info(const tnn_encoding *e, int level, uint32_t *offset, uint32_t *size, float *scale,
                            uint32_t *resolution) {
    if (!e || !e->is_grid) return fail("not a grid encoding");
    if (level < 0 || level >= (int)e->gp.n_levels) return fail("level out of range");
    if (offset) *offset = e->gp.offsets[level];
    if (size) *size = e->gp.offsets[level + 1] - e->gp.offsets[level];
    if (scale) *scale = e->gp.scale[level];
    if (resolution) *resolution = e->gp.resolution[level];
    return 0;
}

int tnn_encoding_initialize_params(tnn_encoding *e, uint64_t seed, void *stream) {
    TNN_GUARD_BEGIN
    if (!e) return fail("encoding is null");
    if (!e->n_params) return 0;
    std::mt19937_64 gen(seed);
    std::uniform_real_distribution<float> dis(-1e-4f, 1e-4f);
    std::vector<float> h(e->n_params);
    for (auto &v : h) v = dis(gen);
    TNN_CUDA(cudaMemcpyAsync(e->params(), h.data(), h.size() * sizeof(float), cudaMemcpyHostToDevice, (cudaStream_t)stream));
    TNN_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return 0;
    TNN_GUARD_END
}

int tnn_encoding_set_params(tnn_encoding *e, const float *params, void *stream) {
    if (!e || !params) return fail("null argument");
    if (!e->n_params) return fail("no encoding params to set");
    if (params == e->params()) return 0; // bound storage: nothing to copy
    TNN_CUDA(cudaMemcpyAsync(e->params(), params, e->n_params * sizeof(float), cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    return 0;
}

int tnn_encoding_get_params(const tnn_encoding *e, float *out, void *stream) {
    if (!e || !out) return fail("null argument");
    if (!e->n_params) return 0;
    TNN_CUDA(cudaMemcpyAsync(out, e->params(), e->n_params * sizeof(float), cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    return 0;
}

int tnn_encoding_forward(tnn_encoding *e, const float *x, void *out, int out_dtype, size_t batch, void *stream) {
    TNN_GUARD_BEGIN
    if (!e) return fail("encoding is null");
    if (batch == 0) return 0;
    if (!x || !out) return fail("null argument");
    if (out_dtype != TNN_DTYPE_FP32 && out_dtype != TNN_DTYPE_BF16 && out_dtype != TNN_DTYPE_FP16)
        return fail("output must be fp32, bf16 or fp16");
    if (batch > 0xFFFFFFFFull / 8) return fail("batch too large");
    if (e->is_grid)
        TNN_CUDA(tnn::launch_grid_fwd(e->gp, x, e->params(), out, out_dtype, batch, (cudaStream_t)stream));
    else if (e->n_frequencies > 0)
        TNN_CUDA(tnn::launch_frequency_fwd(x, out, out_dtype, batch, e->n_in, e->n_frequencies, e->padded,
                                           (cudaStream_t)stream));
    else if (e->sh_degree > 0)
        TNN_CUDA(tnn::launch_spherical_harmonics_fwd(x, out, out_dtype, batch, e->sh_degree, e->padded, (cudaStream_t)stream));
    else
        TNN_CUDA(tnn::launch_identity_fwd(x, out, out_dtype, batch, e->n_in, e->padded, e->scale, e->offset,
                                          (cudaStream_t)stream));
    return 0;
    TNN_GUARD_END
}

int tnn_encoding_backward(tnn_encoding *e, const float *x, const void *dy, int dy_dtype, float *grads, size_t batch,
                          int deterministic, void *stream) {
    TNN_GUARD_BEGIN
    if (!e) return fail("encoding is null");
    if (!e->n_params) return 0; // parameter-free encodings have no gradient (tnn_api.h:372-374)
    if (!grads) return fail("grads is null");
    cudaStream_t s = (cudaStream_t)stream;
    if (batch == 0) return fail("batch_size == 0"); // grid.h:744
    if (!x || !dy) return fail("null argument");
    if (dy_dtype != TNN_DTYPE_FP32 && dy_dtype != TNN_DTYPE_BF16 && dy_dtype != TNN_DTYPE_FP16)
        return fail("dy must be fp32, bf16 or fp16");
    if (batch > 0xFFFFFFFFull / 8) return fail("batch too large");
    if (reinterpret_cast<uintptr_t>(grads) % 16 != 0) return fail("grads must be 16-byte aligned (vector reductions)");
    if (deterministic < 0 || deterministic > 2) return fail("deterministic must be 0, 1 or 2");
    size_t need = tnn::grid_bwd_scratch_bytes(e->gp, batch, deterministic);
    if (need > e->scratch_bytes) {
        TNN_CUDA(cudaStreamSynchronize(s));
        cudaFree(e->scratch);
        e->scratch = nullptr;
        e->scratch_bytes = 0;
        TNN_CUDA(cudaMalloc(&e->scratch, need));
        e->scratch_bytes = need;
    }
    TNN_CUDA(tnn::launch_grid_bwd(e->gp, x, dy, dy_dtype, grads, batch,
                                  deterministic ? e->scratch : nullptr, e->scratch_bytes, s, deterministic));
    return 0;
    TNN_GUARD_END
}

} // extern "C"

extern "C" int tnn_encoding_backward_input(tnn_encoding *e, const float *x, const void *dy, int dy_dtype, float *dx,
                                          size_t batch, void *stream) {
    TNN_GUARD_BEGIN
    if (!e) return fail("encoding is null");
    if (batch == 0) return fail("batch_size == 0");
    if (!x || !dy || !dx) return fail("null argument");
    if (dy_dtype != TNN_DTYPE_FP32 && dy_dtype != TNN_DTYPE_BF16 && dy_dtype != TNN_DTYPE_FP16)
        return fail("dy must be fp32, bf16 or fp16");
    if (batch > 0xFFFFFFFFull / 8) return fail("batch too large");
    cudaStream_t s = (cudaStream_t)stream;
    if (e->sh_degree > 0) return fail("Spherical backward not yet implemented."); // spherical_harmonics.h:66-71
    if (e->is_grid)
        TNN_CUDA(tnn::launch_grid_bwd_input(e->gp, x, e->params(), dy, dy_dtype, dx, batch, s));
    else if (e->n_frequencies > 0)
        TNN_CUDA(tnn::launch_frequency_bwd_input(x, dy, dy_dtype, dx, batch, e->n_in, e->n_frequencies, e->padded, s));
    else
        TNN_CUDA(tnn::launch_identity_bwd_input(dy, dy_dtype, dx, batch, e->n_in, e->padded, e->scale, s));
    return 0;
    TNN_GUARD_END
}

// ======================================================================== network with input encoding
namespace {

// The identity encoding can be folded into the network kernels' first-layer load.
bool foldable(const tnn_encoding *e) {
    return !e->is_grid && e->n_frequencies == 0 && e->sh_degree == 0 && e->n_in <= tnn::kMaxFoldedInputs;
}

// The fused kernel covers the common grids: 2-D / 3-D, two features per level, all features inside the network width.
bool grid_fusable(const tnn_network *n, const tnn_encoding *e) {
    return e->is_grid && e->gp_dev && (e->gp.n_dims == 2 || e->gp.n_dims == 3) && e->gp.features_per_level == 2 &&
           (int)e->gp.n_features <= n->width && e->padded == n->width;
}

int nwe_checks(const tnn_network *n, const tnn_encoding *e, const float *x, size_t batch) {
    if (!n || !e) return fail("null handle");
    if (e->padded != n->width)
        return fail("the encoding's padded output width (" + std::to_string(e->padded) + ") must equal the network width (" +
                    std::to_string(n->width) + ")");
    if (batch && !x) return fail("input is null");
    if (batch % 8 != 0) return fail("Batch size is not divisible by 8.");
    if (reinterpret_cast<uintptr_t>(x) % 4 != 0) return fail("input must be 4-byte aligned");
    return 0;
}

size_t nwe_workspace_bytes(const tnn_network *n, size_t batch) {
    // encoded input, the three-kernel training workspace, dL/d(encoded input)
    return (size_t)(n->n_mat + 4) * batch * n->width * sizeof(__nv_bfloat16);
}

} // namespace

extern "C" {

size_t tnn_network_with_encoding_workspace_bytes(const tnn_network *n, size_t batch) {
    return n ? nwe_workspace_bytes(n, batch) : 0;
}

int tnn_network_with_encoding_forward(tnn_network *n, tnn_encoding *e, const float *x, void *y, void *interm_fwd,
                                      size_t batch, void *stream) {
    TNN_GUARD_BEGIN
    if (int rc = nwe_checks(n, e, x, batch)) return rc;
    if (batch == 0) return 0;
    if (!y && !interm_fwd) return fail("forward needs y or interm_fwd");
    if (foldable(e)) {
        const tnn::EncodedInput enc{x, e->n_in, e->scale, e->offset};
        return run_forward(n, nullptr, y, interm_fwd, batch, stream, false, &enc);
    }
    if (grid_fusable(n, e) && (n->variant & 128)) {
        // hash grid gathered by extra warps of the network kernel straight into its input tile.  Opt-in (variant bit
        // 128): measured at the benchmark grid (3-D, 16 levels, batch 2^20, width 64, 2 hidden layers) the fused
        // kernel takes 0.58 ms against 0.39 ms for encoding kernel + network kernel - the gathers are bound by L2
        // latency and need about 12 000 loads in flight per SM, which the stand-alone kernel reaches with 1 536
        // gathering threads and the fused kernel, whose registers also serve the MMA issuers and epilogues, does not.
        const int rc = run_forward(n, nullptr, y, interm_fwd, batch, stream, false, nullptr, e, x);
        if (rc >= 0) return rc;
    }
    // other encodings: the encoded rows go through matrix 0 of interm_fwd when the caller provides it (that is where
    // the backward pass expects the network input), else through the handle's workspace
    void *encoded = interm_fwd;
    if (!encoded) {
        if (int rc = ensure_workspace(n, batch * n->width * sizeof(__nv_bfloat16), (cudaStream_t)stream)) return rc;
        encoded = n->ws;
    }
    if (int rc = tnn_encoding_forward(e, x, encoded, n->fp16 ? TNN_DTYPE_FP16 : TNN_DTYPE_BF16, batch, stream)) return rc;
    return run_forward(n, encoded, y, interm_fwd, batch, stream, /*copy_input=*/false);
    TNN_GUARD_END
}

int tnn_network_with_encoding_inference(tnn_network *n, tnn_encoding *e, const float *x, void *y, size_t batch,
                                        void *stream) {
    if (!y && batch) return fail("output is null");
    return tnn_network_with_encoding_forward(n, e, x, y, nullptr, batch, stream);
}

static int nwe_train_step_impl(tnn_network *n, tnn_encoding *e, const float *x, const float *targets, int n_targets,
                               size_t batch, float loss_scale, void *grads, int grads_dtype, int pack_transpose,
                               float *encoding_grads, int deterministic, float *loss_sum, void *stream, int *raw) {
    TNN_GUARD_BEGIN
    if (int rc = nwe_checks(n, e, x, batch)) return rc;
    if (foldable(e)) {
        const tnn::EncodedInput enc{x, e->n_in, e->scale, e->offset};
        return train_step_impl(n, nullptr, &enc, targets, n_targets, batch, loss_scale, grads, grads_dtype, pack_transpose,
                               nullptr, loss_sum, stream, raw);
    }
    if (batch == 0) return fail("batch_size == 0");
    const bool want_enc_grads = encoding_grads && e->n_params;
    if (int rc = ensure_workspace(n, nwe_workspace_bytes(n, batch), (cudaStream_t)stream)) return rc;
    // layout: [three-kernel workspace][encoded input][dL/d(encoded input)]
    uint8_t *base = reinterpret_cast<uint8_t *>(n->ws);
    const size_t mat = batch * n->width * sizeof(__nv_bfloat16);
    void *encoded = base + (size_t)(n->n_mat + 2) * mat;
    void *dx = want_enc_grads ? base + (size_t)(n->n_mat + 3) * mat : nullptr;
    const int net_dtype = n->fp16 ? TNN_DTYPE_FP16 : TNN_DTYPE_BF16;
    if (int rc = tnn_encoding_forward(e, x, encoded, net_dtype, batch, stream)) return rc;
    if (int rc = train_step_impl(n, encoded, nullptr, targets, n_targets, batch, loss_scale, grads, grads_dtype,
                                 pack_transpose, dx, loss_sum, stream, raw))
        return rc;
    if (want_enc_grads)
        return tnn_encoding_backward(e, x, dx, net_dtype, encoding_grads, batch, deterministic, stream);
    return 0;
    TNN_GUARD_END
}

int tnn_network_with_encoding_train_step(tnn_network *n, tnn_encoding *e, const float *x, const float *targets,
                                         int n_targets, size_t batch, float loss_scale, void *grads, int grads_dtype,
                                         int pack_transpose, float *encoding_grads, int deterministic, float *loss_sum,
                                         void *stream) {
    return nwe_train_step_impl(n, e, x, targets, n_targets, batch, loss_scale, grads, grads_dtype, pack_transpose,
                               encoding_grads, deterministic, loss_sum, stream, nullptr);
}

} // extern "C"

namespace tnn {
// The training pass as the trainer wants it: per-CTA slabs and loss partials left in the network's buffers.
int train_step_raw(tnn_network *n, tnn_encoding *e, const void *x, const float *targets, int n_targets, size_t batch,
                   float loss_scale, float *encoding_grads, int deterministic, int *n_slabs, int *n_loss_partials,
                   void *stream) {
    int raw[2] = {0, 0};
    int rc;
    if (e)
        rc = nwe_train_step_impl(n, e, (const float *)x, targets, n_targets, batch, loss_scale, nullptr, TNN_DTYPE_FP32, 1,
                                 encoding_grads, deterministic, nullptr, stream, raw);
    else if (!x)
        rc = fail("x and targets are required");
    else
        rc = train_step_impl(n, x, nullptr, targets, n_targets, batch, loss_scale, nullptr, TNN_DTYPE_FP32, 1, nullptr,
                             nullptr, stream, raw);
    *n_slabs = raw[0];
    *n_loss_partials = raw[1];
    return rc;
}
} // namespace tnn
