// L2 loss for callers that are not allowed to allocate device memory.
//
// tnn_l2_loss keeps its per-block partial sums in a buffer it allocates on first use.  Some callers cannot
// tolerate that: a plug-in living inside a host application whose own allocator has already claimed all
// free device memory (a cudaMalloc from the plug-in then fails, or steals from the host's pool), or a
// latency-critical loop in which the implicit device-wide synchronisation of an allocation is unacceptable.
// For them this entry point computes the same loss with the partial sums in a fixed array that is part of
// the library image itself, so nothing is ever allocated or freed - at the price of a size limit and of
// every call on a device sharing that one array.
#include "../../include/tnn_b200.h"

#include "elementwise.h"

#include <string>

namespace tnn {
int api_fail(const std::string &msg, int code); // records the message behind tnn_last_error(), returns code
}

namespace {

constexpr int kStaticPartials = 4096;            // one partial sum per block
constexpr size_t kElemsPerPartial = 32768;       // elements one block reduces
constexpr size_t kMaxElements = (size_t)kStaticPartials * kElemsPerPartial; // 2^27 = batch * stride limit
constexpr int kMaxDevices = 64;

// The scratch array.  It occupies 16 KiB on every GPU that loads the library, until the process exits.
// In host code this name is only a handle for the runtime, not a device address.
static __device__ __align__(256) float g_l2_static_partials[kStaticPartials];

// Device address of the array, looked up once per device.
float *g_partials_addr[kMaxDevices] = {};

} // namespace

extern "C" int tnn_l2_loss_static(const void *pred, const float *target, int n_targets, float *values, void *grads,
                                  size_t batch, int stride, float loss_scale, float *loss_sum, void *stream) {
    if (batch == 0) return 0;
    if (!pred || !target) return tnn::api_fail("null argument", 1);
    if (n_targets <= 0 || n_targets > stride) return tnn::api_fail("n_targets must be in [1, stride]", 1);
    if (loss_scale == 0.0f) return tnn::api_fail("loss_scale must not be 0", 1);
    if (stride % 16 != 0) return tnn::api_fail("stride must be a multiple of 16 (network widths are)", 1);
    {
        auto mis = [](const void *q, uintptr_t a) { return q && reinterpret_cast<uintptr_t>(q) % a != 0; };
        if (mis(pred, 16) || mis(values, 16) || mis(grads, 16))
            return tnn::api_fail("pred, values and grads must be 16-byte aligned", 1);
        if (mis(target, n_targets == stride ? 16 : 4))
            return tnn::api_fail("target must be 16-byte aligned when n_targets == stride (4-byte aligned otherwise)", 1);
    }
    const size_t n_el = batch * (size_t)stride;
    if (n_el > kMaxElements)
        return tnn::api_fail("tnn_l2_loss_static: batch * stride = " + std::to_string(n_el) +
                                 " exceeds the capacity of the static scratch array (" + std::to_string(kMaxElements) +
                                 " elements); use tnn_l2_loss or split the batch",
                             1);
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return tnn::api_fail(std::string("cudaGetDevice: ") + cudaGetErrorString(e), 2);
    if (dev < 0 || dev >= kMaxDevices) return tnn::api_fail("device ordinal out of range", 1);
    if (!g_partials_addr[dev]) {
        // set-up, once per device, with that device current: translate the symbol into a device address
        float *ptr = nullptr;
        e = cudaGetSymbolAddress((void **)&ptr, g_l2_static_partials);
        if (e != cudaSuccess || !ptr)
            return tnn::api_fail(std::string("cudaGetSymbolAddress(g_l2_static_partials): ") + cudaGetErrorString(e), 2);
        g_partials_addr[dev] = ptr;
    }
    const int n_partials = (int)((n_el + kElemsPerPartial - 1) / kElemsPerPartial);
    // every one of the n_partials slots is overwritten by its block and only those slots are summed, so
    // nothing left over from an earlier call can leak into this one and nothing needs clearing
    e = tnn::launch_l2_loss((const __nv_bfloat16 *)pred, /*fp16=*/0, target, n_targets, values, (__nv_bfloat16 *)grads, batch, stride,
                            loss_scale, loss_sum ? g_partials_addr[dev] : nullptr, n_partials, loss_sum,
                            (cudaStream_t)stream);
    if (e != cudaSuccess) return tnn::api_fail(std::string("l2 loss launch: ") + cudaGetErrorString(e), 2);
    return 0;
}
