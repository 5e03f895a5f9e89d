// Trainer and data parallelism behind the C ABI.
//
// The reference's Trainer<T>::training_step (include/trainer.h:23-46) runs forward_pass and backward_pass; its
// training loops add torch's loss and torch.optim.Adam around the module, with one host round trip per piece.
// Here the whole loop body is device work enqueued by ONE call:
//
//   single GPU     fused forward + L2 + backward kernel -> ONE kernel that sums the per-CTA weight-gradient slabs
//                  and loss partials, applies Adam to the fp32 master parameters and rewrites the bf16 operand
//                  images the kernels read
//   data parallel  fused kernel -> ONE kernel that sums the slabs, pushes this rank's gradient into every peer's
//                  window over NVLink (plain peer stores + a flag per block), waits for the peers' blocks, adds the
//                  ranks' gradients in rank order (every rank gets the same bits) and applies Adam + operand refresh.
//                  Without peer windows (ranks on several hosts, no peer access, or a network larger than a window
//                  slot): slab / loss reduction -> ncclAllReduce(sum) of the (L+1) W^2 fp32 gradient buffer ->
//                  Adam + operand refresh.
//
// The reference has no data-parallel training (its MPI benchmarks run independent replicas,
// benchmarks/common_benchmarks.h:53-54); the exchange is what a data-parallel use of its modules needs: one
// all-reduce of the small weight-gradient buffer per step.  A trainable encoding (hash grid) shards its optimiser:
// reduce-scatter of the table gradient, Adam on this rank's slice of the table, all-gather of the table.
//
// NCCL is reached through dlopen, so the library itself links neither NCCL nor MPI: a process that already loaded
// NCCL (PyTorch does) shares that copy.
#include "../../include/tnn_b200.h"

#include "elementwise.h"
#include "handles.h"
#include "mlp_common.cuh"
#include "slab_sum.cuh"

#include <cmath>
#include <cuda_fp16.h>
#include <cstdlib>
#include <cstring>
#include <dlfcn.h>
#include <mutex>
#include <string>
#include <unistd.h>
#include <vector>

// ------------------------------------------------------------------------------------ NCCL by dlopen
namespace {

// The few NCCL entry points used, with the types of nccl.h (ncclComm_t is an opaque pointer, ncclUniqueId a
// 128-byte struct passed by value, enums are ints: ncclFloat32 = 7, ncclSum = 0).
struct NcclUniqueId { char internal[128]; };
struct NcclApi {
    int (*GetUniqueId)(NcclUniqueId *) = nullptr;
    int (*CommInitRank)(void **, int, NcclUniqueId, int) = nullptr;
    int (*CommDestroy)(void *) = nullptr;
    int (*CommCount)(void *, int *) = nullptr;
    int (*CommUserRank)(void *, int *) = nullptr;
    int (*AllReduce)(const void *, void *, size_t, int, int, void *, cudaStream_t) = nullptr;
    int (*ReduceScatter)(const void *, void *, size_t, int, int, void *, cudaStream_t) = nullptr;
    int (*AllGather)(const void *, void *, size_t, int, void *, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
    bool ok = false;
    std::string why;
};
constexpr int kNcclFloat32 = 7, kNcclSum = 0;

NcclApi &nccl() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD); // the copy the process already uses, if any
        if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) {
            api.why = "libnccl.so.2 could not be loaded";
            return;
        }
        auto sym = [&](const char *name) { return dlsym(h, name); };
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
        api.CommCount = reinterpret_cast<decltype(api.CommCount)>(sym("ncclCommCount"));
        api.CommUserRank = reinterpret_cast<decltype(api.CommUserRank)>(sym("ncclCommUserRank"));
        api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
        api.ReduceScatter = reinterpret_cast<decltype(api.ReduceScatter)>(sym("ncclReduceScatter"));
        api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
        api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.CommCount && api.CommUserRank &&
                 api.AllReduce && api.ReduceScatter && api.AllGather && api.GetErrorString;
        if (!api.ok) api.why = "libnccl.so.2 lacks an expected symbol";
    });
    return api;
}

int nccl_fail(const char *what, int rc) {
    return tnn::api_fail(std::string(what) + ": " + (nccl().GetErrorString ? nccl().GetErrorString(rc) : "NCCL error"), 3);
}

#define TNN_CUDA(expr)                                                                                                 \
    do {                                                                                                               \
        cudaError_t e_ = (expr);                                                                                       \
        if (e_ != cudaSuccess) return tnn::api_fail(std::string(#expr) + ": " + cudaGetErrorString(e_), 2);            \
    } while (0)

} // namespace

// Peer window of a communicator: one device buffer per rank, mapped into every rank of the same host (CUDA IPC).
// An element is 8 bytes: {fp32 value, exchange number}, written with ONE 8-byte store, so value and "it has arrived"
// travel together and no fence or separate flag is needed (the low-latency scheme of collective libraries; a
// release fence over outstanding peer stores alone costs several microseconds).  Rank s pushes its contribution of
// exchange number q into slot [q & 1][s] of every rank's window; the receiver polls its own memory until an element
// carries q.  Two slots per source are enough: a rank can start exchange q + 2 only after it finished q + 1, which
// needed every peer's contribution to q + 1, which a peer sends only after its kernel of exchange q has finished
// reading.
constexpr int kMaxPeers = 8;
constexpr size_t kWinSlotFloats = 256 * 1024; // largest gradient buffer exchanged through the window
constexpr int kWinBlock = tnn::kSlabBlock;     // weights per block of the exchange kernel
struct PeerWindow {
    uint2 *slots[kMaxPeers]; // slots[r]: rank r's window as mapped in this process (own window at [rank])
    int rank, world;
};
constexpr size_t win_bytes(int world) { return 2 * (size_t)world * kWinSlotFloats * sizeof(uint2); }

struct tnn_dp_comm {
    void *comm = nullptr; // ncclComm_t
    int rank = 0, world = 1;
    bool owned = false;
    // peer window (all null / false when the ranks cannot map each other's memory)
    void *win = nullptr;               // this rank's window (cudaMalloc)
    void *peer_base[kMaxPeers] = {};   // peers' windows as opened here
    PeerWindow pw{};
    bool peer_ok = false, peer_enabled = true;
    unsigned seq = 0; // exchanges enqueued so far
};

namespace {

struct WinExchange { // what the ranks tell each other when a communicator is made
    cudaIpcMemHandle_t handle;
    char host[64];
    char boot[48];
    int ok;
    int pad[3];
};
static_assert(sizeof(WinExchange) == 192, "exchange record");
constexpr int kNcclInt8 = 0;

void release_peer_window(tnn_dp_comm *c) {
    for (int r = 0; r < kMaxPeers; ++r) {
        if (c->peer_base[r]) cudaIpcCloseMemHandle(c->peer_base[r]);
        c->peer_base[r] = nullptr;
    }
    if (c->win) cudaFree(c->win);
    c->win = nullptr;
    c->peer_ok = false;
    cudaGetLastError();
}

// Collective over the communicator: every rank allocates its window, the IPC handles travel by ncclAllGather,
// every rank maps the others' windows, and a vote (ncclAllReduce) keeps the windows only if every rank mapped
// every peer.  Returns non-zero only when the collective itself failed; "no windows" is not an error.
int setup_peer_window(tnn_dp_comm *c) {
    c->peer_ok = false;
    const char *env = getenv("TNN_DP_PEER_WINDOW");
    if (env && env[0] == '0') return 0; // (the same on every rank)
    if (c->world < 2 || c->world > kMaxPeers) return 0;
    const int world = c->world;
    bool ok = true;
    WinExchange mine{};
    const size_t bytes = win_bytes(world);
    if (cudaMalloc(&c->win, bytes) != cudaSuccess) {
        c->win = nullptr;
        ok = false;
    }
    if (ok && cudaMemset(c->win, 0, bytes) != cudaSuccess) ok = false;
    if (ok && cudaIpcGetMemHandle(&mine.handle, c->win) != cudaSuccess) ok = false;
    cudaGetLastError();
    gethostname(mine.host, sizeof(mine.host) - 1);
    if (FILE *f = fopen("/proc/sys/kernel/random/boot_id", "r")) {
        if (!fgets(mine.boot, sizeof(mine.boot), f)) mine.boot[0] = 0;
        fclose(f);
    }
    mine.ok = ok ? 1 : 0;

    WinExchange *dev = nullptr; // [world] gathered records, then this rank's own
    if (cudaError_t ea = cudaMalloc(&dev, (world + 1) * sizeof(WinExchange)); ea != cudaSuccess) {
        release_peer_window(c);
        return tnn::api_fail(std::string("peer windows: ") + cudaGetErrorString(ea), 2);
    }
    std::vector<WinExchange> all(world);
    int rc = 0;
    cudaError_t e = cudaMemcpy(dev + world, &mine, sizeof(mine), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) rc = nccl().AllGather(dev + world, dev, sizeof(WinExchange), kNcclInt8, c->comm, nullptr);
    if (e == cudaSuccess && rc == 0) e = cudaStreamSynchronize(nullptr);
    if (e == cudaSuccess && rc == 0) e = cudaMemcpy(all.data(), dev, world * sizeof(WinExchange), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess || rc != 0) {
        cudaFree(dev);
        release_peer_window(c);
        return rc ? nccl_fail("ncclAllGather (peer windows)", rc)
                  : tnn::api_fail(std::string("peer windows: ") + cudaGetErrorString(e), 2);
    }
    for (int r = 0; r < world && ok; ++r) {
        if (!all[r].ok || strncmp(all[r].host, mine.host, sizeof(mine.host)) != 0 ||
            strncmp(all[r].boot, mine.boot, sizeof(mine.boot)) != 0)
            ok = false;
    }
    for (int r = 0; r < world && ok; ++r) {
        if (r == c->rank) continue;
        if (cudaIpcOpenMemHandle(&c->peer_base[r], all[r].handle, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            c->peer_base[r] = nullptr;
            ok = false;
        }
    }
    cudaGetLastError();
    // the vote; it also orders every rank's memset before any peer's first store
    float vote = ok ? 1.0f : 0.0f;
    float *dv = reinterpret_cast<float *>(dev);
    e = cudaMemcpy(dv, &vote, sizeof(float), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) rc = nccl().AllReduce(dv, dv, 1, kNcclFloat32, kNcclSum, c->comm, nullptr);
    if (e == cudaSuccess && rc == 0) e = cudaStreamSynchronize(nullptr);
    if (e == cudaSuccess && rc == 0) e = cudaMemcpy(&vote, dv, sizeof(float), cudaMemcpyDeviceToHost);
    cudaFree(dev);
    if (e != cudaSuccess || rc != 0) {
        release_peer_window(c);
        return rc ? nccl_fail("ncclAllReduce (peer windows)", rc)
                  : tnn::api_fail(std::string("peer windows: ") + cudaGetErrorString(e), 2);
    }
    if (vote < (float)world - 0.5f) {
        release_peer_window(c);
        return 0;
    }
    c->pw.rank = c->rank;
    c->pw.world = world;
    for (int r = 0; r < world; ++r) {
        char *base = static_cast<char *>(r == c->rank ? c->win : c->peer_base[r]);
        c->pw.slots[r] = reinterpret_cast<uint2 *>(base);
    }
    c->peer_ok = true;
    return 0;
}

unsigned long long peer_wait_ns() {
    const char *env = getenv("TNN_DP_WAIT_MS");
    const long ms = env ? atol(env) : 0;
    return (unsigned long long)(ms > 0 ? ms : 30000) * 1000000ull;
}

} // namespace

// ------------------------------------------------------------------------------------ kernels
namespace tnn {

__host__ __device__ inline int packed_coord_(int i, int j, int cols) {
    return (i & 1) == 0 ? i * cols + 2 * j : (i - 1) * cols + 2 * j + 1;
}

// Adam (torch.optim.Adam arithmetic, see adam_kernel) on the fp32 master parameters of a network, followed by the
// refresh of everything the kernels read: packed bf16 weights and both swizzled operand images, with the padding
// rows / columns forced to zero (Network.h:171-233).  One thread per weight.
// FROM_SLABS: the gradient is summed here from the per-CTA slabs of the training kernel (fixed order), and block 0
// also sums the loss partials; otherwise it is read from `grads` (already reduced, e.g. across ranks).
// The arithmetic shared by the two optimiser kernels: Adam on weight `pk` with gradient g (already scaled), then the
// refresh of the three 16-bit copies.
template <int W>
__device__ __forceinline__ void adam_and_refresh(int l, int o, int i, int pk, float g, float *__restrict__ master,
                                                 float *__restrict__ m, float *__restrict__ v, int n_mat,
                                                 int one_padded_in, int unpadded_out, float lr, float b1, float b2,
                                                 float eps, float bc1, float bc2_sqrt, int net_fp16,
                                                 __nv_bfloat16 *__restrict__ packed_out, __nv_bfloat16 *__restrict__ wimg,
                                                 __nv_bfloat16 *__restrict__ wimg_t) {
    using T = Tile<W>;
    const float mi = b1 * m[pk] + (1.0f - b1) * g;
    const float vi = b2 * v[pk] + (1.0f - b2) * g * g;
    m[pk] = mi;
    v[pk] = vi;
    const float denom = sqrtf(vi) / bc2_sqrt + eps;
    float p = master[pk] - (lr / bc1) * (mi / denom);
    master[pk] = p;
    if (l == 0 && i >= one_padded_in) p = 0.0f;
    if (l == n_mat - 1 && o >= unpadded_out) p = 0.0f;
    // the 16 bits the kernels read: bf16, or the bits of the fp16 value
    const __nv_bfloat16 b = net_fp16 ? __ushort_as_bfloat16(__half_as_ushort(__float2half_rn(p))) : __float2bfloat16_rn(p);
    packed_out[pk] = b;
    uint8_t *wi = reinterpret_cast<uint8_t *>(wimg) + (size_t)l * T::WGT_BYTES;
    uint8_t *wt = reinterpret_cast<uint8_t *>(wimg_t) + (size_t)l * T::WGT_BYTES;
    *reinterpret_cast<__nv_bfloat16 *>(wi + T::elem_off(i, o, T::WGT_ATOM_BYTES)) = b;
    *reinterpret_cast<__nv_bfloat16 *>(wt + T::elem_off(o, i, T::WGT_ATOM_BYTES)) = b;
}

// Sum of this rank's loss partials by the threads with threadIdx.y == 0 of one block (fixed order).
__device__ __forceinline__ void loss_sum_block(const float *__restrict__ loss_partials, int n_loss,
                                               float *__restrict__ loss_out, float *red) {
    if (threadIdx.y == 0) {
        float local = 0.0f;
        for (int i = threadIdx.x; i < n_loss; i += kSlabBlock) local += loss_partials[i];
        red[threadIdx.x] = local;
    }
    __syncthreads();
    for (int s = kSlabBlock / 2; s > 0; s >>= 1) {
        if (threadIdx.y == 0 && (int)threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.y == 0 && threadIdx.x == 0) *loss_out = red[0];
    __syncthreads();
}

// Blocks of (128, 8) threads when FROM_SLABS (see slab_sum), of (128, 1) otherwise.
template <int W, bool FROM_SLABS>
__global__ void __launch_bounds__(kSlabBlock *kSlabWays)
adam_refresh_kernel(float *__restrict__ master, float *__restrict__ m, float *__restrict__ v, float *__restrict__ grads,
                    const float *__restrict__ slabs, int n_slabs, const float *__restrict__ loss_partials, int n_loss,
                    float *__restrict__ loss_out, int n_mat, int one_padded_in, int unpadded_out, float grad_scale,
                    float lr, float b1, float b2, float eps, float bc1, float bc2_sqrt, int net_fp16,
                    __nv_bfloat16 *__restrict__ packed_out, __nv_bfloat16 *__restrict__ wimg,
                    __nv_bfloat16 *__restrict__ wimg_t, int *__restrict__ counters) {
    __shared__ float part[FROM_SLABS ? kSlabWays : 1][kSlabBlock];
    const int idx = blockIdx.x * kSlabBlock + threadIdx.x; // slab order: (matrix, output feature, input feature)
    const int per = n_mat * W * W;                          // a multiple of the block's 128 weights
    // counters (optional): {optimiser steps done, blocks of this launch that have read it}.  With it the step number
    // - Adam's bias correction - is device state: a CUDA graph that holds this launch advances it at every replay.
    const int step_now = counters ? *reinterpret_cast<volatile int *>(counters) + 1 : 0;
    if (FROM_SLABS && blockIdx.x == 0 && loss_out) loss_sum_block(loss_partials, n_loss, loss_out, part[0]);
    const int l = idx / (W * W);
    const int o = (idx / W) % W; // output feature
    const int i = idx % W;       // input feature
    const int pk = l * W * W + packed_coord_(i, o, W);
    float g;
    if constexpr (FROM_SLABS) {
        g = slab_sum(slabs, n_slabs, per, idx, part); // (holds a block barrier: every thread has read the counter)
    } else {
        g = grads[pk];
        if (counters) __syncthreads();
    }
    if constexpr (FROM_SLABS) {
        if (threadIdx.y != 0) return;
        grads[pk] = g;
    }
    if (counters) { // (only the 128 threads that apply the update pay for the two powf)
        bc1 = 1.0f - powf(b1, (float)step_now);
        bc2_sqrt = sqrtf(1.0f - powf(b2, (float)step_now));
    }
    adam_and_refresh<W>(l, o, i, pk, g * grad_scale, master, m, v, n_mat, one_padded_in, unpadded_out, lr, b1, b2, eps,
                        bc1, bc2_sqrt, net_fp16, packed_out, wimg, wimg_t);
    if (counters && threadIdx.x == 0) {
        // Every thread of this block read the old count before the block barrier above.  The last block to get here
        // therefore knows that every block has read it, and publishes the new one.
        int *ticket = counters + 1;
        if (atomicAdd(ticket, 1) == (int)gridDim.x - 1) {
            *ticket = 0;
            *reinterpret_cast<volatile int *>(counters) = step_now;
        }
    }
}

template <bool FROM_SLABS>
static cudaError_t launch_adam_refresh(int width, float *master, float *m, float *v, float *grads, const float *slabs,
                                       int n_slabs, const float *loss_partials, int n_loss, float *loss_out, int n_mat,
                                       int one_padded_in, int unpadded_out, float grad_scale, int step, float lr, float b1,
                                       float b2, float eps, int net_fp16, __nv_bfloat16 *packed, __nv_bfloat16 *wimg,
                                       __nv_bfloat16 *wimg_t, cudaStream_t s, int *counters = nullptr) {
    const int n = n_mat * width * width;
    const int blocks = n / kSlabBlock;
    const dim3 threads(kSlabBlock, FROM_SLABS ? kSlabWays : 1);
    const float bc1 = 1.0f - powf(b1, (float)step);
    const float bc2_sqrt = sqrtf(1.0f - powf(b2, (float)step));
    count_launch();
#define TNN_CASE(WW)                                                                                                    \
    case WW:                                                                                                            \
        adam_refresh_kernel<WW, FROM_SLABS><<<blocks, threads, 0, s>>>(                                                 \
            master, m, v, grads, slabs, n_slabs, loss_partials, n_loss, loss_out, n_mat, one_padded_in, unpadded_out,   \
            grad_scale, lr, b1, b2, eps, bc1, bc2_sqrt, net_fp16, packed, wimg, wimg_t, counters);                                \
        break;
    switch (width) {
        TNN_CASE(16) TNN_CASE(32) TNN_CASE(64) TNN_CASE(128)
    default: return cudaErrorInvalidValue;
    }
#undef TNN_CASE
    return cudaGetLastError();
}


// ---- data-parallel variant: gradient exchange through the peer windows inside the optimiser kernel
// 8-byte element {value bits, exchange number}: single stores and loads, never torn
__device__ __forceinline__ void st_elem(uint2 *p, float value, unsigned seq) {
    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(value)), "r"(seq) : "memory");
}
__device__ __forceinline__ uint2 ld_elem(const uint2 *p) {
    uint2 v;
    asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// One block = 128 consecutive weights (slab order), (128, 8) threads when FROM_SLABS, (128, 1) otherwise.  Sum the
// slabs (or take the already reduced gradient), store every value together with the exchange number into slot
// [seq & 1][rank] of every rank's window, then - one thread per weight - poll this rank's own window until the element
// of every source rank carries the exchange number (bounded: `wait_ns`), add the world contributions in rank order
// and run Adam + refresh on the sum.  A wait that runs out sets *status and the thread leaves its weight untouched.
template <int W, bool FROM_SLABS>
__global__ void __launch_bounds__(kSlabBlock *kSlabWays)
dp_adam_refresh_kernel(PeerWindow pw, unsigned seq, unsigned long long wait_ns, int *__restrict__ status,
                       float *__restrict__ master, float *__restrict__ m, float *__restrict__ v,
                       float *__restrict__ grads, const float *__restrict__ slabs, int n_slabs,
                       const float *__restrict__ loss_partials, int n_loss, float *__restrict__ loss_out, int n_mat,
                       int one_padded_in, int unpadded_out, float grad_scale, float lr, float b1, float b2, float eps,
                       float bc1, float bc2_sqrt, int net_fp16, __nv_bfloat16 *__restrict__ packed_out,
                       __nv_bfloat16 *__restrict__ wimg, __nv_bfloat16 *__restrict__ wimg_t) {
    __shared__ float part[FROM_SLABS ? kSlabWays : 1][kSlabBlock];
    const int tid = threadIdx.x;
    const int idx = blockIdx.x * kSlabBlock + tid;
    const int per = n_mat * W * W; // a multiple of the block's 128 weights
    const size_t parity = seq & 1u;
    if (FROM_SLABS && blockIdx.x == 0 && loss_out) loss_sum_block(loss_partials, n_loss, loss_out, part[0]);
    const int l = idx / (W * W);
    const int o = (idx / W) % W; // output feature
    const int i = idx % W;       // input feature
    const int pk = l * W * W + packed_coord_(i, o, W);
    float g;
    if constexpr (FROM_SLABS) {
        g = slab_sum(slabs, n_slabs, per, idx, part);
    } else {
        g = grads[pk];
    }
    // push: thread (x, y) stores weight x into the windows of the ranks y, y + 8, ...: slot [parity][rank] of every
    // window (this rank's own included, so that the sum below reads all ranks alike)
    const size_t slot = (parity * pw.world + pw.rank) * kWinSlotFloats + idx;
    if constexpr (FROM_SLABS) {
        if (threadIdx.y == 0) part[0][tid] = g;
        __syncthreads();
        g = part[0][tid];
    }
    for (int r = threadIdx.y; r < pw.world; r += blockDim.y) st_elem(pw.slots[r] + slot, g, seq);
    if (threadIdx.y != 0) return;
    // gather: the elements of all source ranks, in rank order
    const uint2 *own = pw.slots[pw.rank] + parity * pw.world * kWinSlotFloats + idx;
    const unsigned long long t0 = global_timer_ns();
    g = 0.0f;
    for (int r = 0; r < pw.world; ++r) {
        const uint2 *src = own + (size_t)r * kWinSlotFloats;
        uint2 e = ld_elem(src);
        for (unsigned it = 0; e.y != seq; ++it) {
            if ((it & 63u) == 63u) {
                if (global_timer_ns() - t0 > wait_ns) {
                    atomicOr(status, 2);
                    return;
                }
                __nanosleep(20);
            }
            e = ld_elem(src);
        }
        g += __uint_as_float(e.x);
    }
    grads[pk] = g; // the sum over ranks (what the all-reduce path leaves here)
    adam_and_refresh<W>(l, o, i, pk, g * grad_scale, master, m, v, n_mat, one_padded_in, unpadded_out, lr, b1, b2, eps,
                        bc1, bc2_sqrt, net_fp16, packed_out, wimg, wimg_t);
}

template <bool FROM_SLABS>
static cudaError_t launch_dp_adam_refresh(const PeerWindow &pw, unsigned seq, unsigned long long wait_ns, int *status,
                                          int width, float *master, float *m, float *v, float *grads,
                                          const float *slabs, int n_slabs, const float *loss_partials, int n_loss,
                                          float *loss_out, int n_mat, int one_padded_in, int unpadded_out,
                                          float grad_scale, int step, float lr, float b1, float b2, float eps,
                                          int net_fp16, __nv_bfloat16 *packed, __nv_bfloat16 *wimg,
                                          __nv_bfloat16 *wimg_t, cudaStream_t s) {
    const int n = n_mat * width * width;
    const int blocks = n / kWinBlock;
    const dim3 threads(kSlabBlock, FROM_SLABS ? kSlabWays : 1);
    const float bc1 = 1.0f - powf(b1, (float)step);
    const float bc2_sqrt = sqrtf(1.0f - powf(b2, (float)step));
    count_launch();
#define TNN_CASE(WW)                                                                                                    \
    case WW:                                                                                                            \
        dp_adam_refresh_kernel<WW, FROM_SLABS><<<blocks, threads, 0, s>>>(                                            \
            pw, seq, wait_ns, status, master, m, v, grads, slabs, n_slabs, loss_partials, n_loss, loss_out, n_mat,      \
            one_padded_in, unpadded_out, grad_scale, lr, b1, b2, eps, bc1, bc2_sqrt, net_fp16, packed, wimg, wimg_t);   \
        break;
    switch (width) {
        TNN_CASE(16) TNN_CASE(32) TNN_CASE(64) TNN_CASE(128)
    default: return cudaErrorInvalidValue;
    }
#undef TNN_CASE
    return cudaGetLastError();
}
} // namespace tnn

// entry points of capi.cu that hand the raw per-CTA results to the trainer instead of reducing them
namespace tnn {
int train_step_raw(tnn_network *n, tnn_encoding *e, const void *x, const float *targets, int n_targets, size_t batch,
                   float loss_scale, float *encoding_grads, int deterministic, int *n_slabs, int *n_loss_partials,
                   void *stream);
}

// ------------------------------------------------------------------------------------ trainer
struct tnn_trainer {
    tnn_network *net = nullptr;
    tnn_encoding *enc = nullptr;
    float lr = 1e-3f, b1 = 0.9f, b2 = 0.99f, eps = 1e-15f, loss_scale = 1.0f;
    int step = 0;
    float *master = nullptr, *m = nullptr, *v = nullptr, *grads = nullptr; // network: n_params fp32 each (one block)
    float *loss = nullptr;                                                  // one fp32: loss sum of the last step
    int *counters = nullptr; // {optimiser steps done, ticket}: the device-side step count of the optimiser kernel
    // trainable encoding: gradient of the whole table; moments for this rank's slice of it
    float *enc_grads = nullptr, *enc_m = nullptr, *enc_v = nullptr;
    size_t enc_shard = 0;      // table elements whose moments this rank keeps
    bool enc_sharded = false;  // reduce-scatter / sharded Adam / all-gather instead of all-reduce + replicated Adam
    int deterministic_encoding = 0;
    tnn_dp_comm *dp = nullptr;
    int n_slabs = 0, n_loss = 0; // what the last forward_backward left in the network's slab buffers
    bool reduced = false;        // grads / loss already hold the reduced values of the last forward_backward
};

namespace {

int world_of(const tnn_trainer *t) { return t->dp ? t->dp->world : 1; }
int rank_of(const tnn_trainer *t) { return t->dp ? t->dp->rank : 0; }

int alloc_encoding_state(tnn_trainer *t) {
    cudaFree(t->enc_grads);
    cudaFree(t->enc_m);
    cudaFree(t->enc_v);
    t->enc_grads = t->enc_m = t->enc_v = nullptr;
    if (!t->enc || !t->enc->n_params) return 0;
    const size_t n = t->enc->n_params;
    const size_t world = (size_t)world_of(t);
    // the optimiser state is sharded when the table splits into equal 16-byte aligned slices; otherwise every rank
    // keeps the whole state and the gradient is all-reduced
    t->enc_sharded = world > 1 && n % (4 * world) == 0;
    t->enc_shard = t->enc_sharded ? n / world : n;
    TNN_CUDA(cudaMalloc(&t->enc_grads, n * sizeof(float)));
    TNN_CUDA(cudaMemset(t->enc_grads, 0, n * sizeof(float)));
    TNN_CUDA(cudaMalloc(&t->enc_m, t->enc_shard * sizeof(float)));
    TNN_CUDA(cudaMalloc(&t->enc_v, t->enc_shard * sizeof(float)));
    TNN_CUDA(cudaMemset(t->enc_m, 0, t->enc_shard * sizeof(float)));
    TNN_CUDA(cudaMemset(t->enc_v, 0, t->enc_shard * sizeof(float)));
    return 0;
}

} // namespace

extern "C" {

// ---- data parallelism
int tnn_dp_get_unique_id(void *id128) {
    if (!id128) return tnn::api_fail("null argument");
    if (!nccl().ok) return tnn::api_fail("NCCL is not available: " + nccl().why, 3);
    NcclUniqueId id;
    if (int rc = nccl().GetUniqueId(&id)) return nccl_fail("ncclGetUniqueId", rc);
    memcpy(id128, &id, sizeof(id));
    return 0;
}

int tnn_dp_comm_create(const void *id128, int rank, int world, tnn_dp_comm **out) {
    if (!id128 || !out) return tnn::api_fail("null argument");
    *out = nullptr;
    if (world < 1 || rank < 0 || rank >= world) return tnn::api_fail("rank must be in [0, world)");
    if (!nccl().ok) return tnn::api_fail("NCCL is not available: " + nccl().why, 3);
    NcclUniqueId id;
    memcpy(&id, id128, sizeof(id));
    void *comm = nullptr;
    if (int rc = nccl().CommInitRank(&comm, world, id, rank)) return nccl_fail("ncclCommInitRank", rc);
    auto *c = new tnn_dp_comm();
    c->comm = comm;
    c->rank = rank;
    c->world = world;
    c->owned = true;
    if (int rc = setup_peer_window(c)) {
        tnn_dp_comm_destroy(c);
        return rc;
    }
    *out = c;
    return 0;
}

int tnn_dp_init(void *nccl_comm, tnn_dp_comm **out) {
    if (!nccl_comm || !out) return tnn::api_fail("null argument");
    *out = nullptr;
    if (!nccl().ok) return tnn::api_fail("NCCL is not available: " + nccl().why, 3);
    int world = 0, rank = 0;
    if (int rc = nccl().CommCount(nccl_comm, &world)) return nccl_fail("ncclCommCount", rc);
    if (int rc = nccl().CommUserRank(nccl_comm, &rank)) return nccl_fail("ncclCommUserRank", rc);
    auto *c = new tnn_dp_comm();
    c->comm = nccl_comm;
    c->rank = rank;
    c->world = world;
    c->owned = false;
    if (int rc = setup_peer_window(c)) {
        tnn_dp_comm_destroy(c);
        return rc;
    }
    *out = c;
    return 0;
}

int tnn_dp_comm_destroy(tnn_dp_comm *c) {
    if (!c) return 0;
    release_peer_window(c);
    if (c->owned && c->comm && nccl().ok) nccl().CommDestroy(c->comm);
    delete c;
    return 0;
}

int tnn_dp_rank(const tnn_dp_comm *c) { return c ? c->rank : 0; }
int tnn_dp_world_size(const tnn_dp_comm *c) { return c ? c->world : 1; }

int tnn_dp_peer_window(const tnn_dp_comm *c) { return (c && c->peer_ok && c->peer_enabled) ? 1 : 0; }
int tnn_dp_set_peer_window(tnn_dp_comm *c, int enable) {
    if (!c) return tnn::api_fail("communicator is null");
    c->peer_enabled = enable != 0;
    return 0;
}

int tnn_dp_allreduce_sum(tnn_dp_comm *c, float *buf, size_t n, void *stream) {
    if (!buf) return tnn::api_fail("null argument");
    if (!c || c->world == 1 || n == 0) return 0;
    if (int rc = nccl().AllReduce(buf, buf, n, kNcclFloat32, kNcclSum, c->comm, (cudaStream_t)stream))
        return nccl_fail("ncclAllReduce", rc);
    return 0;
}

// ---- trainer
int tnn_trainer_create(tnn_network *net, tnn_encoding *enc, float lr, float beta1, float beta2, float eps,
                       float loss_scale, tnn_trainer **out) {
    if (!net || !out) return tnn::api_fail("null argument");
    *out = nullptr;
    if (loss_scale == 0.0f) return tnn::api_fail("loss_scale must not be 0");
    if (enc && enc->padded != net->width)
        return tnn::api_fail("the encoding's padded output width must equal the network width");
    auto *t = new tnn_trainer();
    t->net = net;
    t->enc = enc;
    t->lr = lr, t->b1 = beta1, t->b2 = beta2, t->eps = eps, t->loss_scale = loss_scale;
    const size_t n = net->n_params;
    cudaError_t e = cudaMalloc(&t->master, (4 * n + 8) * sizeof(float));
    if (e == cudaSuccess) e = cudaMemset(t->master, 0, (4 * n + 8) * sizeof(float));
    if (e != cudaSuccess) {
        delete t;
        return tnn::api_fail(std::string("device allocation failed: ") + cudaGetErrorString(e), 2);
    }
    t->m = t->master + n;
    t->v = t->m + n;
    t->grads = t->v + n;
    t->loss = t->grads + n;
    t->counters = reinterpret_cast<int *>(t->loss + 4);
    // master copy = the network's current (bf16) weights; tnn_trainer_set_master_params replaces it with the fp32 draw
    e = net->fp16 ? tnn::launch_fp16_to_f32(net->packed, t->master, n, nullptr)
                  : tnn::launch_bf16_to_f32(net->packed, t->master, n, nullptr);
    if (e == cudaSuccess) e = cudaStreamSynchronize(nullptr);
    if (e != cudaSuccess) {
        tnn_trainer_destroy(t);
        return tnn::api_fail(std::string("master copy: ") + cudaGetErrorString(e), 2);
    }
    if (int rc = alloc_encoding_state(t)) {
        tnn_trainer_destroy(t);
        return rc;
    }
    *out = t;
    return 0;
}

int tnn_trainer_destroy(tnn_trainer *t) {
    if (!t) return 0;
    cudaFree(t->master);
    cudaFree(t->enc_grads);
    cudaFree(t->enc_m);
    cudaFree(t->enc_v);
    delete t;
    return 0;
}

int tnn_trainer_set_dp(tnn_trainer *t, tnn_dp_comm *comm) {
    if (!t) return tnn::api_fail("trainer is null");
    if (t->step != 0 && t->enc && t->enc->n_params)
        return tnn::api_fail("the communicator of a trainer with a trainable encoding must be set before the first step");
    t->dp = comm;
    return alloc_encoding_state(t); // the encoding's optimiser state is sharded over the ranks
}

int tnn_trainer_set_deterministic_encoding(tnn_trainer *t, int deterministic) {
    if (!t) return tnn::api_fail("trainer is null");
    t->deterministic_encoding = deterministic ? 1 : 0;
    return 0;
}

int tnn_trainer_set_master_params(tnn_trainer *t, const float *packed_fp32, void *stream) {
    if (!t || !packed_fp32) return tnn::api_fail("null argument");
    TNN_CUDA(cudaMemcpyAsync(t->master, packed_fp32, t->net->n_params * sizeof(float), cudaMemcpyDeviceToDevice,
                             (cudaStream_t)stream));
    return tnn_network_set_params(t->net, t->master, TNN_DTYPE_FP32, 1, stream);
}

float *tnn_trainer_master_params(tnn_trainer *t) { return t ? t->master : nullptr; }
float *tnn_trainer_grads(tnn_trainer *t) { return t ? t->grads : nullptr; }
float *tnn_trainer_encoding_grads(tnn_trainer *t) { return t ? t->enc_grads : nullptr; }
float *tnn_trainer_loss(tnn_trainer *t) { return t ? t->loss : nullptr; }
int tnn_trainer_step_count(const tnn_trainer *t) { return t ? t->step : 0; }

int tnn_trainer_forward_backward(tnn_trainer *t, const void *x, const float *targets, int n_targets, size_t batch,
                                 void *stream) {
    if (!t) return tnn::api_fail("trainer is null");
    t->reduced = false;
    if (int rc = tnn::train_step_raw(t->net, t->enc, x, targets, n_targets, batch, t->loss_scale,
                                     (t->enc && t->enc->n_params) ? t->enc_grads : nullptr, t->deterministic_encoding,
                                     &t->n_slabs, &t->n_loss, stream))
        return rc;
    return 0;
}

// Sums the slabs and loss partials the last forward_backward left behind into grads / loss (no optimiser step).
int tnn_trainer_reduce(tnn_trainer *t, void *stream) {
    if (!t) return tnn::api_fail("trainer is null");
    if (t->reduced) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    tnn_network *n = t->net;
    TNN_CUDA(tnn::launch_reduce_dw(n->dw_slabs, t->n_slabs, n->n_mat, n->width, 1, 1.0f, t->grads, nullptr, 0, s,
                                   n->loss_partials, t->n_loss, t->loss));
    t->reduced = true;
    return 0;
}

int tnn_trainer_optimizer_step(tnn_trainer *t, void *stream) {
    if (!t) return tnn::api_fail("trainer is null");
    cudaStream_t s = (cudaStream_t)stream;
    // A single-GPU trainer without a trainable encoding keeps its step count (Adam's bias correction) on the device,
    // so its step can be captured into a CUDA graph and replayed.  With a communicator the exchange number of the
    // peer windows, and with a trainable encoding the step count of its Adam kernel, are host state that goes into
    // kernel arguments: a captured graph would replay stale values.
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    if ((world_of(t) > 1 || (t->enc && t->enc->n_params)) && cudaStreamIsCapturing(s, &capturing) == cudaSuccess &&
        capturing != cudaStreamCaptureStatusNone)
        return tnn::api_fail("tnn_trainer_optimizer_step cannot be captured into a CUDA graph with a communicator or a "
                             "trainable encoding: step count and exchange number are arguments of its kernels");
    tnn_network *n = t->net;
    const int world = world_of(t);
    const float grad_scale = 1.0f / (t->loss_scale * (float)world);
    t->step += 1;
    const bool windowed = world > 1 && tnn_dp_peer_window(t->dp) && n->n_params <= kWinSlotFloats;
    if (world > 1 && !windowed) {
        if (int rc = tnn_trainer_reduce(t, stream)) return rc;
        if (int rc = tnn_dp_allreduce_sum(t->dp, t->grads, n->n_params, stream)) return rc;
    }
    if (windowed) {
        // slab sum + exchange over the peer windows + Adam + refresh in one kernel
        const unsigned seq = ++t->dp->seq;
        if (t->reduced)
            TNN_CUDA(tnn::launch_dp_adam_refresh<false>(t->dp->pw, seq, peer_wait_ns(), n->status, n->width, t->master,
                                                        t->m, t->v, t->grads, nullptr, 0, nullptr, 0, nullptr, n->n_mat,
                                                        n->one_padded_input(), n->output_width, grad_scale, t->step,
                                                        t->lr, t->b1, t->b2, t->eps, n->fp16, n->packed, n->wimg,
                                                        n->wimg_t, s));
        else
            TNN_CUDA(tnn::launch_dp_adam_refresh<true>(t->dp->pw, seq, peer_wait_ns(), n->status, n->width, t->master,
                                                       t->m, t->v, t->grads, n->dw_slabs, t->n_slabs, n->loss_partials,
                                                       t->n_loss, t->loss, n->n_mat, n->one_padded_input(),
                                                       n->output_width, grad_scale, t->step, t->lr, t->b1, t->b2, t->eps,
                                                       n->fp16, n->packed, n->wimg, n->wimg_t, s));
        t->reduced = true;
    } else if (world > 1 || t->reduced) {
        TNN_CUDA(tnn::launch_adam_refresh<false>(n->width, t->master, t->m, t->v, t->grads, nullptr, 0, nullptr, 0, nullptr,
                                                 n->n_mat, n->one_padded_input(), n->output_width, grad_scale, t->step,
                                                 t->lr, t->b1, t->b2, t->eps, n->fp16, n->packed, n->wimg, n->wimg_t, s,
                                                 world == 1 ? t->counters : nullptr));
    } else {
        TNN_CUDA(tnn::launch_adam_refresh<true>(n->width, t->master, t->m, t->v, t->grads, n->dw_slabs, t->n_slabs,
                                                n->loss_partials, t->n_loss, t->loss, n->n_mat, n->one_padded_input(),
                                                n->output_width, grad_scale, t->step, t->lr, t->b1, t->b2, t->eps, n->fp16,
                                                n->packed, n->wimg, n->wimg_t, s, t->counters));
        t->reduced = true;
    }
    if (t->enc && t->enc->n_params) {
        tnn_encoding *e = t->enc;
        float *table = e->params();
        if (!t->enc_sharded) {
            if (world > 1)
                if (int rc = tnn_dp_allreduce_sum(t->dp, t->enc_grads, e->n_params, stream)) return rc;
            TNN_CUDA(tnn::launch_adam(table, t->enc_m, t->enc_v, t->enc_grads, e->n_params, grad_scale, t->step, t->lr,
                                      t->b1, t->b2, t->eps, nullptr, s));
        } else {
            // sharded optimiser: each rank owns enc_shard consecutive table entries
            const size_t off = (size_t)rank_of(t) * t->enc_shard;
            if (int rc = nccl().ReduceScatter(t->enc_grads, t->enc_grads + off, t->enc_shard, kNcclFloat32, kNcclSum,
                                              t->dp->comm, s))
                return nccl_fail("ncclReduceScatter", rc);
            TNN_CUDA(tnn::launch_adam(table + off, t->enc_m, t->enc_v, t->enc_grads + off, t->enc_shard, grad_scale,
                                      t->step, t->lr, t->b1, t->b2, t->eps, nullptr, s));
            if (int rc = nccl().AllGather(table + off, table, t->enc_shard, kNcclFloat32, t->dp->comm, s))
                return nccl_fail("ncclAllGather", rc);
        }
    }
    return 0;
}

int tnn_trainer_training_step(tnn_trainer *t, const void *x, const float *targets, int n_targets, size_t batch,
                              void *stream) {
    if (int rc = tnn_trainer_forward_backward(t, x, targets, n_targets, batch, stream)) return rc;
    return tnn_trainer_optimizer_step(t, stream);
}

} // extern "C"
