// Stand-alone microbenchmark of the tcgen05 building blocks the fused-MLP kernels are designed around.
// Not part of libtnn_b200.so; build and run with
//     python tiny-dpcpp-nn_b200/build.py --microbench && tiny-dpcpp-nn_b200/umma_microbench
// Part 1: cycles per tcgen05.mma (bf16 -> fp32, K = 16) as a function of M, N, where the operands live
//         (shared memory K-major / MN-major, or A in tensor memory) and how the issuing code is written
//         (one thread inside a divergent branch, or a converged warp that elects one lane).
// Part 2: latency of shared-memory round trips (mbarrier test_wait / try_wait, dependent ld.shared,
//         mbarrier arrive) while another warp streams MMAs whose operands come from shared memory.
// One CTA; every wait is bounded.
#include <cstdio>
#include <cuda_runtime.h>

#include "umma.cuh"
using namespace tnn;

constexpr int kSmemBytes = 100 * 1024;

// STYLE 0: single thread in a divergent branch; 1: converged warp + elect, A in shared memory;
// 2: converged warp + elect, A in tensor memory
template <int M, int N, int A_MN, int B_MN, int STYLE> __global__ void mma_rate(int reps, long long *out) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_base_s;
    __shared__ uint32_t abortf;
    for (int i = threadIdx.x; i < 65536 / 4; i += blockDim.x) reinterpret_cast<uint32_t *>(smem)[i] = 0;
    if (threadIdx.x == 0) {
        ptx::mbar_init(&bar, 1);
        abortf = 0;
        ptx::fence_barrier_init();
    }
    if (threadIdx.x < 32) {
        ptx::tmem_alloc(&tmem_base_s, 512);
        ptx::tmem_relinquish();
    }
    ptx::fence_proxy_async_smem();
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tb = tmem_base_s;
    constexpr uint32_t idesc = ptx::make_idesc_bf16(M, N, A_MN, B_MN);
    volatile uint32_t *af = &abortf;
    const uint64_t a = ptx::make_smem_desc(ptx::smem_u32(smem), A_MN ? 16384 : 16, 1024, 2);
    const uint64_t b = ptx::make_smem_desc(ptx::smem_u32(smem) + 32768, B_MN ? 16384 : 16, 1024, 2);
    auto burst = [&]() {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (STYLE == 2)
                ptx::mma_ts(tb, tb + 256 + 8 * k, b + (B_MN ? 128 * k : 2 * k), idesc, 1u);
            else
                ptx::mma_ss(tb, a + (A_MN ? 128 * k : 2 * k), b + (B_MN ? 128 * k : 2 * k), idesc, 1u);
        }
    };
    if (STYLE == 0) {
        if (threadIdx.x == 0) {
            const long long t0 = clock64();
            for (int r = 0; r < reps; ++r) burst();
            const long long t1 = clock64();
            ptx::mma_commit(&bar);
            ptx::mbar_wait(&bar, 0, af);
            const long long t2 = clock64();
            out[0] = t1 - t0;
            out[1] = t2 - t0;
        }
    } else if (threadIdx.x < 32) {
        const long long t0 = clock64();
        for (int r = 0; r < reps; ++r) {
            if (ptx::elect_one()) burst();
            __syncwarp();
        }
        const long long t1 = clock64();
        if (ptx::elect_one()) ptx::mma_commit(&bar);
        __syncwarp();
        ptx::mbar_wait(&bar, 0, af);
        const long long t2 = clock64();
        if (threadIdx.x == 0) {
            out[0] = t1 - t0;
            out[1] = t2 - t0;
        }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x < 32) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tb, 512);
    }
}

template <int M, int N, int A_MN, int B_MN, int STYLE> static int run_rate(long long *d) {
    auto k = mma_rate<M, N, A_MN, B_MN, STYLE>;
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    long long h[2];
    for (int it = 0; it < 2; ++it) {
        k<<<1, 128, kSmemBytes>>>(64, d);
        const cudaError_t e = cudaDeviceSynchronize();
        if (e != cudaSuccess) {
            printf("error: %s\n", cudaGetErrorString(e));
            return 1;
        }
        cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost);
    }
    static const char *style[] = {"single thread", "elected lane ", "elected, A=TMEM"};
    printf("%-16s A %s B %s  M=%3d N=%3d: issue %6.1f, complete %6.1f cycles per MMA  (%.0f flop/cycle)\n", style[STYLE],
           STYLE == 2 ? "tmem" : (A_MN ? "MN  " : "K   "), B_MN ? "MN" : "K ", M, N, h[0] / 256.0, h[1] / 256.0,
           2.0 * M * N * 16 * 256 / h[1]);
    return 0;
}

__global__ void sync_latency(int mma_bursts, int reps, long long *out) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t bar, done_bar, mma_bar;
    __shared__ uint32_t tmem_base_s;
    __shared__ uint32_t abortf;
    __shared__ volatile uint32_t stop;
    for (int i = threadIdx.x; i < 65536 / 4; i += blockDim.x) reinterpret_cast<uint32_t *>(smem)[i] = 0;
    if (threadIdx.x == 0) {
        ptx::mbar_init(&bar, 1);
        ptx::mbar_init(&done_bar, 1);
        ptx::mbar_init(&mma_bar, 1);
        abortf = 0;
        stop = 0;
        ptx::fence_barrier_init();
    }
    if (threadIdx.x < 32) {
        ptx::tmem_alloc(&tmem_base_s, 512);
        ptx::tmem_relinquish();
    }
    ptx::fence_proxy_async_smem();
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tb = tmem_base_s;
    volatile uint32_t *af = &abortf;
    const int warp = threadIdx.x / 32;
    if (warp == 0) {
        // streams bursts of 4 x mma_bursts MMAs (M = 128, N = 64) until told to stop, at most 4000 bursts
        constexpr uint32_t idesc = ptx::make_idesc_bf16(128, 64, 0, 0);
        const uint64_t a = ptx::make_smem_desc(ptx::smem_u32(smem), 16, 1024, 2);
        const uint64_t b = ptx::make_smem_desc(ptx::smem_u32(smem) + 32768, 16, 1024, 2);
        uint32_t par = 0;
        for (int r = 0; mma_bursts && r < 4000 && !stop; ++r) {
            if (ptx::elect_one()) {
                for (int rr = 0; rr < mma_bursts; ++rr) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) ptx::mma_ss(tb, a + 2 * k, b + 2 * k, idesc, 1u);
                }
                ptx::mma_commit(&mma_bar);
            }
            __syncwarp();
            if (!ptx::mbar_wait(&mma_bar, par, af)) break;
            par ^= 1;
        }
    } else if (warp == 1) {
        if (threadIdx.x == 32) ptx::mbar_arrive(&bar); // phase 0 complete: the waits below pass at once
        __syncwarp();
        for (volatile int w = 0; w < 2000; ++w) {
        }
        const long long t0 = clock64();
        uint32_t acc = 0;
        for (int r = 0; r < reps; ++r) acc += ptx::mbar_test_wait(&bar, 0);
        const long long t1 = clock64();
        for (int r = 0; r < reps; ++r) acc += ptx::mbar_try_wait(&bar, 0);
        const long long t2 = clock64();
        volatile uint32_t *sp = reinterpret_cast<volatile uint32_t *>(smem + 49152);
        uint32_t idx = threadIdx.x & 31;
        for (int r = 0; r < reps; ++r) idx = sp[idx] + (threadIdx.x & 31);
        const long long t3 = clock64();
        for (int r = 0; r < reps; ++r)
            if ((threadIdx.x & 31) == 0) ptx::mbar_arrive(&done_bar);
        const long long t4 = clock64();
        if (threadIdx.x == 32) {
            out[0] = t1 - t0;
            out[1] = t2 - t1;
            out[2] = t3 - t2;
            out[3] = t4 - t3;
            out[4] = acc + idx;
        }
        stop = 1;
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x < 32) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tb, 512);
    }
}

int main() {
    long long *d;
    cudaMalloc(&d, 64);
    int rc = 0;
    printf("-- part 1: cycles per tcgen05.mma (256 back-to-back, one accumulator)\n");
    rc |= run_rate<128, 64, 0, 0, 0>(d);
    rc |= run_rate<128, 64, 0, 0, 1>(d);
    rc |= run_rate<128, 64, 0, 1, 1>(d);
    rc |= run_rate<128, 64, 1, 1, 1>(d);
    rc |= run_rate<128, 64, 0, 0, 2>(d);
    rc |= run_rate<128, 64, 0, 1, 2>(d);
    rc |= run_rate<64, 64, 1, 1, 0>(d);
    rc |= run_rate<64, 64, 1, 1, 1>(d);
    rc |= run_rate<64, 64, 0, 0, 2>(d);
    rc |= run_rate<128, 16, 0, 0, 1>(d);
    rc |= run_rate<128, 32, 0, 0, 1>(d);
    rc |= run_rate<128, 128, 0, 0, 1>(d);
    rc |= run_rate<128, 256, 0, 0, 1>(d);
    rc |= run_rate<128, 32, 0, 0, 2>(d);
    rc |= run_rate<128, 128, 0, 0, 2>(d);
    rc |= run_rate<128, 256, 0, 0, 2>(d);
    rc |= run_rate<64, 32, 0, 0, 1>(d);
    rc |= run_rate<64, 16, 0, 0, 1>(d);
    if (rc) return rc;
    printf("-- part 2: shared-memory round trips beside an MMA stream (256 each, cycles per operation)\n");
    cudaFuncSetAttribute(sync_latency, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    for (int on : {0, 1, 4, 64}) {
        long long h[5];
        for (int it = 0; it < 2; ++it) {
            sync_latency<<<1, 64, kSmemBytes>>>(on, 256, d);
            const cudaError_t e = cudaDeviceSynchronize();
            if (e != cudaSuccess) {
                printf("error: %s\n", cudaGetErrorString(e));
                return 1;
            }
            cudaMemcpy(h, d, 40, cudaMemcpyDeviceToHost);
        }
        printf("MMA bursts of %2d x 4: test_wait %6.1f  try_wait %6.1f  dependent ld.shared %6.1f  arrive %6.1f\n", on,
               h[0] / 256.0, h[1] / 256.0, h[2] / 256.0, h[3] / 256.0);
    }
    return 0;
}
