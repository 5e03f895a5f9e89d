// Fully fused MLP forward / inference for sm_100a.
//
// Replaces EsimdKernels::forward_impl_general<INFERENCE> of the reference
// (include/network/kernel_esimd.h:565-640): y = act_out(... act(act(x W0) W1) ... WL), all
// matrices W x W, bf16 operands, fp32 accumulation, rounding to bf16 after every layer.
//
// One persistent CTA per SM walks over 128-row batch tiles.  Roles:
//   warp 0      : TMA producer - stages the weights once, then streams input tiles
//   warp 1      : MMA issuer   - owns TMEM, issues tcgen05.mma for every (tile, layer)
//   warps 2...  : NSLOT epilogue groups of 4 warps; group g owns pipeline slot g
// A slot is one tile in flight: its input buffer, two activation buffers and one fp32
// accumulator of W TMEM columns.  Per layer the group pulls the accumulator out of TMEM,
// applies the activation, rounds to bf16 and writes the next layer's A operand straight
// back to swizzled shared memory (or, with TMEM_A, back to TMEM), so activations never
// leave the SM.  With STORE_ALL every layer's activation is also written to global memory
// by TMA for a later backward pass.
#include "mlp_common.cuh"
#include "mlp_launch.h"

namespace tnn {

template <int W, int NSLOT, bool TMEM_A> struct FwdSmem {
    using T = Tile<W>;
    static constexpr int XBUF = 0;                                     // NSLOT input tiles
    static constexpr int ABUF = XBUF + NSLOT * T::ACT_BYTES;           // NSLOT x 2 activation tiles
    static constexpr int WBUF = ABUF + NSLOT * 2 * T::ACT_BYTES;       // (L+1) weight tiles follow
    static constexpr int tmem_cols_needed = NSLOT * (W + (TMEM_A ? W / 2 : 0));
    static constexpr int tmem_cols =
        tmem_cols_needed <= 32 ? 32 : tmem_cols_needed <= 64 ? 64 : tmem_cols_needed <= 128 ? 128
                                                              : tmem_cols_needed <= 256 ? 256 : 512;
    static_assert(tmem_cols_needed <= 512, "TMEM overflow");
};

struct FwdBarriers {
    uint64_t w_full;
    uint64_t x_full[4];
    uint64_t x_empty[4];
    uint64_t a_ready[4];
    uint64_t acc_full[4];
    uint32_t tmem_base;
    uint32_t abort_flag;
};

template <int W, int NSLOT, bool STORE_ALL, bool TMEM_A, bool B_MN_MAJOR>
__global__ void __launch_bounds__(64 + 128 * NSLOT, 1)
mlp_fwd_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_y,
               const __grid_constant__ CUtensorMap tm_interm, const __nv_bfloat16 *__restrict__ wimg,
               int n_tiles, int n_mat, int act, int out_act, int write_y, int *status) {
    using T = Tile<W>;
    using S = FwdSmem<W, NSLOT, TMEM_A>;
    extern __shared__ uint8_t smem_raw[];
    // operand tiles need 1024-byte alignment (swizzle span)
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ FwdBarriers bars;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int L = n_mat - 1; // index of the output layer
    const uint32_t smem_base = ptx::smem_u32(smem);
    volatile uint32_t *abort_flag = &bars.abort_flag;

    // tiles handled by this CTA: blockIdx.x, blockIdx.x + gridDim.x, ...
    const int my_tiles = (n_tiles > (int)blockIdx.x) ? (n_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

    if (threadIdx.x == 0) {
        ptx::mbar_init(&bars.w_full, 1);
        for (int s = 0; s < NSLOT; ++s) {
            ptx::mbar_init(&bars.x_full[s], 1);
            ptx::mbar_init(&bars.x_empty[s], 1);
            ptx::mbar_init(&bars.a_ready[s], 128);
            ptx::mbar_init(&bars.acc_full[s], 1);
        }
        bars.abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::prefetch_tmap(&tm_x);
        ptx::prefetch_tmap(&tm_y);
        if (STORE_ALL) ptx::prefetch_tmap(&tm_interm);
    }
    if (warp == 1) {
        ptx::tmem_alloc(&bars.tmem_base, S::tmem_cols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = bars.tmem_base;

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        if (lane == 0 && my_tiles > 0) {
            ptx::mbar_arrive_expect_tx(&bars.w_full, (uint32_t)(n_mat * T::WGT_BYTES));
            for (int l = 0; l < n_mat; ++l)
                ptx::bulk_load(smem + S::WBUF + l * T::WGT_BYTES,
                               reinterpret_cast<const uint8_t *>(wimg) + (size_t)l * T::WGT_BYTES, T::WGT_BYTES,
                               &bars.w_full);
            for (int j = 0; j < my_tiles; ++j) {
                const int s = j % NSLOT, t = j / NSLOT;
                const int tile = blockIdx.x + j * gridDim.x;
                if (t >= 1 && !ptx::mbar_wait(&bars.x_empty[s], (t - 1) & 1, abort_flag)) {
                    atomicExch(status, KS_TIMEOUT_PRODUCER | s);
                    break;
                }
                ptx::mbar_arrive_expect_tx(&bars.x_full[s], T::ACT_BYTES);
                for (int a = 0; a < T::KATOMS; ++a)
                    ptx::tma_load_2d(smem + S::XBUF + s * T::ACT_BYTES + a * T::ACT_ATOM_BYTES, &tm_x,
                                     a * T::ATOM_COLS, tile * T::TM, &bars.x_full[s]);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0 && my_tiles > 0) {
            constexpr uint32_t idesc = ptx::make_idesc_bf16(128, W, 0, B_MN_MAJOR ? 1 : 0);
            bool ok = ptx::mbar_wait(&bars.w_full, 0, abort_flag);
            if (!ok) atomicExch(status, KS_TIMEOUT_WEIGHTS);
            const int rounds = (my_tiles + NSLOT - 1) / NSLOT;
            for (int t = 0; ok && t < rounds; ++t) {
                for (int l = 0; ok && l <= L; ++l) {
                    for (int s = 0; s < NSLOT; ++s) {
                        if (t * NSLOT + s >= my_tiles) break;
                        // a_ready completion that must precede this MMA: the epilogue of
                        // (t, l-1), or for l == 0 the last epilogue of the previous tile.
                        const int n = t * n_mat + l - 1;
                        if (l == 0 && !ptx::mbar_wait(&bars.x_full[s], t & 1, abort_flag)) ok = false;
                        if (ok && n >= 0 && !ptx::mbar_wait(&bars.a_ready[s], n & 1, abort_flag)) ok = false;
                        if (!ok) {
                            atomicExch(status, KS_TIMEOUT_MMA | (l << 4) | s);
                            break;
                        }
                        ptx::tc_fence_after_sync();
                        const uint32_t d_tmem = tmem_base + s * W;
                        const uint32_t w_addr = smem_base + S::WBUF + l * T::WGT_BYTES;
                        const uint32_t a_addr = (l == 0) ? smem_base + S::XBUF + s * T::ACT_BYTES
                                                         : smem_base + S::ABUF + (s * 2 + ((l - 1) & 1)) * T::ACT_BYTES;
#pragma unroll
                        for (int ks = 0; ks < T::KSTEPS; ++ks) {
                            const uint64_t bdesc = B_MN_MAJOR ? T::desc_mnmajor(w_addr, ks, T::WGT_ATOM_BYTES)
                                                              : T::desc_kmajor(w_addr, ks, T::WGT_ATOM_BYTES);
                            if (TMEM_A && l > 0) {
                                const uint32_t a_tmem = tmem_base + NSLOT * W + s * (W / 2) + ks * 8;
                                ptx::mma_ts(d_tmem, a_tmem, bdesc, idesc, ks > 0);
                            } else {
                                ptx::mma_ss(d_tmem, T::desc_kmajor(a_addr, ks, T::ACT_ATOM_BYTES), bdesc, idesc, ks > 0);
                            }
                        }
                        ptx::mma_commit(&bars.acc_full[s]);
                        if (l == 0) ptx::mma_commit(&bars.x_empty[s]);
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue groups
        const int g = (warp - 2) >> 2;   // slot owned by this group
        const int quad = warp & 3;       // TMEM lane quarter this warp may touch
        const int row = quad * 32 + lane; // tile row owned by this thread
        const bool leader = ((warp - 2) & 3) == 0 && lane == 0;
        const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
        const int s = g;
        bool ok = true;
        for (int t = 0; ok && t * NSLOT + s < my_tiles; ++t) {
            const int tile = blockIdx.x + (t * NSLOT + s) * gridDim.x;
            for (int l = 0; l <= L; ++l) {
                const int n = t * n_mat + l;
                // the verdict must be warp-uniform: the TMEM accesses below are .aligned
                if (!__all_sync(0xffffffffu, ptx::mbar_wait(&bars.acc_full[s], n & 1, abort_flag))) {
                    if (lane == 0) atomicExch(status, KS_TIMEOUT_EPILOGUE | (l << 4) | s);
                    ok = false;
                    break;
                }
                ptx::tc_fence_after_sync();
                const int a = (l == L) ? out_act : act;
                const bool to_tmem = TMEM_A && l < L;
                uint8_t *abuf = smem + S::ABUF + (s * 2 + (l & 1)) * T::ACT_BYTES;
                if (!to_tmem && (STORE_ALL || TMEM_A || l == 0)) {
                    // the buffer about to be overwritten may still be read by an earlier TMA store
                    if (leader) {
                        if (STORE_ALL && l > 0)
                            ptx::tma_wait_group_read<1>();
                        else
                            ptx::tma_wait_group_read<0>();
                    }
                    ptx::named_bar_sync(1 + g, 128);
                }
                constexpr int CW = (W >= 32) ? 32 : 16; // columns per TMEM load
#pragma unroll
                for (int c0 = 0; c0 < W; c0 += CW) {
                    uint32_t v[CW];
                    if constexpr (CW == 32)
                        ptx::tmem_ld32(tmem_base + lane_addr + s * W + c0, v);
                    else
                        ptx::tmem_ld16(tmem_base + lane_addr + s * W + c0, v);
                    ptx::tmem_ld_wait();
                    uint32_t p[CW / 2];
#pragma unroll
                    for (int i = 0; i < CW / 2; ++i)
                        p[i] = act_pack(a, __uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
                    if (to_tmem) {
                        if constexpr (CW == 32) {
                            ptx::tmem_st16(tmem_base + lane_addr + NSLOT * W + s * (W / 2) + c0 / 2, p);
                        }
                    } else {
#pragma unroll
                        for (int ch = 0; ch < CW / 8; ++ch) {
                            const int c = c0 + ch * 8;
                            uint8_t *dst = abuf + (c / T::ATOM_COLS) * T::ACT_ATOM_BYTES +
                                           T::chunk_off(row, (c % T::ATOM_COLS) / 8);
                            *reinterpret_cast<uint4 *>(dst) =
                                make_uint4(p[ch * 4], p[ch * 4 + 1], p[ch * 4 + 2], p[ch * 4 + 3]);
                        }
                    }
                }
                if (to_tmem)
                    ptx::tmem_st_wait();
                else
                    ptx::fence_proxy_async_smem();
                ptx::tc_fence_before_sync();
                ptx::mbar_arrive(&bars.a_ready[s]);
                if (!to_tmem && (STORE_ALL || l == L)) {
                    ptx::named_bar_sync(1 + g, 128);
                    if (leader) {
                        for (int at = 0; at < T::KATOMS; ++at) {
                            if (STORE_ALL)
                                ptx::tma_store_3d(&tm_interm, abuf + at * T::ACT_ATOM_BYTES, at * T::ATOM_COLS,
                                                  tile * T::TM, l + 1);
                            if (l == L && write_y)
                                ptx::tma_store_2d(&tm_y, abuf + at * T::ACT_ATOM_BYTES, at * T::ATOM_COLS,
                                                  tile * T::TM);
                        }
                        ptx::tma_commit_group();
                    }
                }
            }
        }
        if (leader) ptx::tma_wait_group<0>();
    }

    // ---------------------------------------------------------------- teardown
    if (*abort_flag && threadIdx.x == 0) {
        // give bulk copies that are still in flight time to land before shared memory goes away
        for (int i = 0; i < 2000; ++i) __nanosleep(100);
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, S::tmem_cols);
    }
}

// ---------------------------------------------------------------------- host side
template <int W, int NSLOT, bool STORE_ALL, bool TMEM_A, bool B_MN>
static cudaError_t launch_variant(const FwdLaunch &p) {
    using T = Tile<W>;
    using S = FwdSmem<W, NSLOT, TMEM_A>;
    const size_t smem = (size_t)S::WBUF + (size_t)p.n_mat * T::WGT_BYTES + 1024;
    if (smem > 227 * 1024) return cudaErrorInvalidConfiguration;
    auto kern = mlp_fwd_kernel<W, NSLOT, STORE_ALL, TMEM_A, B_MN>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    const int n_tiles = (int)((p.batch + T::TM - 1) / T::TM);
    const int grid = n_tiles < p.n_sm ? n_tiles : p.n_sm;
    if (grid == 0) return cudaSuccess;
    kern<<<grid, 64 + 128 * NSLOT, smem, p.stream>>>(p.tm_x, p.tm_y, p.tm_interm,
                                                    B_MN ? p.wimg : p.wimg_t, n_tiles, p.n_mat, p.act, p.out_act,
                                                    p.write_y, p.status);
    return cudaGetLastError();
}

template <int W> static cudaError_t launch_w(const FwdLaunch &p) {
    // variant bits: 1 = keep hidden activations in TMEM (inference only), 2 = MN-major weights
    if (p.store_all) {
        return (p.variant & 2) ? launch_variant<W, 2, true, false, true>(p) : launch_variant<W, 2, true, false, false>(p);
    }
    if constexpr (W >= 32) {
        if (p.variant & 1)
            return (p.variant & 2) ? launch_variant<W, 2, false, true, true>(p)
                                   : launch_variant<W, 2, false, true, false>(p);
    }
    return (p.variant & 2) ? launch_variant<W, 2, false, false, true>(p) : launch_variant<W, 2, false, false, false>(p);
}

cudaError_t launch_mlp_fwd(const FwdLaunch &p) {
    switch (p.width) {
    case 16: return launch_w<16>(p);
    case 32: return launch_w<32>(p);
    case 64: return launch_w<64>(p);
    case 128: return launch_w<128>(p);
    default: return cudaErrorInvalidValue;
    }
}

} // namespace tnn
