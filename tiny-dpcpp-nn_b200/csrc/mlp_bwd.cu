// Fully fused MLP backward for sm_100a: delta chain, activation backward and the weight-gradient
// batch reduction in one kernel.
//
// Replaces EsimdKernels::backward_impl of the reference (include/network/kernel_esimd.h:160-240),
// i.e. the chain kernel *and* the oneMKL gemm_batch that follows it:
//     delta_L   = dL/dy (.) act_out'(y)
//     delta_l-1 = (delta_l W_l^T) (.) act'(a_l)          l = L..1, rounded to bf16 per layer
//     dL/dx     = delta_0 W_0^T                          (optional)
//     G_l       = delta_l^T a_l    (out x in)            l = 0..L, summed over the batch
//
// One persistent CTA per SM walks over 128-row batch tiles.  Per tile the forward activations
// a_l arrive by TMA; delta tiles live in shared memory only.  Each delta tile is used twice by the
// tensor cores without being moved: as the K-major A operand of the chain GEMM (M = batch rows) and
// as the MN-major A operand of the weight-gradient GEMM (M = features, K = batch rows).  The
// weight gradients of all layers accumulate in TMEM across all tiles of the CTA and are written
// once, as one fp32 slab per CTA; a small second kernel adds the slabs in a fixed order.
//
// TMEM holds the chain accumulator plus one accumulator per layer, 512 columns in all.  Networks with more
// layers than fit (width 128: three, width 64: seven) run the kernel in several passes; every pass repeats the
// chain and reduces the weight gradients of its own group of layers [dw_lo, dw_hi).  With BIG (width 128, or
// weights that do not fit beside the tiles) the weights are not resident: the issuer streams W_l through a ring
// of two tiles, fetching the next one when it issues a chain GEMM, and fewer tiles are kept in flight.
#include "mlp_common.cuh"
#include "elementwise.h"
#include "mlp_launch.h"

namespace tnn {

constexpr int kBwdMaxRing = 3;
constexpr int kBwdEpiWarps = 8;                      // epilogue: two threads per tile row
constexpr int kBwdEpiThreads = 32 * kBwdEpiWarps;
constexpr int kBwdThreads = 64 + kBwdEpiThreads;     // producer warp, issuer warp, epilogue warps

template <int W, bool BIG> struct BwdSmem {
    using T = Tile<W>;
    static constexpr int NDY = BIG ? 1 : 2;              // dL/dy tiles (this and the next tile)
    static constexpr int RING = BIG ? 2 : 3;             // forward-activation tiles in flight
    static constexpr int DY = 0;
    static constexpr int DP = DY + NDY * T::ACT_BYTES;   // 2 tiles: delta ping-pong (directly behind DY)
    static constexpr int AR = DP + 2 * T::ACT_BYTES;     // RING forward-activation tiles
    static constexpr int WBUF = AR + RING * T::ACT_BYTES;
    static constexpr int DW_M = (W == 128) ? 128 : 64;   // UMMA M of the weight-gradient GEMM
    __host__ __device__ static constexpr int weight_tiles(int n_mat) { return BIG ? 2 : n_mat; }
};

struct BwdBarriers {
    uint64_t w_full;
    uint64_t dy_full[2];
    uint64_t dy_empty[2];
    uint64_t a_full[kBwdMaxRing];
    uint64_t a_empty[kBwdMaxRing];
    uint64_t wring_full[2]; // BIG: weight ring stages
    uint64_t d_ready;  // epilogue -> MMA: next delta tile is in shared memory / accumulator was read
    uint64_t acc_full; // MMA -> epilogue: chain accumulator complete
    uint64_t all_done; // MMA -> epilogue: every weight-gradient MMA of this CTA has completed
    uint32_t tmem_base;
    uint32_t abort_flag;
};

template <int W, bool B_MN_MAJOR, bool BIG, bool HF_>
__global__ void __launch_bounds__(kBwdThreads, 1)
mlp_bwd_kernel(const __grid_constant__ CUtensorMap tm_dy, const __grid_constant__ CUtensorMap tm_interm,
               const __grid_constant__ CUtensorMap tm_a0, const __grid_constant__ CUtensorMap tm_ibwd,
               const __grid_constant__ CUtensorMap tm_dx,
               const __nv_bfloat16 *__restrict__ wimg, float *__restrict__ dw_slabs, int n_tiles, int n_mat, int act,
               int out_act, int store_bwd, int want_dx, int tmem_cols, int dw_lo, int dw_hi, int l_stop, int *status) {
    using T = Tile<W>;
    using S = BwdSmem<W, BIG>;
    constexpr int fp16 = HF_ ? 1 : 0; // element type of operands and activations: bf16 or fp16
    constexpr int kBwdRing = S::RING;
    constexpr int NDY = S::NDY;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ BwdBarriers bars;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int L = n_mat - 1;
    const uint32_t smem_base = ptx::smem_u32(smem);
    volatile uint32_t *abort_flag = &bars.abort_flag;
    const bool has_oact = out_act != ACT_NONE;
    // A pass walks the chain from layer L down to l_stop only: 0 in the pass that stores deltas / dL/dx, the first
    // layer of its weight-gradient group in the others (delta_l below that is of no use to it).
    const int loads_per_tile = (L - l_stop + 1) + (has_oact ? 1 : 0); // a_L..a_{l_stop} (+ y for the output activation)
    const int my_tiles = (n_tiles > (int)blockIdx.x) ? (n_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

    if (threadIdx.x == 0) {
        ptx::mbar_init(&bars.w_full, 1);
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(&bars.dy_full[b], 1);
            ptx::mbar_init(&bars.dy_empty[b], 2); // MMA commit + epilogue leader
            ptx::mbar_init(&bars.wring_full[b], 1);
        }
        for (int r = 0; r < kBwdRing; ++r) {
            ptx::mbar_init(&bars.a_full[r], 1);
            ptx::mbar_init(&bars.a_empty[r], kBwdEpiWarps + 1); // epilogue warps + MMA commit
        }
        ptx::mbar_init(&bars.d_ready, kBwdEpiWarps);
        ptx::mbar_init(&bars.acc_full, 1);
        ptx::mbar_init(&bars.all_done, 1);
        bars.abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::prefetch_tmap(&tm_dy);
        ptx::prefetch_tmap(&tm_interm);
        ptx::prefetch_tmap(&tm_a0);
    }
    if (warp == 1) {
        ptx::tmem_alloc(&bars.tmem_base, (uint32_t)tmem_cols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = bars.tmem_base;
    // TMEM columns: [0, W) chain accumulator, then one W-column weight-gradient accumulator per layer
    const uint32_t acc_tmem = tmem_base;
    auto dw_tmem = [&](int l) { return tmem_base + (uint32_t)(W + (l - dw_lo) * W); }; // dw_lo <= l < dw_hi

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        if (lane == 0 && my_tiles > 0) {
            if constexpr (!BIG) {
                ptx::mbar_arrive_expect_tx(&bars.w_full, (uint32_t)(n_mat * T::WGT_BYTES));
                for (int l = 0; l < n_mat; ++l)
                    ptx::bulk_load(smem + S::WBUF + l * T::WGT_BYTES,
                                   reinterpret_cast<const uint8_t *>(wimg) + (size_t)l * T::WGT_BYTES, T::WGT_BYTES,
                                   &bars.w_full);
            }
            int r = 0; // running index of forward-activation loads
            bool ok = true;
            for (int t = 0; ok && t < my_tiles; ++t) {
                const int tile = blockIdx.x + t * gridDim.x;
                const int b = t % NDY;
                if (t >= NDY && !ptx::mbar_wait(&bars.dy_empty[b], ((t / NDY) - 1) & 1, abort_flag)) {
                    atomicExch(status, KS_TIMEOUT_PRODUCER | 1);
                    break;
                }
                ptx::mbar_arrive_expect_tx(&bars.dy_full[b], T::ACT_BYTES);
                for (int at = 0; at < T::KATOMS; ++at)
                    ptx::tma_load_2d(smem + S::DY + b * T::ACT_BYTES + at * T::ACT_ATOM_BYTES, &tm_dy, at * T::ATOM_COLS,
                                     tile * T::TM, &bars.dy_full[b]);
                for (int j = 0; j < loads_per_tile; ++j, ++r) {
                    // order of use: (y = a_{L+1} if the output activation needs it), a_L, ..., a_0
                    const int mat = has_oact ? (L + 1 - j) : (L - j);
                    const int slot = r % kBwdRing;
                    if (r >= kBwdRing && !ptx::mbar_wait(&bars.a_empty[slot], ((r / kBwdRing) - 1) & 1, abort_flag)) {
                        atomicExch(status, KS_TIMEOUT_PRODUCER | 2);
                        ok = false;
                        break;
                    }
                    ptx::mbar_arrive_expect_tx(&bars.a_full[slot], T::ACT_BYTES);
                    for (int at = 0; at < T::KATOMS; ++at) {
                        uint8_t *dst = smem + S::AR + slot * T::ACT_BYTES + at * T::ACT_ATOM_BYTES;
                        if (mat == 0) // the network input may live outside the activation workspace
                            ptx::tma_load_2d(dst, &tm_a0, at * T::ATOM_COLS, tile * T::TM, &bars.a_full[slot]);
                        else
                            ptx::tma_load_3d(dst, &tm_interm, at * T::ATOM_COLS, tile * T::TM, mat, &bars.a_full[slot]);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (my_tiles > 0) { // all lanes run the loop, one elected lane issues (see ptx::elect_one)
            const uint32_t idesc_chain = ptx::make_idesc_16(128, W, 0, B_MN_MAJOR ? 1 : 0, fp16);
            const uint32_t idesc_dw = ptx::make_idesc_16(S::DW_M, W, 1, 1, fp16);
            // base descriptors; buffers and k-steps are reached with constant adds
            const uint64_t dk_desc0 = T::kdesc_base(smem_base + S::DY);                        // delta tiles, K-major
            const uint64_t dmn_desc0 = T::mndesc_base(smem_base + S::DY, T::ACT_ATOM_BYTES);   // delta tiles, MN-major
            const uint64_t amn_desc0 = T::mndesc_base(smem_base + S::AR, T::ACT_ATOM_BYTES);   // activations, MN-major
            const uint64_t w_desc0 = B_MN_MAJOR ? T::mndesc_base(smem_base + S::WBUF, T::WGT_ATOM_BYTES)
                                                : T::kdesc_base(smem_base + S::WBUF);
            // BIG: chain GEMM number g reads ring stage g & 1; its weights are fetched while GEMM g - 1 is issued
            const int last_chain = (l_stop == 0 && want_dx) ? 0 : l_stop + 1; // lowest layer with a chain GEMM
            [[maybe_unused]] uint32_t wg = 0;
            [[maybe_unused]] auto fetch_weights = [&](int l, uint32_t g) {
                uint64_t *bar = &bars.wring_full[g & 1u];
                ptx::mbar_arrive_expect_tx(bar, (uint32_t)T::WGT_BYTES);
                ptx::bulk_load(smem + S::WBUF + (g & 1u) * T::WGT_BYTES,
                               reinterpret_cast<const uint8_t *>(wimg) + (size_t)l * T::WGT_BYTES, T::WGT_BYTES, bar);
            };
            bool ok = true;
            if constexpr (BIG) {
                if (L >= last_chain) {
                    if (ptx::elect_one()) fetch_weights(L, 0);
                    __syncwarp();
                }
            } else {
                ok = ptx::mbar_wait(&bars.w_full, 0, abort_flag);
            }
            if (!ok && lane == 0) atomicExch(status, KS_TIMEOUT_WEIGHTS);
            int r = 0;  // forward-activation loads consumed
            int dr = 0; // d_ready completions consumed
            for (int t = 0; ok && t < my_tiles; ++t) {
                const int b = t % NDY;
                if (!ptx::mbar_wait(&bars.dy_full[b], (t / NDY) & 1, abort_flag)) ok = false;
                if (ok && has_oact) {
                    // the epilogue rewrites dL/dy in place with the output-activation derivative; y's
                    // ring slot is released by the epilogue threads plus this (empty) commit
                    if (!ptx::mbar_wait(&bars.d_ready, dr & 1, abort_flag)) ok = false;
                    ++dr;
                    if (ptx::elect_one()) ptx::mma_commit(&bars.a_empty[r % kBwdRing]);
                    __syncwarp();
                    ++r;
                }
                if (!ok) {
                    if (lane == 0) atomicExch(status, KS_TIMEOUT_MMA | 1);
                    break;
                }
                for (int l = L; ok && l >= l_stop; --l) {
                    // delta_l: dL/dy buffer for l == L, else ping-pong buffer (L - 1 - l) & 1
                    // (index into the four contiguous delta tiles DY[0], DY[1], DP[0], DP[1])
                    const int d_idx = (l == L) ? b : NDY + ((L - 1 - l) & 1);
                    if (l < L) {
                        if (!ptx::mbar_wait(&bars.d_ready, dr & 1, abort_flag)) {
                            if (lane == 0) atomicExch(status, KS_TIMEOUT_MMA | 2 | (l << 4));
                            ok = false;
                            break;
                        }
                        ++dr;
                    }
                    const bool chain = l > l_stop || (l_stop == 0 && want_dx);
                    uint64_t w_desc = w_desc0 + (uint64_t)(l * T::WGT_UNITS);
                    if constexpr (BIG) {
                        if (chain) {
                            // every earlier chain GEMM is complete (its accumulator was consumed): refill the other
                            // stage with the weights of the next chain GEMM of this CTA, if there is one
                            const int next_l = (l > last_chain) ? l - 1 : L;
                            if (l > last_chain || t + 1 < my_tiles) {
                                if (ptx::elect_one()) fetch_weights(next_l, wg + 1);
                                __syncwarp();
                            }
                            if (!ptx::mbar_wait(&bars.wring_full[wg & 1u], (wg >> 1) & 1u, abort_flag)) {
                                if (lane == 0) atomicExch(status, KS_TIMEOUT_WEIGHTS | 1);
                                ok = false;
                                break;
                            }
                            w_desc = w_desc0 + (uint64_t)((wg & 1u) * T::WGT_UNITS);
                            ++wg;
                        }
                    }
                    ptx::tc_fence_after_sync();
                    if (chain && ptx::elect_one()) {
                        // chain: acc[128 x W] = delta_l[128 x W] * W_l^T
                        T::template issue_chain<B_MN_MAJOR>(acc_tmem, dk_desc0 + (uint64_t)(d_idx * T::ACT_UNITS), w_desc,
                                                            idesc_chain);
                        ptx::mma_commit(&bars.acc_full);
                    }
                    __syncwarp();
                    // weight gradient: G_l[W x W] += delta_l^T[W x 128] * a_l[128 x W]
                    const int slot = r % kBwdRing;
                    if (!ptx::mbar_wait(&bars.a_full[slot], (r / kBwdRing) & 1, abort_flag)) {
                        if (lane == 0) atomicExch(status, KS_TIMEOUT_MMA | 3 | (l << 4));
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after_sync();
                    if (ptx::elect_one()) {
                        if (l >= dw_lo && l < dw_hi) // layers of other passes only release their buffers
                            T::issue_outer(dw_tmem(l), dmn_desc0 + (uint64_t)(d_idx * T::ACT_UNITS),
                                           amn_desc0 + (uint64_t)(slot * T::ACT_UNITS), idesc_dw, t > 0 ? 1u : 0u);
                        ptx::mma_commit(&bars.a_empty[slot]);
                        if (l == L) ptx::mma_commit(&bars.dy_empty[b]);
                    }
                    __syncwarp();
                    ++r;
                }
                if (ok && want_dx) {
                    // the accumulator holding dL/dx must be drained before the next tile reuses it
                    if (!ptx::mbar_wait(&bars.d_ready, dr & 1, abort_flag)) {
                        if (lane == 0) atomicExch(status, KS_TIMEOUT_MMA | 4);
                        ok = false;
                    }
                    ++dr;
                }
            }
            if (ptx::elect_one()) ptx::mma_commit(&bars.all_done);
            __syncwarp();
        }
    } else {
        // ------------------------------------------------------------ epilogue group: two threads per row
        const int quad = warp & 3;            // TMEM lane quarter this warp may touch
        const int half = (warp - 2) >> 2;     // which half of the columns this thread owns
        const int row = quad * 32 + lane;
        const bool leader = (warp == 2) && lane == 0;
        const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
        bool ok = true;
        int r = 0;  // forward-activation loads consumed
        int ac = 0; // acc_full completions consumed
        constexpr int CPT = W / 2;                 // columns per thread
        constexpr int CW = CPT < 32 ? CPT : 32;    // columns per TMEM load
        constexpr int NLD = CPT / CW;
        const int col0 = half * CPT;
        auto chunk_off = [&](int c) { // byte offset of the 16-byte chunk holding columns c..c+7 of this thread's row
            return (c / T::ATOM_COLS) * T::ACT_ATOM_BYTES + T::chunk_off(row, (c % T::ATOM_COLS) / 8);
        };
        auto load_cols = [&](uint32_t taddr, uint32_t (&v)[CW]) {
            if constexpr (CW == 32)
                ptx::tmem_ld32(taddr, v);
            else if constexpr (CW == 16)
                ptx::tmem_ld16(taddr, v);
            else
                ptx::tmem_ld8(taddr, v);
        };

        for (int t = 0; ok && t < my_tiles; ++t) {
            const int tile = blockIdx.x + t * gridDim.x;
            const int b = t % NDY;
            uint8_t *dybuf = smem + S::DY + b * T::ACT_BYTES;
            if (has_oact || store_bwd) {
                if (!__all_sync(0xffffffffu, ptx::mbar_wait(&bars.dy_full[b], (t / NDY) & 1, abort_flag))) {
                    if (lane == 0) atomicExch(status, KS_TIMEOUT_EPILOGUE | 1);
                    ok = false;
                    break;
                }
            }
            if (has_oact) {
                // delta_L = dL/dy (.) act_out'(y), in place
                const int slot = r % kBwdRing;
                if (!__all_sync(0xffffffffu, ptx::mbar_wait(&bars.a_full[slot], (r / kBwdRing) & 1, abort_flag))) {
                    if (lane == 0) atomicExch(status, KS_TIMEOUT_EPILOGUE | 2);
                    ok = false;
                    break;
                }
                const uint8_t *ybuf = smem + S::AR + slot * T::ACT_BYTES;
                dispatch_act_t<HF_>(out_act, [&](auto tag) {
                    constexpr int ACT = decltype(tag)::value;
                    constexpr bool HF = decltype(tag)::half;
#pragma unroll
                    for (int cc = 0; cc < CPT; cc += 8) {
                        const int off = chunk_off(col0 + cc);
                        uint4 d = *reinterpret_cast<const uint4 *>(dybuf + off);
                        const uint4 y = *reinterpret_cast<const uint4 *>(ybuf + off);
                        d.x = act_bwd_pack_t<ACT, HF>(ptx::lo_f32<HF>(d.x), ptx::hi_f32<HF>(d.x), y.x);
                        d.y = act_bwd_pack_t<ACT, HF>(ptx::lo_f32<HF>(d.y), ptx::hi_f32<HF>(d.y), y.y);
                        d.z = act_bwd_pack_t<ACT, HF>(ptx::lo_f32<HF>(d.z), ptx::hi_f32<HF>(d.z), y.z);
                        d.w = act_bwd_pack_t<ACT, HF>(ptx::lo_f32<HF>(d.w), ptx::hi_f32<HF>(d.w), y.w);
                        *reinterpret_cast<uint4 *>(dybuf + off) = d;
                    }
                });
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    ptx::mbar_arrive(&bars.d_ready);
                    ptx::mbar_arrive(&bars.a_empty[slot]);
                }
                ++r;
            }
            if (store_bwd) {
                ptx::named_bar_sync(1, kBwdEpiThreads);
                if (leader) {
                    for (int at = 0; at < T::KATOMS; ++at)
                        ptx::tma_store_3d(&tm_ibwd, dybuf + at * T::ACT_ATOM_BYTES, at * T::ATOM_COLS, tile * T::TM, L);
                    ptx::tma_commit_group();
                }
            }
            for (int l = L; l >= l_stop; --l) {
                const int slot = r % kBwdRing;
                const bool produce = (l > l_stop) || (l_stop == 0 && want_dx); // the accumulator becomes a bf16 tile
                // delta_{l-1} goes to ping-pong buffer (L - l) & 1; dL/dx (l == 0) uses the same rule
                uint8_t *dst = smem + S::DP + ((L - l) & 1) * T::ACT_BYTES;
                if (produce) {
                    if (!__all_sync(0xffffffffu, ptx::mbar_wait(&bars.acc_full, ac & 1, abort_flag))) {
                        if (lane == 0) atomicExch(status, KS_TIMEOUT_EPILOGUE | 3 | (l << 4));
                        ok = false;
                        break;
                    }
                    ++ac;
                    ptx::tc_fence_after_sync();
                }
                const bool need_a = (l > 0) && act != ACT_NONE;
                if (need_a && !__all_sync(0xffffffffu, ptx::mbar_wait(&bars.a_full[slot], (r / kBwdRing) & 1, abort_flag))) {
                    if (lane == 0) atomicExch(status, KS_TIMEOUT_EPILOGUE | 4 | (l << 4));
                    ok = false;
                    break;
                }
                if (produce) {
                    if (store_bwd || want_dx) {
                        // an earlier TMA store may still be reading the buffer that is written next
                        // (with per-layer stores the newest one reads the other ping-pong buffer)
                        if (leader) {
                            if (store_bwd)
                                ptx::tma_wait_group_read<1>();
                            else
                                ptx::tma_wait_group_read<0>();
                        }
                        ptx::named_bar_sync(1, kBwdEpiThreads);
                    }
                    const uint8_t *abuf = smem + S::AR + slot * T::ACT_BYTES;
                    uint32_t v[NLD][CW];
#pragma unroll
                    for (int i = 0; i < NLD; ++i) load_cols(acc_tmem + lane_addr + col0 + i * CW, v[i]);
                    ptx::tmem_ld_wait();
                    dispatch_act_t<HF_>((l > 0) ? act : (int)ACT_NONE, [&](auto tag) {
                        constexpr int ACT = decltype(tag)::value;
                    constexpr bool HF = decltype(tag)::half;
#pragma unroll
                        for (int i = 0; i < NLD; ++i) {
#pragma unroll
                            for (int ch = 0; ch < CW / 8; ++ch) {
                                const int off = chunk_off(col0 + i * CW + ch * 8);
                                uint4 f = make_uint4(0, 0, 0, 0);
                                if constexpr (ACT != ACT_NONE) f = *reinterpret_cast<const uint4 *>(abuf + off);
                                uint4 o;
                                o.x = act_bwd_pack_t<ACT, HF>(__uint_as_float(v[i][ch * 8 + 0]), __uint_as_float(v[i][ch * 8 + 1]), f.x);
                                o.y = act_bwd_pack_t<ACT, HF>(__uint_as_float(v[i][ch * 8 + 2]), __uint_as_float(v[i][ch * 8 + 3]), f.y);
                                o.z = act_bwd_pack_t<ACT, HF>(__uint_as_float(v[i][ch * 8 + 4]), __uint_as_float(v[i][ch * 8 + 5]), f.z);
                                o.w = act_bwd_pack_t<ACT, HF>(__uint_as_float(v[i][ch * 8 + 6]), __uint_as_float(v[i][ch * 8 + 7]), f.w);
                                *reinterpret_cast<uint4 *>(dst + off) = o;
                            }
                        }
                    });
                    ptx::fence_proxy_async_smem();
                    ptx::tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(&bars.d_ready);
                }
                __syncwarp(); // every lane has read its part of the activation tile
                if (lane == 0) ptx::mbar_arrive(&bars.a_empty[slot]);
                ++r;
                if (produce && (store_bwd || l == 0)) {
                    ptx::named_bar_sync(1, kBwdEpiThreads);
                    if (leader) {
                        for (int at = 0; at < T::KATOMS; ++at) {
                            if (l > 0) {
                                if (store_bwd)
                                    ptx::tma_store_3d(&tm_ibwd, dst + at * T::ACT_ATOM_BYTES, at * T::ATOM_COLS,
                                                      tile * T::TM, l - 1);
                            } else {
                                ptx::tma_store_2d(&tm_dx, dst + at * T::ACT_ATOM_BYTES, at * T::ATOM_COLS, tile * T::TM);
                            }
                        }
                        ptx::tma_commit_group();
                    }
                }
            }
            if (!ok) break;
            if (leader) {
                // dL/dy buffer b may be refilled once the store that read it (if any) is done
                if (store_bwd) ptx::tma_wait_group_read<0>();
                ptx::mbar_arrive(&bars.dy_empty[b]);
            }
        }
        if (leader) ptx::tma_wait_group<0>();

        // -------- drain the weight-gradient accumulators into this CTA's slab
        if (ok && my_tiles > 0) {
            if (!__all_sync(0xffffffffu, ptx::mbar_wait(&bars.all_done, 0, abort_flag))) {
                if (lane == 0) atomicExch(status, KS_TIMEOUT_EPILOGUE | 5);
                ok = false;
            }
        }
        if (ok && my_tiles > 0) {
            ptx::tc_fence_after_sync();
            float *slab = dw_slabs + (size_t)blockIdx.x * n_mat * W * W;
            for (int l = dw_lo; l < dw_hi; ++l) {
                // M = 64 accumulators keep row m in lane (m % 16) + 32 * (m / 16); M = 128 in lane m
                const int o = (S::DW_M == 64) ? quad * 16 + lane : quad * 32 + lane;
                const bool valid = (S::DW_M == 64) ? (lane < 16 && o < W) : true;
#pragma unroll
                for (int c0 = col0; c0 < col0 + CPT; c0 += CW) {
                    uint32_t v[CW];
                    load_cols(dw_tmem(l) + lane_addr + c0, v);
                    ptx::tmem_ld_wait();
                    if (valid) {
                        float4 *dstp = reinterpret_cast<float4 *>(slab + ((size_t)l * W + o) * W + c0);
#pragma unroll
                        for (int q4 = 0; q4 < CW / 4; ++q4)
                            dstp[q4] = make_float4(__uint_as_float(v[q4 * 4]), __uint_as_float(v[q4 * 4 + 1]),
                                                   __uint_as_float(v[q4 * 4 + 2]), __uint_as_float(v[q4 * 4 + 3]));
                    }
                }
            }
        }
    }

    if (*abort_flag && threadIdx.x == 0) {
        for (int i = 0; i < 2000; ++i) __nanosleep(100);
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, (uint32_t)tmem_cols);
    }
}

// ---------------------------------------------------------------------- host side
template <int W, bool B_MN, bool BIG, bool HF_> static cudaError_t launch_bwd_t(BwdLaunch &p) {
    using T = Tile<W>;
    using S = BwdSmem<W, BIG>;
    const size_t smem = (size_t)S::WBUF + (size_t)S::weight_tiles(p.n_mat) * T::WGT_BYTES + 1024;
    if (smem > 227 * 1024 - 512) return cudaErrorInvalidConfiguration;
    auto kern = mlp_bwd_kernel<W, B_MN, BIG, HF_>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    const int n_tiles = (int)((p.batch + T::TM - 1) / T::TM);
    const int grid = n_tiles < p.n_sm ? n_tiles : p.n_sm;
    p.grid_out = grid;
    if (grid == 0) return cudaSuccess;
    // weight-gradient accumulators that fit beside the chain accumulator: layers per pass
    const int per_pass = (512 - W) / W;
    for (int lo = 0; lo < p.n_mat; lo += per_pass) {
        const int hi = lo + per_pass < p.n_mat ? lo + per_pass : p.n_mat;
        const int cols_needed = W + (hi - lo) * W;
        int tmem_cols = 32;
        while (tmem_cols < cols_needed) tmem_cols *= 2;
        const int first = lo == 0; // deltas and dL/dx are the same in every pass: store them once
        // K-major weights for the chain are rows = input feature; the MN-major variant reads the transposed image
        count_launch();
        kern<<<grid, kBwdThreads, smem, p.stream>>>(p.tm_dy, p.tm_interm, p.tm_a0, p.tm_ibwd, p.tm_dx,
                                                    B_MN ? p.wimg_t : p.wimg,
                                            p.dw_partials, n_tiles, p.n_mat, p.act, p.out_act, first ? p.store_bwd : 0,
                                            first ? p.want_dx : 0, tmem_cols, lo, hi, first ? 0 : lo, p.status);
        e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

template <int W, bool B_MN, bool BIG> static cudaError_t launch_bwd_variant(BwdLaunch &p) {
    return p.fp16 ? launch_bwd_t<W, B_MN, BIG, true>(p) : launch_bwd_t<W, B_MN, BIG, false>(p);
}

template <int W> static cudaError_t launch_bwd_w(BwdLaunch &p) {
    // variant bit 256 (tests): stream the weights even if they would fit on chip
    cudaError_t e = (p.variant & 256) ? cudaErrorInvalidConfiguration : launch_bwd_variant<W, false, false>(p);
    if (e == cudaErrorInvalidConfiguration) e = launch_bwd_variant<W, false, true>(p); // streamed weights
    return e;
}

cudaError_t launch_mlp_bwd(BwdLaunch &p) {
    switch (p.width) {
    case 16: return launch_bwd_w<16>(p);
    case 32: return launch_bwd_w<32>(p);
    case 64: return launch_bwd_w<64>(p);
    case 128: return launch_bwd_w<128>(p);
    default: return cudaErrorInvalidValue;
    }
}

} // namespace tnn
