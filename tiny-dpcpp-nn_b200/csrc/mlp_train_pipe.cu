// Fused training pass, pipelined over two tiles: while the backward pass of tile t runs, the forward
// pass (and L2 loss) of tile t+1 runs on the same SM.  Same arithmetic as mlp_train.cu - forward
// (reference include/network/kernel_esimd.h:565-640), L2 loss (include/losses/l2.h:19-41), backward chain
// and weight-gradient reduction (kernel_esimd.h:160-240) with no activation ever leaving the SM.
//
// A tile's layer-to-layer chain is strictly serial (GEMM -> epilogue -> GEMM ...), so one tile alone
// leaves the tensor pipe idle most of the time.  Two tiles do not fit in shared memory side by side,
// but a forward pass *fills* its activation buffers in the order 1..L while the backward pass of the
// tile before it *releases* them in the order L..1.  Consecutive tiles therefore use the L+1 activation
// buffers in opposite directions and share them:
//     even tile: a_j -> buffer j-1            odd tile: a_j -> buffer L+1-j
// When the forward stage of tile t+1 reaches layer k it needs exactly the buffer the backward stage of
// tile t released one step earlier.  Per-buffer mbarriers make that hand-over exact.
//
// Roles (640 threads, one CTA per SM):
//   warp 0      TMA producer (weights once, input tiles double-buffered)
//   warp 1      issuer of the forward chain GEMMs       (accumulator F; owns TMEM)
//   warp 2      issuer of the backward chain GEMMs      (accumulator B)
//   warp 3      issuer of the weight-gradient GEMMs     (one accumulator per layer, kept across all tiles)
//   warps 4-11  forward-stage epilogue, two threads per row: activation, bf16, next A operand; L2 loss
//   warps 12-19 backward-stage epilogue, two threads per row: activation backward, next delta tile
#include "mlp_common.cuh"
#include "elementwise.h"
#include "mlp_launch.h"

namespace tnn {

constexpr int kPipeMaxMat = 12; // upper bound of the barrier array; what fits is decided by shared memory and TMEM columns

// TGT: how a tile's fp32 targets reach the loss step.  0: per-thread global loads.  1: full-width rows (128 x W fp32,
// twice the bytes of a bf16 tile) staged by TMA boxes.  2: narrow rows (n_targets < W: 128 * n_targets contiguous
// floats) staged by one plain bulk copy.  4: like 2 for a network with at most 8 live output columns (only the first
// 8-column chunk of a row is evaluated in the loss step).  3: no targets - the upstream gradient dL/dy is given.
// Staged targets go into the delta_L buffer plus one more tile right behind it; the loss step pulls its slice into
// registers before delta_L is written.
template <int W, int TGT> struct PipeSmem {
    using T = Tile<W>;
    // delta tiles first (see mlp_train.cu: the M = 64 weight-gradient GEMM over-reads past them for W < 64)
    static constexpr int DL = 0;                                  // delta_L: forward stage -> backward stage
    static constexpr int NB = (TGT == 1 || TGT == 2 || TGT == 4) ? 2 : 1; // tiles in front of the ping-pong buffers
    static constexpr int TGT_BOX_BYTES = 128 * 128;               // one box: 128 rows x 32 fp32
    static constexpr int TGT_BOXES = W / 32;
    __host__ __device__ static constexpr int DP(int p) { return (NB + p) * T::ACT_BYTES; } // delta ping-pong
    __host__ __device__ static constexpr int X(int b) { return (NB + 2 + b) * T::ACT_BYTES; }  // input tiles
    __host__ __device__ static constexpr int AB(int i) { return (NB + 4 + i) * T::ACT_BYTES; } // L + 1 shared activation buffers
    __host__ __device__ static constexpr int WBUF(int n_mat) { return (NB + 4 + n_mat) * T::ACT_BYTES; }
    static constexpr int GROUP_THREADS = 256; // one epilogue stage: two threads per tile row
    static constexpr int GROUP_WARPS = GROUP_THREADS / 32;
    static constexpr int THREADS = 128 + 2 * GROUP_THREADS;
    static constexpr int CPT = W / 2; // columns per epilogue thread
    // Narrow layers are pure latency chains - an MMA or two per step - and their tiles are small: two CTAs share an SM
    // where shared memory and tensor memory allow (the launcher decides), which doubles the chains in flight.
    static constexpr int CTAS_PER_SM = W <= 32 ? 2 : 1;
};

struct PipeBarriers {
    uint64_t w_full;
    uint64_t x_full[2], x_empty[2];
    uint64_t f_ready, accf_full;       // forward stage <-> its issuer
    uint64_t b_ready, accb_full;       // backward stage <-> its issuer
    uint64_t dl_ready, dl_free;        // delta_L hand-over between the stages
    uint64_t dwgo_f;                   // forward stage -> weight-gradient issuer (delta_L)
    uint64_t dwgo_b[2];                // backward stage -> weight-gradient issuer (alternating, see mlp_train.cu)
    uint64_t chain_issued[2];          // backward issuer -> weight-gradient issuer (alternating)
    uint64_t dp_free[2];               // weight-gradient GEMM that read delta ping-pong buffer p is complete
    uint64_t ab_free[kPipeMaxMat + 1]; // activation buffer i: mask read by the backward stage and weight-gradient GEMM done
    uint64_t all_done;
    uint64_t tgt_full;                 // targets of the current tile have landed
    uint64_t tgt_read;                 // every warp of the forward stage has pulled its targets into registers
    uint32_t tmem_base;
    uint32_t abort_flag;
    float loss_red[8];
};

// (The chain GEMMs read both operands from shared memory.  Feeding their A operand from tensor memory, as the
// inference kernel does, was measured slower here: the activations must be in shared memory anyway for the
// weight-gradient GEMMs and the activation backward, and the extra tcgen05.st in every epilogue step costs more
// than the shorter GEMMs save.)
// DX: the backward stage takes one more step per tile, dL/dinput = delta_0 W_0^T (kernel_esimd.h:213-228), and stores
// it through tm_dx: what a trainable encoding in front of the network needs.
template <int W, int TGT, bool HF_, int MINB, bool DX>
__global__ void __launch_bounds__(PipeSmem<W, TGT>::THREADS, MINB)
mlp_train_pipe_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_tgt,
                      const __grid_constant__ CUtensorMap tm_dx,
                      const __nv_bfloat16 *__restrict__ wimg,
                      const float *__restrict__ targets, int n_targets, float *__restrict__ dw_slabs,
                      float *__restrict__ loss_partials, size_t batch, int n_tiles, int n_mat, int act, int out_act,
                      float loss_scale, float inv_n, const EncodedInput enc, int tmem_cols, int *status) {
    using T = Tile<W>;
    using S = PipeSmem<W, TGT>;
    constexpr int fp16 = HF_ ? 1 : 0; // element type of operands and activations: bf16 or fp16
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ PipeBarriers bars;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int L = n_mat - 1;
    const uint32_t smem_base = ptx::smem_u32(smem);
    volatile uint32_t *abort_flag = &bars.abort_flag;
    const int my_tiles = (n_tiles > (int)blockIdx.x) ? (n_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const uint32_t kTmemCols = (uint32_t)tmem_cols; // power of two covering the accumulators of this network

    // activation buffer of a_j (j = 1..L) of this CTA's t-th tile
    auto ab_index = [L](int t, int j) { return (t & 1) ? L + 1 - j : j - 1; };
    // number of times buffer i was used by the tiles before tile t
    auto ab_prior_uses = [L](int t, int i) { return i == 0 ? (t + 1) / 2 : (i == L ? t / 2 : t); };

    if (threadIdx.x == 0) {
        ptx::mbar_init(&bars.w_full, 1);
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(&bars.x_full[b], 1);
            ptx::mbar_init(&bars.x_empty[b], 2);
            ptx::mbar_init(&bars.dwgo_b[b], S::GROUP_WARPS);
            ptx::mbar_init(&bars.chain_issued[b], 1);
            ptx::mbar_init(&bars.dp_free[b], 1);
        }
        ptx::mbar_init(&bars.f_ready, S::GROUP_WARPS);
        ptx::mbar_init(&bars.accf_full, 1);
        ptx::mbar_init(&bars.b_ready, S::GROUP_WARPS);
        ptx::mbar_init(&bars.accb_full, 1);
        ptx::mbar_init(&bars.dl_ready, S::GROUP_WARPS);
        ptx::mbar_init(&bars.dl_free, 2); // backward chain GEMM + weight-gradient GEMM of layer L
        ptx::mbar_init(&bars.dwgo_f, S::GROUP_WARPS);
        for (int i = 0; i <= kPipeMaxMat; ++i) ptx::mbar_init(&bars.ab_free[i], S::GROUP_WARPS + 1);
        ptx::mbar_init(&bars.all_done, 1);
        ptx::mbar_init(&bars.tgt_full, 1);
        ptx::mbar_init(&bars.tgt_read, S::GROUP_WARPS);
        bars.abort_flag = 0;
        ptx::fence_barrier_init();
        if (!enc.x) ptx::prefetch_tmap(&tm_x);
        if constexpr (TGT == 1 || TGT == 3) ptx::prefetch_tmap(&tm_tgt);
        if constexpr (DX) ptx::prefetch_tmap(&tm_dx);
    }
    if (warp == 1) {
        ptx::tmem_alloc(&bars.tmem_base, kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = bars.tmem_base;
    const uint32_t accf_tmem = tmem_base;     // columns [0, W)
    const uint32_t accb_tmem = tmem_base + W; // columns [W, 2W); weight gradients of layer l at 2W + l W

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        // Weights once; then per tile the input (TMA by lane 0, or - with a folded identity encoding - written by
        // the whole warp from the fp32 coordinates) and the staged targets (lane 0).
        if (lane == 0 && my_tiles > 0) {
            ptx::mbar_arrive_expect_tx(&bars.w_full, (uint32_t)(n_mat * T::WGT_BYTES));
            for (int l = 0; l < n_mat; ++l)
                ptx::bulk_load(smem + S::WBUF(n_mat) + l * T::WGT_BYTES,
                               reinterpret_cast<const uint8_t *>(wimg) + (size_t)l * T::WGT_BYTES, T::WGT_BYTES,
                               &bars.w_full);
        }
        // targets of tile t: the staging area overlaps delta_L, so both GEMMs that read delta_L of the previous tile
        // must be complete (wait), then one thread issues the copy
        auto targets_wait = [&](int t) -> bool {
            if constexpr (TGT != 0) {
                if (t > 0 && !ptx::mbar_wait(&bars.dl_free, (t - 1) & 1, abort_flag)) return false;
            }
            return true;
        };
        auto targets_issue = [&](int tile) {
            if constexpr (TGT == 2 || TGT == 4) {
                const size_t row0 = (size_t)tile * T::TM;
                const uint32_t rows = (uint32_t)(batch - row0 < (size_t)T::TM ? batch - row0 : (size_t)T::TM);
                const uint32_t bytes = rows * (uint32_t)n_targets * 4u; // rows % 8 == 0: a multiple of 16
                ptx::mbar_arrive_expect_tx(&bars.tgt_full, bytes);
                ptx::bulk_load(smem + S::DL, targets + row0 * n_targets, bytes, &bars.tgt_full);
            } else if constexpr (TGT == 1) {
                ptx::mbar_arrive_expect_tx(&bars.tgt_full, (uint32_t)(S::TGT_BOXES * S::TGT_BOX_BYTES));
                for (int bx = 0; bx < S::TGT_BOXES; ++bx)
                    ptx::tma_load_2d(smem + S::DL + bx * S::TGT_BOX_BYTES, &tm_tgt, bx * 32, tile * T::TM, &bars.tgt_full);
            } else if constexpr (TGT == 3) {
                // the upstream gradient dL/dy of the tile lands where delta_L lives, already in operand layout
                ptx::mbar_arrive_expect_tx(&bars.tgt_full, T::ACT_BYTES);
                for (int at = 0; at < T::KATOMS; ++at)
                    ptx::tma_load_2d(smem + S::DL + at * T::ACT_ATOM_BYTES, &tm_tgt, at * T::ATOM_COLS, tile * T::TM,
                                     &bars.tgt_full);
            }
        };
        if (!enc.x) {
            if (lane == 0) {
                for (int t = 0; t < my_tiles; ++t) {
                    const int tile = blockIdx.x + t * gridDim.x;
                    const int b = t & 1;
                    if (t >= 2 && !ptx::mbar_wait(&bars.x_empty[b], ((t >> 1) - 1) & 1, abort_flag)) {
                        atomicExch(status, KS_TIMEOUT_PRODUCER | 1);
                        break;
                    }
                    ptx::mbar_arrive_expect_tx(&bars.x_full[b], T::ACT_BYTES);
                    for (int at = 0; at < T::KATOMS; ++at)
                        ptx::tma_load_2d(smem + S::X(b) + at * T::ACT_ATOM_BYTES, &tm_x, at * T::ATOM_COLS, tile * T::TM,
                                         &bars.x_full[b]);
                    if (!targets_wait(t)) {
                        atomicExch(status, KS_TIMEOUT_PRODUCER | 2);
                        break;
                    }
                    targets_issue(tile);
                }
            }
        } else if (my_tiles > 0) {
            // (every wait below is executed by the whole, converged warp: the hardware then suspends the warp until
            // the barrier flips.  A single polling lane with the others parked at a vote keeps the warp spinning and
            // takes issue slots from the epilogue warps of the same scheduler.)
            fill_tiles_with_ones<W>(smem + S::X(0), 2, lane, fp16);
            __syncwarp();
            IdentityTileEncoder<W> encoder(enc, batch, lane, fp16);
            encoder.fetch((size_t)blockIdx.x * T::TM);
            for (int t = 0; t < my_tiles; ++t) {
                const int tile = blockIdx.x + t * gridDim.x;
                const int b = t & 1;
                if (t >= 2 && !__all_sync(0xffffffffu, ptx::mbar_wait(&bars.x_empty[b], ((t >> 1) - 1) & 1, abort_flag))) {
                    if (lane == 0) atomicExch(status, KS_TIMEOUT_PRODUCER | 1);
                    break;
                }
                encoder.store(smem + S::X(b));
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&bars.x_full[b]);
                // coordinates of the next tile travel while this one is consumed
                if (t + 1 < my_tiles) encoder.fetch((size_t)(tile + gridDim.x) * T::TM);
                if (!__all_sync(0xffffffffu, targets_wait(t))) {
                    if (lane == 0) atomicExch(status, KS_TIMEOUT_PRODUCER | 2);
                    break;
                }
                if (lane == 0) targets_issue(tile);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ forward chain issuer
        if (my_tiles > 0) { // all lanes run the loop, one elected lane issues (see ptx::elect_one)
            const uint32_t idesc = ptx::make_idesc_16(128, W, 0, 1, fp16); // B = W_l read MN-major
            const uint64_t x_desc0 = T::kdesc_base(smem_base + S::X(0));
            const uint64_t ab_desc0 = T::kdesc_base(smem_base + S::AB(0));
            const uint64_t w_desc0 = T::mndesc_base(smem_base + S::WBUF(n_mat), T::WGT_ATOM_BYTES);
            bool ok = ptx::mbar_wait(&bars.w_full, 0, abort_flag);
            if (!ok && lane == 0) atomicExch(status, KS_TIMEOUT_WEIGHTS);
            uint32_t fr_parity = 0;
            for (int t = 0; ok && t < my_tiles; ++t) {
                const int b = t & 1;
                if (t > 0) { // the loss step of the previous tile has drained the accumulator
                    ok = ptx::mbar_wait(&bars.f_ready, fr_parity, abort_flag);
                    fr_parity ^= 1u;
                }
                if (ok) ok = ptx::mbar_wait(&bars.x_full[b], (t >> 1) & 1, abort_flag);
                if (!ok) {
                    if (lane == 0) atomicExch(status, KS_TIMEOUT_MMA | 1);
                    break;
                }
                ptx::tc_fence_after_sync();
                if (ptx::elect_one()) {
                    T::template issue_chain<true>(accf_tmem, x_desc0 + (uint64_t)(b * T::ACT_UNITS), w_desc0, idesc);
                    ptx::mma_commit(&bars.accf_full);
                    ptx::mma_commit(&bars.x_empty[b]);
                }
                __syncwarp();
                // (with dL/dy given and no output activation the output layer is not evaluated: delta_L is dL/dy)
                const int l_last = (TGT == 3 && out_act == ACT_NONE) ? L - 1 : L;
                for (int l = 1; l <= l_last; ++l) {
                    if (!ptx::mbar_wait(&bars.f_ready, fr_parity, abort_flag)) {
                        if (lane == 0) atomicExch(status, KS_TIMEOUT_MMA | 2 | (l << 4));
                        ok = false;
                        break;
                    }
                    fr_parity ^= 1u;
                    ptx::tc_fence_after_sync();
                    if (ptx::elect_one()) {
                        T::template issue_chain<true>(accf_tmem, ab_desc0 + (uint64_t)(ab_index(t, l) * T::ACT_UNITS),
                                                      w_desc0 + (uint64_t)(l * T::WGT_UNITS), idesc);
                        ptx::mma_commit(&bars.accf_full);
                    }
                    __syncwarp();
                }
            }
        }
    } else if (warp == 2) {
        // ------------------------------------------------------------ backward chain issuer
        if (my_tiles > 0) {
            const uint32_t idesc = ptx::make_idesc_16(128, W, 0, 0, fp16); // B = W_l read K-major
            const uint64_t dl_desc = T::kdesc_base(smem_base + S::DL);
            const uint64_t dp_desc0 = T::kdesc_base(smem_base + S::DP(0));
            const uint64_t w_desc0 = T::kdesc_base(smem_base + S::WBUF(n_mat));
            bool ok = ptx::mbar_wait(&bars.w_full, 0, abort_flag);
            uint32_t br_parity = 0, ci_count = 0;
            for (int t = 0; ok && t < my_tiles; ++t) {
                ok = ptx::mbar_wait(&bars.dl_ready, t & 1, abort_flag);
                if (ok && t > 0) { // delta_0 of the previous tile is out: accumulator B is drained
                    ok = ptx::mbar_wait(&bars.b_ready, br_parity, abort_flag);
                    br_parity ^= 1u;
                }
                if (!ok) {
                    if (lane == 0) atomicExch(status, KS_TIMEOUT_MMA | 3);
                    break;
                }
                for (int l = L; l >= 1; --l) {
                    if (l < L) {
                        if (!ptx::mbar_wait(&bars.b_ready, br_parity, abort_flag)) {
                            if (lane == 0) atomicExch(status, KS_TIMEOUT_MMA | 4 | (l << 4));
                            ok = false;
                            break;
                        }
                        br_parity ^= 1u;
                    }
                    ptx::tc_fence_after_sync();
                    const uint64_t d_desc = (l == L) ? dl_desc : dp_desc0 + (uint64_t)(((L - 1 - l) & 1) * T::ACT_UNITS);
                    if (ptx::elect_one()) {
                        T::template issue_chain<false>(accb_tmem, d_desc, w_desc0 + (uint64_t)(l * T::WGT_UNITS), idesc);
                        ptx::mma_commit(&bars.accb_full);
                        if (l == L) ptx::mma_commit(&bars.dl_free);
                        ptx::mbar_arrive(&bars.chain_issued[ci_count & 1u]); // the weight-gradient GEMM of layer l may follow
                    }
                    __syncwarp();
                    ++ci_count;
                }
                if constexpr (DX) { // dL/dinput = delta_0 W_0^T, once delta_0 is written
                    if (ok && !ptx::mbar_wait(&bars.b_ready, br_parity, abort_flag)) {
                        if (lane == 0) atomicExch(status, KS_TIMEOUT_MMA | 6);
                        ok = false;
                    }
                    br_parity ^= 1u;
                    if (!ok) break;
                    ptx::tc_fence_after_sync();
                    const uint64_t d_desc = dp_desc0 + (uint64_t)(((L - 1) & 1) * T::ACT_UNITS); // delta_0
                    if (ptx::elect_one()) {
                        T::template issue_chain<false>(accb_tmem, d_desc, w_desc0, idesc);
                        ptx::mma_commit(&bars.accb_full);
                    }
                    __syncwarp();
                }
            }
        }
    } else if (warp == 3) {
        // ------------------------------------------------------------ weight-gradient issuer
        if (my_tiles > 0) {
            constexpr int DW_M = (W == 128) ? 128 : 64;
            const uint32_t idesc = ptx::make_idesc_16(DW_M, W, 1, 1, fp16);
            const uint64_t x_desc0 = T::mndesc_base(smem_base + S::X(0), T::ACT_ATOM_BYTES);
            const uint64_t ab_desc0 = T::mndesc_base(smem_base + S::AB(0), T::ACT_ATOM_BYTES);
            const uint64_t dl_desc = T::mndesc_base(smem_base + S::DL, T::ACT_ATOM_BYTES);
            const uint64_t dp_desc0 = T::mndesc_base(smem_base + S::DP(0), T::ACT_ATOM_BYTES);
            uint32_t kb = 0; // backward-stage hand-overs consumed
            uint32_t kc = 0; // chain_issued signals consumed
            bool ok = true;
            for (int t = 0; ok && t < my_tiles; ++t) {
                const int b = t & 1;
                for (int l = L; l >= 0; --l) {
                    if (l == L) {
                        ok = ptx::mbar_wait(&bars.dwgo_f, t & 1, abort_flag);
                    } else {
                        ok = ptx::mbar_wait(&bars.dwgo_b[kb & 1u], (kb >> 1) & 1u, abort_flag);
                        ++kb;
                    }
                    if (ok && l >= 1) { // stay behind the chain GEMM that consumes the same delta tile
                        ok = ptx::mbar_wait(&bars.chain_issued[kc & 1u], (kc >> 1) & 1u, abort_flag);
                        ++kc;
                    }
                    if (!ok) {
                        if (lane == 0) atomicExch(status, KS_TIMEOUT_MMA | 5 | (l << 4));
                        break;
                    }
                    ptx::tc_fence_after_sync();
                    const int p = (L - 1 - l) & 1;
                    const uint64_t d_desc = (l == L) ? dl_desc : dp_desc0 + (uint64_t)(p * T::ACT_UNITS);
                    const int ai = (l >= 1) ? ab_index(t, l) : 0;
                    const uint64_t a_desc = (l >= 1) ? ab_desc0 + (uint64_t)(ai * T::ACT_UNITS)
                                                     : x_desc0 + (uint64_t)(b * T::ACT_UNITS);
                    if (ptx::elect_one()) {
                        T::issue_outer(tmem_base + (uint32_t)(2 * W + l * W), d_desc, a_desc, idesc, t > 0 ? 1u : 0u);
                        if (l == L)
                            ptx::mma_commit(&bars.dl_free);
                        else
                            ptx::mma_commit(&bars.dp_free[p]);
                        if (l >= 1)
                            ptx::mma_commit(&bars.ab_free[ai]);
                        else
                            ptx::mma_commit(&bars.x_empty[b]);
                    }
                    __syncwarp();
                }
            }
            if (ptx::elect_one()) ptx::mma_commit(&bars.all_done);
            __syncwarp();
        }
    } else if (warp < 4 + S::GROUP_WARPS) {
        // ------------------------------------------------------------ forward-stage epilogue
        const int gw = warp - 4;
        const int quad = warp & 3;
        const int half = gw >> 2;
        const int row = quad * 32 + lane;
        const int col0 = half * S::CPT;
        constexpr int CPT = S::CPT;
        const uint32_t acc_addr = accf_tmem + ((uint32_t)(quad * 32) << 16) + col0;
        uint32_t af_parity = 0;
        float loss_local = 0.0f;
        bool ok = true;
        auto chunk_at = [&](int ch) {
            const int c = col0 + ch * 8;
            return (c / T::ATOM_COLS) * T::ACT_ATOM_BYTES + T::chunk_off(row, (c % T::ATOM_COLS) / 8);
        };
        auto wait_u = [&](uint64_t *bar, uint32_t parity, int code) { // warp-uniform bounded wait
            const bool r = __all_sync(0xffffffffu, ptx::mbar_wait(bar, parity, abort_flag));
            if (!r && lane == 0) atomicExch(status, KS_TIMEOUT_EPILOGUE | code);
            return r;
        };
        auto load_acc = [&](uint32_t (&v)[CPT]) {
            if constexpr (CPT == 32)
                ptx::tmem_ld32(acc_addr, v);
            else if constexpr (CPT == 16)
                ptx::tmem_ld16(acc_addr, v);
            else
                ptx::tmem_ld8(acc_addr, v);
            ptx::tmem_ld_wait();
        };
        for (int t = 0; ok && t < my_tiles; ++t) {
            const int tile = blockIdx.x + t * gridDim.x;
            const size_t grow = (size_t)tile * T::TM + row;
            const bool row_valid = grow < batch;
            for (int l = 0; l < L && ok; ++l) {
                // Every wait is a shared-memory round trip that queues behind the operand traffic of running
                // GEMMs even when it passes, so the wait for the destination buffer comes first: its latency
                // then hides under the GEMM this step waits for anyway.
                const int bi = ab_index(t, l + 1);
                const int uses = ab_prior_uses(t, bi);
                if (uses > 0 && !wait_u(&bars.ab_free[bi], (uses - 1) & 1, 2 | (l << 4))) {
                    ok = false;
                    break;
                }
                if (!wait_u(&bars.accf_full, af_parity, 1 | (l << 4))) {
                    ok = false;
                    break;
                }
                af_parity ^= 1u;
                ptx::tc_fence_after_sync();
                uint32_t v[CPT];
                load_acc(v);
                uint8_t *dst = smem + S::AB(bi);
                dispatch_act_t<HF_>(act, [&](auto tag) {
                    constexpr int ACT = decltype(tag)::value;
                    constexpr bool HF = decltype(tag)::half;
                    uint32_t pk[CPT / 2];
#pragma unroll
                    for (int q = 0; q < CPT / 2; ++q)
                        pk[q] = act_pack_t<ACT, HF>(__uint_as_float(v[2 * q]), __uint_as_float(v[2 * q + 1]));
#pragma unroll
                    for (int ch = 0; ch < CPT / 8; ++ch)
                        *reinterpret_cast<uint4 *>(dst + chunk_at(ch)) =
                            make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]);
                });
                ptx::fence_proxy_async_smem();
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&bars.f_ready);
            }
            if (!ok) break;
            // ---- output layer + L2 loss.  The target slice is requested before the wait for the last GEMM.
            float tg[CPT];
            if constexpr (TGT == 3) {
                // dL/dy is given: the staged tile IS delta_L (times act_out'(y), applied in place below); every thread
                // touches its own chunks only, so there is no hand-shake before the first write
                if (!wait_u(&bars.tgt_full, t & 1, 8)) {
                    ok = false;
                    break;
                }
            } else if constexpr (TGT != 0) {
                if (!wait_u(&bars.tgt_full, t & 1, 8)) {
                    ok = false;
                    break;
                }
                if constexpr (TGT == 2 || TGT == 4) {
                    // row-major rows of n_targets floats; columns past them (and rows past the batch) compare with 0
                    const float *src = reinterpret_cast<const float *>(smem + S::DL) + row * n_targets;
#pragma unroll
                    for (int q = 0; q < CPT; ++q) tg[q] = 0.0f;
                    constexpr int kTgtCols = (TGT == 4) ? 8 : CPT; // TGT == 4: targets in the first 8 columns only
                    if (col0 < n_targets && row_valid) {
#pragma unroll
                        for (int q = 0; q < kTgtCols; ++q)
                            if (col0 + q < n_targets) tg[q] = src[col0 + q];
                    }
                } else {
                    const uint8_t *src = smem + S::DL + (col0 / 32) * S::TGT_BOX_BYTES + row * 128;
#pragma unroll
                    for (int q4 = 0; q4 < CPT / 4; ++q4) {
                        const int chunk = (col0 % 32) / 4 + q4;
                        const float4 t4 = *reinterpret_cast<const float4 *>(src + ((chunk ^ (row & 7)) << 4));
                        tg[q4 * 4 + 0] = t4.x, tg[q4 * 4 + 1] = t4.y, tg[q4 * 4 + 2] = t4.z, tg[q4 * 4 + 3] = t4.w;
                    }
                }
                // every thread of the stage holds its targets before the first one overwrites the area with delta_L
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&bars.tgt_read);
                if (!wait_u(&bars.tgt_read, t & 1, 9)) {
                    ok = false;
                    break;
                }
            } else if (row_valid && n_targets == W && (reinterpret_cast<uintptr_t>(targets) & 15) == 0) {
#pragma unroll
                for (int q4 = 0; q4 < CPT / 4; ++q4) {
                    const float4 t4 = __ldg(reinterpret_cast<const float4 *>(targets + grow * W + col0) + q4);
                    tg[q4 * 4 + 0] = t4.x, tg[q4 * 4 + 1] = t4.y, tg[q4 * 4 + 2] = t4.z, tg[q4 * 4 + 3] = t4.w;
                }
            } else {
#pragma unroll
                for (int q = 0; q < CPT; ++q)
                    tg[q] = (row_valid && col0 + q < n_targets) ? __ldg(targets + grow * n_targets + col0 + q) : 0.0f;
            }
            uint32_t v[CPT];
            if (!(TGT == 3 && out_act == ACT_NONE)) { // (else: no output-layer GEMM was issued, see the issuer)
                if (!wait_u(&bars.accf_full, af_parity, 3)) {
                    ok = false;
                    break;
                }
                af_parity ^= 1u;
                ptx::tc_fence_after_sync();
                if constexpr (TGT == 4) { // only the first 8 columns of a row are looked at (see below)
                    if (col0 == 0) {
                        uint32_t v8[8];
                        ptx::tmem_ld8(acc_addr, v8);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int k = 0; k < 8; ++k) v[k] = v8[k];
                    }
                } else {
                    load_acc(v);
                }
                // the accumulator is in registers: layer 0 of the next tile may run under the loss arithmetic
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&bars.f_ready);
            }
            if constexpr (TGT == 0) { // delta_L of the previous tile must have been consumed by its two GEMMs
                if (t > 0 && !wait_u(&bars.dl_free, (t - 1) & 1, 4)) {
                    ok = false;
                    break;
                }
            }
            uint8_t *dst = smem + S::DL;
            if constexpr (TGT == 3) {
                // delta_L = dL/dy (.) act_out'(y), in place (rows past the batch were zero-filled by the copy)
                if (out_act != ACT_NONE) {
                    dispatch_act_t<HF_>(out_act, [&](auto tag) {
                        constexpr int ACT = decltype(tag)::value;
                        constexpr bool HF = decltype(tag)::half;
#pragma unroll
                        for (int ch = 0; ch < CPT / 8; ++ch) {
                            uint4 *cell = reinterpret_cast<uint4 *>(dst + chunk_at(ch));
                            const uint4 d = *cell;
                            const uint32_t din[4] = {d.x, d.y, d.z, d.w};
                            uint32_t o[4];
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                const uint32_t y16 = act_pack_t<ACT, HF>(__uint_as_float(v[ch * 8 + 2 * q]),
                                                                         __uint_as_float(v[ch * 8 + 2 * q + 1]));
                                o[q] = act_bwd_pack_t<ACT, HF>(ptx::lo_f32<HF>(din[q]), ptx::hi_f32<HF>(din[q]), y16);
                            }
                            *cell = make_uint4(o[0], o[1], o[2], o[3]);
                        }
                    });
                }
            }
            // rows past the end of the batch contribute neither loss nor gradient
            const float gscale = row_valid ? loss_scale * 2.0f * inv_n : 0.0f;
            float sq = 0.0f;
            if constexpr (TGT != 3)
            dispatch_act_t<HF_>(out_act, [&](auto tag) {
                constexpr int ACT = decltype(tag)::value;
                    constexpr bool HF = decltype(tag)::half;
#pragma unroll
                for (int ch = 0; ch < CPT / 8; ++ch) {
                    if constexpr (TGT == 4) {
                        // At most 8 live output columns (the 3 of an RGB regression): the others hold act_out(0) = 0
                        // under zero weight columns and have no target, so their loss and gradient are exactly zero
                        // and only the first chunk of a row is evaluated.  (Decided at compile time: the same test
                        // as a run-time branch cost more than the arithmetic it saves, this kernel sits at its
                        // register limit.)
                        if (ch > 0 || col0 != 0) {
                            *reinterpret_cast<uint4 *>(dst + chunk_at(ch)) = make_uint4(0u, 0u, 0u, 0u);
                            continue;
                        }
                    }
                    uint32_t o[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        // the prediction as the network stores it (bf16), then the loss on that value
                        const uint32_t y16 = act_pack_t<ACT, HF>(__uint_as_float(v[ch * 8 + 2 * q]),
                                                              __uint_as_float(v[ch * 8 + 2 * q + 1]));
                        const float d0 = ptx::lo_f32<HF>(y16) - tg[ch * 8 + 2 * q];
                        const float d1 = ptx::hi_f32<HF>(y16) - tg[ch * 8 + 2 * q + 1];
                        sq = fmaf(d0, d0, sq);
                        sq = fmaf(d1, d1, sq);
                        const uint32_t g16 = ptx::pack2<HF>(d0 * gscale, d1 * gscale);
                        o[q] = (ACT == ACT_NONE)
                                   ? g16
                                   : act_bwd_pack_t<ACT, HF>(ptx::lo_f32<HF>(g16), ptx::hi_f32<HF>(g16), y16);
                    }
                    *reinterpret_cast<uint4 *>(dst + chunk_at(ch)) = make_uint4(o[0], o[1], o[2], o[3]);
                }
            });
            if (row_valid) loss_local = fmaf(sq, inv_n, loss_local);
            ptx::fence_proxy_async_smem();
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                ptx::mbar_arrive(&bars.dl_ready); // backward chain may start
                ptx::mbar_arrive(&bars.dwgo_f);   // weight gradient of the output layer may start
            }
        }
        // loss partial of this CTA (fixed summation order)
        for (int o = 16; o > 0; o >>= 1) loss_local += __shfl_xor_sync(0xffffffffu, loss_local, o);
        if (lane == 0) bars.loss_red[gw] = loss_local;
        ptx::named_bar_sync(1, S::GROUP_THREADS);
        if (gw == 0 && lane == 0 && loss_partials) {
            float s = 0.0f;
            for (int i = 0; i < S::GROUP_WARPS; ++i) s += bars.loss_red[i];
            loss_partials[blockIdx.x] = s;
        }
    } else {
        // ------------------------------------------------------------ backward-stage epilogue
        const int gw = warp - (4 + S::GROUP_WARPS);
        const int quad = warp & 3;
        const int half = gw >> 2;
        const int row = quad * 32 + lane;
        const int col0 = half * S::CPT;
        constexpr int CPT = S::CPT;
        const uint32_t acc_addr = accb_tmem + ((uint32_t)(quad * 32) << 16) + col0;
        uint32_t ab_parity = 0;
        uint32_t dp_parity = 0, dp_written = 0; // bit p: phase to wait for / buffer p was written before
        uint32_t go_count = 0;
        [[maybe_unused]] bool dx_store_pending = false;
        bool ok = true;
        auto chunk_at = [&](int ch) {
            const int c = col0 + ch * 8;
            return (c / T::ATOM_COLS) * T::ACT_ATOM_BYTES + T::chunk_off(row, (c % T::ATOM_COLS) / 8);
        };
        auto wait_u = [&](uint64_t *bar, uint32_t parity, int code) {
            const bool r = __all_sync(0xffffffffu, ptx::mbar_wait(bar, parity, abort_flag));
            if (!r && lane == 0) atomicExch(status, KS_TIMEOUT_EPILOGUE | code);
            return r;
        };
        for (int t = 0; ok && t < my_tiles; ++t) {
            // the forward stage has finished this tile: its stored activations may be fetched ahead of the GEMMs
            if (!wait_u(&bars.dl_ready, t & 1, 10)) {
                ok = false;
                break;
            }
            for (int l = L; l >= 1 && ok; --l) {
                // The destination buffer and the stored forward activations are ready long before the GEMM of
                // this step completes: wait for the former and fetch the latter first, so that both
                // shared-memory round trips hide under the GEMM (see the forward stage).
                const int p = (L - l) & 1; // delta_{l-1} goes to ping-pong buffer (L - l) & 1
                if constexpr (DX) { // the buffer may still be read by the store of the previous tile's dL/dinput
                    if (dx_store_pending && p == (L & 1)) {
                        if (threadIdx.x == S::THREADS - S::GROUP_THREADS) ptx::tma_wait_group_read<0>();
                        ptx::named_bar_sync(2, S::GROUP_THREADS);
                        dx_store_pending = false;
                    }
                }
                if ((dp_written >> p) & 1u) { // all but the first write wait for the GEMM that read the buffer
                    if (!wait_u(&bars.dp_free[p], (dp_parity >> p) & 1u, 6 | (l << 4))) {
                        ok = false;
                        break;
                    }
                    dp_parity ^= 1u << p;
                }
                dp_written |= 1u << p;
                const int ai = ab_index(t, l);
                const uint8_t *abuf = smem + S::AB(ai);
                uint8_t *dst = smem + S::DP(p);
                uint4 fa[CPT / 8];
#pragma unroll
                for (int ch = 0; ch < CPT / 8; ++ch)
                    fa[ch] = (act != ACT_NONE) ? *reinterpret_cast<const uint4 *>(abuf + chunk_at(ch)) : make_uint4(0, 0, 0, 0);
                if (!wait_u(&bars.accb_full, ab_parity, 5 | (l << 4))) {
                    ok = false;
                    break;
                }
                ab_parity ^= 1u;
                ptx::tc_fence_after_sync();
                uint32_t v[CPT];
                if constexpr (CPT == 32)
                    ptx::tmem_ld32(acc_addr, v);
                else if constexpr (CPT == 16)
                    ptx::tmem_ld16(acc_addr, v);
                else
                    ptx::tmem_ld8(acc_addr, v);
                ptx::tmem_ld_wait();
                dispatch_act_t<HF_>(act, [&](auto tag) {
                    constexpr int ACT = decltype(tag)::value;
                    constexpr bool HF = decltype(tag)::half;
                    uint32_t pk[CPT / 2];
#pragma unroll
                    for (int ch = 0; ch < CPT / 8; ++ch) {
                        const uint4 f = fa[ch];
                        pk[ch * 4 + 0] = act_bwd_pack_t<ACT, HF>(__uint_as_float(v[ch * 8 + 0]), __uint_as_float(v[ch * 8 + 1]), f.x);
                        pk[ch * 4 + 1] = act_bwd_pack_t<ACT, HF>(__uint_as_float(v[ch * 8 + 2]), __uint_as_float(v[ch * 8 + 3]), f.y);
                        pk[ch * 4 + 2] = act_bwd_pack_t<ACT, HF>(__uint_as_float(v[ch * 8 + 4]), __uint_as_float(v[ch * 8 + 5]), f.z);
                        pk[ch * 4 + 3] = act_bwd_pack_t<ACT, HF>(__uint_as_float(v[ch * 8 + 6]), __uint_as_float(v[ch * 8 + 7]), f.w);
                    }
#pragma unroll
                    for (int ch = 0; ch < CPT / 8; ++ch)
                        *reinterpret_cast<uint4 *>(dst + chunk_at(ch)) =
                            make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]);
                });
                ptx::fence_proxy_async_smem();
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    ptx::mbar_arrive(&bars.b_ready);
                    ptx::mbar_arrive(&bars.dwgo_b[go_count & 1u]);
                    ptx::mbar_arrive(&bars.ab_free[ai]); // this stage is done with a_l
                }
                ++go_count;
            }
            if constexpr (DX) {
                // ---- dL/dinput of this tile: delta_0 W_0^T, rounded to the network type, stored by TMA
                if (!ok) break;
                const int p = L & 1; // the buffer that held delta_1
                if (dx_store_pending) { // (a one-hidden-layer network writes this buffer here only)
                    if (threadIdx.x == S::THREADS - S::GROUP_THREADS) ptx::tma_wait_group_read<0>();
                    ptx::named_bar_sync(2, S::GROUP_THREADS);
                    dx_store_pending = false;
                }
                if ((dp_written >> p) & 1u) {
                    if (!wait_u(&bars.dp_free[p], (dp_parity >> p) & 1u, 11)) {
                        ok = false;
                        break;
                    }
                    dp_parity ^= 1u << p;
                }
                dp_written &= ~(1u << p); // no weight-gradient GEMM reads this tile: its reuse waits for the store instead
                if (!wait_u(&bars.accb_full, ab_parity, 12)) {
                    ok = false;
                    break;
                }
                ab_parity ^= 1u;
                ptx::tc_fence_after_sync();
                uint32_t v[CPT];
                if constexpr (CPT == 32)
                    ptx::tmem_ld32(acc_addr, v);
                else if constexpr (CPT == 16)
                    ptx::tmem_ld16(acc_addr, v);
                else
                    ptx::tmem_ld8(acc_addr, v);
                ptx::tmem_ld_wait();
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&bars.b_ready); // accumulator B is drained
                uint8_t *dst = smem + S::DP(p);
#pragma unroll
                for (int ch = 0; ch < CPT / 8; ++ch) {
                    uint32_t o[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        o[q] = ptx::pack2<HF_>(__uint_as_float(v[ch * 8 + 2 * q]), __uint_as_float(v[ch * 8 + 2 * q + 1]));
                    *reinterpret_cast<uint4 *>(dst + chunk_at(ch)) = make_uint4(o[0], o[1], o[2], o[3]);
                }
                ptx::fence_proxy_async_smem();
                ptx::named_bar_sync(2, S::GROUP_THREADS);
                if (threadIdx.x == S::THREADS - S::GROUP_THREADS) {
                    const int tile = blockIdx.x + t * gridDim.x;
                    for (int at = 0; at < T::KATOMS; ++at)
                        ptx::tma_store_2d(&tm_dx, dst + at * T::ACT_ATOM_BYTES, at * T::ATOM_COLS, tile * T::TM);
                    ptx::tma_commit_group();
                }
                dx_store_pending = true;
            }
        }
        if constexpr (DX) {
            if (threadIdx.x == S::THREADS - S::GROUP_THREADS) ptx::tma_wait_group<0>();
        }
        // ---- drain the weight-gradient accumulators into this CTA's slab
        if (ok && my_tiles > 0 && !wait_u(&bars.all_done, 0, 7)) ok = false;
        if (ok && my_tiles > 0) {
            ptx::tc_fence_after_sync();
            float *slab = dw_slabs + (size_t)blockIdx.x * n_mat * W * W;
            const int o = quad * 16 + lane; // M = 64 accumulators keep row m in lane (m % 16) + 32 * (m / 16)
            const bool valid = lane < 16 && o < W;
            for (int l = 0; l < n_mat; ++l) {
                uint32_t v[CPT];
                const uint32_t addr = tmem_base + ((uint32_t)(quad * 32) << 16) + 2 * W + l * W + col0;
                if constexpr (CPT == 32)
                    ptx::tmem_ld32(addr, v);
                else if constexpr (CPT == 16)
                    ptx::tmem_ld16(addr, v);
                else
                    ptx::tmem_ld8(addr, v);
                ptx::tmem_ld_wait();
                if (valid) {
                    float4 *dstp = reinterpret_cast<float4 *>(slab + ((size_t)l * W + o) * W + col0);
#pragma unroll
                    for (int q4 = 0; q4 < CPT / 4; ++q4)
                        dstp[q4] = make_float4(__uint_as_float(v[q4 * 4]), __uint_as_float(v[q4 * 4 + 1]),
                                               __uint_as_float(v[q4 * 4 + 2]), __uint_as_float(v[q4 * 4 + 3]));
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
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------- host side
// 227 KB per CTA minus the statically allocated barriers
constexpr size_t kPipeSmemLimit = 227 * 1024 - 2048;

template <int W, int TGT, bool HF_, int MINB, bool DX> static cudaError_t launch_pipe_d(TrainLaunch &p);
template <int W, int TGT, bool HF_, int MINB> static cudaError_t launch_pipe_b(TrainLaunch &p) {
    return p.want_dx ? launch_pipe_d<W, TGT, HF_, MINB, true>(p) : launch_pipe_d<W, TGT, HF_, MINB, false>(p);
}

template <int W, int TGT, bool HF_> static cudaError_t launch_pipe_t(TrainLaunch &p) {
    using TileT = Tile<W>;
    const size_t smem_probe = (size_t)PipeSmem<W, TGT>::WBUF(p.n_mat) + (size_t)p.n_mat * TileT::WGT_BYTES + 1024;
    int cols = 32;
    while (cols < 2 * W + p.n_mat * W) cols *= 2;
    // two CTAs per SM (registers capped at half the file) only where shared and tensor memory hold two of them
    if constexpr (PipeSmem<W, TGT>::CTAS_PER_SM == 2) {
        if (2 * (smem_probe + 2048) <= 227 * 1024 && 2 * cols <= 512) return launch_pipe_b<W, TGT, HF_, 2>(p);
    }
    return launch_pipe_b<W, TGT, HF_, 1>(p);
}

template <int W, int TGT, bool HF_, int MINB, bool DX> static cudaError_t launch_pipe_d(TrainLaunch &p) {
    using T = Tile<W>;
    using S = PipeSmem<W, TGT>;
    const size_t smem = (size_t)S::WBUF(p.n_mat) + (size_t)p.n_mat * T::WGT_BYTES + 1024;
    const int cols_needed = 2 * W + p.n_mat * W;
    if (smem > kPipeSmemLimit || cols_needed > 512 || p.n_mat > kPipeMaxMat) return cudaErrorInvalidConfiguration;
    int tmem_cols = 32;
    while (tmem_cols < cols_needed) tmem_cols *= 2;
    const int per_sm = MINB;
    auto kern = mlp_train_pipe_kernel<W, TGT, HF_, MINB, DX>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    const int n_tiles = (int)((p.batch + T::TM - 1) / T::TM);
    const int max_ctas = p.n_sm * per_sm <= p.max_slabs ? p.n_sm * per_sm : p.max_slabs;
    const int grid = n_tiles < max_ctas ? n_tiles : max_ctas;
    p.grid_out = grid;
    if (grid == 0) return cudaSuccess;
    const float inv_n = 1.0f / ((float)p.batch * (float)W);
    count_launch();
    kern<<<grid, S::THREADS, smem, p.stream>>>(p.tm_x, (TGT == 1 || TGT == 3) ? p.tm_tgt : p.tm_x, DX ? p.tm_dx : p.tm_x, p.wimg, p.targets, p.n_targets, p.dw_partials, p.loss_partials,
                                               p.batch, n_tiles, p.n_mat, p.act, p.out_act, p.loss_scale, inv_n,
                                               p.enc, tmem_cols, p.status);
    return cudaGetLastError();
}

template <int W, int TGT> static cudaError_t launch_pipe_w(TrainLaunch &p) {
    return p.fp16 ? launch_pipe_t<W, TGT, true>(p) : launch_pipe_t<W, TGT, false>(p);
}

// Whether the pipelined kernel takes a network of this shape with targets / upstream gradients fetched by `tgt_mode`.
template <int W> static bool pipe_fits_w(int n_mat, int tgt_mode) {
    using T = Tile<W>;
    const int nb = (tgt_mode == 1 || tgt_mode == 2 || tgt_mode == 4) ? 2 : 1;
    const size_t smem = (size_t)(nb + 4 + n_mat) * T::ACT_BYTES + (size_t)n_mat * T::WGT_BYTES + 1024;
    return smem <= kPipeSmemLimit && 2 * W + n_mat * W <= 512 && n_mat <= kPipeMaxMat;
}
bool mlp_train_pipe_fits(int width, int n_mat, int tgt_mode) {
    switch (width) {
    case 16: return pipe_fits_w<16>(n_mat, tgt_mode);
    case 32: return pipe_fits_w<32>(n_mat, tgt_mode);
    case 64: return pipe_fits_w<64>(n_mat, tgt_mode);
    default: return false;
    }
}

cudaError_t launch_mlp_train_pipe(TrainLaunch &p) {
    // staged targets (tgt_mode 1: TMA boxes, 2: one bulk copy of narrow rows) need one more tile of shared memory:
    // without room for it the per-thread loads remain
    cudaError_t e = cudaErrorInvalidConfiguration;
    if (p.tgt_mode == 3) { // dL/dy given instead of targets (backward pass that recomputes the forward)
        if (p.width == 16) return launch_pipe_w<16, 3>(p);
        if (p.width == 32) return launch_pipe_w<32, 3>(p);
        if (p.width == 64) return launch_pipe_w<64, 3>(p);
        return e;
    }
    if (p.width == 16) return launch_pipe_w<16, 0>(p); // 64-byte target rows: read directly
    if (p.width != 64 && p.width != 32) return e;
    const bool w64 = p.width == 64;
    if (p.tgt_mode == 1) e = w64 ? launch_pipe_w<64, 1>(p) : launch_pipe_w<32, 1>(p);
    if (p.tgt_mode == 2) e = w64 ? launch_pipe_w<64, 2>(p) : launch_pipe_w<32, 2>(p);
    if (p.tgt_mode == 4) e = w64 ? launch_pipe_w<64, 4>(p) : launch_pipe_w<32, 4>(p);
    if (e == cudaErrorInvalidConfiguration) e = w64 ? launch_pipe_w<64, 0>(p) : launch_pipe_w<32, 0>(p);
    return e;
}

} // namespace tnn
