// Fully fused training pass for sm_100a: forward, L2 loss, backward and the weight-gradient batch
// reduction of a SwiftNet MLP in ONE kernel, with every activation and delta tile living in shared
// memory only.
//
// It computes exactly what the reference's training loops compute with three separate passes over
// global memory - forward_impl (include/network/kernel_esimd.h:565-640) storing every activation,
// L2Loss::Kernel (include/losses/l2.h:19-41), then backward_impl + gemm_batch
// (kernel_esimd.h:160-240) re-reading all of them - but the only global traffic per sample is the
// input row (2 W bytes), the target row and O(1) for the gradients:
//     a_0 = x;  a_l+1 = act(a_l W_l);  y = act_out(a_L W_L)                       (bf16 after each layer)
//     loss += (y - t)^2 / n;  dL/dy = scale 2 (y - t) / n;  delta_L = dL/dy (.) act_out'(y)
//     delta_l-1 = (delta_l W_l^T) (.) act'(a_l);   G_l += delta_l^T a_l          l = L..0
//
// One persistent CTA per SM, one 128-row tile at a time (all of a tile's activations must stay
// resident for its backward pass, which fills shared memory).  Roles:
//   warp 0  TMA producer (weights once, then double-buffered input tiles)
//   warp 1  issuer of the chain GEMMs (forward and backward; owns TMEM)
//   warp 2  issuer of the weight-gradient GEMMs (off the critical path)
//   warps 4-19  epilogue: four threads per tile row, each owns a quarter of the row's columns
// Each weight tile is staged once and used in both directions without a transposed copy: as the
// MN-major B operand of the forward GEMM and as the K-major B operand of the backward GEMM.
#include "mlp_common.cuh"
#include "elementwise.h"
#include "mlp_launch.h"

namespace tnn {

constexpr int kTrainMaxMat = 7; // weight-gradient accumulators that fit in TMEM next to the chain accumulator

template <int W> struct TrainSmem {
    using T = Tile<W>;
    // The delta tiles come first: for W < 64 the weight-gradient GEMM runs with M = 64 and reads up to
    // three atoms past a delta tile (rows it then ignores); those reads must stay inside the allocation.
    __host__ __device__ static constexpr int D(int /*n_mat*/, int p) { return p * T::ACT_BYTES; }
    static constexpr int X = 2 * T::ACT_BYTES; // 2 input tiles
    __host__ __device__ static constexpr int A(int l) { return (4 + (l - 1)) * T::ACT_BYTES; } // a_1..a_L
    __host__ __device__ static constexpr int WBUF(int n_mat) { return (4 + (n_mat - 1)) * T::ACT_BYTES; }
    static constexpr int TPR = 4;                 // epilogue threads per tile row
    static constexpr int EPI_THREADS = 128 * TPR;
    static constexpr int EPI_WARPS = EPI_THREADS / 32;
    static constexpr int THREADS = 128 + EPI_THREADS;
    static constexpr int CPT = W / TPR;           // columns per epilogue thread
};

struct TrainBarriers {
    uint64_t w_full;
    uint64_t x_full[2];
    uint64_t x_empty[2];            // chain GEMM of layer 0 + weight-gradient GEMM of layer 0 have read the tile
    uint64_t a_free[kTrainMaxMat];  // weight-gradient GEMM that read a_l has completed (index l, 1..L)
    uint64_t d_free[2];             // weight-gradient GEMM that read delta buffer p has completed
    uint64_t step_ready;            // epilogue -> chain issuer: next A operand is in shared memory
    // The weight-gradient issuer may trail its two signallers by one hand-over, so these two signals
    // alternate between two barriers: a barrier is then never more than one phase ahead of its waiter.
    uint64_t dw_go[2];              // epilogue -> weight-gradient issuer: next delta tile is ready
    uint64_t chain_issued[2];       // chain issuer -> weight-gradient issuer: the GEMM on the critical path is queued
    uint64_t acc_full;              // chain issuer -> epilogue
    uint64_t all_done;              // weight-gradient issuer -> epilogue: accumulators final
    uint32_t tmem_base;
    uint32_t abort_flag;
    float loss_red[16];
};

template <int W, bool HF_>
__global__ void __launch_bounds__(TrainSmem<W>::THREADS, 1)
mlp_train_kernel(const __grid_constant__ CUtensorMap tm_x, const __nv_bfloat16 *__restrict__ wimg,
                 const float *__restrict__ targets, int n_targets, float *__restrict__ dw_slabs,
                 float *__restrict__ loss_partials, size_t batch, int n_tiles, int n_mat, int act, int out_act,
                 float loss_scale, float inv_n, int tmem_cols, const EncodedInput enc, int *status) {
    using T = Tile<W>;
    using S = TrainSmem<W>;
    constexpr int fp16 = HF_ ? 1 : 0; // element type of operands and activations: bf16 or fp16
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ TrainBarriers bars;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int L = n_mat - 1;
    const uint32_t smem_base = ptx::smem_u32(smem);
    volatile uint32_t *abort_flag = &bars.abort_flag;
    const int my_tiles = (n_tiles > (int)blockIdx.x) ? (n_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

    if (threadIdx.x == 0) {
        ptx::mbar_init(&bars.w_full, 1);
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(&bars.x_full[b], 1);
            ptx::mbar_init(&bars.x_empty[b], 2);
            ptx::mbar_init(&bars.d_free[b], 1);
        }
        for (int l = 0; l < kTrainMaxMat; ++l) ptx::mbar_init(&bars.a_free[l], 1);
        // one arrival per epilogue warp (its lanes fence their own writes, then one lane arrives)
        ptx::mbar_init(&bars.step_ready, S::EPI_WARPS);
        for (int i = 0; i < 2; ++i) {
            ptx::mbar_init(&bars.dw_go[i], S::EPI_WARPS);
            ptx::mbar_init(&bars.chain_issued[i], 1);
        }
        ptx::mbar_init(&bars.acc_full, 1);
        ptx::mbar_init(&bars.all_done, 1);
        bars.abort_flag = 0;
        ptx::fence_barrier_init();
        if (!enc.x) ptx::prefetch_tmap(&tm_x);
    }
    if (warp == 1) {
        ptx::tmem_alloc(&bars.tmem_base, (uint32_t)tmem_cols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = bars.tmem_base;
    const uint32_t acc_tmem = tmem_base; // columns [0, W): chain accumulator; then one W-column block per layer

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        // weights once; then input tiles by TMA (lane 0) or, with a folded identity encoding, written by the whole
        // warp from fp32 coordinates
        if (lane == 0 && my_tiles > 0) {
            ptx::mbar_arrive_expect_tx(&bars.w_full, (uint32_t)(n_mat * T::WGT_BYTES));
            for (int l = 0; l < n_mat; ++l)
                ptx::bulk_load(smem + S::WBUF(n_mat) + l * T::WGT_BYTES,
                               reinterpret_cast<const uint8_t *>(wimg) + (size_t)l * T::WGT_BYTES, T::WGT_BYTES,
                               &bars.w_full);
        }
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
                        ptx::tma_load_2d(smem + S::X + b * T::ACT_BYTES + at * T::ACT_ATOM_BYTES, &tm_x, at * T::ATOM_COLS,
                                         tile * T::TM, &bars.x_full[b]);
                }
            }
        } else if (my_tiles > 0) {
            fill_tiles_with_ones<W>(smem + S::X, 2, lane, fp16);
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
                encoder.store(smem + S::X + b * T::ACT_BYTES);
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&bars.x_full[b]);
                if (t + 1 < my_tiles) encoder.fetch((size_t)(tile + gridDim.x) * T::TM);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ chain-GEMM issuer
        if (my_tiles > 0) { // all lanes run the loop, one elected lane issues (see ptx::elect_one)
            const uint32_t idesc_fwd = ptx::make_idesc_16(128, W, 0, 1, fp16); // B = W_l read MN-major
            const uint32_t idesc_bwd = ptx::make_idesc_16(128, W, 0, 0, fp16); // B = W_l read K-major
            const uint64_t x_desc0 = T::kdesc_base(smem_base + S::X);
            const uint64_t a_desc0 = T::kdesc_base(smem_base + S::A(1));
            const uint64_t d_desc0 = T::kdesc_base(smem_base + S::D(n_mat, 0));
            const uint64_t wk_desc0 = T::kdesc_base(smem_base + S::WBUF(n_mat));
            const uint64_t wmn_desc0 = T::mndesc_base(smem_base + S::WBUF(n_mat), T::WGT_ATOM_BYTES);
            bool ok = ptx::mbar_wait(&bars.w_full, 0, abort_flag);
            if (!ok && lane == 0) atomicExch(status, KS_TIMEOUT_WEIGHTS);
            uint32_t sr_parity = 0;
            uint32_t ci_count = 0; // chain_issued signals sent
            auto signal_chain_issued = [&]() { // called by the elected lane
                ptx::mbar_arrive(&bars.chain_issued[ci_count & 1u]);
            };
            auto wait_step = [&]() {
                const bool r = ptx::mbar_wait(&bars.step_ready, sr_parity, abort_flag);
                sr_parity ^= 1u;
                return r;
            };
            for (int t = 0; ok && t < my_tiles; ++t) {
                const int b = t & 1;
                // the previous tile's last hand-over (delta_0) also says the accumulator is drained
                if (t > 0 && !wait_step()) ok = false;
                if (ok && !ptx::mbar_wait(&bars.x_full[b], (t >> 1) & 1, abort_flag)) ok = false;
                if (!ok) {
                    if (lane == 0) atomicExch(status, KS_TIMEOUT_MMA | 1);
                    break;
                }
                ptx::tc_fence_after_sync();
                if (ptx::elect_one()) {
                    T::template issue_chain<true>(acc_tmem, x_desc0 + (uint64_t)(b * T::ACT_UNITS), wmn_desc0, idesc_fwd);
                    ptx::mma_commit(&bars.acc_full);
                    ptx::mma_commit(&bars.x_empty[b]);
                    // the previous tile's last weight-gradient GEMM (layer 0) may queue behind this one
                    if (t > 0) signal_chain_issued();
                }
                __syncwarp();
                if (t > 0) ++ci_count;
                for (int l = 1; l <= L; ++l) { // forward
                    if (!wait_step()) {
                        if (lane == 0) atomicExch(status, KS_TIMEOUT_MMA | 2 | (l << 4));
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after_sync();
                    if (ptx::elect_one()) {
                        T::template issue_chain<true>(acc_tmem, a_desc0 + (uint64_t)((l - 1) * T::ACT_UNITS),
                                                      wmn_desc0 + (uint64_t)(l * T::WGT_UNITS), idesc_fwd);
                        ptx::mma_commit(&bars.acc_full);
                    }
                    __syncwarp();
                }
                for (int l = L; ok && l >= 1; --l) { // backward: delta_l sits in D[(L - l) & 1]
                    if (!wait_step()) {
                        if (lane == 0) atomicExch(status, KS_TIMEOUT_MMA | 3 | (l << 4));
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after_sync();
                    if (ptx::elect_one()) {
                        T::template issue_chain<false>(acc_tmem, d_desc0 + (uint64_t)(((L - l) & 1) * T::ACT_UNITS),
                                                       wk_desc0 + (uint64_t)(l * T::WGT_UNITS), idesc_bwd);
                        ptx::mma_commit(&bars.acc_full);
                        signal_chain_issued(); // the weight-gradient GEMM of layer l may follow
                    }
                    __syncwarp();
                    ++ci_count;
                }
            }
            if (ok && ptx::elect_one()) signal_chain_issued(); // releases the very last layer-0 weight-gradient GEMM
            __syncwarp();
        }
    } else if (warp == 2) {
        // ------------------------------------------------------------ weight-gradient issuer
        if (my_tiles > 0) {
            constexpr int DW_M = (W == 128) ? 128 : 64;
            const uint32_t idesc_dw = ptx::make_idesc_16(DW_M, W, 1, 1, fp16);
            const uint64_t x_desc0 = T::mndesc_base(smem_base + S::X, T::ACT_ATOM_BYTES);
            const uint64_t a_desc0 = T::mndesc_base(smem_base + S::A(1), T::ACT_ATOM_BYTES);
            const uint64_t d_desc0 = T::mndesc_base(smem_base + S::D(n_mat, 0), T::ACT_ATOM_BYTES);
            uint32_t k = 0; // hand-overs consumed
            bool ok = true;
            for (int t = 0; ok && t < my_tiles; ++t) {
                const int b = t & 1;
                for (int l = L; l >= 0; --l) {
                    const uint32_t kb = k & 1u, kp = (k >> 1) & 1u;
                    ++k;
                    if (!ptx::mbar_wait(&bars.dw_go[kb], kp, abort_flag)) {
                        if (lane == 0) atomicExch(status, KS_TIMEOUT_MMA | 4 | (l << 4));
                        ok = false;
                        break;
                    }
                    // keep the chain GEMM that consumes the same delta tile ahead in the tensor pipe's queue
                    if (!ptx::mbar_wait(&bars.chain_issued[kb], kp, abort_flag)) {
                        if (lane == 0) atomicExch(status, KS_TIMEOUT_MMA | 5 | (l << 4));
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after_sync();
                    const int p = (L - l) & 1;
                    const uint64_t act_desc = (l == 0) ? x_desc0 + (uint64_t)(b * T::ACT_UNITS)
                                                       : a_desc0 + (uint64_t)((l - 1) * T::ACT_UNITS);
                    if (ptx::elect_one()) {
                        T::issue_outer(tmem_base + (uint32_t)(W + l * W), d_desc0 + (uint64_t)(p * T::ACT_UNITS), act_desc,
                                       idesc_dw, t > 0 ? 1u : 0u);
                        ptx::mma_commit(&bars.d_free[p]);
                        if (l == 0)
                            ptx::mma_commit(&bars.x_empty[b]);
                        else
                            ptx::mma_commit(&bars.a_free[l]);
                    }
                    __syncwarp();
                }
            }
            if (ptx::elect_one()) ptx::mma_commit(&bars.all_done);
            __syncwarp();
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------ epilogue: four threads per row
        const int ew = warp - 4;
        const int quad = warp & 3;
        const int part = ew >> 2; // which CPT-column slice of the row
        const int row = quad * 32 + lane;
        const int col0 = part * S::CPT;
        const uint32_t acc_addr = acc_tmem + ((uint32_t)(quad * 32) << 16) + col0;
        constexpr int CPT = S::CPT; // 16 or 8
        uint32_t af_parity = 0;
        uint32_t dfree_parity[2] = {0, 0};
        int dfree_writes[2] = {0, 0}; // writes issued so far to each delta buffer
        float loss_local = 0.0f;
        bool ok = true;

        auto wait_acc = [&](int code) {
            const bool r = __all_sync(0xffffffffu, ptx::mbar_wait(&bars.acc_full, af_parity, abort_flag));
            af_parity ^= 1u;
            if (!r && lane == 0) atomicExch(status, KS_TIMEOUT_EPILOGUE | code);
            return r;
        };
        auto load_acc = [&](uint32_t (&v)[CPT]) {
            if constexpr (CPT == 16)
                ptx::tmem_ld16(acc_addr, v);
            else
                ptx::tmem_ld8(acc_addr, v);
            ptx::tmem_ld_wait();
        };
        // byte offset of this thread's 16-byte chunk `ch` (0 .. CPT/8-1) inside an activation tile
        auto chunk_at = [&](int ch) {
            const int c = col0 + ch * 8;
            return (c / T::ATOM_COLS) * T::ACT_ATOM_BYTES + T::chunk_off(row, (c % T::ATOM_COLS) / 8);
        };
        // hand-over: every lane makes its shared-memory writes visible to the async proxy, then one lane
        // per warp arrives
        uint32_t go_count = 0; // dw_go signals sent
        auto hand_over = [&](bool also_dw) {
            ptx::fence_proxy_async_smem();
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                ptx::mbar_arrive(&bars.step_ready);
                if (also_dw) ptx::mbar_arrive(&bars.dw_go[go_count & 1u]);
            }
            if (also_dw) ++go_count;
        };
        // every write to a delta buffer but its first waits for the weight-gradient GEMM that read it
        auto acquire_dbuf = [&](int p) {
            bool r = true;
            if (dfree_writes[p] > 0) {
                r = __all_sync(0xffffffffu, ptx::mbar_wait(&bars.d_free[p], dfree_parity[p], abort_flag));
                dfree_parity[p] ^= 1u;
            }
            ++dfree_writes[p];
            return r;
        };

        for (int t = 0; ok && t < my_tiles; ++t) {
            const int tile = blockIdx.x + t * gridDim.x;
            const size_t grow = (size_t)tile * T::TM + row; // global row of this thread
            const bool row_valid = grow < batch;
            // this thread's slice of the target row: requested now, consumed after the forward pass
            float tg[CPT];
            if (row_valid && n_targets == W && (reinterpret_cast<uintptr_t>(targets) & 15) == 0) { // 16-byte loads
#pragma unroll
                for (int q4 = 0; q4 < CPT / 4; ++q4) {
                    const float4 t4 = __ldg(reinterpret_cast<const float4 *>(targets + grow * W + col0) + q4);
                    tg[q4 * 4 + 0] = t4.x, tg[q4 * 4 + 1] = t4.y, tg[q4 * 4 + 2] = t4.z, tg[q4 * 4 + 3] = t4.w;
                }
            } else {
                // narrow targets: only the threads whose column slice holds targets load anything
#pragma unroll
                for (int q = 0; q < CPT; ++q) tg[q] = 0.0f;
                if (row_valid && col0 < n_targets) {
#pragma unroll
                    for (int q = 0; q < CPT; ++q)
                        if (col0 + q < n_targets) tg[q] = __ldg(targets + grow * n_targets + col0 + q);
                }
            }
            // ---------------- forward, hidden layers
            for (int l = 0; l < L && ok; ++l) {
                if (!wait_acc(1 | (l << 4))) {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after_sync();
                uint32_t v[CPT];
                load_acc(v);
                // a_{l+1} of the previous tile must have been consumed by its weight-gradient GEMM
                if (t > 0 &&
                    !__all_sync(0xffffffffu, ptx::mbar_wait(&bars.a_free[l + 1], (t - 1) & 1, abort_flag))) {
                    if (lane == 0) atomicExch(status, KS_TIMEOUT_EPILOGUE | 2 | (l << 4));
                    ok = false;
                    break;
                }
                uint8_t *dst = smem + S::A(l + 1);
                dispatch_act_t<HF_>(act, [&](auto tag) {
                    constexpr int ACT = decltype(tag)::value;
                    constexpr bool HF = decltype(tag)::half;
#pragma unroll
                    for (int ch = 0; ch < CPT / 8; ++ch) {
                        uint4 o;
                        o.x = act_pack_t<ACT, HF>(__uint_as_float(v[ch * 8 + 0]), __uint_as_float(v[ch * 8 + 1]));
                        o.y = act_pack_t<ACT, HF>(__uint_as_float(v[ch * 8 + 2]), __uint_as_float(v[ch * 8 + 3]));
                        o.z = act_pack_t<ACT, HF>(__uint_as_float(v[ch * 8 + 4]), __uint_as_float(v[ch * 8 + 5]));
                        o.w = act_pack_t<ACT, HF>(__uint_as_float(v[ch * 8 + 6]), __uint_as_float(v[ch * 8 + 7]));
                        *reinterpret_cast<uint4 *>(dst + chunk_at(ch)) = o;
                    }
                });
                hand_over(false);
            }
            if (!ok) break;
            // ---------------- output layer + L2 loss: delta_L into D[0]
            {
                if (!wait_acc(3)) {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after_sync();
                uint32_t v[CPT];
                load_acc(v);
                if (!acquire_dbuf(0)) {
                    if (lane == 0) atomicExch(status, KS_TIMEOUT_EPILOGUE | 4);
                    ok = false;
                    break;
                }
                uint8_t *dst = smem + S::D(n_mat, 0);
                dispatch_act_t<HF_>(out_act, [&](auto tag) {
                    constexpr int ACT = decltype(tag)::value;
                    constexpr bool HF = decltype(tag)::half;
#pragma unroll
                    for (int ch = 0; ch < CPT / 8; ++ch) {
                        uint32_t o[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            // the prediction as the network stores it (bf16), then the loss on that value
                            const uint32_t y16 = act_pack_t<ACT, HF>(__uint_as_float(v[ch * 8 + 2 * q]),
                                                                  __uint_as_float(v[ch * 8 + 2 * q + 1]));
                            float d0 = ptx::lo_f32<HF>(y16) - tg[ch * 8 + 2 * q];
                            float d1 = ptx::hi_f32<HF>(y16) - tg[ch * 8 + 2 * q + 1];
                            if (!row_valid) d0 = d1 = 0.0f;
                            loss_local += d0 * d0 * inv_n + d1 * d1 * inv_n;
                            const uint32_t g16 =
                                ptx::pack2<HF>(loss_scale * 2.0f * d0 * inv_n, loss_scale * 2.0f * d1 * inv_n);
                            o[q] = (ACT == ACT_NONE)
                                       ? g16
                                       : act_bwd_pack_t<ACT, HF>(ptx::lo_f32<HF>(g16), ptx::hi_f32<HF>(g16), y16);
                        }
                        *reinterpret_cast<uint4 *>(dst + chunk_at(ch)) = make_uint4(o[0], o[1], o[2], o[3]);
                    }
                });
                hand_over(true);
            }
            // ---------------- backward: step l turns (delta_l W_l^T) into delta_{l-1} in D[(L - l + 1) & 1]
            for (int l = L; l >= 1 && ok; --l) {
                if (!wait_acc(5 | (l << 4))) {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after_sync();
                uint32_t v[CPT];
                load_acc(v);
                const int p = (L - l + 1) & 1;
                if (!acquire_dbuf(p)) {
                    if (lane == 0) atomicExch(status, KS_TIMEOUT_EPILOGUE | 6 | (l << 4));
                    ok = false;
                    break;
                }
                const uint8_t *abuf = smem + S::A(l);
                uint8_t *dst = smem + S::D(n_mat, p);
                dispatch_act_t<HF_>(act, [&](auto tag) {
                    constexpr int ACT = decltype(tag)::value;
                    constexpr bool HF = decltype(tag)::half;
#pragma unroll
                    for (int ch = 0; ch < CPT / 8; ++ch) {
                        const int off = chunk_at(ch);
                        uint4 f = make_uint4(0, 0, 0, 0);
                        if constexpr (ACT != ACT_NONE) f = *reinterpret_cast<const uint4 *>(abuf + off);
                        uint4 o;
                        o.x = act_bwd_pack_t<ACT, HF>(__uint_as_float(v[ch * 8 + 0]), __uint_as_float(v[ch * 8 + 1]), f.x);
                        o.y = act_bwd_pack_t<ACT, HF>(__uint_as_float(v[ch * 8 + 2]), __uint_as_float(v[ch * 8 + 3]), f.y);
                        o.z = act_bwd_pack_t<ACT, HF>(__uint_as_float(v[ch * 8 + 4]), __uint_as_float(v[ch * 8 + 5]), f.z);
                        o.w = act_bwd_pack_t<ACT, HF>(__uint_as_float(v[ch * 8 + 6]), __uint_as_float(v[ch * 8 + 7]), f.w);
                        *reinterpret_cast<uint4 *>(dst + off) = o;
                    }
                });
                hand_over(true);
            }
        }

        // ---------------- loss partial of this CTA (fixed summation order)
        for (int o = 16; o > 0; o >>= 1) loss_local += __shfl_xor_sync(0xffffffffu, loss_local, o);
        if (lane == 0) bars.loss_red[ew] = loss_local;
        ptx::named_bar_sync(1, S::EPI_THREADS);
        if (ew == 0 && lane == 0 && loss_partials) {
            float s = 0.0f;
            for (int i = 0; i < S::EPI_WARPS; ++i) s += bars.loss_red[i];
            loss_partials[blockIdx.x] = s;
        }

        // ---------------- drain the weight-gradient accumulators into this CTA's slab
        if (ok && my_tiles > 0) {
            if (!__all_sync(0xffffffffu, ptx::mbar_wait(&bars.all_done, 0, abort_flag))) {
                if (lane == 0) atomicExch(status, KS_TIMEOUT_EPILOGUE | 7);
                ok = false;
            }
        }
        if (ok && my_tiles > 0) {
            ptx::tc_fence_after_sync();
            float *slab = dw_slabs + (size_t)blockIdx.x * n_mat * W * W;
            // M = 64 accumulators keep row m in lane (m % 16) + 32 * (m / 16)
            const int o = quad * 16 + lane;
            const bool valid = lane < 16 && o < W;
            for (int l = 0; l < n_mat; ++l) {
                uint32_t v[CPT];
                if constexpr (CPT == 16)
                    ptx::tmem_ld16(tmem_base + ((uint32_t)(quad * 32) << 16) + W + l * W + col0, v);
                else
                    ptx::tmem_ld8(tmem_base + ((uint32_t)(quad * 32) << 16) + W + l * W + col0, v);
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
        ptx::tmem_dealloc(tmem_base, (uint32_t)tmem_cols);
    }
}

// ---------------------------------------------------------------------- host side
template <int W> static cudaError_t launch_train_w(TrainLaunch &p) {
    using T = Tile<W>;
    using S = TrainSmem<W>;
    const size_t smem = (size_t)S::WBUF(p.n_mat) + (size_t)p.n_mat * T::WGT_BYTES + 1024;
    const int cols_needed = W + p.n_mat * W;
    if (smem > 227 * 1024 || cols_needed > 512 || p.n_mat > kTrainMaxMat) return cudaErrorInvalidConfiguration;
    int tmem_cols = 32;
    while (tmem_cols < cols_needed) tmem_cols *= 2;
    const int n_tiles = (int)((p.batch + T::TM - 1) / T::TM);
    const int grid = n_tiles < p.n_sm ? n_tiles : p.n_sm;
    p.grid_out = grid;
    if (grid == 0) return cudaSuccess;
    const float inv_n = 1.0f / ((float)p.batch * (float)W);
    auto go = [&](auto kern) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        count_launch();
        kern<<<grid, S::THREADS, smem, p.stream>>>(p.tm_x, p.wimg, p.targets, p.n_targets, p.dw_partials,
                                                   p.loss_partials, p.batch, n_tiles, p.n_mat, p.act, p.out_act,
                                                   p.loss_scale, inv_n, tmem_cols, p.enc, p.status);
        return cudaGetLastError();
    };
    return p.fp16 ? go(mlp_train_kernel<W, true>) : go(mlp_train_kernel<W, false>);
}

cudaError_t launch_mlp_train(TrainLaunch &p) {
    if (p.want_dx) return cudaErrorInvalidConfiguration; // dL/dinput: pipelined kernel or the three-kernel path
    switch (p.width) {
    case 32: return launch_train_w<32>(p);
    case 64: return launch_train_w<64>(p);
    default: return cudaErrorInvalidConfiguration; // other widths use the separate forward / backward kernels
    }
}

} // namespace tnn
