// Fully fused MLP forward / inference for sm_100a.
//
// Replaces EsimdKernels::forward_impl_general<INFERENCE> of the reference
// (include/network/kernel_esimd.h:565-640): y = act_out(... act(act(x W0) W1) ... WL), all
// matrices W x W, bf16 operands, fp32 accumulation, rounding to bf16 after every layer.
//
// One persistent CTA per SM walks over 128-row batch tiles with NSLOT tiles in flight.  Roles:
//   warp 0            : TMA producer - stages the weights once, then streams input tiles
//   warps 1..NSLOT    : one MMA issuer per slot (the warp runs converged, an elected lane issues tcgen05.mma)
//   then NSLOT groups : 4 epilogue warps per slot
// A slot is one tile in flight: its input buffer, its activation buffer(s) and one fp32
// accumulator of W TMEM columns.  Per layer the slot's epilogue group pulls the accumulator out
// of TMEM, applies the activation, rounds to bf16 and writes the next layer's A operand back to TMEM
// (TMEM_A, the inference default) or to swizzled shared memory, so activations never leave the SM.
// With the A operand in TMEM a 128 x 64 x 16 MMA reads only its 2 KB weight slice from shared memory
// and runs in 32 cycles; with both operands in shared memory the 6 KB of operand traffic make it 48
// cycles and compete with the epilogue's stores.  With STORE_ALL every layer's activation is also
// written to global memory by TMA for a later backward pass.
//
// Networks whose weights do not fit beside the tiles (width 128, or many layers) run with STREAM_W: every slot
// owns a ring of two weight tiles and its issuer fetches the weights of the next layer (from L2) right before it
// issues the GEMM of the current one, i.e. as soon as the GEMM that read that ring stage is known to be complete.
//
// The layer-to-layer chain of one tile is strictly serial (MMA -> epilogue -> MMA ...), and a
// single thread's dependent instructions cost several cycles each, so throughput comes from
// running the chains of several slots side by side: every slot has its own issuer warp and its
// own epilogue group, and nothing but the tensor pipe and shared memory is shared between them.
#include "mlp_common.cuh"
#include "elementwise.h"
#include "grid_device.cuh"

#include <type_traits>
#include "mlp_launch.h"

namespace tnn {

template <int W, int NSLOT, bool TMEM_A, bool STORE_ALL, bool STREAM_W = false> struct FwdSmem {
    using T = Tile<W>;
    // activation buffers per slot: two (ping-pong) when every layer is also streamed out by TMA,
    // one when the next layer's MMA is the only reader
    static constexpr int NABUF = STORE_ALL ? 2 : 1;
    // With the hidden activations in TMEM the only shared-memory tile a slot writes is its output, once per tile.
    // Streamed-weight configurations, which are short of shared memory, let all slots take turns on one such tile.
    static constexpr bool SHARED_OUT = TMEM_A && !STORE_ALL && STREAM_W && NSLOT > 1;
    static constexpr int ABUF_TILES = SHARED_OUT ? 1 : NSLOT * NABUF;
    static constexpr int XBUF = 0;                                   // NSLOT input tiles
    static constexpr int ABUF = XBUF + NSLOT * T::ACT_BYTES;         // NSLOT x NABUF activation tiles
    static constexpr int WBUF = ABUF + ABUF_TILES * T::ACT_BYTES;    // (L+1) weight tiles follow
    static constexpr int tmem_cols_needed = NSLOT * (W + (TMEM_A ? W / 2 : 0));
    static constexpr int tmem_cols =
        tmem_cols_needed <= 32 ? 32 : tmem_cols_needed <= 64 ? 64 : tmem_cols_needed <= 128 ? 128
                                                              : tmem_cols_needed <= 256 ? 256 : 512;
    static constexpr bool fits_tmem = tmem_cols_needed <= 512;
    static constexpr int THREADS = 32 * (1 + NSLOT) + 128 * NSLOT;
    // weight tiles behind WBUF: all n_mat of them, or a ring of two per slot
    __host__ __device__ static constexpr int weight_tiles(int n_mat) { return STREAM_W ? 2 * NSLOT : n_mat; }
};

constexpr int kMaxSlots = 6;

struct FwdBarriers {
    uint64_t w_full;
    uint64_t x_full[kMaxSlots];
    uint64_t x_empty[kMaxSlots];
    uint64_t a_ready[kMaxSlots];
    uint64_t acc_full[kMaxSlots];
    uint64_t wring_full[kMaxSlots][2]; // STREAM_W: weight ring stages of every slot
    uint32_t tmem_base;
    uint32_t abort_flag;
    uint32_t out_lock; // SHARED_OUT: 1 while a slot owns the output tile
};

// NENC > 0: the network input is the hash-grid encoding of fp32 positions, produced on the SM by NENC extra warps
// (NetworkWithInputEncoding of the reference, dpcpp_bindings/tiny_dpcpp_nn/modules.py:357-421, without the
// batch x W matrix between the two modules).  Each encoder warp owns 32 rows of the tile at one level at a time -
// level parameters are warp-uniform and sit in shared memory - gathers the 2^D corners, interpolates
// (include/encodings/grid.h:64-133, same arithmetic as the stand-alone encoding kernel) and writes the rounded
// features straight into the swizzled input tile that layer 0's MMA reads; columns past the features stay zero.
constexpr int kGridEncWarps = 8;

template <int D>
__device__ __forceinline__ void encode_grid_rows(uint8_t *xt, int row, int level0, const GridCommon &gc,
                                                 const GridLevelInfo *levels, int n_levels, const float *__restrict__ table,
                                                 const float (&xin)[D], bool valid, int fp16, int atom_cols,
                                                 int atom_bytes, int row_bytes, int chunks) {
#pragma unroll 2
    for (int level = level0; level < n_levels; level += 2) {
        float r[2];
        grid_level_features<D, 2>(gc, levels[level], (uint32_t)level, table, xin, r);
        if (!valid) r[0] = r[1] = 0.0f;
        const uint32_t packed = fp16 ? ptx::pack_f16x2(r[0], r[1]) : ptx::pack_bf16x2(r[0], r[1]);
        const int col = level * 2;
        const int chunk = (col % atom_cols) / 8;
        const int off = (col / atom_cols) * atom_bytes + row * row_bytes +
                        ((chunk ^ (((row * row_bytes) >> 7) & (chunks - 1))) << 4) + (col % 8) * 2;
        *reinterpret_cast<uint32_t *>(xt + off) = packed;
    }
}

// LIVE8 (inference with the hidden activations in tensor memory): the network has at most 8 real outputs and
// act_out(0) = 0, so the output columns from the 9th on are exactly zero (zero weight columns).  The output tile of
// a slot is zeroed once and the output layer's epilogue step - a code region of its own, selected at compile time -
// converts and writes the first 8-column chunk of a row only.
template <int W, int NSLOT, bool STORE_ALL, bool TMEM_A, bool B_MN_MAJOR, bool STREAM_W, int NENC, bool HF_, bool LIVE8>
__global__ void __launch_bounds__(FwdSmem<W, NSLOT, TMEM_A, STORE_ALL>::THREADS + 32 * NENC, 1)
mlp_fwd_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_y,
               const __grid_constant__ CUtensorMap tm_interm, const __nv_bfloat16 *__restrict__ wimg,
               const GridParams *__restrict__ gp, const float *__restrict__ table, const float *__restrict__ coords,
               int n_tiles, int n_mat, int act, int out_act, int write_y, size_t batch, const EncodedInput enc, int *status) {
    using T = Tile<W>;
    using S = FwdSmem<W, NSLOT, TMEM_A, STORE_ALL, STREAM_W>;
    constexpr int fp16 = HF_ ? 1 : 0; // element type of operands and activations: bf16 or fp16
    static_assert(NSLOT <= kMaxSlots, "too many slots");
    extern __shared__ uint8_t smem_raw[];
    // operand tiles need 1024-byte alignment (swizzle span)
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ FwdBarriers bars;
    __shared__ GridLevelInfo enc_levels[NENC ? kMaxGridLevels : 1];

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int L = n_mat - 1; // index of the output layer
    const uint32_t smem_base = ptx::smem_u32(smem);
    volatile uint32_t *abort_flag = &bars.abort_flag;
    // Inference with a folded identity encoding: the input tile of a slot is written by that slot's issuer warp, in
    // the shadow of its first epilogue step.  (One producer warp encoding for all slots needs about 1 800 cycles per
    // tile - waits, conversions, stores and fences in sequence - which is the whole tile period of this kernel.)
    const bool ISSUER_ENCODES = !STORE_ALL && NENC == 0 && enc.x != nullptr;

    // tiles handled by this CTA: blockIdx.x, blockIdx.x + gridDim.x, ...; local tile j runs in slot j % NSLOT
    const int my_tiles = (n_tiles > (int)blockIdx.x) ? (n_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

    if (threadIdx.x == 0) {
        ptx::mbar_init(&bars.w_full, 1);
        for (int s = 0; s < NSLOT; ++s) {
            ptx::mbar_init(&bars.x_full[s], NENC ? NENC : 1); // one arrival per encoder warp, or the producer's
            ptx::mbar_init(&bars.x_empty[s], 1);
            ptx::mbar_init(&bars.a_ready[s], 4); // one arrival per epilogue warp
            ptx::mbar_init(&bars.acc_full[s], 1);
            ptx::mbar_init(&bars.wring_full[s][0], 1);
            ptx::mbar_init(&bars.wring_full[s][1], 1);
        }
        bars.abort_flag = 0;
        bars.out_lock = 0;
        ptx::fence_barrier_init();
        if (!enc.x && !NENC) ptx::prefetch_tmap(&tm_x);
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
        // weights once (unless streamed); then input tiles by TMA (lane 0) or, with a folded identity encoding, written
        // by the whole warp from fp32 coordinates (with STORE_ALL the encoded tile is also stored as matrix 0 of the
        // activations)
        if constexpr (!STREAM_W) {
            if (lane == 0 && my_tiles > 0) {
                ptx::mbar_arrive_expect_tx(&bars.w_full, (uint32_t)(n_mat * T::WGT_BYTES));
                for (int l = 0; l < n_mat; ++l)
                    ptx::bulk_load(smem + S::WBUF + l * T::WGT_BYTES,
                                   reinterpret_cast<const uint8_t *>(wimg) + (size_t)l * T::WGT_BYTES, T::WGT_BYTES,
                                   &bars.w_full);
            }
        }
        if constexpr (NENC > 0) {
            // the encoder warps produce the input tiles
        } else if (!enc.x) {
            if (lane == 0) {
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
        } else if (ISSUER_ENCODES) {
            // each slot's issuer warp writes its own input tiles (below)
        } else if (my_tiles > 0) {
            fill_tiles_with_ones<W>(smem + S::XBUF, NSLOT, lane, fp16);
            __syncwarp();
            IdentityTileEncoder<W> encoder(enc, batch, lane, fp16);
            encoder.fetch((size_t)blockIdx.x * T::TM);
            for (int j = 0; j < my_tiles; ++j) {
                const int s = j % NSLOT, t = j / NSLOT;
                const int tile = blockIdx.x + j * gridDim.x;
                if (t >= 1 && !__all_sync(0xffffffffu, ptx::mbar_wait(&bars.x_empty[s], (t - 1) & 1, abort_flag))) {
                    if (lane == 0) atomicExch(status, KS_TIMEOUT_PRODUCER | s);
                    break;
                }
                uint8_t *xt = smem + S::XBUF + s * T::ACT_BYTES;
                if (STORE_ALL && j >= NSLOT) { // the store of this slot's previous tile has read the buffer
                    if (lane == 0) ptx::tma_wait_group_read<NSLOT - 1>();
                    __syncwarp();
                }
                encoder.store(xt);
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    ptx::mbar_arrive(&bars.x_full[s]);
                    if (STORE_ALL) {
                        for (int a = 0; a < T::KATOMS; ++a)
                            ptx::tma_store_3d(&tm_interm, xt + a * T::ACT_ATOM_BYTES, a * T::ATOM_COLS, tile * T::TM, 0);
                        ptx::tma_commit_group();
                    }
                }
                // coordinates of the next tile travel while this one is consumed
                if (j + 1 < my_tiles) encoder.fetch((size_t)(tile + gridDim.x) * T::TM);
            }
            if (STORE_ALL && lane == 0) ptx::tma_wait_group<0>();
        }
    } else if (warp <= NSLOT) {
        // ------------------------------------------------------------ MMA issuer of slot s
        const int s = warp - 1;
        if (my_tiles > s) { // all lanes run the loop, one elected lane issues (see ptx::elect_one)
            const uint32_t idesc = ptx::make_idesc_16(128, W, 0, B_MN_MAJOR ? 1 : 0, fp16);
            // every descriptor this thread will ever need, as bases that are stepped by constants
            const uint64_t x_desc = T::kdesc_base(smem_base + S::XBUF + s * T::ACT_BYTES);
            const uint64_t a_desc0 = T::kdesc_base(smem_base + S::ABUF + s * S::NABUF * T::ACT_BYTES);
            // resident weights: tile l of the image; streamed: stage 0 of this slot's ring
            const uint32_t w_smem0 = smem_base + S::WBUF + (STREAM_W ? s * 2 * T::WGT_BYTES : 0);
            const uint64_t w_desc0 =
                B_MN_MAJOR ? T::mndesc_base(w_smem0, T::WGT_ATOM_BYTES) : T::kdesc_base(w_smem0);
            [[maybe_unused]] uint32_t wg = 0; // STREAM_W: GEMMs issued so far = ring position of the current weights
            [[maybe_unused]] auto fetch_weights = [&](int l, uint32_t g) { // W_l into ring stage g & 1 (elected lane)
                uint64_t *bar = &bars.wring_full[s][g & 1u];
                ptx::mbar_arrive_expect_tx(bar, (uint32_t)T::WGT_BYTES);
                ptx::bulk_load(smem + S::WBUF + (s * 2 + (g & 1u)) * T::WGT_BYTES,
                               reinterpret_cast<const uint8_t *>(wimg) + (size_t)l * T::WGT_BYTES, T::WGT_BYTES, bar);
            };
            const uint32_t d_tmem = tmem_base + s * W;
            [[maybe_unused]] const uint32_t a_tmem = tmem_base + NSLOT * W + s * (W / 2);
            uint64_t *const a_ready = &bars.a_ready[s];
            uint64_t *const acc_full = &bars.acc_full[s];
            bool ok = true;
            if constexpr (STREAM_W) {
                if (ptx::elect_one()) fetch_weights(0, 0);
                __syncwarp();
            } else {
                ok = ptx::mbar_wait(&bars.w_full, 0, abort_flag);
            }
            if (!ok && lane == 0) atomicExch(status, KS_TIMEOUT_WEIGHTS);
            uint32_t ar_parity = 0; // parity of the next a_ready completion to wait for
            uint32_t xf_parity = 0;
            const int my_slot_tiles = (my_tiles - s + NSLOT - 1) / NSLOT;
            // ISSUER_ENCODES: coordinates of this slot's next tile wait in registers
            IdentityTileEncoder<W> encoder(enc, batch, lane, fp16);
            uint8_t *const xt = smem + S::XBUF + s * T::ACT_BYTES;
            if (ISSUER_ENCODES) {
                encoder.fetch((size_t)(blockIdx.x + s * gridDim.x) * T::TM);
                fill_tiles_with_ones<W>(xt, 1, lane, fp16);
                __syncwarp();
                encoder.store(xt);
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (my_slot_tiles > 1) encoder.fetch((size_t)(blockIdx.x + (s + NSLOT) * gridDim.x) * T::TM);
            }
            for (int t = 0; ok && t < my_slot_tiles; ++t) {
                // layer 0: needs the input tile and (from the second tile on) the drained accumulator
                if (!ISSUER_ENCODES) {
                    ok = ptx::mbar_wait(&bars.x_full[s], xf_parity, abort_flag);
                    xf_parity ^= 1u;
                }
                if (ok && t > 0) {
                    ok = ptx::mbar_wait(a_ready, ar_parity, abort_flag);
                    ar_parity ^= 1u;
                }
                if (!ok) {
                    if (lane == 0) atomicExch(status, KS_TIMEOUT_MMA | s);
                    break;
                }
                if constexpr (STREAM_W) {
                    // the GEMM that read the other ring stage is complete (its accumulator was drained): refill it
                    // (next in this slot's sequence: W_1, or W_0 of its next tile for a single-matrix network)
                    if (L >= 1 || t + 1 < my_slot_tiles) {
                        if (ptx::elect_one()) fetch_weights(L >= 1 ? 1 : 0, wg + 1);
                        __syncwarp();
                    }
                    if (!ptx::mbar_wait(&bars.wring_full[s][wg & 1u], (wg >> 1) & 1u, abort_flag)) {
                        if (lane == 0) atomicExch(status, KS_TIMEOUT_WEIGHTS | 1);
                        break;
                    }
                }
                ptx::tc_fence_after_sync();
                if (ptx::elect_one()) {
                    T::template issue_chain<B_MN_MAJOR>(d_tmem, x_desc,
                                                        w_desc0 + (STREAM_W ? (uint64_t)((wg & 1u) * T::WGT_UNITS) : 0), idesc);
                    ptx::mma_commit(acc_full);
                    ptx::mma_commit(&bars.x_empty[s]);
                }
                __syncwarp();
                ++wg;
                if (ISSUER_ENCODES && t + 1 < my_slot_tiles) {
                    // once layer 0 has read the input tile, write the slot's next one while the epilogue works
                    if (!ptx::mbar_wait(&bars.x_empty[s], t & 1, abort_flag)) {
                        if (lane == 0) atomicExch(status, KS_TIMEOUT_PRODUCER | s);
                        ok = false;
                        break;
                    }
                    encoder.store(xt);
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (t + 2 < my_slot_tiles)
                        encoder.fetch((size_t)(blockIdx.x + (s + (t + 2) * NSLOT) * gridDim.x) * T::TM);
                }
                uint64_t w_desc = w_desc0;
                for (int l = 1; l <= L; ++l) {
                    w_desc += T::WGT_UNITS;
                    if (!ptx::mbar_wait(a_ready, ar_parity, abort_flag)) {
                        if (lane == 0) atomicExch(status, KS_TIMEOUT_MMA | (l << 4) | s);
                        ok = false;
                        break;
                    }
                    ar_parity ^= 1u;
                    if constexpr (STREAM_W) {
                        // next in this slot's sequence: W_{l+1}, or W_0 for its next tile
                        if (l < L || t + 1 < my_slot_tiles) {
                            if (ptx::elect_one()) fetch_weights(l < L ? l + 1 : 0, wg + 1);
                            __syncwarp();
                        }
                        if (!ptx::mbar_wait(&bars.wring_full[s][wg & 1u], (wg >> 1) & 1u, abort_flag)) {
                            if (lane == 0) atomicExch(status, KS_TIMEOUT_WEIGHTS | 2);
                            ok = false;
                            break;
                        }
                        w_desc = w_desc0 + (uint64_t)((wg & 1u) * T::WGT_UNITS);
                    }
                    ptx::tc_fence_after_sync();
                    if (ptx::elect_one()) {
                        if constexpr (TMEM_A) {
                            T::template issue_chain_ts<B_MN_MAJOR>(d_tmem, a_tmem, w_desc, idesc);
                        } else {
                            const uint64_t a_desc = a_desc0 + (uint64_t)(((l - 1) & (S::NABUF - 1)) * T::ACT_UNITS);
                            T::template issue_chain<B_MN_MAJOR>(d_tmem, a_desc, w_desc, idesc);
                        }
                        ptx::mma_commit(acc_full);
                    }
                    __syncwarp();
                    ++wg;
                }
            }
        }
    } else if (warp < 1 + NSLOT + 4 * NSLOT) {
        // ------------------------------------------------------------ epilogue group of slot s
        const int ew = warp - (1 + NSLOT);  // epilogue warp index
        const int s = ew >> 2;              // slot owned by this group
        const int quad = warp & 3;          // TMEM lane quarter this warp may touch
        const int row = quad * 32 + lane;   // tile row owned by this thread
        const bool leader = (ew & 3) == 0 && lane == 0;
        const uint32_t acc_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + s * W;
        [[maybe_unused]] const uint32_t a_tmem = tmem_base + ((uint32_t)(quad * 32) << 16) + NSLOT * W + s * (W / 2);
        uint64_t *const a_ready = &bars.a_ready[s];
        uint64_t *const acc_full = &bars.acc_full[s];
        uint32_t af_parity = 0;
        bool ok = true;
        if constexpr (LIVE8) {
            // this thread's row of the slot's output tile: zeros now, only its first chunk is written per tile
            uint8_t *out_tile = smem + S::ABUF + s * S::NABUF * T::ACT_BYTES;
            for (int at = 0; at < T::KATOMS; ++at)
                for (int ch = 0; ch < T::CHUNKS; ++ch)
                    *reinterpret_cast<uint4 *>(out_tile + at * T::ACT_ATOM_BYTES + T::chunk_off(row, ch)) =
                        make_uint4(0u, 0u, 0u, 0u);
        }
        for (int j = s; ok && j < my_tiles; j += NSLOT) {
            const int tile = blockIdx.x + j * gridDim.x;
            // One epilogue step; `last` (a compile-time tag) tells the output layer from the hidden ones, so that each
            // call site is a straight-line body of its own: where the result goes (tensor memory for the next GEMM or
            // shared memory for the store) is then no run-time question inside the per-element code.
            auto epi_step = [&](int l, auto last) -> bool {
                constexpr bool IS_LAST = decltype(last)::value;
                // the verdict must be warp-uniform: the TMEM accesses below are .aligned
                if (!__all_sync(0xffffffffu, ptx::mbar_wait(acc_full, af_parity, abort_flag))) {
                    if (lane == 0) atomicExch(status, KS_TIMEOUT_EPILOGUE | (l << 4) | s);
                    return false;
                }
                af_parity ^= 1u;
                ptx::tc_fence_after_sync();
                const int a = IS_LAST ? out_act : act;
                constexpr bool to_tmem = TMEM_A && !IS_LAST;
                uint8_t *abuf = smem + S::ABUF +
                                (S::SHARED_OUT ? 0 : (s * S::NABUF + (l & (S::NABUF - 1))) * T::ACT_BYTES);
                constexpr int CW = (W >= 32) ? 32 : 16; // columns per TMEM load
                constexpr int NLD = W / CW;
                uint32_t v[NLD][CW];
#pragma unroll
                for (int i = 0; i < NLD; ++i) {
                    if constexpr (CW == 32)
                        ptx::tmem_ld32(acc_addr + i * CW, v[i]);
                    else
                        ptx::tmem_ld16(acc_addr + i * CW, v[i]);
                }
                if constexpr (S::SHARED_OUT) {
                    if (IS_LAST) {
                        // take the shared output tile: the previous owner releases it once its store has read it
                        if (leader) {
                            bool got = false;
                            for (uint32_t it = 0; it < (1u << 22); ++it) {
                                if (atomicCAS(&bars.out_lock, 0u, 1u) == 0u) {
                                    got = true;
                                    break;
                                }
                                if ((it & 63u) == 63u && *abort_flag) break;
                                __nanosleep(32);
                            }
                            if (!got) {
                                *abort_flag = 1u;
                                atomicExch(status, KS_TIMEOUT_EPILOGUE | 0x80 | s);
                            }
                        }
                        // (one verdict for the whole group: nobody is left alone at a later barrier)
                        if (ptx::named_bar_red_or(1 + s, 128, *abort_flag != 0)) {
                            return false;
                        }
                    }
                } else if (!to_tmem && (STORE_ALL || TMEM_A || l == 0)) {
                    // the buffer about to be overwritten may still be read by an earlier TMA store: with
                    // per-layer stores the newest one reads the other ping-pong buffer, otherwise only the
                    // previous tile's output store can be pending
                    if (leader) {
                        if (STORE_ALL && l > 0)
                            ptx::tma_wait_group_read<1>();
                        else
                            ptx::tma_wait_group_read<0>();
                    }
                    ptx::named_bar_sync(1 + s, 128);
                }
                ptx::tmem_ld_wait();
                if constexpr (TMEM_A && IS_LAST) {
                    // output layer: the accumulator is in registers and nothing else is handed to the issuer, so the
                    // first GEMM of the slot's next tile may run under the conversion and the store of this one
                    // (measured neutral to 6 % slower at width 16, whose kernels keep the arrival behind the stores)
                    ptx::tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(a_ready);
                }
                dispatch_act_t<HF_>(a, [&](auto tag) {
                    constexpr int ACT = decltype(tag)::value;
                    constexpr bool HF = decltype(tag)::half;
#pragma unroll
                    for (int i = 0; i < NLD; ++i) {
                        const int c0 = i * CW;
                        uint32_t p[CW / 2];
#pragma unroll
                        for (int q = 0; q < CW / 2; ++q)
                            p[q] = act_pack_t<ACT, HF>(__uint_as_float(v[i][2 * q]), __uint_as_float(v[i][2 * q + 1]));
                        if (to_tmem) {
                            if constexpr (CW == 32) ptx::tmem_st16(a_tmem + c0 / 2, p);
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
                });
                if (to_tmem)
                    ptx::tmem_st_wait();
                else
                    ptx::fence_proxy_async_smem();
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0 && !(TMEM_A && IS_LAST)) ptx::mbar_arrive(a_ready);
                if (!to_tmem && (STORE_ALL || IS_LAST)) {
                    ptx::named_bar_sync(1 + s, 128);
                    if (leader) {
                        for (int at = 0; at < T::KATOMS; ++at) {
                            if (STORE_ALL)
                                ptx::tma_store_3d(&tm_interm, abuf + at * T::ACT_ATOM_BYTES, at * T::ATOM_COLS,
                                                  tile * T::TM, l + 1);
                            if (IS_LAST && write_y)
                                ptx::tma_store_2d(&tm_y, abuf + at * T::ACT_ATOM_BYTES, at * T::ATOM_COLS,
                                                  tile * T::TM);
                        }
                        ptx::tma_commit_group();
                        if constexpr (S::SHARED_OUT) {
                            ptx::tma_wait_group_read<0>(); // the store has read the tile: hand it to the next slot
                            __threadfence_block();
                            atomicExch(&bars.out_lock, 0u);
                        }
                    }
                }
                return true;
            };
            for (int l = 0; ok && l < L; ++l) ok = epi_step(l, std::false_type{});
            if constexpr (!LIVE8) {
                if (ok) ok = epi_step(L, std::true_type{});
            }
            if constexpr (LIVE8) {
                if (!ok) break;
                // ---- output layer, first 8 columns only
                if (!__all_sync(0xffffffffu, ptx::mbar_wait(acc_full, af_parity, abort_flag))) {
                    if (lane == 0) atomicExch(status, KS_TIMEOUT_EPILOGUE | (L << 4) | s);
                    ok = false;
                    break;
                }
                af_parity ^= 1u;
                ptx::tc_fence_after_sync();
                uint32_t v8[8];
                ptx::tmem_ld8(acc_addr, v8);
                uint8_t *out_tile = smem + S::ABUF + s * S::NABUF * T::ACT_BYTES;
                // the previous tile's output store must have read the tile before its first chunk is overwritten
                if (leader) ptx::tma_wait_group_read<0>();
                ptx::named_bar_sync(1 + s, 128);
                ptx::tmem_ld_wait();
                dispatch_act_t<HF_>(out_act, [&](auto tag) {
                    constexpr int ACT = decltype(tag)::value;
                    constexpr bool HF = decltype(tag)::half;
                    uint32_t p[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        p[q] = act_pack_t<ACT, HF>(__uint_as_float(v8[2 * q]), __uint_as_float(v8[2 * q + 1]));
                    *reinterpret_cast<uint4 *>(out_tile + T::chunk_off(row, 0)) = make_uint4(p[0], p[1], p[2], p[3]);
                });
                ptx::fence_proxy_async_smem();
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(a_ready);
                ptx::named_bar_sync(1 + s, 128);
                if (leader) {
                    if (write_y)
                        for (int at = 0; at < T::KATOMS; ++at)
                            ptx::tma_store_2d(&tm_y, out_tile + at * T::ACT_ATOM_BYTES, at * T::ATOM_COLS, tile * T::TM);
                    ptx::tma_commit_group();
                }
            }
        }
        if (leader) ptx::tma_wait_group<0>();
    } else if constexpr (NENC > 0) {
        // ------------------------------------------------------------ hash-grid encoder warps
        const int ew = warp - (1 + NSLOT + 4 * NSLOT); // 0 .. NENC-1
        const int row = (ew & 3) * 32 + lane;          // tile row owned by this thread
        const int level0 = ew >> 2;                     // this warp takes levels level0, level0 + 2, ...
        const int etid = ew * 32 + lane;
        const GridParams &g = *gp;
        const int n_levels = (int)g.n_levels;
        const int n_dims = (int)g.n_dims;
        for (int l = etid; l < n_levels; l += 32 * NENC) enc_levels[l] = grid_level_info(g, (uint32_t)l);
        const GridCommon gc = grid_common(g);
        // all NSLOT input tiles start as zeros: the padding columns are never written again
        for (int i = etid; i < NSLOT * (T::ACT_BYTES / 16); i += 32 * NENC)
            reinterpret_cast<uint4 *>(smem + S::XBUF)[i] = make_uint4(0, 0, 0, 0);
        ptx::named_bar_sync(8, 32 * NENC);
        float xin[3] = {0.0f, 0.0f, 0.0f};
        auto fetch = [&](int tile) {
            const size_t grow = (size_t)tile * T::TM + row;
            for (int d = 0; d < 3; ++d) xin[d] = (d < n_dims && grow < batch) ? __ldg(coords + grow * n_dims + d) : 0.0f;
        };
        if (my_tiles > 0) fetch(blockIdx.x);
        for (int j = 0; j < my_tiles; ++j) {
            const int s = j % NSLOT, t = j / NSLOT;
            const int tile = blockIdx.x + j * gridDim.x;
            if (t >= 1 && !__all_sync(0xffffffffu, ptx::mbar_wait(&bars.x_empty[s], (t - 1) & 1, abort_flag))) {
                if (lane == 0) atomicExch(status, KS_TIMEOUT_PRODUCER | 0x40 | s);
                break;
            }
            uint8_t *xt = smem + S::XBUF + s * T::ACT_BYTES;
            if (STORE_ALL && j >= NSLOT) { // the store of this slot's previous tile has read the buffer
                if (etid == 0) ptx::tma_wait_group_read<NSLOT - 1>();
                ptx::named_bar_sync(8, 32 * NENC);
            }
            const bool valid = (size_t)tile * T::TM + row < batch;
            if (n_dims == 3) {
                encode_grid_rows<3>(xt, row, level0, gc, enc_levels, n_levels, table, xin, valid, fp16, T::ATOM_COLS,
                                    T::ACT_ATOM_BYTES, T::ROW_BYTES, T::CHUNKS);
            } else {
                const float x2[2] = {xin[0], xin[1]};
                encode_grid_rows<2>(xt, row, level0, gc, enc_levels, n_levels, table, x2, valid, fp16, T::ATOM_COLS,
                                    T::ACT_ATOM_BYTES, T::ROW_BYTES, T::CHUNKS);
            }
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&bars.x_full[s]);
            if (STORE_ALL) { // the encoded tile is matrix 0 of the stored activations
                ptx::named_bar_sync(8, 32 * NENC);
                if (etid == 0) {
                    for (int a = 0; a < T::KATOMS; ++a)
                        ptx::tma_store_3d(&tm_interm, xt + a * T::ACT_ATOM_BYTES, a * T::ATOM_COLS, tile * T::TM, 0);
                    ptx::tma_commit_group();
                }
            }
            if (j + 1 < my_tiles) fetch(tile + gridDim.x);
        }
        if (STORE_ALL && etid == 0) ptx::tma_wait_group<0>();
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
template <int W, int NSLOT, bool STORE_ALL, bool TMEM_A, bool B_MN, bool STREAM_W, int NENC, bool HF_, bool LIVE8>
static cudaError_t launch_variant_t(const FwdLaunch &p) {
    using T = Tile<W>;
    using S = FwdSmem<W, NSLOT, TMEM_A, STORE_ALL, STREAM_W>;
    const size_t smem = (size_t)S::WBUF + (size_t)S::weight_tiles(p.n_mat) * T::WGT_BYTES + 1024;
    if (smem > 227 * 1024 - 1024 || !S::fits_tmem) return cudaErrorInvalidConfiguration;
    auto kern = mlp_fwd_kernel<W, NSLOT, STORE_ALL, TMEM_A, B_MN, STREAM_W, NENC, HF_, LIVE8>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    const int n_tiles = (int)((p.batch + T::TM - 1) / T::TM);
    const int grid = n_tiles < p.n_sm ? n_tiles : p.n_sm;
    if (grid == 0) return cudaSuccess;
    count_launch();
    kern<<<grid, S::THREADS + 32 * NENC, smem, p.stream>>>(p.tm_x, p.tm_y, p.tm_interm, B_MN ? p.wimg : p.wimg_t, p.grid_params,
                                                           p.grid_table, p.grid_x, n_tiles, p.n_mat,
                                               p.act, p.out_act, p.write_y, p.batch, p.enc, p.status);
    return cudaGetLastError();
}

template <int W, int NSLOT, bool STORE_ALL, bool TMEM_A, bool B_MN, bool STREAM_W = false, int NENC = 0, bool LIVE8 = false>
static cudaError_t launch_variant(const FwdLaunch &p) {
    return p.fp16 ? launch_variant_t<W, NSLOT, STORE_ALL, TMEM_A, B_MN, STREAM_W, NENC, true, LIVE8>(p)
                  : launch_variant_t<W, NSLOT, STORE_ALL, TMEM_A, B_MN, STREAM_W, NENC, false, LIVE8>(p);
}

// fused hash-grid encoding: two tiles in flight (the gathers, not the GEMMs, set the pace), weights resident
template <int W> static cudaError_t launch_grid_w(const FwdLaunch &p) {
    if (p.store_all) return launch_variant<W, 2, true, false, false, false, kGridEncWarps>(p);
    return launch_variant<W, 2, false, (W >= 32), false, false, kGridEncWarps>(p);
}

template <int W> static cudaError_t launch_w(const FwdLaunch &p) {
    if (p.grid_params) return launch_grid_w<W>(p);
    // variant bit 256 (tests): stream the weights through the per-slot rings even if they would fit on chip
    const bool force_stream = (p.variant & 256) != 0;
    cudaError_t e = cudaErrorInvalidConfiguration;
    if (p.store_all) {
        if (!force_stream) {
            e = launch_variant<W, 3, true, false, false>(p);
            if (e == cudaErrorInvalidConfiguration) e = launch_variant<W, 2, true, false, false>(p);
        }
        // weights do not fit beside the tiles: per-slot weight rings
        if (e == cudaErrorInvalidConfiguration) e = launch_variant<W, 2, true, false, false, true>(p);
        if (e == cudaErrorInvalidConfiguration) e = launch_variant<W, 1, true, false, false, true>(p);
        return e;
    }
    // inference: hidden activations in tensor memory where the A operand can live there (W >= 32)
    constexpr bool TA = W >= 32;
    if (!force_stream) {
        if constexpr (W == 32) {
            if (p.live8) e = launch_variant<W, 6, false, TA, false, false, 0, true>(p);
        }
        if constexpr (W <= 32) {
            // narrow layers are pure latency chains (one or two MMAs per layer): six tiles in flight
            if (e == cudaErrorInvalidConfiguration) e = launch_variant<W, 6, false, TA, false>(p);
        }
        // measured at W = 64, batch 2^22: four tiles in flight win up to 4 hidden layers (0.170 / 0.213 ms at 2 / 4),
        // three from 6 on (0.261 vs 0.272 ms at 6, 0.337 vs 0.465 ms at 8 layers)
        if constexpr (W == 64) {
            if (e == cudaErrorInvalidConfiguration && p.live8)
                e = p.n_mat >= 7 ? launch_variant<W, 3, false, TA, false, false, 0, true>(p)
                                 : launch_variant<W, 4, false, TA, false, false, 0, true>(p);
        }
        if (e == cudaErrorInvalidConfiguration && p.n_mat >= 7) e = launch_variant<W, 3, false, TA, false>(p);
        if (e == cudaErrorInvalidConfiguration) e = launch_variant<W, 4, false, TA, false>(p);
        if (e == cudaErrorInvalidConfiguration) e = launch_variant<W, 2, false, TA, false>(p);
    }
    if (e == cudaErrorInvalidConfiguration) e = launch_variant<W, 2, false, TA, false, true>(p);
    if (e == cudaErrorInvalidConfiguration) e = launch_variant<W, 1, false, TA, false, true>(p);
    return e;
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
