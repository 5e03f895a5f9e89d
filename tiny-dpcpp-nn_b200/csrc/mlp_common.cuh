// Shared definitions of the fused-MLP kernels: tile geometry, the swizzled shared-memory
// layout that both TMA and the tcgen05 descriptors agree on, and activation helpers.
#pragma once
#include "mlp_launch.h"
#include "umma.cuh"

namespace tnn {

// Same enumerator order as the reference's `enum class Activation` (include/common/common.h:28-38).
enum Activation : int {
    ACT_RELU = 0,
    ACT_LEAKY_RELU = 1,
    ACT_EXPONENTIAL = 2,
    ACT_SINE = 3,
    ACT_SIGMOID = 4,
    ACT_SQUAREPLUS = 5,
    ACT_SOFTPLUS = 6,
    ACT_TANH = 7,
    ACT_NONE = 8,
};

// Error words written by a kernel that gave up on a bounded wait.
enum KernelStatus : int {
    KS_OK = 0,
    KS_TIMEOUT_PRODUCER = 0x100,
    KS_TIMEOUT_MMA = 0x200,
    KS_TIMEOUT_EPILOGUE = 0x300,
    KS_TIMEOUT_WEIGHTS = 0x400,
};

// Geometry of one batch tile (128 rows, the UMMA M) of a width-W network.
//
// A tile of `rows` x W bf16 is kept in shared memory as KATOMS column blocks ("atoms") of
// `rows` x ATOM_COLS; inside an atom a row occupies ROW_BYTES contiguous bytes and its
// 16-byte chunks are XOR-swizzled with the row index, exactly the pattern TMA writes for
// CU_TENSOR_MAP_SWIZZLE_{32,64,128}B and the pattern a UMMA descriptor of the matching
// swizzle mode reads.  The same bytes can be consumed
//   * as a K-major operand  (MMA row = stored row,  K = stored column), or
//   * as an MN-major operand (MMA row = stored column, K = stored row).
template <int W> struct Tile {
    static_assert(W == 16 || W == 32 || W == 64 || W == 128, "width must be 16, 32, 64 or 128");
    static constexpr int TM = 128;
    static constexpr int ROW_BYTES = (2 * W < 128) ? 2 * W : 128;
    static constexpr int KATOMS = (2 * W) / ROW_BYTES;
    static constexpr int ATOM_COLS = ROW_BYTES / 2;
    static constexpr int CHUNKS = ROW_BYTES / 16;
    static constexpr int ACT_ATOM_BYTES = TM * ROW_BYTES;
    static constexpr int ACT_BYTES = ACT_ATOM_BYTES * KATOMS; // 128 x W bf16
    static constexpr int WGT_ATOM_BYTES = W * ROW_BYTES;
    static constexpr int WGT_BYTES = WGT_ATOM_BYTES * KATOMS; // W x W bf16
    static constexpr uint32_t SWZ = ptx::swizzle_code(ROW_BYTES);
    static constexpr int SBO = 8 * ROW_BYTES;
    static constexpr int KSTEPS = W / 16; // one tcgen05.mma consumes K = 16 bf16

    // byte offset of the 16-byte chunk `chunk` (0..CHUNKS-1) of row `r` inside an atom
    __host__ __device__ static constexpr int chunk_off(int r, int chunk) {
        return r * ROW_BYTES + ((chunk ^ (((r * ROW_BYTES) >> 7) & (CHUNKS - 1))) << 4);
    }
    // byte offset of element (r, c) of a `rows`-row tile
    __host__ __device__ static constexpr int elem_off(int r, int c, int atom_bytes) {
        return (c / ATOM_COLS) * atom_bytes + chunk_off(r, (c % ATOM_COLS) / 8) + (c % 8) * 2;
    }

    // Descriptor arithmetic.  A descriptor's low 14 bits hold (address >> 4), so stepping to the next
    // k-step or the next buffer is a plain 64-bit add of a compile-time constant to a base descriptor;
    // the MMA issuer is a single thread, every instruction it saves shortens the layer-to-layer chain.
    static constexpr int KPA = ATOM_COLS / 16;              // k-steps inside one K-major atom
    static constexpr uint32_t K_STEP = 2;                    // 32 bytes: one k-step inside a K-major row
    static constexpr uint32_t MN_STEP = ROW_BYTES;           // 16 stored rows: one k-step of an MN-major operand
    static constexpr uint32_t ACT_UNITS = ACT_BYTES >> 4;    // one activation tile, in descriptor units
    static constexpr uint32_t WGT_UNITS = WGT_BYTES >> 4;
    __device__ static uint64_t kdesc_base(uint32_t base) { return ptx::make_smem_desc(base, 16, SBO, SWZ); }
    __device__ static uint64_t mndesc_base(uint32_t base, int atom_bytes) {
        return ptx::make_smem_desc(base, atom_bytes, SBO, SWZ);
    }
    // D[128 x W] = A[128 x W] * B, A K-major in an activation tile, B a weight tile (K- or MN-major).
    template <bool B_MN> __device__ static void issue_chain(uint32_t d_tmem, uint64_t a_base, uint64_t w_base,
                                                            uint32_t idesc) {
#pragma unroll
        for (int at = 0; at < KATOMS; ++at) {
            const uint64_t a0 = a_base + (uint64_t)(at * (ACT_ATOM_BYTES >> 4));
            const uint64_t b0 = w_base + (uint64_t)(B_MN ? at * KPA * MN_STEP : at * (WGT_ATOM_BYTES >> 4));
#pragma unroll
            for (int k = 0; k < KPA; ++k)
                ptx::mma_ss(d_tmem, a0 + (uint64_t)(k * K_STEP), b0 + (uint64_t)(k * (B_MN ? MN_STEP : K_STEP)), idesc,
                            (at > 0 || k > 0) ? 1u : 0u);
        }
    }
    // same with the A operand in tensor memory (two bf16 per 32-bit column: 8 columns per k-step)
    template <bool B_MN> __device__ static void issue_chain_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t w_base,
                                                               uint32_t idesc) {
#pragma unroll
        for (int at = 0; at < KATOMS; ++at) {
            const uint64_t b0 = w_base + (uint64_t)(B_MN ? at * KPA * MN_STEP : at * (WGT_ATOM_BYTES >> 4));
#pragma unroll
            for (int k = 0; k < KPA; ++k)
                ptx::mma_ts(d_tmem, a_tmem + (at * KPA + k) * 8, b0 + (uint64_t)(k * (B_MN ? MN_STEP : K_STEP)), idesc,
                            (at > 0 || k > 0) ? 1u : 0u);
        }
    }
    // D[M x W] (+)= A^T B over the 128 stored rows of two activation tiles, both MN-major.
    __device__ static void issue_outer(uint32_t d_tmem, uint64_t a_base, uint64_t b_base, uint32_t idesc,
                                       uint32_t accumulate) {
#pragma unroll
        for (int k = 0; k < TM / 16; ++k)
            ptx::mma_ss(d_tmem, a_base + (uint64_t)(k * MN_STEP), b_base + (uint64_t)(k * MN_STEP), idesc,
                        (k > 0) ? 1u : accumulate);
    }
};

// Network input produced inside the kernel from fp32 coordinates: the identity encoding
// (include/encodings/identity.h:63-77: out[i, j] = j < n_in ? x * scale + offset : 1) folded into the first-layer
// load, so the batch x W bf16 matrix the reference materialises between the two modules never exists.
// (struct EncodedInput: mlp_launch.h)

// Whole warp: fill `n_tiles` consecutive input tiles with bf16 ones (the padding value of the encoding).
template <int W> __device__ __forceinline__ void fill_tiles_with_ones(uint8_t *tiles, int n_tiles, int lane, int fp16) {
    const uint32_t one2 = fp16 ? 0x3C003C00u : 0x3F803F80u; // two 1.0 in fp16 / bf16
    const uint4 ones = make_uint4(one2, one2, one2, one2);
    for (int i = lane; i < n_tiles * (Tile<W>::ACT_BYTES / 16); i += 32) reinterpret_cast<uint4 *>(tiles)[i] = ones;
}
// Whole warp: produces the encoded columns (the first one or two 16-byte chunks of every row; the rest of the tile
// keeps its ones) of one input tile.  fetch() starts the global loads of a tile's coordinates into registers - issued
// a tile ahead, so that their latency hides under the tile being consumed - and store() converts and writes them.
// Rows past the end of the batch become zeros.  Lane i owns rows i, i + 32, i + 64, i + 96.
template <int W> struct IdentityTileEncoder {
    using T = Tile<W>;
    static constexpr int kRegInputs = 4; // coordinates per row kept in registers between fetch and store
    const EncodedInput e;
    const size_t batch;
    const int lane;
    int fp16 = 0;
    size_t row0 = 0;
    float v[4][kRegInputs];
    __device__ IdentityTileEncoder(const EncodedInput &enc, size_t batch_, int lane_, int fp16_ = 0)
        : e(enc), batch(batch_), lane(lane_), fp16(fp16_) {}
    __device__ __forceinline__ void fetch(size_t first_row) {
        row0 = first_row;
        if (e.n_in > kRegInputs) return; // wide inputs are read in store()
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const size_t grow = row0 + lane + 32 * i;
#pragma unroll
            for (int j = 0; j < kRegInputs; ++j)
                v[i][j] = (j < e.n_in && grow < batch) ? __ldg(e.x + grow * e.n_in + j) : 0.0f;
        }
    }
    __device__ __forceinline__ uint4 pack8(const float (&o)[8]) const {
        return fp16 ? make_uint4(ptx::pack_f16x2(o[0], o[1]), ptx::pack_f16x2(o[2], o[3]), ptx::pack_f16x2(o[4], o[5]),
                                 ptx::pack_f16x2(o[6], o[7]))
                    : make_uint4(ptx::pack_bf16x2(o[0], o[1]), ptx::pack_bf16x2(o[2], o[3]), ptx::pack_bf16x2(o[4], o[5]),
                                 ptx::pack_bf16x2(o[6], o[7]));
    }
    __device__ __forceinline__ void store(uint8_t *xtile) {
        if (e.n_in <= kRegInputs) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = lane + 32 * i;
                const bool valid = row0 + r < batch;
                float o[8];
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    o[j] = (j < kRegInputs && j < e.n_in) ? (valid ? __fadd_rn(__fmul_rn(v[i][j < kRegInputs ? j : 0], e.scale), e.offset) : 0.0f)
                                                        : 1.0f;
                *reinterpret_cast<uint4 *>(xtile + T::chunk_off(r, 0)) = pack8(o);
            }
            return;
        }
        const int n_chunks = (e.n_in + 7) >> 3;
        for (int r = lane; r < T::TM; r += 32) {
            const size_t grow = row0 + r;
            const bool valid = grow < batch;
            for (int c = 0; c < n_chunks; ++c) {
                float o[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int col = c * 8 + j;
                    o[j] = col < e.n_in ? (valid ? __fadd_rn(__fmul_rn(__ldg(e.x + grow * e.n_in + col), e.scale), e.offset) : 0.0f)
                                        : 1.0f;
                }
                *reinterpret_cast<uint4 *>(xtile + T::chunk_off(r, c)) = pack8(o);
            }
        }
    }
};

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + __expf(-x)); }

// Compile-time activation / element-type tags.  The epilogues select the activation (and whether the network
// computes in bf16 or fp16) ONCE per tile step with a uniform branch and then run a straight-line body specialised
// for it: a run-time `act` inside the per-element code makes the compiler evaluate every activation (including the
// exp and the division of the sigmoid) for every element and select afterwards, which multiplied the epilogue's length.
template <int A, bool H = false> struct ActTag {
    static constexpr int value = A;
    static constexpr bool half = H;
};
template <class F> __device__ __forceinline__ void dispatch_act(int act, int fp16, F &&f) {
    if (!fp16) {
        if (act == ACT_RELU)
            f(ActTag<ACT_RELU, false>{});
        else if (act == ACT_SIGMOID)
            f(ActTag<ACT_SIGMOID, false>{});
        else
            f(ActTag<ACT_NONE, false>{});
    } else {
        if (act == ACT_RELU)
            f(ActTag<ACT_RELU, true>{});
        else if (act == ACT_SIGMOID)
            f(ActTag<ACT_SIGMOID, true>{});
        else
            f(ActTag<ACT_NONE, true>{});
    }
}
// Element type fixed at compile time (the kernels are instantiated per type): dispatch over the activation only.
template <bool H, class F> __device__ __forceinline__ void dispatch_act_t(int act, F &&f) {
    if (act == ACT_RELU)
        f(ActTag<ACT_RELU, H>{});
    else if (act == ACT_SIGMOID)
        f(ActTag<ACT_SIGMOID, H>{});
    else
        f(ActTag<ACT_NONE, H>{});
}
template <int A, bool H = false> __device__ __forceinline__ uint32_t act_pack_t(float lo, float hi) {
    if constexpr (A == ACT_RELU) return ptx::pack2_relu<H>(lo, hi);
    if constexpr (A == ACT_SIGMOID) return ptx::pack2<H>(1.0f / (1.0f + __expf(-lo)), 1.0f / (1.0f + __expf(-hi)));
    return ptx::pack2<H>(lo, hi);
}
template <int A, bool H = false> __device__ __forceinline__ uint32_t act_bwd_pack_t(float lo, float hi, uint32_t fwd) {
    if constexpr (A == ACT_RELU) {
        // keep the gradient where the stored activation is > 0: one packed compare gives 0xffff per kept half
        if constexpr (H) {
            __half2 f2;
            memcpy(&f2, &fwd, sizeof(f2));
            return ptx::pack2<H>(lo, hi) & __hgt2_mask(f2, __floats2half2_rn(0.0f, 0.0f));
        } else {
            __nv_bfloat162 f2;
            memcpy(&f2, &fwd, sizeof(f2));
            return ptx::pack2<H>(lo, hi) & __hgt2_mask(f2, __floats2bfloat162_rn(0.0f, 0.0f));
        }
    } else if constexpr (A == ACT_SIGMOID) {
        const float sl = ptx::lo_f32<H>(fwd), sh = ptx::hi_f32<H>(fwd);
        lo *= sl * (1.0f - sl);
        hi *= sh * (1.0f - sh);
    }
    return ptx::pack2<H>(lo, hi);
}

// Forward activation on two fp32 accumulators, rounded to a bf16 pair.  The reference rounds
// to the storage type first and then clamps (kernel_esimd.h:443-458); max(bf16(x), 0) and
// bf16(max(x, 0)) are the same value.  Sigmoid is evaluated in fp32 and then rounded.
__device__ __forceinline__ uint32_t act_pack(int act, float lo, float hi) {
    if (act == ACT_RELU) return ptx::pack_bf16x2_relu(lo, hi);
    if (act == ACT_SIGMOID) return ptx::pack_bf16x2(sigmoidf_(lo), sigmoidf_(hi));
    return ptx::pack_bf16x2(lo, hi);
}

// Backward activation (kernel_esimd.h:460-487): `fwd` holds the two stored forward
// activations of the same elements.  ReLU zeroes where the stored activation is <= 0;
// sigmoid multiplies by s (1 - s) in fp32.
__device__ __forceinline__ uint32_t act_bwd_pack(int act, float lo, float hi, uint32_t fwd) {
    if (act == ACT_RELU) {
        if (!(ptx::bf16lo_to_f32(fwd) > 0.0f)) lo = 0.0f;
        if (!(ptx::bf16hi_to_f32(fwd) > 0.0f)) hi = 0.0f;
    } else if (act == ACT_SIGMOID) {
        const float sl = ptx::bf16lo_to_f32(fwd), sh = ptx::bf16hi_to_f32(fwd);
        lo *= sl * (1.0f - sl);
        hi *= sh * (1.0f - sh);
    }
    return ptx::pack_bf16x2(lo, hi);
}

} // namespace tnn
