// Atomic-free, deterministic hash-grid backward (parameter gradients): a segmented reduction.
//
// The reference scatters w_c * dL/dy into the gradient table with fp32 atomics
// (include/encodings/grid.h:137-245), so its sums have no fixed order.  Here the same sum is
// evaluated without a single atomic, as a segmented reduction with a fixed order, in three kernels per group of
// levels.  It is the third backward mode of the C ABI (deterministic = 2): bit-reproducible like the fixed-point
// reductions of grid_bwd_fixed.cu but about three times slower at the benchmark grid (every level is a random
// scatter of 8.4 M contributions into at most 2^19 entries - the 1.6 GB of (entry, value) records have to be written
// and read back before any sum can be formed), so it is not what the trainer uses.
//
//   partition  every CTA takes a tile of 16384 consecutive contributions (sample-major, corner-minor)
//              of one level, computes their table indices and weighted gradients, and writes them
//              *stably sorted by bucket* (a bucket = 2^shift consecutive table entries) into the
//              tile's own record area, together with the tile's bucket offsets.  Ranks come from
//              warp match/ballot arithmetic and per-warp counters - no atomics, order preserved.
//   accumulate one warp per (bucket, tile group): walks the bucket's segments of its tiles and adds the
//              records, 32 per round, into a warp-private shared-memory accumulator; records of one
//              round that hit the same entry are ranked by lane and added one after the other, so
//              every entry sees its additions in an order fixed by the record layout.  The result
//              goes straight to the gradient table, or to a per-group partial table when coarse
//              levels are split over several groups for parallelism.
//   combine    adds the per-group partial tables in group order.
//
// The summation order per table entry depends only on the record layout (itself a pure function of
// the inputs), never on scheduling, so two runs give identical bits.
#include "grid.h"
#include "elementwise.h"
#include "grid_device.cuh"

#include <algorithm>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <vector>

namespace tnn {

namespace {

constexpr int kTile = 16384;     // contributions per partition CTA
constexpr int kWarpsA = 8;       // warps of a partition CTA
constexpr int kRounds = kTile / (kWarpsA * 32);
constexpr int kMaxBuckets = 1024; // per level; keeps the per-warp counters small enough for 4 CTAs per SM
constexpr int kTargetUnits = 4096; // accumulate warps wanted per level
constexpr int kPassLevels = 16;  // levels handled by one launch triple
constexpr int kWarpsB = 8;       // warps (= units) of an accumulate CTA
constexpr size_t kScratchCap = (size_t)1 << 30;

struct DetLevel {
    uint32_t level;
    uint32_t shift;           // log2(entries per bucket)
    uint32_t n_buckets;
    uint32_t groups;          // tile groups (1 = write the gradient table directly)
    uint32_t tiles_per_group;
    uint32_t T;               // table entries of the level
    uint32_t unit_start;      // first accumulate unit of this level
    uint32_t pad;
    size_t rec_off, offs_off, part_off; // byte offsets into the scratch buffer
};

struct DetPass {
    int n_levels;
    uint32_t n_tiles;
    uint32_t total_units;
    uint32_t corner_shift;    // log2(contributions per sample)
    uint64_t n_contrib;       // batch * corners
    DetLevel lv[kPassLevels];
};

struct LevelPlan {
    uint32_t shift, n_buckets, groups, tiles_per_group;
    size_t rec_bytes, offs_bytes, part_bytes;
};

LevelPlan plan_level(uint32_t T, uint32_t F, uint32_t n_tiles) {
    LevelPlan lp{};
    lp.shift = 7;
    while (((T + (1u << lp.shift) - 1) >> lp.shift) > (uint32_t)kMaxBuckets) ++lp.shift;
    lp.n_buckets = (T + (1u << lp.shift) - 1) >> lp.shift;
    uint32_t g = (kTargetUnits + lp.n_buckets - 1) / lp.n_buckets;
    g = std::max(1u, std::min(g, n_tiles));
    lp.tiles_per_group = (n_tiles + g - 1) / g;
    lp.groups = (n_tiles + lp.tiles_per_group - 1) / lp.tiles_per_group;
    lp.rec_bytes = (size_t)n_tiles * kTile * (4 + 4 * (size_t)F);
    lp.offs_bytes = (size_t)n_tiles * (lp.n_buckets + 1) * 4;
    lp.part_bytes = lp.groups > 1 ? (size_t)lp.groups * T * F * 4 : 0;
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    lp.rec_bytes = up(lp.rec_bytes), lp.offs_bytes = up(lp.offs_bytes), lp.part_bytes = up(lp.part_bytes);
    return lp;
}

uint32_t corners_of(const GridParams &p) { return p.interpolation == INTERP_NEAREST ? 1u : (1u << p.n_dims); }

// table index and weighted gradient of contribution c of one level
template <int D, int F, typename DyT>
__device__ __forceinline__ bool contribution(const GridParams &p, uint32_t level, uint32_t hsize, uint32_t res,
                                             float scale, uint64_t c, uint64_t n_contrib, uint32_t corner_shift,
                                             const float *__restrict__ x, const DyT *__restrict__ dy, uint32_t &index,
                                             float (&val)[F]) {
    if (c >= n_contrib) return false;
    const uint64_t i = c >> corner_shift;
    const uint32_t corner = (uint32_t)c & ((1u << corner_shift) - 1u);
    float w[D], xin[D];
    uint32_t g[D];
#pragma unroll
    for (int d = 0; d < D; ++d) xin[d] = __ldg(x + i * D + d);
    grid_pos<D>(xin, scale, p.interpolation, w, g);
    float weight = 1.0f;
    if (corner_shift > 0) {
#pragma unroll
        for (int d = 0; d < D; ++d) {
            if ((corner & (1u << d)) == 0) {
                weight = __fmul_rn(weight, __fsub_rn(1.0f, w[d]));
            } else {
                weight = __fmul_rn(weight, w[d]);
                g[d] += 1u;
            }
        }
    }
    index = grid_index<D>(p.grid_type, p.hash_type, hsize, res, g);
#pragma unroll
    for (int f = 0; f < F; ++f) val[f] = __fmul_rn(weight, (float)dy[i * p.padded_width + level * F + f]);
    return true;
}

template <int D, int F, typename DyT>
__global__ void __launch_bounds__(kWarpsA * 32)
grid_bwd_partition_kernel(const GridParams p, const DetPass ps, const float *__restrict__ x,
                          const DyT *__restrict__ dy, uint8_t *__restrict__ scratch) {
    extern __shared__ uint8_t sm_raw[];
    const DetLevel lv = ps.lv[blockIdx.y];
    const uint32_t NB = lv.n_buckets; // bucket NB collects the padding of the last tile
    uint16_t *cnt = reinterpret_cast<uint16_t *>(sm_raw);                           // [kWarpsA][NB + 1]
    const size_t cnt_bytes = ((size_t)kWarpsA * (NB + 1) * 2 + 15) & ~(size_t)15;
    uint32_t *seg = reinterpret_cast<uint32_t *>(sm_raw + cnt_bytes);                // [NB + 2]
    const size_t seg_bytes = ((size_t)(NB + 2) * 4 + 15) & ~(size_t)15;
    uint16_t *ranks = reinterpret_cast<uint16_t *>(sm_raw + cnt_bytes + seg_bytes);  // [kRounds][threads]
    __shared__ uint32_t chunk_sum[kWarpsA * 32];

    const uint32_t tile = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t hsize = p.offsets[lv.level + 1] - p.offsets[lv.level];
    const uint32_t res = p.resolution[lv.level];
    const float scale = p.scale[lv.level];
    const uint64_t c0 = (uint64_t)tile * kTile + (uint64_t)warp * (kTile / kWarpsA);

    for (uint32_t i = threadIdx.x; i < kWarpsA * (NB + 1); i += blockDim.x) cnt[i] = 0;
    __syncthreads();

    // ---- phase 1: stable rank of every contribution among the equal-bucket ones of its warp
    uint16_t *wcnt = cnt + (size_t)warp * (NB + 1);
#pragma unroll 1
    for (int r = 0; r < kRounds; ++r) {
        uint32_t index;
        float val[F];
        const bool valid = contribution<D, F, DyT>(p, lv.level, hsize, res, scale, c0 + r * 32 + lane, ps.n_contrib,
                                                    ps.corner_shift, x, dy, index, val);
        const uint32_t bucket = valid ? (index >> lv.shift) : NB;
        const uint32_t peers = __match_any_sync(0xffffffffu, bucket);
        const uint32_t below = __popc(peers & ((1u << lane) - 1u));
        const int leader = __ffs(peers) - 1;
        uint32_t old = 0;
        if (lane == leader) {
            old = wcnt[bucket];
            wcnt[bucket] = (uint16_t)(old + __popc(peers));
        }
        old = __shfl_sync(0xffffffffu, old, leader);
        ranks[r * (kWarpsA * 32) + threadIdx.x] = (uint16_t)(old + below);
        __syncwarp();
    }
    __syncthreads();

    // ---- phase 2: per bucket, exclusive prefix over the warps; then exclusive scan over the buckets
    const uint32_t n_b = NB + 1;
    const uint32_t per_thread = (n_b + blockDim.x - 1) / blockDim.x;
    const uint32_t b_lo = threadIdx.x * per_thread;
    const uint32_t b_hi = min(b_lo + per_thread, n_b);
    uint32_t local = 0;
    for (uint32_t b = b_lo; b < b_hi; ++b) {
        uint32_t running = 0;
        for (int w = 0; w < kWarpsA; ++w) {
            const uint32_t t = cnt[(size_t)w * n_b + b];
            cnt[(size_t)w * n_b + b] = (uint16_t)running;
            running += t;
        }
        seg[b] = running;
        local += running;
    }
    chunk_sum[threadIdx.x] = local;
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t run = 0;
        for (int i = 0; i < kWarpsA * 32; ++i) {
            const uint32_t t = chunk_sum[i];
            chunk_sum[i] = run;
            run += t;
        }
    }
    __syncthreads();
    {
        uint32_t run = chunk_sum[threadIdx.x];
        for (uint32_t b = b_lo; b < b_hi; ++b) {
            const uint32_t t = seg[b];
            seg[b] = run;
            run += t;
        }
    }
    __syncthreads();
    uint32_t *offs = reinterpret_cast<uint32_t *>(scratch + lv.offs_off) + (size_t)tile * n_b;
    for (uint32_t b = threadIdx.x; b < n_b; b += blockDim.x) offs[b] = seg[b];

    // ---- phase 3: recompute and write every record to its sorted position inside the tile's area
    // a record = {entry index inside its bucket, F weighted gradients}, stored contiguously
    uint32_t *rec = reinterpret_cast<uint32_t *>(scratch + lv.rec_off);
#pragma unroll 1
    for (int r = 0; r < kRounds; ++r) {
        uint32_t index;
        float val[F];
        const bool valid = contribution<D, F, DyT>(p, lv.level, hsize, res, scale, c0 + r * 32 + lane, ps.n_contrib,
                                                    ps.corner_shift, x, dy, index, val);
        if (!valid) continue;
        const uint32_t bucket = index >> lv.shift;
        const uint32_t rk = ranks[r * (kWarpsA * 32) + threadIdx.x];
        const size_t pos = (size_t)tile * kTile + seg[bucket] + wcnt[bucket] + rk;
        uint32_t *r_out = rec + pos * (1 + F);
        r_out[0] = index & ((1u << lv.shift) - 1u);
#pragma unroll
        for (int f = 0; f < F; ++f) r_out[1 + f] = __float_as_uint(val[f]);
    }
}

template <int F>
__global__ void __launch_bounds__(kWarpsB * 32)
grid_bwd_accumulate_kernel(const GridParams p, const DetPass ps, const uint8_t *__restrict__ scratch,
                           float *__restrict__ grads, uint8_t *__restrict__ scratch_out) {
    extern __shared__ float acc_all[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t unit = blockIdx.x * kWarpsB + warp;
    if (unit >= ps.total_units) return;
    int li = 0;
    while (li + 1 < ps.n_levels && unit >= ps.lv[li + 1].unit_start) ++li;
    const DetLevel lv = ps.lv[li];
    const uint32_t local = unit - lv.unit_start;
    const uint32_t b = local % lv.n_buckets;
    const uint32_t g = local / lv.n_buckets;
    const uint32_t E = 1u << lv.shift;
    // the accumulator stride is the largest bucket of the pass so every warp has room
    uint32_t e_max = 0;
    for (int i = 0; i < ps.n_levels; ++i) e_max = max(e_max, 1u << ps.lv[i].shift);
    float *acc = acc_all + (size_t)warp * e_max * F;
    for (uint32_t i = lane; i < E * F; i += 32) acc[i] = 0.0f;
    __syncwarp();

    const uint32_t n_b = lv.n_buckets + 1;
    const uint32_t *offs = reinterpret_cast<const uint32_t *>(scratch + lv.offs_off);
    const uint32_t *rec = reinterpret_cast<const uint32_t *>(scratch + lv.rec_off);
    const uint32_t t0 = g * lv.tiles_per_group;
    const uint32_t t1 = min(t0 + lv.tiles_per_group, ps.n_tiles);

    // One round adds up to 32 records (one per lane) into the accumulator.  Lanes whose records hit the
    // same entry are ranked by lane and take turns, so the additions into an entry happen in lane order;
    // lanes with distinct entries add at once.  The order is a fixed function of the record layout.
    auto add_round = [&](bool active, uint32_t m, const float (&v)[F]) {
        const uint32_t key = active ? m : (0x80000000u | (uint32_t)lane);
        const uint32_t peers = __match_any_sync(0xffffffffu, key);
        const uint32_t rank = __popc(peers & ((1u << lane) - 1u));
        const uint32_t max_rank = __reduce_max_sync(0xffffffffu, active ? rank : 0u);
        for (uint32_t r = 0; r <= max_rank; ++r) {
            if (active && rank == r) {
#pragma unroll
                for (int f = 0; f < F; ++f) acc[m * F + f] += v[f];
            }
            __syncwarp();
        }
    };

    constexpr int R = 8; // records of its segment every lane pre-loads
    for (uint32_t tb = t0; tb < t1; tb += 32) {
        // every lane looks up the segment of one tile and pre-loads its first R records
        const uint32_t my_tile = tb + lane;
        uint32_t s = 0, n = 0;
        if (my_tile < t1) {
            s = __ldg(offs + (size_t)my_tile * n_b + b);
            n = __ldg(offs + (size_t)my_tile * n_b + b + 1) - s;
        }
        uint32_t mr[R];
        float vr[R][F];
        const uint32_t *seg_rec = rec + ((size_t)my_tile * kTile + s) * (1 + F);
#pragma unroll
        for (int k = 0; k < R; ++k) {
            mr[k] = 0;
#pragma unroll
            for (int f = 0; f < F; ++f) vr[k][f] = 0.0f;
            if ((uint32_t)k < n) {
                mr[k] = __ldg(seg_rec + k * (1 + F));
#pragma unroll
                for (int f = 0; f < F; ++f) vr[k][f] = __uint_as_float(__ldg(seg_rec + k * (1 + F) + 1 + f));
            }
        }
        const uint32_t n_max = __reduce_max_sync(0xffffffffu, n);
#pragma unroll
        for (int k = 0; k < R; ++k)
            if ((uint32_t)k < n_max) add_round((uint32_t)k < n, mr[k], vr[k]); // k-th record of each segment, in tile order
        if (n_max > (uint32_t)R) {
            // long segments (coarse levels): stream the rest of each, 32 records per round
            const uint32_t tiles_here = min(32u, t1 - tb);
            for (uint32_t t = 0; t < tiles_here; ++t) {
                const uint32_t nt = __shfl_sync(0xffffffffu, n, t);
                if (nt <= (uint32_t)R) continue;
                const uint32_t st = __shfl_sync(0xffffffffu, s, t);
                const uint32_t *trec = rec + (size_t)(tb + t) * kTile * (1 + F);
                for (uint32_t i = st + R; i < st + nt; i += 32) {
                    const uint32_t idx = i + lane;
                    const bool act = idx < st + nt;
                    uint32_t mm = 0;
                    float vv[F];
#pragma unroll
                    for (int f = 0; f < F; ++f) vv[f] = 0.0f;
                    if (act) {
                        mm = __ldg(trec + (size_t)idx * (1 + F));
#pragma unroll
                        for (int f = 0; f < F; ++f) vv[f] = __uint_as_float(__ldg(trec + (size_t)idx * (1 + F) + 1 + f));
                    }
                    add_round(act, mm, vv);
                }
            }
        }
    }
    __syncwarp();
    float *dst = lv.groups > 1 ? reinterpret_cast<float *>(scratch_out + lv.part_off) + (size_t)g * lv.T * F
                               : grads + (size_t)p.offsets[lv.level] * F;
    for (uint32_t i = lane; i < E * F; i += 32) {
        const uint32_t entry = b * E + i / F;
        if (entry < lv.T) dst[(size_t)entry * F + (i % F)] = acc[i];
    }
}

__global__ void grid_bwd_combine_kernel(const GridParams p, const DetPass ps, const uint8_t *__restrict__ scratch,
                                        float *__restrict__ grads) {
    const DetLevel lv = ps.lv[blockIdx.y];
    if (lv.groups <= 1) return;
    const uint32_t F = p.features_per_level;
    const size_t n = (size_t)lv.T * F;
    const float *part = reinterpret_cast<const float *>(scratch + lv.part_off);
    float *dst = grads + (size_t)p.offsets[lv.level] * F;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float s = 0.0f;
        for (uint32_t g = 0; g < lv.groups; ++g) s += part[(size_t)g * n + i];
        dst[i] = s;
    }
}

struct PassLayout {
    size_t slot_bytes;
    int levels_per_pass;
};

PassLayout layout_for(const GridParams &p, size_t batch) {
    const uint32_t corners = corners_of(p);
    const uint64_t n_contrib = (uint64_t)batch * corners;
    const uint32_t n_tiles = (uint32_t)((n_contrib + kTile - 1) / kTile);
    size_t slot = 0;
    for (uint32_t l = 0; l < p.n_levels; ++l) {
        const LevelPlan lp = plan_level(p.offsets[l + 1] - p.offsets[l], p.features_per_level, n_tiles);
        slot = std::max(slot, lp.rec_bytes + lp.offs_bytes + lp.part_bytes);
    }
    int per_pass = (int)std::max<size_t>(1, std::min<size_t>(kScratchCap / std::max<size_t>(slot, 1), kPassLevels));
    per_pass = std::min<int>(per_pass, (int)p.n_levels);
    return {slot, per_pass};
}

template <int D, int F>
cudaError_t run_det(const GridParams &p, const float *x, const void *dy, int dy_dtype, float *grads, size_t batch,
                    void *scratch, size_t scratch_bytes, cudaStream_t stream) {
    const PassLayout lay = layout_for(p, batch);
    if (scratch_bytes < lay.slot_bytes * lay.levels_per_pass) return cudaErrorInvalidValue;
    const uint32_t corners = corners_of(p);
    const uint64_t n_contrib = (uint64_t)batch * corners;
    const uint32_t n_tiles = (uint32_t)((n_contrib + kTile - 1) / kTile);
    const float max_level = (p.max_level * (float)p.n_features) / (float)F;
    uint8_t *sc = reinterpret_cast<uint8_t *>(scratch);

    // levels switched off by max_level keep a zero gradient (grid.h:155)
    std::vector<uint32_t> active;
    for (uint32_t l = 0; l < p.n_levels; ++l) {
        if ((float)l >= max_level + 1e-3f) {
            const size_t off = (size_t)p.offsets[l] * F, n = (size_t)(p.offsets[l + 1] - p.offsets[l]) * F;
            cudaError_t e = cudaMemsetAsync(grads + off, 0, n * sizeof(float), stream);
            if (e != cudaSuccess) return e;
        } else {
            active.push_back(l);
        }
    }
    for (size_t first = 0; first < active.size(); first += lay.levels_per_pass) {
        DetPass ps{};
        ps.n_levels = (int)std::min<size_t>(lay.levels_per_pass, active.size() - first);
        ps.n_tiles = n_tiles;
        ps.corner_shift = (p.interpolation == INTERP_NEAREST) ? 0u : p.n_dims;
        ps.n_contrib = n_contrib;
        uint32_t units = 0, nb_max = 0, e_max = 0;
        bool any_groups = false;
        uint32_t t_max = 0;
        for (int i = 0; i < ps.n_levels; ++i) {
            const uint32_t l = active[first + i];
            const uint32_t T = p.offsets[l + 1] - p.offsets[l];
            const LevelPlan lp = plan_level(T, F, n_tiles);
            DetLevel &d = ps.lv[i];
            d.level = l, d.shift = lp.shift, d.n_buckets = lp.n_buckets, d.groups = lp.groups;
            d.tiles_per_group = lp.tiles_per_group, d.T = T, d.unit_start = units;
            d.rec_off = (size_t)i * lay.slot_bytes;
            d.offs_off = d.rec_off + lp.rec_bytes;
            d.part_off = d.offs_off + lp.offs_bytes;
            units += lp.n_buckets * lp.groups;
            nb_max = std::max(nb_max, lp.n_buckets);
            e_max = std::max(e_max, 1u << lp.shift);
            any_groups |= lp.groups > 1;
            t_max = std::max(t_max, T);
        }
        ps.total_units = units;
        const size_t smem_a = (((size_t)kWarpsA * (nb_max + 1) * 2 + 15) & ~(size_t)15) +
                              (((size_t)(nb_max + 2) * 4 + 15) & ~(size_t)15) + (size_t)kTile * 2;
        const size_t smem_b = (size_t)kWarpsB * e_max * F * sizeof(float);
        if (smem_a > 200 * 1024 || smem_b > 200 * 1024) return cudaErrorInvalidConfiguration;
        dim3 grid_a(n_tiles, ps.n_levels);
        cudaError_t e;
        count_launch(any_groups ? 3 : 2);
        if (dy_dtype == 0) {
            auto k = grid_bwd_partition_kernel<D, F, __nv_bfloat16>;
            if ((e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_a)) != cudaSuccess) return e;
            k<<<grid_a, kWarpsA * 32, smem_a, stream>>>(p, ps, x, (const __nv_bfloat16 *)dy, sc);
        } else if (dy_dtype == 1) {
            auto k = grid_bwd_partition_kernel<D, F, __half>;
            if ((e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_a)) != cudaSuccess) return e;
            k<<<grid_a, kWarpsA * 32, smem_a, stream>>>(p, ps, x, (const __half *)dy, sc);
        } else {
            auto k = grid_bwd_partition_kernel<D, F, float>;
            if ((e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_a)) != cudaSuccess) return e;
            k<<<grid_a, kWarpsA * 32, smem_a, stream>>>(p, ps, x, (const float *)dy, sc);
        }
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
        auto kb = grid_bwd_accumulate_kernel<F>;
        if ((e = cudaFuncSetAttribute(kb, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_b)) != cudaSuccess) return e;
        kb<<<(units + kWarpsB - 1) / kWarpsB, kWarpsB * 32, smem_b, stream>>>(p, ps, sc, grads, sc);
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
        if (any_groups) {
            dim3 grid_c((unsigned)std::min<size_t>(((size_t)t_max * F + 255) / 256, 1024), ps.n_levels);
            grid_bwd_combine_kernel<<<grid_c, 256, 0, stream>>>(p, ps, sc, grads);
            if ((e = cudaGetLastError()) != cudaSuccess) return e;
        }
    }
    return cudaSuccess;
}

} // namespace

size_t grid_bwd_segmented_scratch_bytes(const GridParams &p, size_t batch) {
    const PassLayout lay = layout_for(p, batch);
    return lay.slot_bytes * lay.levels_per_pass;
}

cudaError_t launch_grid_bwd_segmented(const GridParams &p, const float *x, const void *dy, int dy_dtype, float *grads,
                                      size_t batch, void *scratch, size_t scratch_bytes, cudaStream_t stream) {
    const int key = (int)p.n_dims * 16 + (int)p.features_per_level;
    switch (key) {
    case 2 * 16 + 1: return run_det<2, 1>(p, x, dy, dy_dtype, grads, batch, scratch, scratch_bytes, stream);
    case 2 * 16 + 2: return run_det<2, 2>(p, x, dy, dy_dtype, grads, batch, scratch, scratch_bytes, stream);
    case 2 * 16 + 4: return run_det<2, 4>(p, x, dy, dy_dtype, grads, batch, scratch, scratch_bytes, stream);
    case 2 * 16 + 8: return run_det<2, 8>(p, x, dy, dy_dtype, grads, batch, scratch, scratch_bytes, stream);
    case 3 * 16 + 1: return run_det<3, 1>(p, x, dy, dy_dtype, grads, batch, scratch, scratch_bytes, stream);
    case 3 * 16 + 2: return run_det<3, 2>(p, x, dy, dy_dtype, grads, batch, scratch, scratch_bytes, stream);
    case 3 * 16 + 4: return run_det<3, 4>(p, x, dy, dy_dtype, grads, batch, scratch, scratch_bytes, stream);
    case 3 * 16 + 8: return run_det<3, 8>(p, x, dy, dy_dtype, grads, batch, scratch, scratch_bytes, stream);
    default: return cudaErrorInvalidValue;
    }
}

} // namespace tnn
