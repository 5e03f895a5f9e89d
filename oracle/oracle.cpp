// TEST INFRASTRUCTURE - CPU restatement of the reference algorithms of the hot path.
//
// This file is the checker the parity tests compare the CUDA kernels against, and the CPU
// baseline bench.py times.  It is never linked into or called from the product library.
// Every function names the reference source (intel/tiny-dpcpp-nn, path:line) it restates.
//
// Pinning: the MLP restatement is checked against the reference's own host MLP (test/mlp.h,
// compiled unmodified into oracle/_ref by oracle/build_oracle.py) and against the closed-form
// expectations of test/doctest_swiftnet.cpp:44-96; the grid restatement against the known-answer
// vector of test/doctest_encodings.cpp:234-285; packing against test/doctest_packing.cpp:21-46;
// L2 against test/doctest_losses.cpp:46-47.  The grid *backward* has no value fixture in the
// reference (its CSV fixtures are not in the repository): parity unpinned by fixtures for that
// function; it is pinned only through linearity / adjointness with the pinned forward.
//
// Build: g++ -O3 -march=native -fopenmp -shared -fPIC oracle.cpp -o liboracle.so
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

// Same enumerator order as include/common/common.h:28-38.
enum { ACT_RELU = 0, ACT_SIGMOID = 4, ACT_NONE = 8 };

inline float bf16_round(float v) {
    // round-to-nearest-even to 8 bits of mantissa, like static_cast<bf16>(float)
    uint32_t u;
    std::memcpy(&u, &v, 4);
    if ((u & 0x7F800000u) == 0x7F800000u) return v; // inf / nan unchanged
    const uint32_t lsb = (u >> 16) & 1u;
    u += 0x7FFFu + lsb;
    u &= 0xFFFF0000u;
    float r;
    std::memcpy(&r, &u, 4);
    return r;
}

inline float fp16_round(float v) {
    // round-to-nearest-even to IEEE half precision (11 significant bits, subnormals below 2^-14, overflow to inf),
    // like static_cast<sycl::half>(float)
    return (float)(_Float16)v;
}

// storage rounding of the device type T: mode 0 = none, 1 = bf16, 2 = fp16
inline float round16(float v, int mode) { return mode == 2 ? fp16_round(v) : mode == 1 ? bf16_round(v) : v; }

inline void set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

} // namespace

extern "C" {

int oracle_max_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

float oracle_bf16_round(float v) { return bf16_round(v); }
float oracle_fp16_round(float v) { return fp16_round(v); }

// ---------------------------------------------------------------------------------------------
// Weight packing: source/common/common.cpp:33-66 (to/fromPackedLayoutCoord) and
// include/common/common.h:174-212 (vertical_pack / get_packed_weights).
// ---------------------------------------------------------------------------------------------
unsigned oracle_to_packed_coord(unsigned idx, unsigned rows, unsigned cols) {
    (void)rows;
    const int i = idx / cols, j = idx % cols;
    return (i % 2 == 0) ? i * cols + 2 * j : (i - 1) * cols + 2 * j + 1;
}
unsigned oracle_from_packed_coord(unsigned idx, unsigned rows, unsigned cols) {
    (void)rows;
    const int i = idx / (cols * 2), j = idx % (cols * 2);
    return (j % 2 == 0) ? (i * 2) * cols + j / 2 : (i * 2 + 1) * cols + (j - 1) / 2;
}
// n_mat matrices of width x width, unpacked (in x out row-major) -> packed.
void oracle_pack_weights(const float *unpacked, int n_mat, int width, float *packed) {
    for (int l = 0; l < n_mat; ++l)
        for (int idx = 0; idx < width * width; ++idx)
            packed[l * width * width + oracle_to_packed_coord(idx, width, width)] = unpacked[l * width * width + idx];
}

// ---------------------------------------------------------------------------------------------
// Fused MLP forward: include/network/kernel_esimd.h:565-640 (forward_impl_general) with the
// activation rules of 443-458.  x: batch x W.  w: n_mat matrices (in x out, row-major, unpacked).
// interm: (n_mat + 1) matrices batch x W; matrix 0 = x, matrix l + 1 = activation of layer l.
// bf16 != 0: every stored activation is rounded like the device type T (1 = bf16, 2 = fp16); accumulation is
// done in double, the device's fp32 accumulation differs from it by less than one bf16 ulp.
// bf16 == 0: plain double-precision network, the arithmetic of test/mlp.h:234-282.
// ---------------------------------------------------------------------------------------------
void oracle_mlp_forward(const float *x, const float *w, int n_mat, int W, int act, int out_act, size_t batch, int bf16,
                        float *interm, int n_threads) {
    set_threads(n_threads);
    std::memcpy(interm, x, batch * W * sizeof(float));
#pragma omp parallel for schedule(static)
    for (long long b = 0; b < (long long)batch; ++b) {
        std::vector<double> cur(W), nxt(W);
        for (int k = 0; k < W; ++k) cur[k] = x[b * W + k];
        for (int l = 0; l < n_mat; ++l) {
            const float *wl = w + (size_t)l * W * W;
            for (int n = 0; n < W; ++n) nxt[n] = 0.0;
            for (int k = 0; k < W; ++k) {
                const double a = cur[k];
                if (a == 0.0) continue;
                const float *wr = wl + (size_t)k * W;
                for (int n = 0; n < W; ++n) nxt[n] += a * (double)wr[n];
            }
            const int a_ = (l == n_mat - 1) ? out_act : act;
            float *dst = interm + ((size_t)(l + 1) * batch + b) * W;
            for (int n = 0; n < W; ++n) {
                double v = nxt[n];
                if (a_ == ACT_SIGMOID) v = 1.0 / (1.0 + std::exp(-v));
                if (bf16) v = round16((float)v, bf16);
                if (a_ == ACT_RELU) v = std::max(v, 0.0);
                dst[n] = (float)v;
                cur[n] = v;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Fused MLP backward: include/network/kernel_esimd.h:160-240 (chain kernel + gemm_batch) with the
// backward activation rules of 460-487 (ReLU mask = stored activation <= 0; sigmoid s (1 - s)).
// dy: batch x W = dL/d(output).  interm: forward activations as written by oracle_mlp_forward.
// interm_bwd (optional): n_mat matrices, matrix l = dL/d(pre-activation of layer l).
// grads: n_mat matrices (out x in) = interm_bwd[l]^T interm_fwd[l], accumulated in double, not rounded.
// dx (optional): batch x W.
// ---------------------------------------------------------------------------------------------
void oracle_mlp_backward(const float *dy, const float *interm, const float *w, int n_mat, int W, int act, int out_act,
                         size_t batch, int bf16, float *interm_bwd, double *grads, float *dx, int n_threads) {
    set_threads(n_threads);
    const int L = n_mat - 1;
    const size_t gsz = (size_t)n_mat * W * W;
    std::fill(grads, grads + gsz, 0.0);
    int nt = 1;
#ifdef _OPENMP
    nt = omp_get_max_threads();
#endif
    std::vector<std::vector<double>> partial(nt, std::vector<double>(gsz, 0.0));
#pragma omp parallel
    {
        int tid = 0;
#ifdef _OPENMP
        tid = omp_get_thread_num();
#endif
        std::vector<double> &g = partial[tid];
        std::vector<double> delta(W), prev(W);
#pragma omp for schedule(static)
        for (long long b = 0; b < (long long)batch; ++b) {
            const float *y = interm + ((size_t)(L + 1) * batch + b) * W;
            for (int n = 0; n < W; ++n) {
                double d = dy[b * W + n];
                if (out_act == ACT_RELU) {
                    if (y[n] <= 0.0f) d = 0.0;
                } else if (out_act == ACT_SIGMOID) {
                    d *= (double)y[n] * (1.0 - (double)y[n]);
                }
                if (bf16) d = round16((float)d, bf16);
                delta[n] = d;
            }
            for (int l = L; l >= 0; --l) {
                const float *al = interm + ((size_t)l * batch + b) * W;
                if (interm_bwd)
                    for (int n = 0; n < W; ++n) interm_bwd[((size_t)l * batch + b) * W + n] = (float)delta[n];
                double *gl = g.data() + (size_t)l * W * W;
                for (int o = 0; o < W; ++o) {
                    const double d = delta[o];
                    if (d == 0.0) continue;
                    for (int i = 0; i < W; ++i) gl[(size_t)o * W + i] += d * (double)al[i];
                }
                if (l == 0 && !dx) break;
                // prev[k] = sum_n delta[n] * W_l[k][n]
                const float *wl = w + (size_t)l * W * W;
                for (int k = 0; k < W; ++k) {
                    double s = 0.0;
                    const float *wr = wl + (size_t)k * W;
                    for (int n = 0; n < W; ++n) s += delta[n] * (double)wr[n];
                    if (l > 0) {
                        if (act == ACT_RELU) {
                            if (al[k] <= 0.0f) s = 0.0;
                        } else if (act == ACT_SIGMOID) {
                            s *= (double)al[k] * (1.0 - (double)al[k]);
                        }
                    }
                    if (bf16) s = round16((float)s, bf16);
                    prev[k] = s;
                }
                if (l == 0) {
                    for (int k = 0; k < W; ++k) dx[b * W + k] = (float)prev[k];
                } else {
                    delta.swap(prev);
                }
            }
        }
    }
    for (int t = 0; t < nt; ++t)
        for (size_t i = 0; i < gsz; ++i) grads[i] += partial[t][i];
}

// ---------------------------------------------------------------------------------------------
// L2 loss: include/losses/l2.h:19-25.  n_elements = batch * stride.
// ---------------------------------------------------------------------------------------------
void oracle_l2_loss(const float *pred, const float *target, int n_targets, size_t batch, int stride, float loss_scale,
                    float *values, float *grads, int bf16_grads) {
    const float inv_n = 1.0f / (float)(batch * (size_t)stride);
    for (size_t b = 0; b < batch; ++b)
        for (int c = 0; c < stride; ++c) {
            const float t = c < n_targets ? target[b * n_targets + c] : 0.0f;
            const float diff = pred[b * stride + c] - t;
            if (values) values[b * stride + c] = diff * diff * inv_n;
            if (grads) {
                const float g = loss_scale * 2 * diff * inv_n;
                grads[b * stride + c] = round16(g, bf16_grads);
            }
        }
}

// ---------------------------------------------------------------------------------------------
// Adam, torch.optim.Adam semantics (no weight decay / amsgrad); `step` counts from 1.
// ---------------------------------------------------------------------------------------------
void oracle_adam(float *p, float *m, float *v, const float *g, size_t n, int step, float lr, float b1, float b2,
                 float eps) {
    const double bc1 = 1.0 - std::pow((double)b1, step);
    const double bc2 = 1.0 - std::pow((double)b2, step);
    for (size_t i = 0; i < n; ++i) {
        m[i] = b1 * m[i] + (1.0f - b1) * g[i];
        v[i] = b2 * v[i] + (1.0f - b2) * g[i] * g[i];
        const double denom = std::sqrt((double)v[i]) / std::sqrt(bc2) + (double)eps;
        p[i] = (float)((double)p[i] - ((double)lr / bc1) * ((double)m[i] / denom));
    }
}

// ---------------------------------------------------------------------------------------------
// Identity encoding: include/encodings/identity.h:63-77.
// ---------------------------------------------------------------------------------------------
void oracle_identity_forward(const float *x, size_t batch, int n_in, int padded, float scale, float offset, float *out) {
    for (size_t b = 0; b < batch; ++b)
        for (int j = 0; j < padded; ++j) out[b * padded + j] = j < n_in ? x[b * n_in + j] * scale + offset : 1.0f;
}

// ---------------------------------------------------------------------------------------------
// Frequency encoding: include/encodings/frequency.h:63-80.  The reference forms the argument as
// float * size_t (float) * M_PI (double) + phase (float) and rounds it to float before the sine.
// ---------------------------------------------------------------------------------------------
void oracle_frequency_forward(const float *x, size_t batch, int n_in, int n_freq, int padded, float *out) {
    const int n_out = n_in * n_freq * 2;
    for (size_t b = 0; b < batch; ++b)
        for (int j = 0; j < padded; ++j) {
            if (j >= n_out) {
                out[b * padded + j] = 1.0f;
                continue;
            }
            const int feature = j / (n_freq * 2);
            const int log2_frequency = (j / 2) % n_freq;
            const float phase_shift = (float)((j % 2) * (M_PI / 2.0));
            const float arg = (float)((double)(x[b * n_in + feature] * (float)((size_t)1 << log2_frequency)) * M_PI + phase_shift);
            out[b * padded + j] = std::sin(arg);
        }
}

// dL/dinput of the frequency encoding: include/encodings/frequency.h:72-73 (dy/dx = 2^f pi cos(arg)) and 91-131
// (dL/dx_j = sum over the 2 F outputs of feature j of dL/dy * dy/dx).  Accumulated in double.
void oracle_frequency_backward_input(const float *x, const float *dy, size_t batch, int n_in, int n_freq, int padded,
                                     float *dx) {
    for (size_t b = 0; b < batch; ++b)
        for (int f = 0; f < n_in; ++f) {
            double acc = 0.0;
            for (int k = 0; k < 2 * n_freq; ++k) {
                const int j = f * 2 * n_freq + k;
                const int log2_frequency = (j / 2) % n_freq;
                const float phase_shift = (float)((j % 2) * (M_PI / 2.0));
                const float scale = (float)((size_t)1 << log2_frequency);
                const float arg = (float)((double)(x[b * n_in + f] * scale) * M_PI + phase_shift);
                acc += (double)dy[b * padded + j] * (double)scale * M_PI * std::cos((double)arg);
            }
            dx[b * n_in + f] = (float)acc;
        }
}

// ---------------------------------------------------------------------------------------------
// Spherical harmonics: include/encodings/spherical_harmonics.h:28-64 encodes the direction 2 x - 1 with the
// degree^2 real spherical harmonics (order l (l + 1) + m), padded with ones.  The reference evaluates generated
// polynomials (include/common/common_device.h:33-206, "generated ... based on the recurrence relations in appendix A1
// of Sloan, Stupid Spherical Harmonics Tricks"); this restatement evaluates the same functions from that published
// definition in double precision:
//   Y_l^m = sqrt(2) K_l^m (-1)^m Q_l^m(z) Re (x + i y)^m,  Y_l^-m = ... Im (x + i y)^m,  Y_l^0 = K_l^0 Q_l^0(z),
//   K_l^m = sqrt((2 l + 1) (l - m)! / (4 pi (l + m)!)),  Q_l^m = d^m P_l / dz^m.
// ---------------------------------------------------------------------------------------------
void oracle_spherical_harmonics_forward(const float *in, size_t batch, int degree, int padded, float *out) {
    for (size_t b = 0; b < batch; ++b) {
        // the inputs are mapped in fp32 like the device code (x * 2.f - 1.f)
        const double x = (double)(in[b * 3 + 0] * 2.0f - 1.0f), y = (double)(in[b * 3 + 1] * 2.0f - 1.0f),
                     z = (double)(in[b * 3 + 2] * 2.0f - 1.0f);
        float *o = out + b * padded;
        for (int j = degree * degree; j < padded; ++j) o[j] = 1.0f;
        double c = 1.0, s = 0.0, qmm = 1.0;
        for (int m = 0; m < degree; ++m) {
            if (m > 0) {
                const double cn = c * x - s * y;
                s = c * y + s * x;
                c = cn;
                qmm *= (double)(2 * m - 1);
            }
            double q2 = 0.0, q1 = 0.0;
            for (int l = m; l < degree; ++l) {
                double q;
                if (l == m)
                    q = qmm;
                else if (l == m + 1)
                    q = (2 * m + 1) * z * q1;
                else
                    q = ((2 * l - 1) * z * q1 - (l + m - 1) * q2) / (double)(l - m);
                q2 = q1;
                q1 = q;
                double ratio = 1.0;
                for (int i = l - m + 1; i <= l + m; ++i) ratio /= (double)i;
                double k = std::sqrt((2.0 * l + 1.0) / (4.0 * M_PI) * ratio);
                if (m > 0) k *= std::sqrt(2.0) * ((m & 1) ? -1.0 : 1.0);
                if (m == 0) {
                    o[l * (l + 1)] = (float)(k * q);
                } else {
                    o[l * (l + 1) + m] = (float)(k * q * c);
                    o[l * (l + 1) - m] = (float)(k * q * s);
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Hash grid.  Level table: include/encodings/grid.h:588-659; scale / resolution:
// include/common/common_device.h:767-775; hash and index: common_device.h:700-765 (all uint32,
// wrapping); forward: grid.h:37-135; backward: grid.h:137-245.
// ---------------------------------------------------------------------------------------------
struct OracleGrid {
    uint32_t n_levels, F, D, base_resolution;
    float log2_per_level_scale;
    int grid_type;     // 0 Hash, 1 Dense, 2 Tiled
    int hash_type;     // 0 Prime, 1 CoherentPrime, 2 ReversedPrime, 3 Rng
    int interpolation; // 0 Nearest, 1 Linear, 2 Smoothstep
    uint32_t offsets[129];
};

static float grid_scale(uint32_t level, float log2_pls, uint32_t base) {
    return std::exp2(level * log2_pls) * base - 1.0f;
}
static uint32_t grid_resolution(float scale) { return (uint32_t)std::ceil(scale) + 1; }
static uint32_t powi(uint32_t base, uint32_t e) {
    uint32_t r = 1;
    for (uint32_t i = 0; i < e; ++i) r *= base;
    return r;
}

uint32_t oracle_grid_init(OracleGrid *g, uint32_t n_levels, uint32_t F, uint32_t D, uint32_t log2_hashmap_size,
                          uint32_t base_resolution, float per_level_scale, int grid_type, int hash_type,
                          int interpolation) {
    g->n_levels = n_levels, g->F = F, g->D = D, g->base_resolution = base_resolution;
    if (per_level_scale <= 0.0f) // default of grid.h:1035-1041
        per_level_scale = (grid_type == 1 && n_levels > 1)
                              ? std::exp(std::log(256.0f / (float)base_resolution) / (n_levels - 1))
                              : 2.0f;
    g->log2_per_level_scale = std::log2(per_level_scale);
    g->grid_type = grid_type, g->hash_type = hash_type, g->interpolation = interpolation;
    uint32_t offset = 0;
    for (uint32_t i = 0; i < n_levels; ++i) {
        const uint32_t resolution = grid_resolution(grid_scale(i, g->log2_per_level_scale, base_resolution));
        const uint32_t max_params = std::numeric_limits<uint32_t>::max() / 2;
        uint32_t params_in_level =
            std::pow((float)resolution, (float)D) > (float)max_params ? max_params : powi(resolution, D);
        params_in_level = (params_in_level + 7u) / 8u * 8u;
        if (grid_type == 2)
            params_in_level = std::min(params_in_level, powi(base_resolution, D));
        else if (grid_type == 0)
            params_in_level = std::min(params_in_level, 1u << log2_hashmap_size);
        g->offsets[i] = offset;
        offset += params_in_level;
    }
    g->offsets[n_levels] = offset;
    return offset;
}

static uint32_t grid_hash(int hash_type, uint32_t D, const uint32_t *pos) {
    static const uint32_t prime[7] = {1958374283u, 2654435761u, 805459861u, 3674653429u,
                                      2097192037u, 1434869437u, 2165219737u};
    static const uint32_t coherent[7] = {1u,          2654435761u, 805459861u, 3674653429u,
                                         2097192037u, 1434869437u, 2165219737u};
    static const uint32_t reversed[7] = {2165219737u, 1434869437u, 2097192037u, 3674653429u,
                                         805459861u,  2654435761u, 1958374283u};
    const uint32_t *f = hash_type == 0 ? prime : hash_type == 1 ? coherent : hash_type == 2 ? reversed : nullptr;
    if (!f) return 0;
    uint32_t r = 0;
    for (uint32_t i = 0; i < D; ++i) r ^= pos[i] * f[i];
    return r;
}

static uint32_t grid_index(const OracleGrid *g, uint32_t hashmap_size, uint32_t res, const uint32_t *pos) {
    uint32_t stride = 1, index = 0;
    for (uint32_t dim = 0; dim < g->D && stride <= hashmap_size; ++dim) {
        index += pos[dim] * stride;
        stride *= res;
    }
    if (g->grid_type == 0 && hashmap_size < stride) index = grid_hash(g->hash_type, g->D, pos);
    return index % hashmap_size;
}

static void grid_position(const OracleGrid *g, const float *x, float scale, float *pos, uint32_t *pos_grid) {
    for (uint32_t d = 0; d < g->D; ++d) {
        pos[d] = std::fma(scale, x[d], 0.5f);
        const float tmp = std::floor(pos[d]);
        pos_grid[d] = (uint32_t)(int)tmp;
        pos[d] -= tmp;
        if (g->interpolation == 2) pos[d] = pos[d] * pos[d] * (3.0f - 2.0f * pos[d]);
    }
}

// x: batch x D.  table: offsets[n_levels] * F floats.  out: batch x padded (columns >= n_levels F zeroed).
void oracle_grid_forward(const OracleGrid *g, const float *x, const float *table, size_t batch, int padded, float *out,
                         int n_threads) {
    set_threads(n_threads);
    const uint32_t F = g->F, D = g->D;
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < (long long)batch; ++i) {
        float *orow = out + (size_t)i * padded;
        for (int c = g->n_levels * F; c < padded; ++c) orow[c] = 0.0f;
        for (uint32_t level = 0; level < g->n_levels; ++level) {
            const float *grid = table + (size_t)g->offsets[level] * F;
            const uint32_t hashmap_size = g->offsets[level + 1] - g->offsets[level];
            const float scale = grid_scale(level, g->log2_per_level_scale, g->base_resolution);
            const uint32_t resolution = grid_resolution(scale);
            float pos[3];
            uint32_t pos_grid[3];
            grid_position(g, x + (size_t)i * D, scale, pos, pos_grid);
            float result[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            if (g->interpolation == 0) {
                const uint32_t idx = grid_index(g, hashmap_size, resolution, pos_grid);
                for (uint32_t f = 0; f < F; ++f) result[f] = grid[(size_t)idx * F + f];
            } else {
                for (uint32_t c = 0; c < (1u << D); ++c) {
                    float weight = 1.0f;
                    uint32_t local[3];
                    for (uint32_t d = 0; d < D; ++d) {
                        if ((c & (1u << d)) == 0) {
                            weight *= 1 - pos[d];
                            local[d] = pos_grid[d];
                        } else {
                            weight *= pos[d];
                            local[d] = pos_grid[d] + 1;
                        }
                    }
                    const uint32_t idx = grid_index(g, hashmap_size, resolution, local);
                    for (uint32_t f = 0; f < F; ++f) result[f] = std::fma(weight, grid[(size_t)idx * F + f], result[f]);
                }
            }
            for (uint32_t f = 0; f < F; ++f) orow[level * F + f] = result[f];
        }
    }
}

// dL/dinput of the grid: the derivative of the interpolation formula above with respect to x (the quantity
// kernel_grid_backward_input, grid.h:247-268, forms from a stored dy/dx), accumulated in double:
//   dL/dx_d = sum_l scale_l sum_c (+-1)_(c_d) [smoothstep: 6 p (1 - p)] prod_(e != d) w_e(c) <dL/dy_l, table_l[index(g + c)]>
void oracle_grid_backward_input(const OracleGrid *g, const float *x, const float *table, const float *dy, size_t batch,
                                int padded, float *dx, int n_threads) {
    set_threads(n_threads);
    const uint32_t F = g->F, D = g->D;
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < (long long)batch; ++i) {
        double acc[3] = {0, 0, 0};
        for (uint32_t level = 0; level < g->n_levels && g->interpolation != 0; ++level) {
            const float *grid = table + (size_t)g->offsets[level] * F;
            const uint32_t hashmap_size = g->offsets[level + 1] - g->offsets[level];
            const float scale = grid_scale(level, g->log2_per_level_scale, g->base_resolution);
            const uint32_t resolution = grid_resolution(scale);
            double w[3], dw[3];
            uint32_t pos_grid[3];
            for (uint32_t d = 0; d < D; ++d) {
                float p = std::fma(scale, x[(size_t)i * D + d], 0.5f);
                const float fl = std::floor(p);
                pos_grid[d] = (uint32_t)(int)fl;
                p -= fl;
                dw[d] = g->interpolation == 2 ? 6.0 * p * (1.0 - p) : 1.0;
                w[d] = g->interpolation == 2 ? (double)p * p * (3.0 - 2.0 * p) : (double)p;
            }
            for (uint32_t c = 0; c < (1u << D); ++c) {
                uint32_t local[3];
                for (uint32_t d = 0; d < D; ++d) local[d] = pos_grid[d] + ((c >> d) & 1u);
                const uint32_t idx = grid_index(g, hashmap_size, resolution, local);
                double v = 0.0;
                for (uint32_t f = 0; f < F; ++f)
                    v += (double)dy[(size_t)i * padded + level * F + f] * (double)grid[(size_t)idx * F + f];
                for (uint32_t d = 0; d < D; ++d) {
                    double wd = ((c >> d) & 1u) ? dw[d] : -dw[d];
                    for (uint32_t e = 0; e < D; ++e)
                        if (e != d) wd *= ((c >> e) & 1u) ? w[e] : 1.0 - w[e];
                    acc[d] += (double)scale * wd * v;
                }
            }
        }
        for (uint32_t d = 0; d < D; ++d) dx[(size_t)i * D + d] = (float)acc[d];
    }
}

// dy: batch x padded.  grads: offsets[n_levels] * F doubles, overwritten (the reference memsets and then
// adds float atomics in an unspecified order; the sum is accumulated here in double, sample order).
// Parallel over levels, so no two threads touch the same entry.
void oracle_grid_backward(const OracleGrid *g, const float *x, const float *dy, size_t batch, int padded, double *grads,
                          int n_threads) {
    set_threads(n_threads);
    const uint32_t F = g->F, D = g->D;
    std::fill(grads, grads + (size_t)g->offsets[g->n_levels] * F, 0.0);
#pragma omp parallel for schedule(dynamic, 1)
    for (int level = 0; level < (int)g->n_levels; ++level) {
        double *gl = grads + (size_t)g->offsets[level] * F;
        const uint32_t hashmap_size = g->offsets[level + 1] - g->offsets[level];
        const float scale = grid_scale(level, g->log2_per_level_scale, g->base_resolution);
        const uint32_t resolution = grid_resolution(scale);
        for (size_t i = 0; i < batch; ++i) {
            float pos[3];
            uint32_t pos_grid[3];
            grid_position(g, x + i * D, scale, pos, pos_grid);
            const float *grad = dy + i * padded + level * F;
            if (g->interpolation == 0) {
                const uint32_t idx = grid_index(g, hashmap_size, resolution, pos_grid);
                for (uint32_t f = 0; f < F; ++f) gl[(size_t)idx * F + f] += grad[f];
                continue;
            }
            for (uint32_t c = 0; c < (1u << D); ++c) {
                float weight = 1.0f;
                uint32_t local[3];
                for (uint32_t d = 0; d < D; ++d) {
                    if ((c & (1u << d)) == 0) {
                        weight *= 1 - pos[d];
                        local[d] = pos_grid[d];
                    } else {
                        weight *= pos[d];
                        local[d] = pos_grid[d] + 1;
                    }
                }
                const uint32_t idx = grid_index(g, hashmap_size, resolution, local);
                for (uint32_t f = 0; f < F; ++f) gl[(size_t)idx * F + f] += (double)(weight * grad[f]);
            }
        }
    }
}

} // extern "C"
