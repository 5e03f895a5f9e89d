"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

They stand in for the reference's benchmark workloads (constant-filled tensors of
benchmarks/benchmark_inference.h:39-48, the NeRF / image shapes of benchmarks/benchmark_all.cpp:53-104
and the image of samples/); everything is drawn on the host with numpy's PCG64 so the oracle and the
GPU see the same arrays.
"""
import numpy as np

from oracle import oracle as O


def xavier_weights(n_mat, width, seed):
    """n_mat matrices (in x out), uniform(+-sqrt(6 / (2 width))) - Network.h:271-295 with equal fans."""
    rng = np.random.default_rng(seed)
    bound = np.sqrt(6.0 / (2 * width))
    return rng.uniform(-bound, bound, (n_mat, width, width)).astype(np.float32)


def uniform_inputs(batch, width, seed=100, lo=-1.0, hi=1.0):
    return np.random.default_rng(seed).uniform(lo, hi, (batch, width)).astype(np.float32)


def mlp_case(width, n_hidden, batch, w_seed=0, x_seed=100):
    """Weights and inputs already rounded to bf16 (stored as float32)."""
    w = O.bf16_round(xavier_weights(n_hidden + 1, width, w_seed))
    x = O.bf16_round(uniform_inputs(batch, width, x_seed))
    return w, x


def grid_table(n_params, seed=3):
    return np.random.default_rng(seed).uniform(-1e-4, 1e-4, n_params).astype(np.float32)


def sinusoid_targets(points, n_out, n_waves, fmax, seed):
    """t_c(p) = sum_k a_kc sin(2 pi f_k . p + phi_k): the smooth stand-in for image / field targets."""
    rng = np.random.default_rng(seed)
    d = points.shape[1]
    f = rng.uniform(1.0, fmax, (n_waves, d))
    phi = rng.uniform(0.0, 2 * np.pi, n_waves)
    a = rng.uniform(-1.0, 1.0, (n_waves, n_out)) / n_waves
    phase = 2 * np.pi * points.astype(np.float64) @ f.T + phi
    return (np.sin(phase) @ a).astype(np.float32)
