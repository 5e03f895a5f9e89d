"""TEST INFRASTRUCTURE.  ctypes / numpy front end of the CPU oracle (oracle.cpp) and of the
reference's own host MLP (oracle/_ref/libref_mlp.so, built from the reference's test/mlp.h).

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this module.
"""
import ctypes
import os

import numpy as np

from . import build_oracle

_HERE = os.path.dirname(os.path.abspath(__file__))

ACT = {"relu": 0, "sigmoid": 4, "none": 8, "linear": 8}
GRID_TYPE = {"Hash": 0, "Dense": 1, "Tiled": 2}
HASH_TYPE = {"Prime": 0, "CoherentPrime": 1, "ReversedPrime": 2, "Rng": 3}
INTERP = {"Nearest": 0, "Linear": 1, "Smoothstep": 2}

_lib = None
_ref = None


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a, t=ctypes.c_float):
    return a.ctypes.data_as(ctypes.POINTER(t))


def lib():
    global _lib
    if _lib is None:
        path, _ = build_oracle.build()
        _lib = ctypes.CDLL(path)
        _lib.oracle_bf16_round.restype = ctypes.c_float
        _lib.oracle_bf16_round.argtypes = [ctypes.c_float]
        _lib.oracle_to_packed_coord.restype = ctypes.c_uint
        _lib.oracle_from_packed_coord.restype = ctypes.c_uint
        _lib.oracle_grid_init.restype = ctypes.c_uint32
        _lib.oracle_max_threads.restype = ctypes.c_int
    return _lib


def ref_lib():
    """The reference's own host MLP, or None when it was not built (no reference checkout)."""
    global _ref
    if _ref is None:
        _, path = build_oracle.build()
        if path is None:
            return None
        _ref = ctypes.CDLL(path)
        _ref.ref_mlp_run_batch.restype = ctypes.c_long
    return _ref


def max_threads():
    return lib().oracle_max_threads()


def bf16_round(a):
    """Round-to-nearest-even to bfloat16, returned as float32 (vectorised)."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    finite = (u & 0x7F800000) != 0x7F800000
    r = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    out = np.where(finite, r, u.astype(np.uint32)).astype(np.uint32)
    return out.view(np.float32).reshape(a.shape)


def to_packed_coord(idx, rows, cols):
    return lib().oracle_to_packed_coord(ctypes.c_uint(idx), ctypes.c_uint(rows), ctypes.c_uint(cols))


def from_packed_coord(idx, rows, cols):
    return lib().oracle_from_packed_coord(ctypes.c_uint(idx), ctypes.c_uint(rows), ctypes.c_uint(cols))


def pack_weights(unpacked, n_mat, width):
    """n_mat matrices (in x out, row-major) -> the reference's packed layout."""
    u = _f32(unpacked).reshape(-1)
    assert u.size == n_mat * width * width
    p = np.empty_like(u)
    lib().oracle_pack_weights(_ptr(u), ctypes.c_int(n_mat), ctypes.c_int(width), _ptr(p))
    return p


def unpack_weights(packed, n_mat, width):
    p = np.asarray(packed).reshape(n_mat, width * width)
    idx = np.array([to_packed_coord(i, width, width) for i in range(width * width)])
    return p[:, idx].reshape(-1)


def _mode(bf16):
    """Storage rounding of the device type: False / 0 none, True / 1 / "bf16" bfloat16, 2 / "fp16" half."""
    if bf16 in ("fp16", "float16", 2):
        return 2
    return 1 if bf16 else 0


def fp16_round(a):
    """Round-to-nearest-even to IEEE half, returned as float32."""
    return np.ascontiguousarray(a, dtype=np.float32).astype(np.float16).astype(np.float32)


def round16(a, dtype):
    return fp16_round(a) if _mode(dtype) == 2 else bf16_round(a)


def mlp_forward(x, w, n_mat, width, act, out_act, bf16=True, n_threads=0):
    """Returns interm_fwd as array (n_mat + 1, batch, width); [0] = input, [-1] = output.
    bf16: True / "bf16" or "fp16" = the device type whose rounding every stored activation gets; False = none."""
    x = _f32(x)
    w = _f32(w).reshape(-1)
    batch = x.shape[0]
    interm = np.empty((n_mat + 1, batch, width), dtype=np.float32)
    lib().oracle_mlp_forward(_ptr(x), _ptr(w), ctypes.c_int(n_mat), ctypes.c_int(width), ctypes.c_int(ACT[act]),
                             ctypes.c_int(ACT[out_act]), ctypes.c_size_t(batch), ctypes.c_int(_mode(bf16)),
                             _ptr(interm), ctypes.c_int(n_threads))
    return interm


def mlp_backward(dy, interm, w, n_mat, width, act, out_act, bf16=True, want_dx=True, n_threads=0):
    """Returns (interm_bwd (n_mat, batch, width), grads (n_mat, width(out), width(in)) float64, dx or None)."""
    dy = _f32(dy)
    interm = _f32(interm)
    w = _f32(w).reshape(-1)
    batch = dy.shape[0]
    ibwd = np.empty((n_mat, batch, width), dtype=np.float32)
    grads = np.empty((n_mat, width, width), dtype=np.float64)
    dx = np.empty((batch, width), dtype=np.float32) if want_dx else None
    lib().oracle_mlp_backward(_ptr(dy), _ptr(interm), _ptr(w), ctypes.c_int(n_mat), ctypes.c_int(width),
                              ctypes.c_int(ACT[act]), ctypes.c_int(ACT[out_act]), ctypes.c_size_t(batch),
                              ctypes.c_int(_mode(bf16)), _ptr(ibwd), _ptr(grads, ctypes.c_double),
                              _ptr(dx) if want_dx else None, ctypes.c_int(n_threads))
    return ibwd, grads, dx


def l2_loss(pred, target, loss_scale=1.0, bf16_grads=False):
    pred = _f32(pred)
    target = _f32(target)
    batch, stride = pred.shape
    values = np.empty_like(pred)
    grads = np.empty_like(pred)
    lib().oracle_l2_loss(_ptr(pred), _ptr(target), ctypes.c_int(target.shape[1]), ctypes.c_size_t(batch),
                         ctypes.c_int(stride), ctypes.c_float(loss_scale), _ptr(values), _ptr(grads),
                         ctypes.c_int(_mode(bf16_grads)))
    return values, grads


def adam(p, m, v, g, step, lr=1e-3, b1=0.9, b2=0.99, eps=1e-15):
    """In-place Adam step on float32 arrays."""
    for a in (p, m, v):
        assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    g = _f32(g)
    lib().oracle_adam(_ptr(p), _ptr(m), _ptr(v), _ptr(g), ctypes.c_size_t(p.size), ctypes.c_int(step),
                      ctypes.c_float(lr), ctypes.c_float(b1), ctypes.c_float(b2), ctypes.c_float(eps))


def identity_forward(x, padded, scale=1.0, offset=0.0):
    x = _f32(x)
    out = np.empty((x.shape[0], padded), dtype=np.float32)
    lib().oracle_identity_forward(_ptr(x), ctypes.c_size_t(x.shape[0]), ctypes.c_int(x.shape[1]), ctypes.c_int(padded),
                                  ctypes.c_float(scale), ctypes.c_float(offset), _ptr(out))
    return out


def frequency_forward(x, n_frequencies, padded=None):
    """include/encodings/frequency.h:63-80: sin / cos pairs of n_frequencies octaves per input feature, padded with 1."""
    x = _f32(x)
    padded = padded or x.shape[1] * n_frequencies * 2
    out = np.empty((x.shape[0], padded), dtype=np.float32)
    lib().oracle_frequency_forward(_ptr(x), ctypes.c_size_t(x.shape[0]), ctypes.c_int(x.shape[1]),
                                   ctypes.c_int(n_frequencies), ctypes.c_int(padded), _ptr(out))
    return out


def frequency_backward_input(x, dy, n_frequencies):
    """include/encodings/frequency.h:91-131: dL/dinput (batch x n_in) from dL/dy (batch x padded)."""
    x, dy = _f32(x), _f32(dy)
    dx = np.empty_like(x)
    lib().oracle_frequency_backward_input(_ptr(x), _ptr(dy), ctypes.c_size_t(x.shape[0]), ctypes.c_int(x.shape[1]),
                                          ctypes.c_int(n_frequencies), ctypes.c_int(dy.shape[1]), _ptr(dx))
    return dx


def spherical_harmonics_forward(x, degree, padded=None):
    """include/encodings/spherical_harmonics.h:28-64: degree^2 real spherical harmonics of 2 x - 1, padded with 1."""
    x = _f32(x)
    assert x.shape[1] == 3 and 1 <= degree <= 8
    padded = padded or degree * degree
    out = np.empty((x.shape[0], padded), dtype=np.float32)
    lib().oracle_spherical_harmonics_forward(_ptr(x), ctypes.c_size_t(x.shape[0]), ctypes.c_int(degree),
                                             ctypes.c_int(padded), _ptr(out))
    return out


class _GridStruct(ctypes.Structure):
    _fields_ = [("n_levels", ctypes.c_uint32), ("F", ctypes.c_uint32), ("D", ctypes.c_uint32),
                ("base_resolution", ctypes.c_uint32), ("log2_per_level_scale", ctypes.c_float),
                ("grid_type", ctypes.c_int), ("hash_type", ctypes.c_int), ("interpolation", ctypes.c_int),
                ("offsets", ctypes.c_uint32 * 129)]


class Grid:
    """Hash-grid oracle with the reference's configuration keys and defaults (grid.h:1010-1047)."""

    def __init__(self, n_dims_to_encode=2, n_levels=16, n_features_per_level=2, log2_hashmap_size=19,
                 base_resolution=16, per_level_scale=None, type="Hash", hash="CoherentPrime", interpolation="Linear"):
        if per_level_scale is None:
            per_level_scale = 0.0  # oracle_grid_init then applies the default of grid.h:1035-1041
        self.s = _GridStruct()
        self.n_entries = lib().oracle_grid_init(ctypes.byref(self.s), ctypes.c_uint32(n_levels),
                                                ctypes.c_uint32(n_features_per_level), ctypes.c_uint32(n_dims_to_encode),
                                                ctypes.c_uint32(log2_hashmap_size), ctypes.c_uint32(base_resolution),
                                                ctypes.c_float(per_level_scale), ctypes.c_int(GRID_TYPE[type]),
                                                ctypes.c_int(HASH_TYPE[hash]), ctypes.c_int(INTERP[interpolation]))
        self.F = n_features_per_level
        self.D = n_dims_to_encode
        self.n_levels = n_levels
        self.n_params = self.n_entries * self.F
        self.offsets = np.array(self.s.offsets[: n_levels + 1], dtype=np.int64)

    def forward(self, x, table, padded=None, n_threads=0):
        x = _f32(x)
        table = _f32(table).reshape(-1)
        assert table.size == self.n_params and x.shape[1] == self.D
        padded = padded or self.n_levels * self.F
        out = np.empty((x.shape[0], padded), dtype=np.float32)
        lib().oracle_grid_forward(ctypes.byref(self.s), _ptr(x), _ptr(table), ctypes.c_size_t(x.shape[0]),
                                  ctypes.c_int(padded), _ptr(out), ctypes.c_int(n_threads))
        return out

    def backward_input(self, x, table, dy, n_threads=0):
        """dL/dinput (batch x D) from dL/dy (batch x padded): derivative of the interpolation with respect to x."""
        x, dy = _f32(x), _f32(dy)
        table = _f32(table).reshape(-1)
        dx = np.empty_like(x)
        lib().oracle_grid_backward_input(ctypes.byref(self.s), _ptr(x), _ptr(table), _ptr(dy), ctypes.c_size_t(x.shape[0]),
                                         ctypes.c_int(dy.shape[1]), _ptr(dx), ctypes.c_int(n_threads))
        return dx

    def backward(self, x, dy, n_threads=0):
        x = _f32(x)
        dy = _f32(dy)
        grads = np.empty(self.n_params, dtype=np.float64)
        lib().oracle_grid_backward(ctypes.byref(self.s), _ptr(x), _ptr(dy), ctypes.c_size_t(x.shape[0]),
                                   ctypes.c_int(dy.shape[1]), _ptr(grads, ctypes.c_double), ctypes.c_int(n_threads))
        return grads


# ------------------------------------------------------------------ reference host MLP (test/mlp.h)
def ref_mlp_sample(width, n_mat, act, out_act, x, target, weights=None, init_mode=1, in_dim=None, out_dim=None,
                   batch=1, loss_scale=1.0):
    """One sample through the reference's mlp_cpp::MLP<double>.  Returns a dict of float64 arrays."""
    r = ref_lib()
    if r is None:
        raise RuntimeError("oracle/_ref/libref_mlp.so is not available")
    in_dim = in_dim or width
    out_dim = out_dim or width
    x = np.ascontiguousarray(x, dtype=np.float64)
    target = np.ascontiguousarray(target, dtype=np.float64)
    w = None if weights is None else np.ascontiguousarray(weights, dtype=np.float64).reshape(-1)
    d = ctypes.c_double
    out = {
        "fwd": np.empty((n_mat + 1, width)), "weights": np.empty((n_mat, width, width)),
        "grads": np.empty((n_mat, width, width)), "loss_grads": np.empty((n_mat, width)),
        "dl_dinput": np.empty(width), "loss": np.empty(width),
    }
    rc = r.ref_mlp_sample(ctypes.c_int(in_dim), ctypes.c_int(width), ctypes.c_int(out_dim), ctypes.c_int(n_mat),
                          ctypes.c_int(batch), ctypes.c_int(ACT[act]), ctypes.c_int(ACT[out_act]),
                          None if w is None else _ptr(w, d), ctypes.c_int(init_mode), _ptr(x, d), _ptr(target, d),
                          ctypes.c_double(loss_scale), _ptr(out["fwd"], d), _ptr(out["weights"], d),
                          _ptr(out["grads"], d), _ptr(out["loss_grads"], d), _ptr(out["dl_dinput"], d),
                          _ptr(out["loss"], d))
    if rc != 0:
        raise RuntimeError("ref_mlp_sample failed")
    return out


def ref_mlp_run_batch(width, n_mat, act, out_act, weights, x, target, do_backward):
    """Throughput helper: runs every row of x through the reference MLP; returns samples processed."""
    r = ref_lib()
    w = np.ascontiguousarray(weights, dtype=np.float64).reshape(-1)
    x = np.ascontiguousarray(x, dtype=np.float64)
    target = np.ascontiguousarray(target, dtype=np.float64)
    d = ctypes.c_double
    chk = ctypes.c_double(0.0)
    return r.ref_mlp_run_batch(ctypes.c_int(width), ctypes.c_int(n_mat), ctypes.c_int(ACT[act]),
                               ctypes.c_int(ACT[out_act]), _ptr(w, d), _ptr(x, d), _ptr(target, d),
                               ctypes.c_long(x.shape[0]), ctypes.c_int(1 if do_backward else 0), ctypes.byref(chk))


def within_tolerance(value, target, tol):
    """areVectorsWithinTolerance of the reference (include/common/result_check.h:83-102):
    max|a - b| / max(|a|_inf, |b|_inf) <= tol (absolute when the target is all zero)."""
    value = np.asarray(value, dtype=np.float64).reshape(-1)
    target = np.asarray(target, dtype=np.float64).reshape(-1)
    diff = np.max(np.abs(value - target)) if value.size else 0.0
    inf_t = np.max(np.abs(target)) if target.size else 0.0
    inf_v = np.max(np.abs(value)) if value.size else 0.0
    rel = diff if inf_t == 0.0 else diff / max(inf_t, inf_v)
    return rel <= tol, rel
