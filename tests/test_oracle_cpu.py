"""CPU tests: the oracle against the reference's golden vectors, known-answer tests and closed forms."""
import json
import os

import math

import numpy as np
import pytest

from oracle import oracle as O
from tests import synth

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
ACT_NAME = {0: "relu", 4: "sigmoid", 8: "none"}


def test_grid_known_answer_vector():
    """test/doctest_encodings.cpp:234-285."""
    kat = json.load(open(os.path.join(GOLDEN, "grid_kat.json")))
    c = kat["config"]
    g = O.Grid(n_dims_to_encode=c["n_dims_to_encode"], n_levels=c["n_levels"],
               n_features_per_level=c["n_features_per_level"], log2_hashmap_size=c["log2_hashmap_size"],
               base_resolution=c["base_resolution"], per_level_scale=c["per_level_scale"], type=c["type"])
    assert g.n_params == kat["n_params"]
    n = g.n_params
    table = (np.arange(n, dtype=np.float64) / (n / 2.0) - 1.0).astype(np.float32)
    out = g.forward(np.array([kat["input"]], dtype=np.float32), table, padded=kat["padded_output_width"])
    ok, rel = O.within_tolerance(out[0], kat["expected"], kat["tolerance"])
    assert ok, rel


def test_grid_level_table():
    """Level sizes of the benchmark grid: 16 levels x 2 features, 2^19 entries cap, base 16, scale 2."""
    g = O.Grid(n_dims_to_encode=3)
    sizes = np.diff(g.offsets)
    assert list(sizes[:3]) == [4096, 32768, 262144]
    assert all(s == 524288 for s in sizes[3:])
    assert g.n_entries == 7114752


def test_grid_backward_zero_upstream_gives_zero_gradient():
    """test/doctest_encodings.cpp:286-341."""
    g = O.Grid(n_dims_to_encode=3)
    grads = g.backward(np.ones((1, 3), np.float32), np.zeros((1, 32), np.float32))
    assert not grads.any()


def test_grid_backward_is_adjoint_of_forward():
    """<forward(x; T), dy> == <T, backward(x, dy)> for every table T: pins the backward to the pinned forward."""
    g = O.Grid(n_dims_to_encode=3, n_levels=6, log2_hashmap_size=12, base_resolution=4)
    rng = np.random.default_rng(0)
    x = rng.uniform(0, 1, (256, 3)).astype(np.float32)
    table = rng.uniform(-1, 1, g.n_params).astype(np.float32)
    dy = rng.uniform(-1, 1, (256, 12)).astype(np.float32)
    lhs = float((g.forward(x, table).astype(np.float64) * dy).sum())
    rhs = float((table.astype(np.float64) * g.backward(x, dy)).sum())
    assert abs(lhs - rhs) <= 1e-5 * max(abs(lhs), 1.0)


def test_grid_backward_hand_checked_fixture():
    """tests/golden/grid_backward_handcheck.json: the parameter gradient of five samples on a 2-level 2-D dense grid,
    derived by explicit corner enumeration in tests/golden/make_grid_backward_fixture.py (independent of the oracle;
    two entries worked by hand in that file).  Pins the oracle's backward, which the reference's own tests cannot
    (their backward fixtures are CSV files that are not in the reference repository)."""
    k = json.load(open(os.path.join(GOLDEN, "grid_backward_handcheck.json")))
    c = k["config"]
    g = O.Grid(n_dims_to_encode=c["n_dims_to_encode"], n_levels=c["n_levels"],
               n_features_per_level=c["n_features_per_level"], log2_hashmap_size=c["log2_hashmap_size"],
               base_resolution=c["base_resolution"], per_level_scale=c["per_level_scale"], type=c["type"])
    assert g.n_params == k["n_params"] and list(g.offsets) == [0, 16, 80]
    grads = g.backward(np.array(k["x"], np.float32), np.array(k["dy"], np.float32))
    assert np.array_equal(grads, np.array(k["expected_grad"]))  # binary fractions: exact
    # the two entries worked by hand in the generator's docstring
    assert grads[10 * 2] == 1.0 + 0.0625 + 0.5 * 0.0625 and grads[52 * 2] == 3.0 and grads[52 * 2 + 1] == 4.0


@pytest.mark.parametrize("dims,interp,gtype", [(2, "Linear", "Hash"), (3, "Smoothstep", "Hash"),
                                               (2, "Nearest", "Dense"), (3, "Linear", "Tiled")])
def test_grid_variants_run(dims, interp, gtype):
    g = O.Grid(n_dims_to_encode=dims, n_levels=4, log2_hashmap_size=10, base_resolution=4, type=gtype,
               interpolation=interp)
    rng = np.random.default_rng(1)
    x = rng.uniform(0, 1, (64, dims)).astype(np.float32)
    t = rng.uniform(-1, 1, g.n_params).astype(np.float32)
    out = g.forward(x, t, padded=16)
    assert out.shape == (64, 16) and not out[:, 8:].any() and np.isfinite(out).all()


def test_packing_known_vectors():
    """test/python/test_packing.py:9-27 and test/doctest_packing.cpp:21-72."""
    kat = json.load(open(os.path.join(GOLDEN, "packing_kat.json")))
    un = np.array(kat["unpacked_4x4"], dtype=np.float32)
    assert np.array_equal(O.pack_weights(un, 1, 4).reshape(4, 4), np.array(kat["packed_4x4"], dtype=np.float32))
    w = np.arange(1, 513, dtype=np.float32)  # three 16 x 16 matrices (input, hidden... here input + output + one more)
    p = O.pack_weights(w[:512], 2, 16)
    assert list(p[:32]) == kat["packed_16_first_row_pair"]
    assert list(p[-32:]) == kat["packed_16_last_row_pair"]
    for idx, rows, cols, exp in kat["coord_points"]:
        assert O.to_packed_coord(idx, rows, cols) == exp
        assert O.from_packed_coord(exp, rows, cols) == idx
    assert np.array_equal(O.unpack_weights(p, 2, 16), w[:512])


def test_l2_loss_closed_form():
    """test/doctest_losses.cpp:22-52: value = (p - t)^2 / n, gradient = scale * 2 (p - t) / n."""
    for out_dim, batch, scale, p, t in [(16, 8, 1.0, 0.5, 0.25), (64, 16, 128.0, -1.0, 2.0)]:
        n = out_dim * batch
        values, grads = O.l2_loss(np.full((batch, out_dim), p), np.full((batch, out_dim), t), scale)
        assert np.allclose(values, (p - t) ** 2 / n, rtol=1e-6)
        assert np.allclose(grads, scale * 2 * (p - t) / n, rtol=1e-6)


def test_adam_matches_torch():
    import torch

    rng = np.random.default_rng(5)
    p0 = rng.normal(size=1000).astype(np.float32)
    p, m, v = p0.copy(), np.zeros_like(p0), np.zeros_like(p0)
    tp = torch.nn.Parameter(torch.from_numpy(p0.copy()))
    opt = torch.optim.Adam([tp], lr=1e-3, betas=(0.9, 0.99), eps=1e-15)
    for step in range(1, 6):
        g = rng.normal(size=1000).astype(np.float32) * 1e-3
        O.adam(p, m, v, g, step)
        tp.grad = torch.from_numpy(g.copy())
        opt.step()
    assert np.allclose(p, tp.detach().numpy(), rtol=1e-5, atol=1e-7)


def test_mlp_one_layer_constant_weights_closed_form():
    """test/doctest_swiftnet.cpp:44-51, 83-96: constant weights 0.01, input 1 => hidden = 0.01 * in,
    output = 0.01 * in * width * 0.01 on the real output columns."""
    W, in_w, out_w = 64, 64, 16
    w = np.full((2, W, W), 0.01, dtype=np.float32)
    w[1][:, out_w:] = 0.0
    interm = O.mlp_forward(np.ones((8, W), np.float32), w, 2, W, "relu", "none", bf16=True)
    assert np.allclose(interm[1], 0.01 * in_w, rtol=1e-2)
    assert np.allclose(interm[2][:, :out_w], 0.01 * in_w * W * 0.01, rtol=1e-2)
    assert not interm[2][:, out_w:].any()


def _golden_cases():
    z = np.load(os.path.join(GOLDEN, "mlp_ref_vectors.npz"))
    n = len([k for k in z.files if k.endswith("_cfg")])
    for ci in range(n):
        k = f"c{ci}"
        W, nh, a, oa = [int(v) for v in z[k + "_cfg"]]
        w = synth.xavier_weights(nh + 1, W, int(z[k + "_wseed"][0]))
        yield dict(W=W, nh=nh, act=ACT_NAME[a], oact=ACT_NAME[oa], w=w, x=z[k + "_x"], t=z[k + "_t"],
                   fwd=z[k + "_fwd"], grads=z[k + "_grads"], lgrads=z[k + "_lgrads"], dldi=z[k + "_dldi"])


def test_mlp_restatement_matches_reference_fixture():
    """The double-precision restatement reproduces the outputs of the reference's test/mlp.h
    (tests/golden/mlp_ref_vectors.npz, made by tests/golden/make_golden.py)."""
    for c in _golden_cases():
        n_mat = c["nh"] + 1
        interm = O.mlp_forward(c["x"], c["w"], n_mat, c["W"], c["act"], c["oact"], bf16=False)
        for b in range(c["x"].shape[0]):
            ok, rel = O.within_tolerance(interm[:, b, :], c["fwd"][b], 1e-5)
            assert ok, rel
            dy = (2 * (interm[-1, b] - c["t"][b]) / c["W"])[None, :]  # mlp.h:303-310 with batch 1
            ib, gr, dx = O.mlp_backward(dy, interm[:, b:b + 1, :], c["w"], n_mat, c["W"], c["act"], c["oact"],
                                        bf16=False)
            assert O.within_tolerance(ib[:, 0, :], c["lgrads"][b], 1e-5)[0]
            assert O.within_tolerance(dx[0], c["dldi"][b], 1e-5)[0]
            if b == 0:
                assert O.within_tolerance(gr, c["grads"][0], 1e-5)[0]


def test_bf16_faithful_restatement_within_reference_tolerance_of_double():
    """The bf16 rounding points move the result by less than the reference's own 1e-2 tolerance
    (test/doctest_swiftnet.cpp:931-966 compares the device against the double MLP at 1e-2)."""
    for c in _golden_cases():
        n_mat = c["nh"] + 1
        w16, x16 = O.bf16_round(c["w"]), O.bf16_round(c["x"])
        a = O.mlp_forward(x16, w16, n_mat, c["W"], c["act"], c["oact"], bf16=True)
        b = O.mlp_forward(x16, w16, n_mat, c["W"], c["act"], c["oact"], bf16=False)
        ok, rel = O.within_tolerance(a[-1], b[-1], 1e-2)
        assert ok, rel


def test_reference_host_mlp_live_when_available():
    """Where the reference's mlp.h could be compiled (oracle/_ref), check against it directly as well."""
    if O.ref_lib() is None:
        pytest.skip("oracle/_ref/libref_mlp.so not built on this machine")
    W, n_mat = 32, 3
    w = synth.xavier_weights(n_mat, W, 77).astype(np.float64)
    rng = np.random.default_rng(78)
    x, t = rng.uniform(-1, 1, W), rng.uniform(-1, 1, W)
    r = O.ref_mlp_sample(W, n_mat, "relu", "none", x, t, weights=w)
    interm = O.mlp_forward(x[None, :], w, n_mat, W, "relu", "none", bf16=False)
    assert O.within_tolerance(interm[:, 0, :], r["fwd"], 1e-5)[0]
    # the reference's own weight initialisation (mt19937 seed 42) exported in the (in x out) order
    r2 = O.ref_mlp_sample(W, n_mat, "relu", "none", x, t, weights=None, init_mode=1)
    interm2 = O.mlp_forward(x[None, :], r2["weights"], n_mat, W, "relu", "none", bf16=False)
    assert O.within_tolerance(interm2[:, 0, :], r2["fwd"], 1e-5)[0]


def test_frequency_encoding_closed_forms():
    """The reference's expectations (test/doctest_encodings.cpp:486-560, test/python/test_encodings.py:611-633):
    sin / cos of pi x 2^k per feature, padding columns 1, tolerance 1e-4."""
    out = O.frequency_forward(np.array([[1.234]], np.float32), 1, padded=4)
    assert np.allclose(out[0], [math.sin(math.pi * 1.234), math.cos(math.pi * 1.234), 1, 1], atol=1e-4)
    x = np.arange(6, dtype=np.float32).reshape(2, 3)
    out = O.frequency_forward(x, 2, padded=14)
    exp = np.ones((2, 14))
    for r in range(2):
        for f in range(3):
            for k in range(2):
                exp[r, f * 4 + 2 * k] = math.sin(math.pi * (1 << k) * x[r, f])
                exp[r, f * 4 + 2 * k + 1] = math.cos(math.pi * (1 << k) * x[r, f])
    assert O.within_tolerance(out, exp.astype(np.float32), 1e-4)[0]
    assert np.abs(out - exp).max() < 1e-4


def test_identity_pads_with_ones():
    """include/encodings/identity.h:63-77, test/doctest_encodings.cpp:156-195."""
    x = np.array([[0.25, 0.5]], dtype=np.float32)
    out = O.identity_forward(x, 8, scale=2.0, offset=1.0)
    assert np.allclose(out[0], [1.5, 2.0, 1, 1, 1, 1, 1, 1])


def test_spherical_harmonics_known_answer_and_definition():
    """test/python/test_encodings.py:377-573 (degree 4, input ones -> direction (1, 1, 1)) and
    test/doctest_encodings.cpp:197-231 (degree 1, padded with ones); beyond degree 4 the reference has no vectors, so
    the restatement is checked against an independent evaluation of the defining formula (scipy's complex spherical
    harmonics, which carry the same Condon-Shortley phase) on the unit sphere, and against orthonormality."""
    kat = [0.2821, -0.4886, 0.4886, -0.4886, 1.0925, -1.0925, 0.6308, -1.0925, 0.0, -1.1801, 2.8906, -1.8282, 0.7464,
           -1.8282, 0.0, 1.1801]
    out = O.spherical_harmonics_forward(np.ones((10, 3), np.float32), 4)
    assert np.allclose(out, np.array(kat, np.float32)[None, :], atol=1e-3)
    x = np.arange(6, dtype=np.float32).reshape(2, 3)
    assert np.allclose(O.spherical_harmonics_forward(x, 1, padded=3), [[0.2821, 1.0, 1.0]] * 2, atol=1e-3)
    from scipy.special import sph_harm_y

    rng = np.random.default_rng(0)
    v = rng.normal(size=(500, 3))
    v /= np.linalg.norm(v, axis=1, keepdims=True)
    inp = ((v + 1) / 2).astype(np.float32)
    out = O.spherical_harmonics_forward(inp, 8)
    d = inp.astype(np.float64) * 2 - 1
    az, pol = np.arctan2(d[:, 1], d[:, 0]), np.arccos(np.clip(d[:, 2] / np.linalg.norm(d, axis=1), -1, 1))
    for l in range(8):
        for m in range(-l, l + 1):
            y = sph_harm_y(l, abs(m), pol, az)
            ref = np.sqrt(2) * y.real if m > 0 else (np.sqrt(2) * y.imag if m < 0 else y.real)
            assert np.abs(out[:, l * (l + 1) + m] - ref).max() < 2e-5, (l, m)
    # orthonormality over the sphere (Monte-Carlo, 200k directions): the Gram matrix is the identity
    v = rng.normal(size=(200000, 3))
    v /= np.linalg.norm(v, axis=1, keepdims=True)
    y = O.spherical_harmonics_forward(((v + 1) / 2).astype(np.float32), 8).astype(np.float64)
    gram = 4 * np.pi * (y.T @ y) / len(v)
    assert np.abs(gram - np.eye(64)).max() < 0.05


def test_frequency_backward_input_is_the_derivative_of_the_forward():
    """include/encodings/frequency.h:72-73, 91-131: dL/dx = sum_k dL/dy_k 2^f pi cos(arg_k); checked against central
    differences of the pinned forward."""
    rng = np.random.default_rng(3)
    x = rng.uniform(-1, 1, (7, 2)).astype(np.float32)
    dy = rng.uniform(-1, 1, (7, 2 * 3 * 2 + 4)).astype(np.float32)  # padded output: the padding carries no gradient
    dx = O.frequency_backward_input(x, dy, 3)
    eps = 1e-3
    for j in range(2):
        xp, xm = x.copy(), x.copy()
        xp[:, j] += eps
        xm[:, j] -= eps
        fp = O.frequency_forward(xp, 3, padded=16).astype(np.float64)
        fm = O.frequency_forward(xm, 3, padded=16).astype(np.float64)
        num = ((fp - fm) * dy).sum(1) / (xp[:, j].astype(np.float64) - xm[:, j])
        assert np.allclose(num, dx[:, j], rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("interp", ["Linear", "Smoothstep"])
def test_grid_backward_input_is_the_derivative_of_the_forward(interp):
    """dL/dinput of the grid against central differences of the pinned forward (2-D and 3-D)."""
    for dims in (2, 3):
        g = O.Grid(n_dims_to_encode=dims, n_levels=4, log2_hashmap_size=12, base_resolution=4, interpolation=interp)
        rng = np.random.default_rng(dims)
        x = rng.uniform(0.05, 0.95, (32, dims)).astype(np.float32)
        t = rng.uniform(-1, 1, g.n_params).astype(np.float32)
        dy = rng.uniform(-1, 1, (32, 8)).astype(np.float32)
        dx = g.backward_input(x, t, dy)
        eps = 1e-4
        for d in range(dims):
            xp, xm = x.copy(), x.copy()
            xp[:, d] += eps
            xm[:, d] -= eps
            num = ((g.forward(xp, t).astype(np.float64) - g.forward(xm, t).astype(np.float64)) * dy).sum(1) \
                / (xp[:, d].astype(np.float64) - xm[:, d])
            # (a sample within eps of a cell boundary sees a kink: allow a few outliers)
            close = np.isclose(num, dx[:, d], rtol=5e-3, atol=5e-3 * np.abs(dx).max())
            assert close.mean() >= 0.9, (dims, d, close.mean())
    assert not O.Grid(n_dims_to_encode=2, n_levels=2, interpolation="Nearest").backward_input(
        x[:, :2], np.zeros(O.Grid(n_dims_to_encode=2, n_levels=2, interpolation="Nearest").n_params, np.float32),
        dy[:, :4]).any()
