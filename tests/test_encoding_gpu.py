"""GPU parity tests of the hash-grid and identity encodings, L2 loss and Adam, through the C ABI."""
import json
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")
from oracle import oracle as O  # noqa: E402
from tests import synth  # noqa: E402

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
BENCH_GRID = dict(otype="HashGrid", n_dims_to_encode=3, n_levels=16, n_features_per_level=2, log2_hashmap_size=19,
                  base_resolution=16, per_level_scale=2.0)


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()


def test_grid_known_answer_vector(tnn_lib):
    """test/doctest_encodings.cpp:234-285 on the device."""
    kat = json.load(open(os.path.join(GOLDEN, "grid_kat.json")))
    enc = tnn_lib.create_encoding("HashGrid", kat["config"], kat["padded_output_width"], seed=1)
    n = enc.n_params()
    assert n == kat["n_params"]
    enc.set_params(_t(np.arange(n, dtype=np.float64) / (n / 2.0) - 1.0))
    out = enc.fwd(torch.ones((1, 3), device="cuda")).cpu().numpy()
    ok, rel = O.within_tolerance(out[0], kat["expected"], kat["tolerance"])
    assert ok, rel


def test_grid_level_table_matches_oracle(tnn_lib):
    enc = tnn_lib.create_encoding("HashGrid", BENCH_GRID, 64, seed=1)
    g = O.Grid(n_dims_to_encode=3)
    for l in range(16):
        off, size, scale, res = enc.level_info(l)
        assert off == g.offsets[l] and size == g.offsets[l + 1] - g.offsets[l]
        assert res == 16 * 2 ** l


@pytest.mark.parametrize("cfg", [
    dict(n_dims_to_encode=3),
    dict(n_dims_to_encode=2),
    dict(n_dims_to_encode=3, n_levels=8, n_features_per_level=4, log2_hashmap_size=14, base_resolution=8,
         per_level_scale=1.5),
    dict(n_dims_to_encode=2, n_levels=4, n_features_per_level=1, log2_hashmap_size=12, interpolation="Smoothstep"),
    dict(n_dims_to_encode=3, n_levels=4, n_features_per_level=8, log2_hashmap_size=10, base_resolution=4,
         interpolation="Nearest"),
    dict(n_dims_to_encode=2, n_levels=5, type="Dense", base_resolution=4),
    dict(n_dims_to_encode=3, n_levels=4, type="Tiled", base_resolution=8, hash="Prime"),
])
def test_grid_forward_bit_exact_and_backward(tnn_lib, cfg):
    """Forward: bit-exact against the restatement (same fp32 operation order).  Backward: the sum is
    order-dependent in fp32, so it is compared at 1e-5 relative against a double accumulation; the
    deterministic path must also repeat bit for bit."""
    g = O.Grid(**cfg)
    full = dict(otype="HashGrid", **cfg)
    F, NL = g.F, g.n_levels
    padded = ((NL * F + 15) // 16) * 16
    enc = tnn_lib.create_encoding("HashGrid", full, padded, seed=3)
    assert enc.n_params() == g.n_params
    rng = np.random.default_rng(100)
    for batch in (1, 37, 4096):
        x = rng.uniform(0, 1, (batch, g.D)).astype(np.float32)
        table = rng.uniform(-1, 1, g.n_params).astype(np.float32)
        enc.set_params(_t(table))
        ref = g.forward(x, table, padded=padded)
        out = enc.fwd(_t(x)).cpu().numpy()
        assert np.array_equal(out, ref)
        out16 = enc.fwd(_t(x), out_dtype=torch.bfloat16).float().cpu().numpy()
        assert np.array_equal(out16, O.bf16_round(ref))
        dy = rng.uniform(-1, 1, (batch, padded)).astype(np.float32)
        gref = g.backward(x, dy)
        for det in (False, True, 2):  # fp32 atomics, fixed-point atomics, atomic-free segmented reduction
            _, grads = enc.bwd_with_encoding_grad(_t(dy), _t(x), False, False, deterministic=det)
            ok, rel = O.within_tolerance(grads.cpu().numpy().reshape(-1), gref, 1e-5)
            assert ok, (det, rel)
        for det in (True, 2):
            _, g1 = enc.bwd_with_encoding_grad(_t(dy), _t(x), False, False, deterministic=det)
            _, g2 = enc.bwd_with_encoding_grad(_t(dy), _t(x), False, False, deterministic=det)
            assert torch.equal(g1, g2)


@pytest.mark.parametrize("deterministic", [False, True, 2])
@pytest.mark.parametrize("dy_dtype", [torch.float32, torch.bfloat16])
def test_grid_backward_hand_checked_fixture(tnn_lib, deterministic, dy_dtype):
    """The hand-derived gradient of tests/golden/grid_backward_handcheck.json (see make_grid_backward_fixture.py) on
    the device, through both backward paths: every weight and upstream value is a binary fraction, so the sums are
    exact in fp32 (and in bf16 for the upstream values) whatever the order."""
    k = json.load(open(os.path.join(GOLDEN, "grid_backward_handcheck.json")))
    enc = tnn_lib.create_encoding("HashGrid", dict(otype="HashGrid", **k["config"]), None, seed=1)
    assert enc.n_params() == k["n_params"]
    x, dy = _t(k["x"]), _t(k["dy"]).to(dy_dtype)
    _, g = enc.bwd_with_encoding_grad(dy, x, False, False, deterministic=deterministic)
    assert np.array_equal(g.cpu().numpy().reshape(-1), np.array(k["expected_grad"], dtype=np.float32))


def test_grid_odd_padded_width(tnn_lib):
    """A padded output width that is odd leaves every second row unaligned for two-feature vector stores: the kernel
    must fall back to scalar stores (any padded width >= the natural one is valid, grid.h:683-694)."""
    cfg = dict(n_dims_to_encode=3, n_levels=16, n_features_per_level=2, log2_hashmap_size=12, base_resolution=4)
    g = O.Grid(**cfg)
    enc = tnn_lib.create_encoding("HashGrid", dict(otype="HashGrid", **cfg), 33, seed=1)
    table = synth.grid_table(g.n_params)
    enc.set_params(_t(table))
    p = np.random.default_rng(4).uniform(0, 1, (257, 3)).astype(np.float32)
    ref = g.forward(p, table, padded=33)
    assert np.array_equal(enc.fwd(_t(p)).cpu().numpy(), ref)
    out16 = enc.fwd(_t(p), out_dtype=torch.bfloat16).float().cpu().numpy()
    assert np.array_equal(out16, O.bf16_round(ref))


def test_grid_deterministic_backward_reports_non_finite_upstream(tnn_lib):
    """An inf or NaN in dL/dy must not disappear in the integer accumulation: every gradient of the call is NaN, so a
    loss-scale overflow check on the gradients still fires (the fp32 path propagates it into the entries it touches)."""
    cfg = dict(n_dims_to_encode=2, n_levels=4, n_features_per_level=2, log2_hashmap_size=10, base_resolution=4)
    enc = tnn_lib.create_encoding("HashGrid", dict(otype="HashGrid", **cfg), None, seed=1)
    x = torch.rand((64, 2), device="cuda")
    dy = torch.rand((64, 8), device="cuda")
    dy[5, 3] = float("nan")
    _, g = enc.bwd_with_encoding_grad(dy, x, False, False, deterministic=True)
    assert torch.isnan(g).all()
    _, g = enc.bwd_with_encoding_grad(dy, x, False, False, deterministic=False)
    assert torch.isnan(g).any()
    dy[5, 3] = 0.25
    _, g = enc.bwd_with_encoding_grad(dy, x, False, False, deterministic=True)
    assert torch.isfinite(g).all()


def test_grid_backward_zero_upstream(tnn_lib):
    """test/doctest_encodings.cpp:286-341: zero upstream gradient => zero gradients, parameters untouched."""
    enc = tnn_lib.create_encoding("HashGrid", BENCH_GRID, 32, seed=1)
    enc.set_params(torch.ones(enc.n_params(), device="cuda"))
    _, grads = enc.bwd_with_encoding_grad(torch.zeros((8, 32), device="cuda"), torch.ones((8, 3), device="cuda"),
                                          False, False)
    assert not grads.any().item()
    assert torch.equal(enc.get_params().reshape(-1), torch.ones(enc.n_params(), device="cuda"))


@pytest.mark.parametrize("cfg", [
    dict(n_dims_to_encode=3, n_levels=6, base_resolution=2, log2_hashmap_size=12),          # levels 0, 1 of 6
    dict(n_dims_to_encode=3, n_levels=5, base_resolution=2, log2_hashmap_size=6),           # every level (hashed too)
    dict(n_dims_to_encode=2, n_levels=6, n_features_per_level=4, base_resolution=2, log2_hashmap_size=10),
    dict(n_dims_to_encode=3, n_levels=3, n_features_per_level=1, base_resolution=2, interpolation="Nearest"),
])
def test_grid_backward_with_coarse_levels_in_shared_memory(tnn_lib, cfg):
    """At 2^16 samples the first levels of these small grids get thousands of contributions per entry: the backward
    kernels accumulate them per CTA in shared memory and add each copy to the table gradient once.  Same sums as the
    oracle's (1e-5 against its double accumulation), the fixed-point path still repeats bit for bit, with fp32 and
    bf16 upstream gradients."""
    g = O.Grid(**cfg)
    F, NL = g.F, g.n_levels
    padded = ((NL * F + 15) // 16) * 16
    enc = tnn_lib.create_encoding("HashGrid", dict(otype="HashGrid", **cfg), padded, seed=3)
    batch = 1 << 16
    rng = np.random.default_rng(7)
    x = rng.uniform(0, 1, (batch, g.D)).astype(np.float32)
    dy = O.bf16_round(rng.uniform(-1, 1, (batch, padded)).astype(np.float32))
    gref = g.backward(x, dy)
    for dt in (torch.float32, torch.bfloat16):
        for det in (False, True):
            _, grads = enc.bwd_with_encoding_grad(_t(dy).to(dt), _t(x), False, False, deterministic=det)
            ok, rel = O.within_tolerance(grads.cpu().numpy().reshape(-1), gref, 1e-5)
            assert ok, (dt, det, rel)
    _, g1 = enc.bwd_with_encoding_grad(_t(dy), _t(x), False, False, deterministic=True)
    _, g2 = enc.bwd_with_encoding_grad(_t(dy), _t(x), False, False, deterministic=True)
    assert torch.equal(g1, g2)


def test_grid_benchmark_config_against_oracle(tnn_lib):
    """Benchmark grid (16 x 2, T = 2^19, base 16) at 2^16 samples, bf16 dy as the network hands it over."""
    g = O.Grid(n_dims_to_encode=3)
    enc = tnn_lib.create_encoding("HashGrid", BENCH_GRID, 64, seed=3)
    batch = 1 << 16
    x = synth.uniform_inputs(batch, 3, 100, 0.0, 1.0)
    table = synth.grid_table(g.n_params, 3)
    enc.set_params(_t(table))
    assert np.array_equal(enc.fwd(_t(x)).cpu().numpy(), g.forward(x, table, padded=64))
    dy = O.bf16_round(np.random.default_rng(5).uniform(-1, 1, (batch, 64)).astype(np.float32) / batch)
    _, grads = enc.bwd_with_encoding_grad(_t(dy).to(torch.bfloat16), _t(x), False, False)
    ok, rel = O.within_tolerance(grads.cpu().numpy().reshape(-1), g.backward(x, dy), 1e-5)
    assert ok, rel


def test_grid_adjoint_property_at_full_size(tnn_lib):
    """Size-independent check at the benchmark batch (2^20): <forward(x; T), dy> == <T, backward(x, dy)>."""
    enc = tnn_lib.create_encoding("HashGrid", BENCH_GRID, 64, seed=3)
    batch = 1 << 20
    gen = torch.Generator(device="cuda").manual_seed(100)
    x = torch.rand((batch, 3), device="cuda", generator=gen)
    table = torch.rand(enc.n_params(), device="cuda", generator=gen) * 2 - 1
    enc.set_params(table)
    dy = torch.rand((batch, 64), device="cuda", generator=gen) * 2 - 1
    out = enc.fwd(x)
    _, grads = enc.bwd_with_encoding_grad(dy, x, False, False)
    lhs = (out.double() * dy.double()).sum().item()
    rhs = (table.double() * grads.reshape(-1).double()).sum().item()
    assert abs(lhs - rhs) <= 1e-5 * abs(lhs)


def test_bound_parameter_storage_is_used_in_place(tnn_lib):
    """tnn_encoding_bind_params: the kernels read the caller's tensor; in-place updates need no set_params."""
    cfg = dict(otype="HashGrid", n_dims_to_encode=2, n_levels=4, n_features_per_level=2, log2_hashmap_size=10,
               base_resolution=4, per_level_scale=2.0)
    enc = tnn_lib.create_encoding("HashGrid", cfg, 8, seed=1)
    x = _t(synth.uniform_inputs(256, 2, 5, 0.0, 1.0))
    table = torch.rand(enc.n_params(), device="cuda") - 0.5
    enc.set_params(table)
    ref = enc.fwd(x).clone()
    bound = table.clone()
    enc.bind_params(bound)
    assert torch.equal(enc.fwd(x), ref)
    bound.mul_(2.0)  # an optimiser step would do this
    assert torch.equal(enc.fwd(x), enc.fwd(x)) and torch.allclose(enc.fwd(x), 2.0 * ref)
    assert torch.equal(enc.get_params().reshape(-1), bound)
    enc.bind_params(None)  # back to the handle's own table, which still holds the first values
    assert torch.equal(enc.fwd(x), ref)


def test_identity_encoding(tnn_lib):
    """include/encodings/identity.h:63-77; test/doctest_encodings.cpp:156-195: pads with ones."""
    enc = tnn_lib.create_encoding("Identity", dict(otype="Identity", n_dims_to_encode=2, scale=1.0, offset=0.0), 64)
    assert enc.n_params() == 0 and enc.n_output_dims() == 64
    x = synth.uniform_inputs(1000, 2, 100, 0.0, 1.0)
    assert np.array_equal(enc.fwd(_t(x)).cpu().numpy(), O.identity_forward(x, 64))
    out16 = enc.fwd(_t(x), out_dtype=torch.bfloat16).float().cpu().numpy()
    assert np.array_equal(out16, O.bf16_round(O.identity_forward(x, 64)))


def test_frequency_encoding(tnn_lib):
    """include/encodings/frequency.h:63-80; expectations of test/doctest_encodings.cpp:486-560 (1e-4)."""
    import math
    enc = tnn_lib.create_encoding("Frequency", dict(otype="Frequency", n_frequencies=1, n_dims_to_encode=1), 4)
    assert enc.n_params() == 0 and enc.n_output_dims() == 4
    out = enc.fwd(_t(np.array([[1.234]], np.float32))).cpu().numpy()
    assert np.allclose(out[0], [math.sin(math.pi * 1.234), math.cos(math.pi * 1.234), 1, 1], atol=1e-4)
    enc = tnn_lib.create_encoding("Frequency", dict(otype="Frequency", n_frequencies=2, n_dims_to_encode=3), 14)
    x = np.arange(6, dtype=np.float32).reshape(2, 3)
    assert np.abs(enc.fwd(_t(x)).cpu().numpy() - O.frequency_forward(x, 2, padded=14)).max() < 1e-4
    # NeRF-style use: 3-D positions in [0, 1], 12 octaves, padded to the network width, bf16 for the MLP
    enc = tnn_lib.create_encoding("Frequency", dict(otype="Frequency", n_frequencies=12, n_dims_to_encode=3), 128)
    x = synth.uniform_inputs(4096 + 8, 3, 100, 0.0, 1.0)
    ref = O.frequency_forward(x, 12, padded=128)
    # arguments reach 2^11 pi: the device sine and the host sine agree to a few fp32 ulps of the argument
    assert np.abs(enc.fwd(_t(x)).cpu().numpy() - ref).max() < 1e-4
    out16 = enc.fwd(_t(x), out_dtype=torch.bfloat16).float().cpu().numpy()
    assert np.abs(out16 - ref).max() < 1e-2
    assert enc.bwd_with_encoding_grad(_t(ref), _t(x), False, False) == (None, None)


def test_frequency_backward_input(tnn_lib):
    """include/encodings/frequency.h:91-131 on the device, fp32 and bf16 upstream gradients."""
    enc = tnn_lib.create_encoding("Frequency", dict(n_dims_to_encode=3, n_frequencies=4), 32)
    rng = np.random.default_rng(2)
    x = rng.uniform(-1, 1, (1000, 3)).astype(np.float32)
    dy = rng.uniform(-1, 1, (1000, 32)).astype(np.float32)
    ref = O.frequency_backward_input(x, dy, 4)
    got = enc.bwd_input(_t(dy), _t(x)).cpu().numpy()
    assert np.allclose(got, ref, rtol=1e-4, atol=1e-4 * np.abs(ref).max())
    dyb = O.bf16_round(dy)
    got = enc.bwd_input(_t(dyb).to(torch.bfloat16), _t(x)).cpu().numpy()
    assert np.allclose(got, O.frequency_backward_input(x, dyb, 4), rtol=1e-4, atol=1e-4 * np.abs(ref).max())


def test_identity_backward_input(tnn_lib):
    enc = tnn_lib.create_encoding("Identity", dict(n_dims_to_encode=3, scale=2.0, offset=0.5), 16)
    dy = torch.rand((64, 16), device="cuda")
    x = torch.rand((64, 3), device="cuda")
    assert torch.equal(enc.bwd_input(dy, x), dy[:, :3] * 2.0)


@pytest.mark.parametrize("cfg", [dict(n_dims_to_encode=3), dict(n_dims_to_encode=2, interpolation="Smoothstep"),
                                 dict(n_dims_to_encode=3, n_levels=4, n_features_per_level=4, log2_hashmap_size=12)])
def test_grid_backward_input(tnn_lib, cfg):
    """dL/dinput of the hash grid (the product kernel_grid_backward_input forms, grid.h:247-268) against the oracle's
    double-precision derivative of the interpolation."""
    g = O.Grid(**cfg)
    enc = tnn_lib.create_encoding("HashGrid", dict(otype="HashGrid", **cfg), None, seed=1)
    table = np.random.default_rng(5).uniform(-1, 1, g.n_params).astype(np.float32)
    enc.set_params(_t(table))
    rng = np.random.default_rng(6)
    x = rng.uniform(0, 1, (2000, g.D)).astype(np.float32)
    dy = rng.uniform(-1, 1, (2000, g.n_levels * g.F)).astype(np.float32)
    ref = g.backward_input(x, table, dy)
    got = enc.bwd_input(_t(dy), _t(x)).cpu().numpy()
    ok, rel = O.within_tolerance(got, ref, 1e-4)
    assert ok, rel


def test_spherical_harmonics_encoding(tnn_lib):
    """include/encodings/spherical_harmonics.h:28-64: known answers of the reference's tests (degree 4 at ones,
    degree 1 padded) and the oracle on random inputs for every degree, fp32 and bf16 output."""
    enc = tnn_lib.create_encoding("SphericalHarmonics", dict(n_dims_to_encode=3, degree=4), None)
    kat = [0.2821, -0.4886, 0.4886, -0.4886, 1.0925, -1.0925, 0.6308, -1.0925, 0.0, -1.1801, 2.8906, -1.8282, 0.7464,
           -1.8282, 0.0, 1.1801]
    out = enc.fwd(torch.ones((10, 3), device="cuda")).cpu().numpy()
    assert out.shape == (10, 16) and np.allclose(out, np.array(kat, np.float32)[None, :], atol=1e-3)
    enc1 = tnn_lib.create_encoding("SphericalHarmonics", dict(n_dims_to_encode=3, degree=1), 3)
    out = enc1.fwd(_t(np.arange(6).reshape(2, 3))).cpu().numpy()
    assert np.allclose(out, [[0.2821, 1.0, 1.0]] * 2, atol=1e-3)
    x = np.random.default_rng(8).uniform(0, 1, (999, 3)).astype(np.float32)
    for degree in range(1, 9):
        enc = tnn_lib.create_encoding("SphericalHarmonics", dict(n_dims_to_encode=3, degree=degree), 64)
        ref = O.spherical_harmonics_forward(x, degree, padded=64)
        got = enc.fwd(_t(x)).cpu().numpy()
        assert np.abs(got - ref).max() <= 2e-5 * max(1.0, np.abs(ref).max()), degree
        got16 = enc.fwd(_t(x), out_dtype=torch.bfloat16).float().cpu().numpy()
        assert np.abs(got16 - ref).max() <= 1e-2 * np.abs(ref).max()
    with pytest.raises(tnn_lib.TnnError, match="not yet implemented"):
        enc.bwd_input(torch.zeros((8, 64), device="cuda"), torch.zeros((8, 3), device="cuda"))
    for bad in (dict(n_dims_to_encode=2, degree=4), dict(n_dims_to_encode=3, degree=9), dict(n_dims_to_encode=3, degree=0),
                dict(n_dims_to_encode=3)):
        with pytest.raises(tnn_lib.TnnError):
            tnn_lib.create_encoding("SphericalHarmonics", bad, None)


def test_grid_forward_fp16_output_and_wide_padding(tnn_lib):
    """fp16 output rows (for fp16 networks) and a padded width too wide for the tiled kernel's staging buffer."""
    cfg = dict(n_dims_to_encode=3, n_levels=8, n_features_per_level=2, log2_hashmap_size=12, base_resolution=4)
    g = O.Grid(**cfg)
    table = synth.grid_table(g.n_params) * 1e3
    p = np.random.default_rng(4).uniform(0, 1, (700, 3)).astype(np.float32)
    for padded in (16, 64, 400):
        enc = tnn_lib.create_encoding("HashGrid", dict(otype="HashGrid", **cfg), padded, seed=1)
        enc.set_params(_t(table))
        ref = g.forward(p, table, padded=padded)
        assert np.array_equal(enc.fwd(_t(p)).cpu().numpy(), ref)
        assert np.array_equal(enc.fwd(_t(p), out_dtype=torch.float16).float().cpu().numpy(), O.fp16_round(ref))
        assert np.array_equal(enc.fwd(_t(p), out_dtype=torch.bfloat16).float().cpu().numpy(), O.bf16_round(ref))


def test_unaligned_pointers_are_refused_not_faulted(tnn_lib):
    """The L2 and grid-backward kernels move 16 bytes at a time: an offset view handed through the ABI must come back
    as an error code with a message, never as a misaligned-address fault on the device."""
    lib = tnn_lib.load()
    s = tnn_lib.stream_ptr()
    pred = torch.zeros(64 * 64 + 8, dtype=torch.bfloat16, device="cuda")
    target = torch.zeros(64 * 64 + 4, dtype=torch.float32, device="cuda")
    grads = torch.zeros(64 * 64 + 8, dtype=torch.bfloat16, device="cuda")
    loss = torch.zeros(1, device="cuda")
    ok = lib.tnn_l2_loss(tnn_lib.dptr(pred), tnn_lib.dptr(target), 64, None, tnn_lib.dptr(grads), 64, 64, 1.0,
                         tnn_lib.dptr(loss), s)
    assert ok == 0
    for fn in (lib.tnn_l2_loss, lib.tnn_l2_loss_static):
        assert fn(tnn_lib.dptr(pred[1:]), tnn_lib.dptr(target), 64, None, tnn_lib.dptr(grads), 64, 64, 1.0,
                  tnn_lib.dptr(loss), s) != 0
        assert b"16-byte aligned" in lib.tnn_last_error()
        assert fn(tnn_lib.dptr(pred), tnn_lib.dptr(target[1:]), 64, None, tnn_lib.dptr(grads), 64, 64, 1.0,
                  tnn_lib.dptr(loss), s) != 0
        # narrow targets only need 4-byte alignment
        assert fn(tnn_lib.dptr(pred), tnn_lib.dptr(target[1:]), 3, None, tnn_lib.dptr(grads), 64, 64, 1.0,
                  tnn_lib.dptr(loss), s) == 0
    enc = tnn_lib.create_encoding("HashGrid", dict(otype="HashGrid", n_dims_to_encode=2, n_levels=2), None, seed=1)
    g = torch.zeros(enc.n_params() + 4, device="cuda")
    x = torch.rand((8, 2), device="cuda")
    dy = torch.rand((8, 4), device="cuda")
    rc = lib.tnn_encoding_backward(enc._h, tnn_lib.dptr(x), tnn_lib.dptr(dy), 2, tnn_lib.dptr(g[1:]), 8, 0, s)
    assert rc != 0 and b"16-byte aligned" in lib.tnn_last_error()
    torch.cuda.synchronize()  # the context is intact


def test_encoding_errors(tnn_lib):
    with pytest.raises(tnn_lib.TnnError, match="Unknown encoding type"):
        tnn_lib.create_encoding("OneBlob", dict(otype="OneBlob", n_dims_to_encode=3))
    with pytest.raises(tnn_lib.TnnError, match="simultaneously"):
        tnn_lib.create_encoding("HashGrid", dict(otype="HashGrid", n_levels=4, n_features=8))
    with pytest.raises(tnn_lib.TnnError, match="2 or 3"):
        tnn_lib.create_encoding("HashGrid", dict(otype="HashGrid", n_dims_to_encode=4))
    enc = tnn_lib.create_encoding("HashGrid", dict(otype="HashGrid", n_dims_to_encode=2, n_levels=2), 16)
    with pytest.raises(tnn_lib.TnnError):
        enc.fwd(torch.zeros((4, 3), device="cuda"))


def test_l2_loss_and_adam(tnn_lib):
    """include/losses/l2.h:19-41 and torch.optim.Adam semantics."""
    rng = np.random.default_rng(11)
    batch, stride = 4096, 64
    pred = O.bf16_round(rng.uniform(-1, 1, (batch, stride)).astype(np.float32))
    target = rng.uniform(-1, 1, (batch, stride)).astype(np.float32)
    vals, grads = O.l2_loss(pred, target, 1.0, bf16_grads=True)
    loss_sum, g, v = tnn_lib.l2_loss(_t(pred).to(torch.bfloat16), _t(target), 1.0, want_values=True)
    assert np.allclose(v.cpu().numpy(), vals, rtol=1e-6, atol=1e-12)
    assert np.array_equal(g.float().cpu().numpy(), grads)
    assert abs(loss_sum.item() - vals.astype(np.float64).sum()) <= 1e-5 * vals.sum()
    # narrow targets: the padding columns compare against zero
    t3 = target[:, :3].copy()
    vals3, _ = O.l2_loss(pred, t3, 1.0)
    _, _, v3 = tnn_lib.l2_loss(_t(pred).to(torch.bfloat16), _t(t3), 1.0, want_values=True)
    assert np.allclose(v3.cpu().numpy(), vals3, rtol=1e-6, atol=1e-12)

    n = 10000
    p0 = rng.normal(size=n).astype(np.float32)
    p, m, vv = p0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
    tp, tm, tv = _t(p0), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    ref = torch.nn.Parameter(torch.from_numpy(p0.copy()))
    opt = torch.optim.Adam([ref], lr=1e-3, betas=(0.9, 0.99), eps=1e-15)
    for step in range(1, 6):
        gr = (rng.normal(size=n) * 1e-3).astype(np.float32)
        O.adam(p, m, vv, gr, step)
        tnn_lib.adam_step(tp, tm, tv, _t(gr), step)
        ref.grad = torch.from_numpy(gr.copy())
        opt.step()
    assert np.allclose(tp.cpu().numpy(), p, rtol=1e-5, atol=1e-7)
    assert np.allclose(tp.cpu().numpy(), ref.detach().numpy(), rtol=1e-5, atol=1e-7)
    # table-sized vectors take the 16-byte path plus a scalar tail: same arithmetic
    n = (1 << 17) + 3
    p0 = rng.normal(size=n).astype(np.float32)
    p, m, vv = p0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
    tp, tm, tv = _t(p0), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    for step in range(1, 4):
        gr = (rng.normal(size=n) * 1e-3).astype(np.float32)
        O.adam(p, m, vv, gr, step)
        tnn_lib.adam_step(tp, tm, tv, _t(gr), step)
    assert np.allclose(tp.cpu().numpy(), p, rtol=1e-5, atol=1e-7)
    assert np.allclose(tm.cpu().numpy(), m, rtol=1e-5, atol=1e-9) and np.allclose(tv.cpu().numpy(), vv, rtol=1e-5, atol=1e-12)
