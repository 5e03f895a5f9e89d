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
        for det in (False, True):
            _, grads = enc.bwd_with_encoding_grad(_t(dy), _t(x), False, False, deterministic=det)
            ok, rel = O.within_tolerance(grads.cpu().numpy().reshape(-1), gref, 1e-5)
            assert ok, (det, rel)
        _, g1 = enc.bwd_with_encoding_grad(_t(dy), _t(x), False, False, deterministic=True)
        _, g2 = enc.bwd_with_encoding_grad(_t(dy), _t(x), False, False, deterministic=True)
        assert torch.equal(g1, g2)


def test_grid_backward_zero_upstream(tnn_lib):
    """test/doctest_encodings.cpp:286-341: zero upstream gradient => zero gradients, parameters untouched."""
    enc = tnn_lib.create_encoding("HashGrid", BENCH_GRID, 32, seed=1)
    enc.set_params(torch.ones(enc.n_params(), device="cuda"))
    _, grads = enc.bwd_with_encoding_grad(torch.zeros((8, 32), device="cuda"), torch.ones((8, 3), device="cuda"),
                                          False, False)
    assert not grads.any().item()
    assert torch.equal(enc.get_params().reshape(-1), torch.ones(enc.n_params(), device="cuda"))


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


def test_encoding_errors(tnn_lib):
    with pytest.raises(tnn_lib.TnnError, match="outside the scope"):
        tnn_lib.create_encoding("SphericalHarmonics", dict(otype="SphericalHarmonics", degree=4, n_dims_to_encode=3))
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
