"""GPU parity tests of the fused MLP kernels, called through the C ABI, against the CPU oracle.

Tolerance: the reference's own - max|a - b| / max(|a|_inf, |b|_inf) <= 1e-2
(include/common/result_check.h:83-102, used at test/doctest_swiftnet.cpp:931-1248).
"""
import ctypes
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")
from oracle import oracle as O  # noqa: E402
from tests import synth  # noqa: E402

pytestmark = pytest.mark.gpu
TOL = 1e-2
A = {"relu": 0, "sigmoid": 4, "none": 8}
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _bf16(t):
    return torch.from_numpy(np.ascontiguousarray(t, dtype=np.float32)).cuda().to(torch.bfloat16)


def _net(L, W, nh, act, oact, w, in_w=None, out_w=None, use_bias=True):
    net = L.create_network(in_w or W, out_w or W, nh, A[act], A[oact], W, "torch.bfloat16", use_bias, seed=1)
    net.set_params(torch.from_numpy(np.ascontiguousarray(w, dtype=np.float32).reshape(-1)).cuda(), False)
    return net


def _check(value, target, tol=TOL):
    ok, rel = O.within_tolerance(value, target, tol)
    assert ok, f"relative error {rel:.3e} > {tol}"


@pytest.mark.parametrize("W", [16, 32, 64])
@pytest.mark.parametrize("nh", [1, 2, 4])
@pytest.mark.parametrize("act,oact", [("relu", "none"), ("none", "none"), ("sigmoid", "sigmoid"), ("relu", "relu"),
                                      ("none", "sigmoid"), ("sigmoid", "none")])
def test_forward_backward_matrix(tnn_lib, W, nh, act, oact):
    """The reference's forward / interm_bwd / dL/dinput / weight-gradient matrix
    (test/doctest_swiftnet.cpp:931-1210): batch {8..64} -> here 8, 64 and a ragged multi-tile batch."""
    for batch in (8, 64, 128 * 3 + 40):
        w, x = synth.mlp_case(W, nh, batch, w_seed=2, x_seed=100 + batch)
        n_mat = nh + 1
        net = _net(tnn_lib, W, nh, act, oact, w)
        interm = O.mlp_forward(x, w, n_mat, W, act, oact, bf16=True)
        xt = _bf16(x)
        y_inf = net.inference(xt)
        _check(y_inf.float().cpu().numpy(), interm[-1])
        y = net.fwd(xt)
        ig = net.interm_fwd().float().cpu().numpy()
        assert np.array_equal(ig[0], x)  # matrix 0 is the input copy
        for l in range(1, n_mat + 1):
            _check(ig[l], interm[l])
        assert np.array_equal(y.float().cpu().numpy(), ig[-1])
        rng = np.random.default_rng(7 + batch)
        dy = O.bf16_round((rng.uniform(-1, 1, (batch, W)) / batch).astype(np.float32))
        # the oracle continues from the activations the device stored, so one flipped bf16 rounding in the
        # forward pass is not counted twice
        ib, gr, dx = O.mlp_backward(dy, ig, w, n_mat, W, act, oact, bf16=True)
        dxg, g = net.bwd_no_encoding_grad(_bf16(dy), False, True, want_interm_bwd=True, grads_dtype=torch.float32)
        assert net.status() == 0
        g = g.cpu().numpy().reshape(n_mat, W, W)
        ibg = net._interm_bwd.float().cpu().numpy()
        for l in range(n_mat):
            _check(ibg[l], ib[l])
            _check(g[l], gr[l])
        _check(dxg.float().cpu().numpy().reshape(batch, W), dx)
        # the same backward pass from the input alone: one fused kernel recomputes the activations on chip
        assert net.recompute_supported()
        dxr, gr2 = net.bwd_from_input(xt, _bf16(dy), False, True, grads_dtype=torch.float32)
        assert net.status() == 0
        gr2 = gr2.cpu().numpy().reshape(n_mat, W, W)
        for l in range(n_mat):
            _check(gr2[l], gr[l])
        _check(dxr.float().cpu().numpy().reshape(batch, W), dx)
        _, gp = net.bwd_from_input(xt, _bf16(dy), True, False, grads_dtype=torch.float32)
        assert np.allclose(O.unpack_weights(gp.cpu().numpy().reshape(-1), n_mat, W).reshape(n_mat, W, W),
                           np.transpose(gr2, (0, 2, 1)), rtol=0, atol=0)


def test_backward_from_input_limits(tnn_lib):
    """Networks that do not fit the fused training kernel say so (and the stored-activation path serves them)."""
    w, _ = synth.mlp_case(128, 2, 8, w_seed=2, x_seed=1)
    assert not _net(tnn_lib, 128, 2, "relu", "none", w).recompute_supported()
    w, x = synth.mlp_case(64, 8, 64, w_seed=2, x_seed=1)
    net = _net(tnn_lib, 64, 8, "relu", "none", w)
    assert not net.recompute_supported()
    with pytest.raises(tnn_lib.TnnError, match="does not fit the fused kernel"):
        net.bwd_from_input(_bf16(x), _bf16(x), False, False)


@pytest.mark.parametrize("W,nh,variant,act,oact", [
    (128, 2, 0, "relu", "none"), (128, 4, 0, "relu", "none"), (128, 8, 0, "relu", "none"), (64, 8, 0, "relu", "none"),
    (32, 8, 0, "relu", "none"), (16, 8, 0, "relu", "none"), (64, 4, 256, "relu", "none"), (32, 2, 256, "relu", "none"),
    (128, 4, 0, "sigmoid", "sigmoid"), (64, 8, 0, "none", "relu"), (64, 2, 256, "sigmoid", "sigmoid")])
def test_wide_and_deep_networks(tnn_lib, W, nh, variant, act, oact):
    """The reference's sweep (benchmarks/benchmark_all.cpp: widths 16..128, up to 8+ hidden layers): networks whose
    weights do not stay resident (streamed through per-slot rings; variant 256 forces that path) and whose weight
    gradients need more than one pass over the tensor-memory accumulators."""
    for batch in (64, 128 * 150 + 8):
        w, x = synth.mlp_case(W, nh, batch, w_seed=3, x_seed=200 + batch)
        n_mat = nh + 1
        net = _net(tnn_lib, W, nh, act, oact, w)
        net.set_variant(variant)
        interm = O.mlp_forward(x, w, n_mat, W, act, oact, bf16=True)
        xt = _bf16(x)
        _check(net.inference(xt).float().cpu().numpy(), interm[-1])
        net.fwd(xt)
        ig = net.interm_fwd().float().cpu().numpy()
        for l in range(1, n_mat + 1):
            _check(ig[l], interm[l])
        dy = O.bf16_round((np.random.default_rng(9).uniform(-1, 1, (batch, W)) / batch).astype(np.float32))
        ib, gr, dx = O.mlp_backward(dy, ig, w, n_mat, W, act, oact, bf16=True)
        dxg, g = net.bwd_no_encoding_grad(_bf16(dy), False, True, want_interm_bwd=True, grads_dtype=torch.float32)
        assert net.status() == 0
        g = g.cpu().numpy().reshape(n_mat, W, W)
        ibg = net._interm_bwd.float().cpu().numpy()
        for l in range(n_mat):
            _check(ibg[l], ib[l])
            _check(g[l], gr[l])
        _check(dxg.float().cpu().numpy().reshape(batch, W), dx)


def test_inference_benchmark_self_check(tnn_lib):
    """benchmarks/benchmark_inference.h:39-48, 71: weights 1 / W, input 0.1, linear => every output is 0.1."""
    W, nh, batch = 64, 4, 1 << 12
    w = np.full((nh + 1, W, W), 1.0 / W, dtype=np.float32)
    net = _net(tnn_lib, W, nh, "none", "none", w)
    y = net.inference(_bf16(np.full((batch, W), 0.1, np.float32))).float().cpu().numpy()
    assert np.allclose(y, 0.1, rtol=1e-2)


def test_one_layer_constant_weights_padded_output(tnn_lib):
    """test/doctest_swiftnet.cpp:44-51, 83-96 with output width 16 < network width: padded columns are zero."""
    W, in_w, out_w, batch = 64, 64, 16, 64
    net = tnn_lib.create_network(in_w, out_w, 1, A["relu"], A["none"], W, "torch.bfloat16", True, seed=0)
    net.set_params(torch.full((2 * W * W,), 0.01, device="cuda"), False)
    y = net.inference(_bf16(np.ones((batch, W), np.float32))).float().cpu().numpy()
    assert np.allclose(y[:, :out_w], 0.01 * in_w * W * 0.01, rtol=1e-2)
    assert not y[:, out_w:].any()


def test_input_padding_rows_are_zeroed(tnn_lib):
    """Network.h:171-233: with 3 real inputs and bias, rows 16.. of the first matrix are zero; without
    bias rows 3.. are zero."""
    W = 64
    for use_bias, first_zero in ((True, 16), (False, 3)):
        net = tnn_lib.create_network(3, W, 1, A["relu"], A["none"], W, "torch.bfloat16", use_bias, seed=0)
        net.set_params(torch.ones(2 * W * W, device="cuda"), False)
        w0 = O.unpack_weights(net.get_params().float().cpu().numpy().reshape(-1), 2, W).reshape(2, W, W)[0]
        assert w0[:first_zero].all() and not w0[first_zero:].any()


def test_params_roundtrip_packed_and_unpacked(tnn_lib):
    """set_params(unpacked) -> get_params() is the packed vector; set_params(packed) is the identity
    (tnn_api.h:622-641, common.h:184-212)."""
    W, nh = 32, 2
    w = O.bf16_round(synth.xavier_weights(nh + 1, W, 9))
    net = _net(tnn_lib, W, nh, "relu", "none", w)
    packed = net.get_params().float().cpu().numpy().reshape(-1)
    assert np.array_equal(packed, O.pack_weights(w, nh + 1, W))
    net.set_params(torch.from_numpy(packed).cuda().to(torch.bfloat16), True)
    assert np.array_equal(net.get_params().float().cpu().numpy().reshape(-1), packed)


def test_packed_transposed_gradient_layout(tnn_lib):
    """pack_transpose_gradient (tnn_api.h:599-603): gradients come back in the weights' own layout."""
    W, nh, batch = 64, 2, 256
    w, x = synth.mlp_case(W, nh, batch)
    net = _net(tnn_lib, W, nh, "relu", "none", w)
    net.fwd(_bf16(x))
    dy = _bf16(np.random.default_rng(3).uniform(-1, 1, (batch, W)).astype(np.float32) / batch)
    _, g = net.bwd_no_encoding_grad(dy, False, False, grads_dtype=torch.float32)
    _, gp = net.bwd_no_encoding_grad(dy, True, False, grads_dtype=torch.float32)
    g = g.cpu().numpy().reshape(nh + 1, W, W)
    exp = O.pack_weights(np.ascontiguousarray(np.transpose(g, (0, 2, 1))), nh + 1, W)
    assert np.array_equal(gp.cpu().numpy().reshape(-1), exp)
    # bf16 gradients, as the reference returns them
    _, gb = net.bwd_no_encoding_grad(dy, True, False, grads_dtype=torch.bfloat16)
    _check(gb.float().cpu().numpy().reshape(-1), exp)


def test_backward_is_bitwise_reproducible(tnn_lib):
    """The weight-gradient reduction has a fixed summation order."""
    W, nh, batch = 64, 4, 128 * 400
    w, x = synth.mlp_case(W, nh, batch)
    net = _net(tnn_lib, W, nh, "relu", "none", w)
    net.fwd(_bf16(x))
    dy = _bf16(np.random.default_rng(4).uniform(-1, 1, (batch, W)).astype(np.float32) / batch)
    g1 = net.bwd_no_encoding_grad(dy, True, False, grads_dtype=torch.float32)[1].clone()
    g2 = net.bwd_no_encoding_grad(dy, True, False, grads_dtype=torch.float32)[1]
    assert torch.equal(g1, g2)


def test_reference_fixture_through_the_device(tnn_lib):
    """Outputs of the reference's own host MLP (tests/golden/mlp_ref_vectors.npz) vs the device, 1e-2."""
    z = np.load(os.path.join(GOLDEN, "mlp_ref_vectors.npz"))
    names = {0: "relu", 4: "sigmoid", 8: "none"}
    for ci in range(len([k for k in z.files if k.endswith("_cfg")])):
        k = f"c{ci}"
        W, nh, a, oa = [int(v) for v in z[k + "_cfg"]]
        w = synth.xavier_weights(nh + 1, W, int(z[k + "_wseed"][0]))
        net = _net(tnn_lib, W, nh, names[a], names[oa], w)
        x = np.zeros((8, W), np.float32)
        x[: z[k + "_x"].shape[0]] = z[k + "_x"]
        y = net.inference(_bf16(x)).float().cpu().numpy()
        _check(y[: z[k + "_x"].shape[0]], z[k + "_fwd"][:, -1, :])


def test_edge_cases_and_errors(tnn_lib):
    W, nh = 64, 2
    w, x = synth.mlp_case(W, nh, 16)
    net = _net(tnn_lib, W, nh, "relu", "none", w)
    # empty batch: nothing to do, empty result
    assert net.inference(torch.empty((0, W), dtype=torch.bfloat16, device="cuda")).shape == (0, W)
    # batch not divisible by 8: SwiftNetMLP.h:293-302
    with pytest.raises(tnn_lib.TnnError, match="divisible by 8"):
        net.inference(_bf16(x[:12]))
    # wrong width
    with pytest.raises(tnn_lib.TnnError):
        net.inference(_bf16(x[:, :32]))
    # backward without forward of the same batch
    net.fwd(_bf16(x))
    with pytest.raises(tnn_lib.TnnError):
        net.bwd_no_encoding_grad(_bf16(np.zeros((8, W), np.float32)), True, True)
    # wrong parameter count: Network.h:94-101
    with pytest.raises(tnn_lib.TnnError, match="does not match"):
        net.set_params(torch.zeros(5, device="cuda"), False)


def test_linearity_at_full_size(tnn_lib):
    """Size-independent property at the benchmark batch (2^22): a linear network is linear -
    f(2x) = 2 f(x) exactly in bf16 (scaling by 2 commutes with rounding) - and rows are independent."""
    W, nh, batch = 64, 4, 1 << 22
    w = O.bf16_round(synth.xavier_weights(nh + 1, W, 0))
    net = _net(tnn_lib, W, nh, "none", "none", w)
    g = torch.Generator(device="cuda").manual_seed(100)
    x = (torch.rand((batch, W), device="cuda", generator=g) * 2 - 1).to(torch.bfloat16)
    y1 = net.inference(x)
    y2 = net.inference(x * 2)
    assert torch.equal(y2, y1 * 2)
    # independence of rows: any slice run alone gives the same bits
    y_slice = net.inference(x[128 * 1000: 128 * 1000 + 4096].contiguous())
    assert torch.equal(y_slice, y1[128 * 1000: 128 * 1000 + 4096])
    # spot check of rows against the oracle
    idx = torch.arange(0, batch, batch // 64, device="cuda")
    xs = x[idx].float().cpu().numpy()
    interm = O.mlp_forward(xs, w, nh + 1, W, "none", "none", bf16=True)
    _check(y1[idx].float().cpu().numpy(), interm[-1])
