"""GPU parity tests of the benchmark configurations as configurations, through the C ABI, against the CPU oracle:

  C1  inference, 64 -> 4 x 64 ReLU -> 64, Xavier weights seed 0, inputs seed 100, batch 2^17 (whole batch)
  C2  fused training step of the same network at batch 2^20 (whole batch), and a short Adam trajectory
  C4  hash grid -> 2 x 64 network -> 3 outputs: the gradient that reaches the table through the network's dL/dinput
  C5  2-D coordinates -> identity encoding padded to 64 (folded into the first-layer load) -> 4 x 64 -> 3 outputs
      with narrow (3-column) targets staged by bulk copies, and the data-parallel step over NCCL on two GPUs

Reference tests these stand in for: test/doctest_swiftnet.cpp:931-1248 (forward / backward against mlp.h),
test/python/test_compare_torch_dpcpp.py:92-157 (training trajectories against torch)."""
import os
import socket
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
from oracle import oracle as O  # noqa: E402
from tests import synth  # noqa: E402

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
A = {"relu": 0, "sigmoid": 4, "none": 8}
TOL = 1e-2  # include/common/result_check.h:83-102 as used by test/doctest_swiftnet.cpp
W, NH = 64, 4
N_MAT = NH + 1


def _bf16(t):
    return torch.from_numpy(np.ascontiguousarray(t, dtype=np.float32)).cuda().to(torch.bfloat16)


def _check(value, target, tol=TOL, what=""):
    ok, rel = O.within_tolerance(value, target, tol)
    assert ok, (what, rel)


def _oracle_step(x, t, w, n_mat=N_MAT, act="relu", oact="none", want_dx=False):
    """Loss sum, packed weight gradients (n_mat x W^2) and optionally dL/dx of the oracle for encoded rows x."""
    interm = O.mlp_forward(x, w, n_mat, W, act, oact, bf16=True)
    tpad = np.zeros((x.shape[0], W), np.float32)
    tpad[:, : t.shape[1]] = t
    vals, dy = O.l2_loss(interm[-1], tpad, 1.0, bf16_grads=True)
    _, gr, dx = O.mlp_backward(dy, interm, w, n_mat, W, act, oact, bf16=True, want_dx=want_dx)
    packed = O.pack_weights(np.ascontiguousarray(np.transpose(gr, (0, 2, 1))).astype(np.float32), n_mat, W)
    return float(vals.astype(np.float64).sum()), packed.reshape(n_mat, W * W), dx, interm


def _c5_case(batch, seed=100):
    """Coordinates, targets and weights of the image-regression configuration (bench.py holds the same recipe)."""
    q = np.random.default_rng(seed).uniform(0, 1, (batch, 2)).astype(np.float32)
    t = synth.sinusoid_targets(q, 3, 16, 32.0, seed=7)
    w = O.bf16_round(synth.xavier_weights(N_MAT, W, 6))
    w[-1][:, 3:] = 0.0  # Network::set_weights_matrices zeroes the padded output columns (Network.h:171-233)
    return q, t, w


def _c5_modules(tnn_lib, w):
    net = tnn_lib.create_network(W, 3, NH, A["relu"], A["none"], W, "torch.bfloat16", True, seed=1)
    net.set_params(torch.from_numpy(w.reshape(-1)).cuda(), False)
    enc = tnn_lib.create_encoding("Identity", dict(n_dims_to_encode=2, scale=1.0, offset=0.0), W)
    return net, enc


# ------------------------------------------------------------------------------------------------ C1
def test_c1_inference_whole_batch(tnn_lib):
    batch = 1 << 17
    w, x = synth.mlp_case(W, NH, batch, w_seed=0, x_seed=100)
    net = tnn_lib.create_network(W, W, NH, A["relu"], A["none"], W, "torch.bfloat16", True, seed=0)
    net.set_params(torch.from_numpy(w.reshape(-1)).cuda(), False)
    y = net.inference(_bf16(x)).float().cpu().numpy()
    assert net.status() == 0
    ref = O.mlp_forward(x, w, N_MAT, W, "relu", "none", bf16=True)[-1]
    _check(y, ref, what="C1 output")
    # row by row as well: no row may be off by more than the tolerance on its own scale
    scale = np.maximum(np.abs(ref).max(axis=1), 1e-3)
    assert (np.abs(y - ref).max(axis=1) / scale).max() <= 5e-2


# ------------------------------------------------------------------------------------------------ C2
def test_c2_fused_training_step_whole_batch(tnn_lib):
    from tiny_dpcpp_nn.trainer import Trainer

    batch = 1 << 20
    w, x = synth.mlp_case(W, NH, batch, w_seed=0, x_seed=100)
    t = synth.uniform_inputs(batch, W, seed=1)
    net = tnn_lib.create_network(W, W, NH, A["relu"], A["none"], W, "torch.bfloat16", True, seed=0)
    net.set_params(torch.from_numpy(w.reshape(-1)).cuda(), False)
    tr = Trainer(net)
    loss = tr.forward_backward(_bf16(x), torch.from_numpy(t).cuda()).item()
    assert net.status() == 0
    exp_loss, exp_grads, _, _ = _oracle_step(x, t, w)
    assert abs(loss - exp_loss) <= 1e-4 * abs(exp_loss)
    g = tr.grads.cpu().numpy().reshape(N_MAT, W * W)
    for l in range(N_MAT):
        _check(g[l], exp_grads[l], what=f"C2 dW[{l}]")


def test_c2_adam_trajectory_matches_oracle(tnn_lib):
    """Three full steps (fused kernel, Adam on the fp32 master copy, bf16 weight refresh) against the oracle taking
    the same three steps on its own gradients.  Adam normalises the gradient, so a weight whose gradient is within
    rounding noise of zero can move the other way (by up to 2 lr per step); all others must agree closely."""
    from tiny_dpcpp_nn.trainer import Trainer

    batch, steps, lr = 1 << 14, 3, 1e-3
    w0 = synth.xavier_weights(N_MAT, W, 0)
    x = O.bf16_round(synth.uniform_inputs(batch, W, seed=100))
    t = synth.uniform_inputs(batch, W, seed=1)
    net = tnn_lib.create_network(W, W, NH, A["relu"], A["none"], W, "torch.bfloat16", True, seed=0)
    tr = Trainer(net, lr=lr, betas=(0.9, 0.99), eps=1e-15)
    p = O.pack_weights(w0, N_MAT, W).copy()
    tr.set_master_params(torch.from_numpy(p.copy()).cuda())
    m, v = np.zeros_like(p), np.zeros_like(p)
    xt, tt = _bf16(x), torch.from_numpy(t).cuda()
    for step in range(1, steps + 1):
        w_work = O.bf16_round(O.unpack_weights(p, N_MAT, W)).reshape(N_MAT, W, W)  # what the kernels read
        exp_loss, exp_grads, _, _ = _oracle_step(x, t, w_work)
        loss = tr.training_step(xt, tt).item()
        assert abs(loss - exp_loss) <= 2e-3 * abs(exp_loss), (step, loss, exp_loss)
        O.adam(p, m, v, exp_grads.reshape(-1).astype(np.float32), step, lr=lr)
    assert net.status() == 0 and tr.step == steps
    diff = np.abs(tr.master.cpu().numpy() - p)
    assert diff.max() <= 2.1 * lr * steps
    assert (diff <= 2e-5).mean() >= 0.99, (diff <= 2e-5).mean()
    # the weights the kernels read are the rounded master copy
    assert np.array_equal(net.get_params().float().cpu().numpy().reshape(-1), O.bf16_round(tr.master.cpu().numpy()))


# ------------------------------------------------------------------------------------------------ C5
@pytest.mark.parametrize("variant", [0, 64, 16])
def test_c5_step_with_folded_identity_encoding_and_narrow_targets(tnn_lib, variant):
    """Coordinates in, 3 targets per row: the encoded matrix never exists (variants 0 / 64: fused kernels; 16: the
    forward kernel encodes and stores it as matrix 0 for the backward kernel)."""
    from tiny_dpcpp_nn.trainer import Trainer

    batch = 128 * 148 * 2 + 72  # more than two tiles per SM and a ragged last tile
    q, t, w = _c5_case(batch)
    net, enc = _c5_modules(tnn_lib, w)
    net.set_variant(variant)
    tr = Trainer(net, encoding=enc)
    loss = tr.forward_backward(torch.from_numpy(q).cuda(), torch.from_numpy(t).cuda()).item()
    assert net.status() == 0
    x = O.bf16_round(O.identity_forward(q, W))
    exp_loss, exp_grads, _, _ = _oracle_step(x, t, w)
    assert abs(loss - exp_loss) <= 1e-4 * abs(exp_loss)
    g = tr.grads.cpu().numpy().reshape(N_MAT, W * W)
    for l in range(N_MAT):
        _check(g[l], exp_grads[l], what=f"C5 dW[{l}] variant {variant}")


def test_c5_step_equals_the_two_module_path(tnn_lib):
    """Folded encoding + narrow staged targets give the very bits of: identity kernel -> bf16 matrix -> training step
    with the same targets (both run the same GEMMs on the same operands)."""
    from tiny_dpcpp_nn.trainer import Trainer

    batch = 128 * 37 + 8
    q, t, w = _c5_case(batch, seed=3)
    net, enc = _c5_modules(tnn_lib, w)
    qt, tt = torch.from_numpy(q).cuda(), torch.from_numpy(t).cuda()
    fused = Trainer(net, encoding=enc)
    l1 = fused.forward_backward(qt, tt).clone()
    g1 = fused.grads.clone()
    plain = Trainer(net)
    l2 = plain.forward_backward(enc.fwd(qt, out_dtype=torch.bfloat16), tt)
    assert torch.equal(g1, plain.grads) and torch.equal(l1, l2)


def test_c5_inference_and_stored_forward(tnn_lib):
    batch = 128 * 300 + 8
    q, _, w = _c5_case(batch, seed=5)
    net, enc = _c5_modules(tnn_lib, w)
    qt = torch.from_numpy(q).cuda()
    x = O.bf16_round(O.identity_forward(q, W))
    interm = O.mlp_forward(x, w, N_MAT, W, "relu", "none", bf16=True)
    y = tnn_lib.nwe_inference(net, enc, qt).float().cpu().numpy()
    _check(y, interm[-1], what="C5 inference")
    assert np.all(y[:, 3:] == 0.0)  # padded output columns
    out = tnn_lib.nwe_forward(net, enc, qt).float().cpu().numpy()
    ig = net.interm_fwd().float().cpu().numpy()
    assert np.array_equal(ig[0], x)  # matrix 0 = the encoded input, bit for bit
    for l in range(1, N_MAT + 1):
        _check(ig[l], interm[l], what=f"C5 a[{l}]")
    assert np.array_equal(out, ig[-1])
    assert net.status() == 0


@pytest.mark.parametrize("n_in, batch, shift", [(2, 128 * 9 + 40, 0), (3, 128 * 5 + 48, 0), (1, 136, 0), (4, 128 * 700, 0),
                                                (2, 128 * 3 + 8, 1), (3, 24, 0), (7, 128 * 150 + 16, 0)])
def test_folded_identity_forward_equals_the_two_module_path(tnn_lib, n_in, batch, shift):
    """Inference (input tiles written by the issuer warps) and stored forward (by the producer warp) from fp32
    coordinates give the bits of identity kernel -> network: ragged last tiles, fewer tiles than slots, a coordinate
    pointer that is only 4-byte aligned, more coordinates than the encoder keeps in registers."""
    rng = np.random.default_rng(40 + n_in)
    w = O.bf16_round(synth.xavier_weights(N_MAT, W, 9))
    net = tnn_lib.create_network(n_in, 3, NH, A["relu"], A["none"], W, "torch.bfloat16", True, seed=1)
    net.set_params(torch.from_numpy(w.reshape(-1)).cuda(), False)
    enc = tnn_lib.create_encoding("Identity", {"n_dims_to_encode": n_in, "scale": 1.5, "offset": -0.25}, W)
    store = torch.from_numpy(rng.uniform(0, 1, batch * n_in + 4).astype(np.float32)).cuda()
    q = store[shift:shift + batch * n_in].view(batch, n_in)
    y_two = net.inference(enc.fwd(q, out_dtype=torch.bfloat16)).clone()
    y = tnn_lib.nwe_inference(net, enc, q)
    assert torch.equal(y, y_two)
    out = tnn_lib.nwe_forward(net, enc, q)
    assert torch.equal(out, y_two) and torch.equal(net.interm_fwd()[0], enc.fwd(q, out_dtype=torch.bfloat16))
    assert net.status() == 0


def test_narrow_targets_other_widths_and_alignments(tnn_lib):
    """Bulk-staged narrow targets at W = 32, an unaligned target pointer (falls back to per-thread loads), 63 of 64."""
    from tiny_dpcpp_nn.trainer import Trainer

    for width, nh, nt, offset in ((32, 3, 5, 0), (64, 2, 63, 0), (64, 4, 3, 1), (32, 2, 31, 0)):
        batch = 128 * 9 + 16
        w, x = synth.mlp_case(width, nh, batch, w_seed=8)
        t = synth.uniform_inputs(batch, nt, seed=2)
        net = tnn_lib.create_network(width, width, nh, A["relu"], A["none"], width, "torch.bfloat16", True, seed=1)
        net.set_params(torch.from_numpy(w.reshape(-1)).cuda(), False)
        tr = Trainer(net)
        buf = torch.empty(batch * nt + 4, dtype=torch.float32, device="cuda")
        tt = buf[offset:offset + batch * nt].view(batch, nt)  # offset 1: only 4-byte aligned
        tt.copy_(torch.from_numpy(t))
        loss = tr.forward_backward(_bf16(x), tt).item()
        assert net.status() == 0
        interm = O.mlp_forward(x, w, nh + 1, width, "relu", "none", bf16=True)
        tpad = np.zeros((batch, width), np.float32)
        tpad[:, :nt] = t
        vals, dy = O.l2_loss(interm[-1], tpad, 1.0, bf16_grads=True)
        _, gr, _ = O.mlp_backward(dy, interm, w, nh + 1, width, "relu", "none", bf16=True, want_dx=False)
        packed = O.pack_weights(np.ascontiguousarray(np.transpose(gr, (0, 2, 1))).astype(np.float32), nh + 1, width)
        assert abs(loss - float(vals.astype(np.float64).sum())) <= 1e-4 * abs(loss)
        _check(tr.grads.cpu().numpy(), packed, what=f"W{width} nt{nt}")


@pytest.mark.parametrize("out_w, nt, oact, width", [(8, 8, "none", 64), (8, 5, "relu", 64), (9, 9, "none", 64),
                                                     (3, 3, "relu", 64), (1, 1, "none", 32), (8, 3, "none", 32)])
def test_few_live_output_columns(tnn_lib, out_w, nt, oact, width):
    """Networks with at most 8 real outputs and a linear or ReLU output layer: the padded output columns are exactly
    zero and the fused kernel evaluates the loss on the first 8-column chunk of a row only (9 outputs: all columns).
    Loss and gradients as the oracle computes them over all columns."""
    from tiny_dpcpp_nn.trainer import Trainer

    nh, batch = 2, 128 * 5 + 24
    w, x = synth.mlp_case(width, nh, batch, w_seed=11)
    w[-1][:, out_w:] = 0.0  # what Network::set_weights_matrices makes of the padded output columns
    t = synth.uniform_inputs(batch, nt, seed=3)
    net = tnn_lib.create_network(width, out_w, nh, A["relu"], A[oact], width, "torch.bfloat16", True, seed=1)
    net.set_params(torch.from_numpy(w.reshape(-1)).cuda(), False)
    tr = Trainer(net)
    loss = tr.forward_backward(_bf16(x), torch.from_numpy(t).cuda()).item()
    assert net.status() == 0
    interm = O.mlp_forward(x, w, nh + 1, width, "relu", oact, bf16=True)
    tpad = np.zeros((batch, width), np.float32)
    tpad[:, :nt] = t
    vals, dy = O.l2_loss(interm[-1], tpad, 1.0, bf16_grads=True)
    _, gr, _ = O.mlp_backward(dy, interm, w, nh + 1, width, "relu", oact, bf16=True, want_dx=False)
    packed = O.pack_weights(np.ascontiguousarray(np.transpose(gr, (0, 2, 1))).astype(np.float32), nh + 1, width)
    assert abs(loss - float(vals.astype(np.float64).sum())) <= 1e-4 * abs(loss)
    _check(tr.grads.cpu().numpy(), packed, what=f"out {out_w} targets {nt} {oact}")


@pytest.mark.parametrize("width, nh, out_w, oact", [(64, 4, 3, "none"), (64, 2, 8, "relu"), (64, 8, 1, "none"),
                                                    (32, 3, 3, "none"), (32, 2, 5, "relu"), (64, 4, 9, "none"),
                                                    (64, 4, 3, "sigmoid"), (16, 2, 3, "none")])
def test_inference_of_networks_with_few_outputs(tnn_lib, width, nh, out_w, oact):
    """Inference of networks with at most 8 real outputs (linear / ReLU output: the output layer's epilogue writes the
    first chunk of a row only) gives the bits of the stored forward pass, whose kernel has no such path, zeros in the
    padded columns, and the oracle's values; 9 outputs, a sigmoid output and width 16 take the generic path."""
    for batch in (8, 128 + 16, 128 * 21 + 8, 128 * 148 * 5):  # fewer tiles than slots, ragged, several tiles per slot
        w, x = synth.mlp_case(width, nh, batch, w_seed=12)
        w[-1][:, out_w:] = 0.0
        net = tnn_lib.create_network(width, out_w, nh, A["relu"], A[oact], width, "torch.bfloat16", True, seed=1)
        net.set_params(torch.from_numpy(w.reshape(-1)).cuda(), False)
        xt = _bf16(x)
        y = net.inference(xt)
        assert torch.equal(y, net.fwd(xt)) and net.status() == 0
        if oact != "sigmoid":
            assert torch.all(y[:, out_w:] == 0)
        if batch <= 128 * 21 + 8:
            interm = O.mlp_forward(x, w, nh + 1, width, "relu", oact, bf16=True)
            _check(y.float().cpu().numpy(), interm[-1], what=f"W{width} L{nh} out {out_w} {oact} batch {batch}")


def test_workspace_lent_by_the_caller(tnn_lib):
    """The three-kernel path on a caller-owned workspace: no allocation inside the step; too small a workspace is an
    error with a message, not a reallocation."""
    import ctypes

    from tiny_dpcpp_nn.trainer import Trainer

    lib = tnn_lib.load()
    batch, width, nh = 4096, 128, 2  # width 128 trains through forward / loss / backward kernels
    w, x = synth.mlp_case(width, nh, batch, w_seed=8)
    t = synth.uniform_inputs(batch, width, seed=2)
    net = tnn_lib.create_network(width, width, nh, A["relu"], A["none"], width, "torch.bfloat16", True, seed=1)
    net.set_params(torch.from_numpy(w.reshape(-1)).cuda(), False)
    need = lib.tnn_network_workspace_bytes(net._h, batch)
    assert need == (nh + 1 + 2) * batch * width * 2
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    tnn_lib.check(lib.tnn_network_set_workspace(net._h, tnn_lib.dptr(ws), need))
    tr = Trainer(net)
    tr.forward_backward(_bf16(x), torch.from_numpy(t).cuda())
    g_lent = tr.grads.clone()
    tnn_lib.check(lib.tnn_network_set_workspace(net._h, tnn_lib.dptr(ws), need // 2))
    with pytest.raises(tnn_lib.TnnError, match="too small"):
        tr.forward_backward(_bf16(x), torch.from_numpy(t).cuda())
    tnn_lib.check(lib.tnn_network_set_workspace(net._h, None, 0))  # back to the library's own
    tr.forward_backward(_bf16(x), torch.from_numpy(t).cuda())
    assert torch.equal(g_lent, tr.grads) and net.status() == 0
    assert isinstance(lib.tnn_launch_count(), int) and lib.tnn_launch_count() > 0
    del ctypes


# ------------------------------------------------------------------------------------------------ C4
GRID_CFG = dict(otype="HashGrid", n_dims_to_encode=3, n_levels=16, n_features_per_level=2, log2_hashmap_size=19,
                base_resolution=16, per_level_scale=2.0)


def test_c4_table_gradient_through_the_network(tnn_lib):
    """Hash grid -> 2 x 64 ReLU network -> 3 outputs, one training pass through the C ABI: network weight gradients
    and the table gradient (dL/dinput of the network scattered back through the trilinear weights) against the
    oracle's chain (grid forward -> bf16 -> MLP forward -> L2 -> MLP backward with dL/dx -> bf16 -> grid backward)."""
    from tiny_dpcpp_nn.trainer import Trainer

    batch, nh = 1 << 14, 2
    n_mat = nh + 1
    grid = O.Grid(n_dims_to_encode=3, per_level_scale=2.0)
    rng = np.random.default_rng(100)
    pts = rng.uniform(0, 1, (batch, 3)).astype(np.float32)
    table = rng.uniform(-0.5, 0.5, grid.n_params).astype(np.float32)  # large enough for a non-trivial signal
    t = synth.sinusoid_targets(pts, 3, 8, 8.0, seed=5)
    w = O.bf16_round(synth.xavier_weights(n_mat, W, 4))
    w[0][32:, :] = 0.0  # rows beyond the 32 encoded features carry no signal (one_padded_input = 32)
    w[-1][:, 3:] = 0.0
    net = tnn_lib.create_network(32, 3, nh, A["relu"], A["none"], W, "torch.bfloat16", True, seed=1)
    net.set_params(torch.from_numpy(w.reshape(-1)).cuda(), False)
    enc = tnn_lib.create_encoding("HashGrid", GRID_CFG, W, seed=3)
    enc.set_params(torch.from_numpy(table).cuda())
    tr = Trainer(net, encoding=enc)
    tr.set_deterministic_encoding(True)
    loss = tr.forward_backward(torch.from_numpy(pts).cuda(), torch.from_numpy(t).cuda()).item()
    assert net.status() == 0
    x = O.bf16_round(grid.forward(pts, table, padded=W))
    exp_loss, exp_grads, dx, _ = _oracle_step(x, t, w, n_mat=n_mat, want_dx=True)
    assert abs(loss - exp_loss) <= 1e-3 * abs(exp_loss)
    g = tr.grads.cpu().numpy().reshape(n_mat, W * W)
    for l in range(n_mat):
        _check(g[l], exp_grads[l], what=f"C4 dW[{l}]")
    exp_table = grid.backward(pts, O.bf16_round(dx)[:, :32])
    got = tr.encoding_grads.cpu().numpy().astype(np.float64)
    for l in range(16):
        a, b = grid.offsets[l] * 2, grid.offsets[l + 1] * 2
        _check(got[a:b], exp_table[a:b], what=f"C4 table gradient, level {l}")


@pytest.mark.parametrize("width,nh,nt", [(64, 1, 3), (64, 2, 64), (64, 4, 3), (32, 3, 5), (32, 1, 32), (16, 2, 2)])
def test_dl_dinput_of_the_fused_training_kernel(tnn_lib, width, nh, nt):
    """The pipelined training kernel's extra backward step (dL/dinput = delta_0 W_0^T, stored by TMA) feeds a trainable
    encoding: the table gradient it produces must equal the one of the forward / loss / backward kernel path
    (variant 16), and the network gradients must be unchanged."""
    from tiny_dpcpp_nn.trainer import Trainer

    batch = 128 * 150 + 72
    cfg = dict(otype="HashGrid", n_dims_to_encode=3, n_levels=width // 4, n_features_per_level=2, log2_hashmap_size=12,
               base_resolution=4, per_level_scale=1.5)
    w = O.bf16_round(synth.xavier_weights(nh + 1, width, 9))
    rng = np.random.default_rng(5)
    pts = torch.from_numpy(rng.uniform(0, 1, (batch, 3)).astype(np.float32)).cuda()
    t = torch.from_numpy(rng.uniform(-1, 1, (batch, nt)).astype(np.float32)).cuda()
    out = []
    for variant in (0, 16):
        net = tnn_lib.create_network(width // 2, min(nt, width), nh, A["relu"], A["none"], width, "torch.bfloat16", True, seed=1)
        net.set_params(torch.from_numpy(w.reshape(-1)).cuda(), False)
        net.set_variant(variant)
        enc = tnn_lib.create_encoding("HashGrid", cfg, width, seed=3)
        enc.set_params(torch.from_numpy(np.random.default_rng(2).uniform(-0.5, 0.5, enc.n_params()).astype(np.float32)).cuda())
        tr = Trainer(net, encoding=enc)
        tr.set_deterministic_encoding(True)
        loss = tr.forward_backward(pts, t).item()
        assert net.status() == 0
        out.append((loss, tr.grads.clone(), tr.encoding_grads.clone()))
    assert abs(out[0][0] - out[1][0]) <= 1e-5 * abs(out[1][0])
    _check(out[0][1].cpu().numpy(), out[1][1].cpu().numpy(), what="network gradients")
    assert out[1][2].abs().max() > 0
    _check(out[0][2].cpu().numpy(), out[1][2].cpu().numpy(), what="table gradient through the fused kernel's dL/dinput")


@pytest.mark.parametrize("dims", [3, 2])
def test_c4_fused_encoding_forward_equals_the_two_kernel_path(tnn_lib, dims):
    """Hash grid gathered by extra warps of the network kernel straight into its input tile: inference and the stored
    forward pass return the bits of (encoding kernel -> bf16 matrix -> network kernel), and matrix 0 of the stored
    activations is the encoded input."""
    nh = 2
    cfg = dict(GRID_CFG, n_dims_to_encode=dims)
    batch = 128 * 148 + 128 * 7 + 8
    net = tnn_lib.create_network(32, 3, nh, A["relu"], A["none"], W, "torch.bfloat16", True, seed=4)
    enc = tnn_lib.create_encoding("HashGrid", cfg, W, seed=3)
    grid = O.Grid(n_dims_to_encode=dims, per_level_scale=2.0)
    table = np.random.default_rng(1).uniform(-0.5, 0.5, grid.n_params).astype(np.float32)
    enc.set_params(torch.from_numpy(table).cuda())
    pts = torch.rand((batch, dims), device="cuda")
    encoded = enc.fwd(pts, out_dtype=torch.bfloat16)
    assert np.array_equal(encoded.float().cpu().numpy(), O.bf16_round(grid.forward(pts.cpu().numpy(), table, padded=W)))
    y_two = net.inference(encoded)
    assert torch.equal(tnn_lib.nwe_inference(net, enc, pts), y_two)  # default: encoding kernel, then network kernel
    launches = tnn_lib.load().tnn_launch_count()
    net.set_variant(128)  # the grid is gathered inside the network kernel: one launch
    y_fused = tnn_lib.nwe_inference(net, enc, pts)
    assert tnn_lib.load().tnn_launch_count() == launches + 1
    assert torch.equal(y_fused, y_two) and net.status() == 0
    out = tnn_lib.nwe_forward(net, enc, pts)
    ig = net.interm_fwd()
    assert torch.equal(ig[0], encoded) and torch.equal(out, y_two)


# ------------------------------------------------------------------------------------------------ data parallel, NCCL
def _dp_worker(rank, world, port, out_dir, batch, steps, window):
    for p in (ROOT, os.path.join(ROOT, "tiny-dpcpp-nn_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    from tiny_dpcpp_nn import _lib as L
    from tiny_dpcpp_nn.parallel import shard_rows
    from tiny_dpcpp_nn.trainer import Trainer

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    q, t, w = _c5_case(batch)
    a, b = shard_rows(batch, rank, world)
    net, enc = _c5_modules(L, w)
    tr = Trainer(net, lr=1e-3, process_group=dist.group.WORLD, world_size=world, encoding=enc)
    tr.set_master_params(torch.from_numpy(O.pack_weights(w, N_MAT, W)).cuda())
    if not window:
        tr.set_peer_window(False)
    qt, tt = torch.from_numpy(q[a:b]).cuda(), torch.from_numpy(t[a:b]).cuda()
    for i in range(steps):
        if i % 2 == 0:
            tr.training_step(qt, tt)
        else:  # the two halves of a step as separate calls: the exchange starts from the reduced gradient
            tr.forward_backward(qt, tt)
            tr.optimizer_step()
    torch.cuda.synchronize()
    with open(os.path.join(out_dir, f"window{rank}.txt"), "w") as f:
        f.write(str(int(tr.peer_window)))
    np.save(os.path.join(out_dir, f"master{rank}.npy"), tr.master.cpu().numpy())
    np.save(os.path.join(out_dir, f"grads{rank}.npy"), tr.grads.cpu().numpy())
    assert net.status() == 0
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["window", "nccl"])
def test_data_parallel_step_equals_single_gpu_full_batch(tnn_lib, tmp_path, exchange):
    """Two ranks, each on its half of the batch, the weight-gradient buffer summed over the ranks once per step -
    inside the optimiser kernel through the peer windows, or by one NCCL all-reduce: after the steps both ranks hold
    identical bits, and they equal (within the kernel tolerance) a single-GPU trainer that saw the whole batch."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    from tiny_dpcpp_nn.trainer import Trainer

    batch, steps, world = 128 * 64, 4, 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_dp_worker, args=(world, port, str(tmp_path), batch, steps, exchange == "window"), nprocs=world, join=True)
    active = [int((tmp_path / f"window{r}.txt").read_text()) for r in range(world)]
    if exchange == "window" and active != [1] * world:
        pytest.skip("the ranks of this host cannot map each other's memory: no peer windows")
    assert exchange == "window" or active == [0] * world
    m0, m1 = np.load(tmp_path / "master0.npy"), np.load(tmp_path / "master1.npy")
    g0, g1 = np.load(tmp_path / "grads0.npy"), np.load(tmp_path / "grads1.npy")
    assert np.array_equal(m0, m1) and np.array_equal(g0, g1)  # replicas stay bit-identical
    q, t, w = _c5_case(batch)
    net, enc = _c5_modules(tnn_lib, w)
    tr = Trainer(net, lr=1e-3, encoding=enc)
    tr.set_master_params(torch.from_numpy(O.pack_weights(w, N_MAT, W)).cuda())
    qt, tt = torch.from_numpy(q).cuda(), torch.from_numpy(t).cuda()
    for _ in range(steps):
        tr.training_step(qt, tt)
    # gradient of the last step: sum over the ranks = world x the full-batch mean gradient
    _check(g0 / world, tr.grads.cpu().numpy(), what="DP gradient")
    diff = np.abs(m0 - tr.master.cpu().numpy())
    assert diff.max() <= 2.1e-3 * steps and (diff <= 2e-5).mean() >= 0.98


def _dp_timeout_worker(rank, world, port, out_dir):
    for p in (ROOT, os.path.join(ROOT, "tiny-dpcpp-nn_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", TNN_DP_WAIT_MS="300")
    import time

    import torch.distributed as dist

    from tiny_dpcpp_nn import _lib as L
    from tiny_dpcpp_nn.trainer import Trainer

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    batch = 128 * 8
    q, t, w = _c5_case(batch)
    net, enc = _c5_modules(L, w)
    tr = Trainer(net, lr=1e-3, process_group=dist.group.WORLD, world_size=world, encoding=enc)
    qt, tt = torch.from_numpy(q).cuda(), torch.from_numpy(t).cuda()
    seen = [int(tr.peer_window)]
    tr.training_step(qt, tt)
    seen.append(net.status())  # 0: both ranks arrived together
    dist.barrier()
    if rank == 1:
        time.sleep(2.0)  # rank 0 waits 300 ms for this rank's gradient, then gives up
    tr.training_step(qt, tt)
    seen.append(net.status())  # rank 0: 2 (wait ran out, its weights of this step untouched), rank 1: 0
    dist.barrier()
    tr.training_step(qt, tt)
    seen.append(net.status())  # the context and the windows are usable afterwards
    with open(os.path.join(out_dir, f"timeout{rank}.txt"), "w") as f:
        f.write(" ".join(str(v) for v in seen))
    dist.barrier()
    dist.destroy_process_group()


def test_peer_window_wait_gives_up_and_reports(tnn_lib, tmp_path):
    """A rank whose peer is late by more than TNN_DP_WAIT_MS: the exchange kernel stops polling, leaves its weights
    alone and sets bit 2 of the status word; nothing hangs or faults and the next step runs normally."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_dp_timeout_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r0 = [int(v) for v in (tmp_path / "timeout0.txt").read_text().split()]
    r1 = [int(v) for v in (tmp_path / "timeout1.txt").read_text().split()]
    if r0[0] != 1 or r1[0] != 1:
        pytest.skip("the ranks of this host cannot map each other's memory: no peer windows")
    assert r0[1:] == [0, 2, 0] and r1[1:] == [0, 0, 0]


def _dp_grid_worker(rank, world, port, out_dir, batch, steps):
    for p in (ROOT, os.path.join(ROOT, "tiny-dpcpp-nn_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    from tiny_dpcpp_nn import _lib as L
    from tiny_dpcpp_nn.parallel import shard_rows
    from tiny_dpcpp_nn.trainer import Trainer

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    net, enc, pts, t = _c4_setup(L, batch)
    a, b = shard_rows(batch, rank, world)
    tr = Trainer(net, lr=1e-2, process_group=dist.group.WORLD, world_size=world, encoding=enc)
    tr.set_deterministic_encoding(True)
    for _ in range(steps):
        tr.training_step(pts[a:b].contiguous(), t[a:b].contiguous())
    torch.cuda.synchronize()
    np.save(os.path.join(out_dir, f"table{rank}.npy"), enc.get_params().cpu().numpy())
    np.save(os.path.join(out_dir, f"net{rank}.npy"), tr.master.cpu().numpy())
    assert net.status() == 0
    dist.barrier()
    dist.destroy_process_group()


def _c4_setup(L, batch):
    """The hash-grid model with seeded weights and table, same on every rank."""
    nh = 2
    w = O.bf16_round(synth.xavier_weights(nh + 1, W, 4))
    net = L.create_network(32, 3, nh, A["relu"], A["none"], W, "torch.bfloat16", True, seed=1)
    net.set_params(torch.from_numpy(w.reshape(-1)).cuda(), False)
    cfg = dict(GRID_CFG, log2_hashmap_size=14)
    enc = L.create_encoding("HashGrid", cfg, W, seed=3)
    n = enc.n_params()
    enc.set_params(torch.from_numpy(np.random.default_rng(2).uniform(-0.5, 0.5, n).astype(np.float32)).cuda())
    rng = np.random.default_rng(100)
    pts = torch.from_numpy(rng.uniform(0, 1, (batch, 3)).astype(np.float32)).cuda()
    t = torch.from_numpy(synth.sinusoid_targets(pts.cpu().numpy(), 3, 8, 8.0, seed=5)).cuda()
    return net, enc, pts, t


def test_data_parallel_hash_grid_training_over_nccl(tnn_lib, tmp_path):
    """Two ranks train the hash-grid model on halves of the batch: network gradients all-reduced, table gradient
    reduce-scattered, Adam on each rank's slice of the table, table all-gathered.  Both ranks end with identical
    tables and weights, equal (to the kernels' tolerance) to a single-GPU trainer on the whole batch."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    from tiny_dpcpp_nn.trainer import Trainer

    batch, steps, world = 128 * 32, 2, 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_dp_grid_worker, args=(world, port, str(tmp_path), batch, steps), nprocs=world, join=True)
    t0, t1 = np.load(tmp_path / "table0.npy"), np.load(tmp_path / "table1.npy")
    n0, n1 = np.load(tmp_path / "net0.npy"), np.load(tmp_path / "net1.npy")
    assert np.array_equal(t0, t1) and np.array_equal(n0, n1)
    net, enc, pts, t = _c4_setup(tnn_lib, batch)
    tr = Trainer(net, lr=1e-2, encoding=enc)
    tr.set_deterministic_encoding(True)
    for _ in range(steps):
        tr.training_step(pts, t)
    ref = enc.get_params().cpu().numpy()
    # Adam moves every touched entry by about lr per step whatever the gradient's size: entries whose gradient is
    # within rounding noise of zero may differ by up to 2 lr per step, all others agree closely
    diff = np.abs(t0 - ref)
    assert diff.max() <= 2.1e-2 * steps and (diff <= 1e-4).mean() >= 0.98, ((diff <= 1e-4).mean(), diff.max())
