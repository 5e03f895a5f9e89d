"""GPU parity tests of fp16 networks (the reference's sycl::half instantiations,
include/network/kernel_esimd.h:643-721, with loss scale 128 as in dpcpp_bindings/tiny_dpcpp_nn/modules.py:158-161)
through the C ABI, against the CPU oracle rounding every stored value to IEEE half.  Same cases as the reference's
fp16 parametrisations of test/python/test_compare_torch_dpcpp.py:92-157."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
from oracle import oracle as O  # noqa: E402
from tests import synth  # noqa: E402

pytestmark = pytest.mark.gpu
A = {"relu": 0, "sigmoid": 4, "none": 8}
TOL = 1e-2


def _h(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda().to(torch.float16)


def _check(v, t, what=""):
    ok, rel = O.within_tolerance(v, t, TOL)
    assert ok, (what, rel)


def _case(W, nh, batch, w_seed=0):
    w = O.fp16_round(synth.xavier_weights(nh + 1, W, w_seed))
    x = O.fp16_round(synth.uniform_inputs(batch, W, 100))
    return w, x


@pytest.mark.parametrize("W,nh,act,oact", [(64, 4, "relu", "none"), (64, 2, "sigmoid", "sigmoid"), (32, 3, "relu", "none"),
                                          (16, 2, "relu", "none"), (128, 2, "relu", "none"), (64, 8, "none", "relu"),
                                          (128, 4, "sigmoid", "none")])
def test_fp16_forward_backward_matches_oracle(tnn_lib, W, nh, act, oact):
    batch = 128 * 150 + 8
    n_mat = nh + 1
    w, x = _case(W, nh, batch, w_seed=3)
    net = tnn_lib.create_network(W, W, nh, A[act], A[oact], W, "torch.float16", True, seed=1)
    net.set_params(torch.from_numpy(w.reshape(-1)).cuda(), False)
    assert net.get_params().dtype == torch.float16
    interm = O.mlp_forward(x, w, n_mat, W, act, oact, bf16="fp16")
    xt = _h(x)
    _check(net.inference(xt).float().cpu().numpy(), interm[-1], "inference")
    net.fwd(xt)
    ig = net.interm_fwd().float().cpu().numpy()
    assert np.array_equal(ig[0], x)
    for l in range(1, n_mat + 1):
        _check(ig[l], interm[l], f"a[{l}]")
    # loss-scaled upstream gradient, as the Python layer sends it (x 128)
    dy = O.fp16_round((np.random.default_rng(9).uniform(-1, 1, (batch, W)) * 128.0 / batch).astype(np.float32))
    ib, gr, dx = O.mlp_backward(dy, ig, w, n_mat, W, act, oact, bf16="fp16")
    dxg, g = net.bwd_no_encoding_grad(_h(dy), False, True, want_interm_bwd=True, grads_dtype=torch.float32)
    assert net.status() == 0
    g = g.cpu().numpy().reshape(n_mat, W, W)
    for l in range(n_mat):
        _check(net._interm_bwd[l].float().cpu().numpy(), ib[l], f"delta[{l}]")
        _check(g[l], gr[l], f"dW[{l}]")
    _check(dxg.float().cpu().numpy().reshape(batch, W), dx, "dx")
    # gradients in the network's own type, like the reference returns them
    _, g16 = net.bwd_no_encoding_grad(_h(dy), False, False)
    assert g16.dtype == torch.float16
    _check(g16.float().cpu().numpy().reshape(-1), gr.reshape(-1), "dW fp16")


@pytest.mark.parametrize("variant", [0, 64, 16])
@pytest.mark.parametrize("W,nh,nt", [(64, 4, 64), (64, 4, 3), (32, 2, 32)])
def test_fp16_fused_training_step_with_loss_scale(tnn_lib, variant, W, nh, nt):
    from tiny_dpcpp_nn.trainer import Trainer

    batch, scale = 128 * 40 + 8, 128.0
    n_mat = nh + 1
    w, x = _case(W, nh, batch, w_seed=5)
    t = synth.uniform_inputs(batch, nt, seed=1)
    net = tnn_lib.create_network(W, W, nh, A["relu"], A["none"], W, "torch.float16", True, seed=1)
    net.set_variant(variant)
    net.set_params(torch.from_numpy(w.reshape(-1)).cuda(), False)
    tr = Trainer(net, loss_scale=scale)
    loss = tr.forward_backward(_h(x), torch.from_numpy(t).cuda()).item()
    assert net.status() == 0
    interm = O.mlp_forward(x, w, n_mat, W, "relu", "none", bf16="fp16")
    tpad = np.zeros((batch, W), np.float32)
    tpad[:, :nt] = t
    vals, dy = O.l2_loss(interm[-1], tpad, scale, bf16_grads="fp16")
    _, gr, _ = O.mlp_backward(dy, interm, w, n_mat, W, "relu", "none", bf16="fp16", want_dx=False)
    packed = O.pack_weights(np.ascontiguousarray(np.transpose(gr, (0, 2, 1))).astype(np.float32), n_mat, W)
    assert abs(loss - float(vals.astype(np.float64).sum())) <= 1e-3 * abs(loss)
    _check(tr.grads.cpu().numpy(), packed, "scaled gradient")
    # one optimiser step: the gradient is unscaled again, the refreshed weights are the fp16-rounded master copy
    tr.optimizer_step()
    assert np.array_equal(net.get_params().float().cpu().numpy().reshape(-1), O.fp16_round(tr.master.cpu().numpy()))


def test_fp16_identity_fold_and_module(tnn_lib):
    """NetworkWithInputEncoding in fp16: folded identity encoding == the two-module path; loss scale 128 applied and
    removed by the module (modules.py:158-161 of the reference)."""
    import tiny_dpcpp_nn as tnn

    net_cfg = {"n_neurons": 64, "n_hidden_layers": 2, "activation": "relu", "output_activation": "none"}
    model = tnn.NetworkWithInputEncoding(2, 3, net_cfg, {"otype": "Identity", "scale": 1.0, "offset": 0.0},
                                         dtype=torch.float16, seed=5)
    assert model.network.loss_scale == 128.0 and model._foldable()
    x = torch.rand((512, 2), device="cuda")
    tgt = torch.rand((512, 3), device="cuda")
    grads = []
    for fn in (model, model.network_with_encoding):
        model.zero_grad(set_to_none=True)
        out = fn(x)
        assert out.dtype == torch.float16
        ((out.float() - tgt) ** 2).mean().backward()
        grads.append(model.params.grad.clone())
    assert torch.equal(grads[0], grads[1]) and torch.isfinite(grads[0]).all() and grads[0].abs().sum() > 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_network_module_matches_torch_linear_stack(tnn_lib, dtype):
    """test/python/test_compare_torch_dpcpp.py:92-157: forward and parameter gradients of the module against a torch
    MLP holding the same (rounded) weights, both dtypes."""
    import tiny_dpcpp_nn as tnn

    W, nh, batch = 64, 3, 2048
    net = tnn.Network(W, W, {"n_neurons": W, "n_hidden_layers": nh, "activation": "relu", "output_activation": "none"},
                      dtype=dtype, seed=3)
    x = (torch.rand((batch, W), device="cuda") * 2 - 1).to(dtype)
    y = net(x)
    assert y.dtype == dtype
    packed = net.get_params().float().cpu().numpy().reshape(-1)
    w = O.unpack_weights(packed, nh + 1, W).reshape(nh + 1, W, W)
    ref = x.float().cpu().numpy()
    for l in range(nh + 1):
        ref = ref @ w[l]
        if l < nh:
            ref = np.maximum(ref, 0)
        ref = O.round16(ref.astype(np.float32), "fp16" if dtype == torch.float16 else "bf16")
    _check(y.detach().float().cpu().numpy(), ref, "module forward")
    (y.float() ** 2).mean().backward()
    assert torch.isfinite(net.params.grad).all() and net.params.grad.abs().sum() > 0
