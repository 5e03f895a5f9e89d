"""GPU tests of the torch.nn.Module front end (tiny_dpcpp_nn.Network / Encoding / NetworkWithInputEncoding)
against a plain torch.nn.Linear stack, in the manner of the reference's test/python/test_compare_torch_dpcpp.py
(forward rtol 2e-2: 185-248; gradients rtol 1e-2 with an absolute floor of 5e-4: src/utils.py:9-33)."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
from oracle import oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu


class TorchMLP(torch.nn.Module):
    """Reference network: Linear layers without bias; the bias is the column of ones the input is padded with
    (test/python/src/mlp.py of the reference builds the same thing)."""

    def __init__(self, width, n_hidden, act, out_act, round_weights=False):
        super().__init__()
        self.layers = torch.nn.ModuleList([torch.nn.Linear(width, width, bias=False) for _ in range(n_hidden + 1)])
        self.act, self.out_act = act, out_act
        # the device computes with the bf16 rounding of its fp32 master weights; a model whose weights are being
        # trained has to do the same to stay comparable (updates smaller than a bf16 step change nothing at first)
        self.round_weights = round_weights

    @staticmethod
    def _a(name, x):
        return torch.relu(x) if name == "relu" else torch.sigmoid(x) if name == "sigmoid" else x

    def forward(self, x):
        for i, layer in enumerate(self.layers):
            w = layer.weight.to(torch.bfloat16).to(torch.float32) if self.round_weights else layer.weight
            x = torch.nn.functional.linear(x, w)
            x = self._a(self.out_act if i == len(self.layers) - 1 else self.act, x)
            x = x.to(torch.bfloat16).to(torch.float32)  # the fused kernels round every layer to bf16
        return x


def _close(a, b, rtol, atol):
    return np.allclose(a, b, rtol=rtol, atol=atol) or O.within_tolerance(a, b, rtol)[0]


@pytest.mark.parametrize("in_dim,out_dim", [(64, 64), (3, 1), (16, 3)])
@pytest.mark.parametrize("act,oact", [("relu", "linear"), ("sigmoid", "sigmoid"), ("linear", "linear")])
@pytest.mark.parametrize("width,n_hidden", [(64, 4), (32, 2), (16, 1)])
def test_network_forward_and_gradients_match_torch(tnn_lib, in_dim, out_dim, act, oact, width, n_hidden):
    import tiny_dpcpp_nn as tnn

    if in_dim > width or out_dim > width:
        pytest.skip("input / output wider than the network")
    cfg = {"n_neurons": width, "n_hidden_layers": n_hidden, "activation": act, "output_activation": oact}
    net = tnn.Network(in_dim, out_dim, cfg, dtype=torch.bfloat16, seed=7)
    # load the same weights into the torch model: unpack the packed parameter vector (in x out per matrix)
    packed = net.params.detach().float().cpu().numpy().reshape(-1)
    w = O.unpack_weights(packed, n_hidden + 1, width).reshape(n_hidden + 1, width, width)
    ref = TorchMLP(width, n_hidden, "none" if act == "linear" else act, "none" if oact == "linear" else oact).cuda()
    with torch.no_grad():
        for l, layer in enumerate(ref.layers):
            layer.weight.copy_(torch.from_numpy(w[l].T.copy()))  # Linear stores (out x in)
    batch = 1 << 10
    gen = torch.Generator(device="cuda").manual_seed(0)
    x = (torch.rand((batch, in_dim), device="cuda", generator=gen) * 2 - 1)
    xr = x.to(torch.bfloat16).float()
    xpad = torch.nn.functional.pad(xr, [0, width - in_dim], value=1.0) if in_dim < width else xr

    y = net(x)
    y_ref = ref(xpad)[:, :out_dim]
    assert y.shape == (batch, out_dim)
    assert _close(y.float().detach().cpu().numpy(), y_ref.detach().cpu().numpy(), 2e-2, 1e-3)

    target = torch.rand((batch, out_dim), device="cuda", generator=gen)
    loss = ((y.float() - target) ** 2).mean()
    loss.backward()
    loss_ref = ((y_ref - target) ** 2).mean()
    loss_ref.backward()
    g = O.unpack_weights(net.params.grad.float().cpu().numpy().reshape(-1), n_hidden + 1, width)
    g = g.reshape(n_hidden + 1, width, width)
    for l, layer in enumerate(ref.layers):
        gr = layer.weight.grad.cpu().numpy().T  # back to (in x out)
        assert _close(g[l], gr, 2e-2, 5e-4), f"layer {l}"


def test_network_eval_mode_uses_inference_and_handles_ragged_batches(tnn_lib):
    import tiny_dpcpp_nn as tnn

    cfg = {"n_neurons": 64, "n_hidden_layers": 2, "activation": "relu", "output_activation": "linear"}
    net = tnn.Network(5, 2, cfg, dtype=torch.bfloat16, seed=1)
    x = torch.rand((13, 5), device="cuda")  # 13 rows: padded to 16 inside (modules.py:215-223)
    y_train = net(x)
    net.eval()
    with torch.no_grad():
        y_eval = net(x)
    assert y_train.shape == (13, 2) and torch.equal(y_train.detach(), y_eval)


def test_grid_encoding_module_and_chain(tnn_lib):
    import tiny_dpcpp_nn as tnn

    enc_cfg = {"otype": "HashGrid", "type": "Hash", "n_levels": 8, "n_features_per_level": 2, "log2_hashmap_size": 15,
               "base_resolution": 16, "per_level_scale": 2.0}
    enc = tnn.Encoding(3, enc_cfg, seed=3)
    g = O.Grid(n_dims_to_encode=3, n_levels=8, log2_hashmap_size=15)
    x = torch.rand((1000, 3), device="cuda")
    out = enc(x)
    table = enc.params.detach().cpu().numpy().reshape(-1)
    ref = g.forward(x.cpu().numpy(), table)
    assert np.array_equal(out.detach().cpu().numpy(), ref)
    dy = torch.rand_like(out)
    out.backward(dy)
    gref = g.backward(x.cpu().numpy(), dy.cpu().numpy())
    ok, rel = O.within_tolerance(enc.params.grad.cpu().numpy().reshape(-1), gref, 1e-5)
    assert ok, rel

    net_cfg = {"n_neurons": 64, "n_hidden_layers": 2, "activation": "relu", "output_activation": "linear"}
    model = tnn.NetworkWithInputEncoding(3, 3, net_cfg, enc_cfg, dtype=torch.bfloat16, seed=4)
    opt = torch.optim.Adam(model.parameters(), lr=1e-2, betas=(0.9, 0.99), eps=1e-15)
    pts = torch.rand((1 << 12, 3), device="cuda")
    tgt = torch.sin(6.28 * pts)
    losses = []
    for _ in range(60):
        opt.zero_grad()
        loss = ((model(pts).float() - tgt) ** 2).mean()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < 0.5 * losses[0], (losses[0], losses[-1])


def test_identity_encoding_feeds_network(tnn_lib):
    import tiny_dpcpp_nn as tnn

    enc = tnn.Encoding(2, {"otype": "Identity", "scale": 1.0, "offset": 0.0}, n_output_dims=64)
    x = torch.rand((64, 2), device="cuda")
    out = enc(x)
    assert out.shape == (64, 64)
    assert torch.equal(out[:, :2], x) and torch.all(out[:, 2:] == 1.0)


def test_regression_with_sgd_tracks_torch(tnn_lib):
    """test/python/test_training.py:57-182: the module and a torch MLP with the same weights are trained side by
    side with plain SGD on a linear target; after every step outputs, loss, gradient mass and parameter mass agree."""
    import tiny_dpcpp_nn as tnn

    width, n_hidden, lr, steps = 32, 1, 5e-3, 30
    cfg = {"n_neurons": width, "n_hidden_layers": n_hidden, "activation": "relu", "output_activation": "linear"}
    net = tnn.Network(width, 1, cfg, dtype=torch.bfloat16, seed=3)
    packed = net.params.detach().float().cpu().numpy().reshape(-1)
    w = O.unpack_weights(packed, n_hidden + 1, width).reshape(n_hidden + 1, width, width)
    ref = TorchMLP(width, n_hidden, "relu", "none", round_weights=True).cuda()
    with torch.no_grad():
        for l, layer in enumerate(ref.layers):
            layer.weight.copy_(torch.from_numpy(w[l].T.copy()))
    x = torch.ones((8, width), device="cuda")
    labels = 0.5 * x[:, :1]
    first_loss = None
    for step in range(steps):
        y = net(x).float()
        loss = ((y - labels) ** 2).mean()
        net.zero_grad()
        loss.backward()
        before = net.params.detach().clone()
        with torch.no_grad():
            net.params.copy_(net.params - lr * net.params.grad)
        assert step > 0 or not torch.equal(before, net.params.detach())  # (later on the loss may reach exactly 0)

        y_ref = ref(x)[:, :1]
        loss_ref = ((y_ref - labels) ** 2).mean()
        ref.zero_grad()
        loss_ref.backward()
        grad_mass_ref = sum(layer.weight.grad.abs().sum().item() for layer in ref.layers)
        with torch.no_grad():
            for layer in ref.layers:
                layer.weight.copy_(layer.weight - lr * layer.weight.grad)

        first_loss = loss.item() if first_loss is None else first_loss
        assert torch.allclose(y.detach(), y_ref.detach(), rtol=5e-2, atol=5e-3), step
        assert abs(loss.item() - loss_ref.item()) <= 5e-2 * abs(loss_ref.item()) + 1e-4, step
        grad_mass = net.params.grad.float().abs().sum().item()
        assert abs(grad_mass - grad_mass_ref) <= 5e-2 * grad_mass_ref + 1e-3, step
    assert loss.item() < 0.5 * first_loss  # and the regression made progress
    mass = net.params.detach().float().abs().sum().item()
    mass_ref = sum(layer.weight.detach().abs().sum().item() for layer in ref.layers)
    assert abs(mass - mass_ref) <= 1e-2 * mass_ref


def test_set_params_roundtrip_through_the_module(tnn_lib):
    """test/python/test_set_param.py:22-75: a constant parameter vector set through the module is what the module
    reports afterwards, and the forward pass uses it (linear network, input 0.1: closed form)."""
    import tiny_dpcpp_nn as tnn

    width, n_hidden = 16, 3
    cfg = {"n_neurons": width, "n_hidden_layers": n_hidden, "activation": "none", "output_activation": "none"}
    net = tnn.Network(width, width, cfg, dtype=torch.bfloat16)
    val = 0.123
    vals = torch.full((width * width * (n_hidden + 1), 1), val, device="cuda", dtype=torch.bfloat16)
    net.set_params(vals)
    assert torch.allclose(net.params.detach().to(torch.bfloat16).reshape(-1, 1), vals)
    y = net(torch.full((8, width), 0.1, device="cuda")).float()
    # every layer multiplies by 16 x bf16(0.123), rounded to bf16 after each layer
    expect = torch.tensor(0.1, dtype=torch.bfloat16).float()
    wv = torch.tensor(val, dtype=torch.bfloat16).float()
    for _ in range(n_hidden + 1):
        expect = (expect * wv * width).to(torch.bfloat16).float()
    assert torch.allclose(y, torch.full_like(y, expect.item()), rtol=2e-2)


def test_network_with_identity_encoding_runs_folded_and_equals_the_sequential_path(tnn_lib):
    """NetworkWithInputEncoding (modules.py:357-421 of the reference) with an Identity encoding: the single-kernel
    path (encoding folded into the first-layer load) returns the bits of the two-module Sequential path, in eval and
    in training mode, and the same parameter gradient; ragged batches are padded to 8 rows."""
    import tiny_dpcpp_nn as tnn

    net_cfg = {"n_neurons": 64, "n_hidden_layers": 4, "activation": "relu", "output_activation": "none"}
    enc_cfg = {"otype": "Identity", "scale": 1.0, "offset": 0.0}
    model = tnn.NetworkWithInputEncoding(2, 3, net_cfg, enc_cfg, seed=11)
    assert model._foldable()
    x = torch.rand((1000 + 3, 2), device="cuda")
    tgt = torch.rand((1000 + 3, 3), device="cuda")
    model.eval()
    with torch.no_grad():
        y_folded = model(x)
        y_seq = model.network_with_encoding(x)
    assert y_folded.shape == (1003, 3) and torch.equal(y_folded, y_seq)
    model.train()
    grads = []
    for fn in (model, model.network_with_encoding):
        model.zero_grad(set_to_none=True)
        out = fn(x)
        ((out.float() - tgt) ** 2).mean().backward()
        grads.append(model.params.grad.clone())
        assert torch.equal(out, y_seq)
    assert torch.equal(grads[0], grads[1]) and grads[0].abs().sum() > 0


def test_network_with_grid_encoding_fused_forward_equals_the_sequential_path(tnn_lib):
    """NetworkWithInputEncoding with a HashGrid through the single-operator path of the module (one call into the
    library per pass; with variant bit 128 the grid is gathered inside the network kernel) returns the bits of the
    Sequential path; the table and network gradients agree (the table gradient is summed with floating-point
    reductions in memory on both paths, so to rounding only)."""
    import tiny_dpcpp_nn as tnn

    net_cfg = {"n_neurons": 64, "n_hidden_layers": 2, "activation": "relu", "output_activation": "none"}
    enc_cfg = {"otype": "HashGrid", "n_levels": 16, "n_features_per_level": 2, "log2_hashmap_size": 15,
               "base_resolution": 16, "per_level_scale": 1.5}
    model = tnn.NetworkWithInputEncoding(3, 3, net_cfg, enc_cfg, seed=7)
    assert model._fusable()
    with torch.no_grad():
        model.encoding.params.mul_(1e3)  # default initial values are +-1e-4: make the features matter
    x = torch.rand((4096 + 5, 3), device="cuda")
    tgt = torch.rand((4096 + 5, 3), device="cuda")
    model.eval()
    with torch.no_grad():
        ref = model.network_with_encoding(x)
        assert torch.equal(model(x), ref)
        model.network.tnn_module.set_variant(128)
        assert torch.equal(model(x), ref)
    model.train()
    res = []
    for fn in (model, model.network_with_encoding):
        model.zero_grad(set_to_none=True)
        out = fn(x)
        ((out.float() - tgt) ** 2).mean().backward()
        res.append((out.clone(), model.network.params.grad.clone(), model.encoding.params.grad.clone()))
    assert torch.equal(res[0][0], res[1][0]) and torch.equal(res[0][1], res[1][1])
    ga, gb = res[0][2], res[1][2]
    assert ga.abs().sum() > 0 and (ga - gb).abs().max() <= 1e-5 * ga.abs().max()
