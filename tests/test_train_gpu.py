"""GPU parity tests of the fused training step (forward + L2 loss + backward + weight gradients in one
kernel), of the Adam step and of the Trainer, through the C ABI, against the CPU oracle."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
from oracle import oracle as O  # noqa: E402
from tests import synth  # noqa: E402

pytestmark = pytest.mark.gpu
A = {"relu": 0, "sigmoid": 4, "none": 8}
TOL = 1e-2  # include/common/result_check.h:83-102 as used by test/doctest_swiftnet.cpp


def _bf16(t):
    return torch.from_numpy(np.ascontiguousarray(t, dtype=np.float32)).cuda().to(torch.bfloat16)


def _oracle_step(x, t, w, W, nh, act, oact):
    n_mat = nh + 1
    interm = O.mlp_forward(x, w, n_mat, W, act, oact, bf16=True)
    tpad = np.zeros((x.shape[0], W), np.float32)
    tpad[:, : t.shape[1]] = t
    vals, dy = O.l2_loss(interm[-1], tpad, 1.0, bf16_grads=True)
    _, gr, _ = O.mlp_backward(dy, interm, w, n_mat, W, act, oact, bf16=True, want_dx=False)
    packed = O.pack_weights(np.ascontiguousarray(np.transpose(gr, (0, 2, 1))).astype(np.float32), n_mat, W)
    return float(vals.astype(np.float64).sum()), packed.reshape(n_mat, W * W)


# variant 0: pipelined fused kernel, 64: single-tile fused kernel, 16: forward / loss / backward kernels
@pytest.mark.parametrize("variant", [0, 64, 16])
@pytest.mark.parametrize("W,nh,act,oact,batch,nt", [
    (64, 4, "relu", "none", 128 * 148 * 2 + 72, 64),
    (64, 2, "sigmoid", "sigmoid", 8000, 3),
    (64, 1, "none", "relu", 8, 64),
    (64, 5, "relu", "none", 4096, 64),
    (32, 4, "relu", "none", 4096, 32),
    (32, 2, "sigmoid", "none", 4096, 5),
    (16, 2, "relu", "none", 4096, 16),
    (64, 6, "relu", "none", 4096, 64),
    (64, 8, "relu", "none", 4096, 64),
    (32, 8, "relu", "none", 128 * 150 + 8, 32),
    (32, 10, "sigmoid", "none", 4096, 7),
    (128, 2, "relu", "none", 4096, 128),
    (128, 4, "relu", "none", 128 * 150 + 8, 128),
])
def test_train_step_matches_oracle(tnn_lib, variant, W, nh, act, oact, batch, nt):
    from tiny_dpcpp_nn.trainer import Trainer

    w, x = synth.mlp_case(W, nh, batch, w_seed=5)
    t = synth.uniform_inputs(batch, nt, seed=1)
    net = tnn_lib.create_network(W, W, nh, A[act], A[oact], W, "torch.bfloat16", True, seed=1)
    net.set_variant(variant)
    net.set_params(torch.from_numpy(w.reshape(-1)).cuda(), False)
    tr = Trainer(net)
    loss = tr.forward_backward(_bf16(x), torch.from_numpy(t).cuda())
    assert net.status() == 0
    exp_loss, exp_grads = _oracle_step(x, t, w, W, nh, act, oact)
    assert abs(loss.item() - exp_loss) <= 1e-4 * abs(exp_loss)
    g = tr.grads.cpu().numpy().reshape(nh + 1, W * W)
    for l in range(nh + 1):
        ok, rel = O.within_tolerance(g[l], exp_grads[l], TOL)
        assert ok, (l, rel)


def test_train_step_is_bitwise_reproducible(tnn_lib):
    from tiny_dpcpp_nn.trainer import Trainer

    W, nh, batch = 64, 4, 128 * 300
    w, x = synth.mlp_case(W, nh, batch)
    t = synth.uniform_inputs(batch, W, seed=1)
    net = tnn_lib.create_network(W, W, nh, A["relu"], A["none"], W, "torch.bfloat16", True, seed=1)
    net.set_params(torch.from_numpy(w.reshape(-1)).cuda(), False)
    tr = Trainer(net)
    xt, tt = _bf16(x), torch.from_numpy(t).cuda()
    l1 = tr.forward_backward(xt, tt).clone()
    g1 = tr.grads.clone()
    l2 = tr.forward_backward(xt, tt)
    assert torch.equal(g1, tr.grads) and torch.equal(l1, l2)


def test_network_adam_step_matches_oracle_and_refreshes_weights(tnn_lib):
    W, nh = 64, 2
    n_mat = nh + 1
    w = synth.xavier_weights(n_mat, W, 3)
    net = tnn_lib.create_network(W, W, nh, A["relu"], A["none"], W, "torch.bfloat16", True, seed=1)
    packed = O.pack_weights(w, n_mat, W)
    master = torch.from_numpy(packed.copy()).cuda()
    m, v = torch.zeros_like(master), torch.zeros_like(master)
    p, pm, pv = packed.copy(), np.zeros_like(packed), np.zeros_like(packed)
    rng = np.random.default_rng(0)
    for step in range(1, 4):
        g = (rng.normal(size=packed.size) * 1e-2).astype(np.float32)
        O.adam(p, pm, pv, g, step)
        net.adam_step(master, m, v, torch.from_numpy(g).cuda(), step)
    assert np.allclose(master.cpu().numpy(), p, rtol=1e-5, atol=1e-7)
    # the bf16 working copy the kernels read is the rounded master copy
    assert np.array_equal(net.get_params().float().cpu().numpy().reshape(-1), O.bf16_round(master.cpu().numpy()))


def test_trainer_reduces_the_loss(tnn_lib):
    """Fixed batch, 100 Adam steps (lr 1e-3, beta 0.9 / 0.99, eps 1e-15): the L2 loss must fall, as in the
    reference's convergence tests (test/python/test_training.py:261-456)."""
    from tiny_dpcpp_nn.trainer import Trainer

    W, nh, batch = 64, 4, 1 << 14
    x = synth.uniform_inputs(batch, W, seed=100)
    t = synth.sinusoid_targets(x[:, :3], W, 8, 4.0, seed=5)
    net = tnn_lib.create_network(W, W, nh, A["relu"], A["none"], W, "torch.bfloat16", True, seed=0)
    tr = Trainer(net, lr=1e-3, betas=(0.9, 0.99), eps=1e-15)
    xt, tt = _bf16(x), torch.from_numpy(t).cuda()
    first = tr.training_step(xt, tt).item()
    for _ in range(99):
        last = tr.training_step(xt, tt).item()
    assert net.status() == 0
    assert last < 0.7 * first, (first, last)


def test_training_step_replays_from_a_cuda_graph(tnn_lib):
    """A single-GPU trainer counts its optimiser steps on the device, so the whole training step (fused kernel +
    optimiser kernel) is capturable: three replays of the captured step leave the bits of three eager steps of a twin
    trainer (Adam's bias correction advances with every replay)."""
    from tiny_dpcpp_nn.trainer import Trainer

    W, nh, batch = 64, 2, 128 * 9
    x = synth.uniform_inputs(batch, W, seed=3)
    t = synth.uniform_inputs(batch, W, seed=4)
    w = synth.xavier_weights(nh + 1, W, 5)
    xt, tt = _bf16(x), torch.from_numpy(t).cuda()
    trainers = []
    for _ in range(2):
        net = tnn_lib.create_network(W, W, nh, A["relu"], A["none"], W, "torch.bfloat16", True, seed=0)
        tr = Trainer(net, lr=1e-2)
        tr.set_master_params(torch.from_numpy(O.pack_weights(w, nh + 1, W)).cuda())
        trainers.append((net, tr))
    (net_e, eager), (net_g, graphed) = trainers
    for _ in range(4):
        eager.training_step(xt, tt)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        graphed.training_step(xt, tt)  # step 1, eager, on the capturing stream (warm-up)
        with torch.cuda.graph(graph, stream=side):
            graphed.training_step(xt, tt)  # captured, not executed
    for _ in range(3):
        graph.replay()  # steps 2, 3, 4
    torch.cuda.synchronize()
    assert torch.equal(graphed.master, eager.master) and torch.equal(graphed.grads, eager.grads)
    assert torch.equal(net_g.get_params(), net_e.get_params())
    assert net_e.status() == 0 and net_g.status() == 0
