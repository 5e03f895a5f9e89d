"""CPU test of the data-parallel semantics with two gloo ranks: every rank computes the gradient of ITS
mean loss on its row shard (here with the oracle standing in for the GPU kernel), the ranks all-reduce
(sum) the gradient buffer and scale by 1 / world - the result must equal the gradient of the mean loss
over the whole batch, and every rank must hold the same bits afterwards."""
import os
import socket
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
W, NH, BATCH, WORLD = 32, 2, 512, 2


def _grads(x, t, w):
    from oracle import oracle as O

    interm = O.mlp_forward(x, w, NH + 1, W, "relu", "none", bf16=True)
    _, dy = O.l2_loss(interm[-1], t, 1.0, bf16_grads=True)
    return O.mlp_backward(dy, interm, w, NH + 1, W, "relu", "none", bf16=True, want_dx=False)[1]


def _worker(rank, port, out_dir):
    for p in (ROOT, os.path.join(ROOT, "tiny-dpcpp-nn_b200")):
        sys.path.insert(0, p)
    from tests import synth
    from tiny_dpcpp_nn.parallel import allreduce_sum_, shard_rows

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    w, x = synth.mlp_case(W, NH, BATCH, w_seed=6)
    t = synth.uniform_inputs(BATCH, W, seed=1)
    a, b = shard_rows(BATCH, rank, WORLD)
    g = torch.from_numpy(_grads(x[a:b], t[a:b], w).astype(np.float32).reshape(-1))
    allreduce_sum_(g, dist.group.WORLD)
    g /= WORLD
    np.save(os.path.join(out_dir, f"g{rank}.npy"), g.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gradient_average_equals_full_batch_gradient(tmp_path):
    from oracle import oracle as O
    from tests import synth

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(port, str(tmp_path)), nprocs=WORLD, join=True)
    g0, g1 = np.load(tmp_path / "g0.npy"), np.load(tmp_path / "g1.npy")
    assert np.array_equal(g0, g1)
    w, x = synth.mlp_case(W, NH, BATCH, w_seed=6)
    t = synth.uniform_inputs(BATCH, W, seed=1)
    full = _grads(x, t, w).reshape(-1)
    # the per-shard dL/dy is rounded to bf16 at a different scale than the full-batch one: 1e-2 like the kernels
    ok, rel = O.within_tolerance(g0, full, 1e-2)
    assert ok, rel


def _sharded_adam_worker(rank, port, out_dir):
    """The optimiser of a trainable encoding under data parallelism: reduce-scatter of the table gradient, Adam on this
    rank's slice of the table (with its slice of the moments), all-gather of the table - against all-reduce + Adam on
    the whole table, which every rank could also do (the oracle's Adam stands in for the device kernel)."""
    for p in (ROOT, os.path.join(ROOT, "tiny-dpcpp-nn_b200")):
        sys.path.insert(0, p)
    from oracle import oracle as O

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    n, steps = 4096, 3
    shard = n // WORLD
    table = np.random.default_rng(0).uniform(-1e-4, 1e-4, n).astype(np.float32)  # identical on every rank
    full = table.copy()
    fm, fv = np.zeros(n, np.float32), np.zeros(n, np.float32)
    sm, sv = np.zeros(shard, np.float32), np.zeros(shard, np.float32)
    for step in range(1, steps + 1):
        g = np.random.default_rng(10 * step + rank).normal(size=n).astype(np.float32)  # this rank's gradient
        total = torch.from_numpy(g.copy())
        dist.all_reduce(total)
        mean = (total.numpy() / WORLD).astype(np.float32)
        O.adam(full, fm, fv, mean, step)  # replicated optimiser
        # sharded optimiser: this rank's slice of the summed gradient (what a reduce-scatter delivers) ...
        mine = np.ascontiguousarray(table[rank * shard:(rank + 1) * shard])
        O.adam(mine, sm, sv, np.ascontiguousarray(mean[rank * shard:(rank + 1) * shard]), step)
        # ... and an all-gather of the updated slices
        parts = [torch.empty(shard) for _ in range(WORLD)]
        dist.all_gather(parts, torch.from_numpy(mine))
        table = torch.cat(parts).numpy().copy()
    np.save(os.path.join(out_dir, f"sharded{rank}.npy"), table)
    np.save(os.path.join(out_dir, f"full{rank}.npy"), full)
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_adam_equals_replicated_adam(tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_sharded_adam_worker, args=(port, str(tmp_path)), nprocs=WORLD, join=True)
    s0, s1 = np.load(tmp_path / "sharded0.npy"), np.load(tmp_path / "sharded1.npy")
    f0 = np.load(tmp_path / "full0.npy")
    assert np.array_equal(s0, s1)   # every rank holds the same table after the all-gather
    assert np.array_equal(s0, f0)   # and it is the table of the replicated optimiser, bit for bit


def test_shard_rows_cover_the_batch():
    from tiny_dpcpp_nn.parallel import shard_rows

    for n, world in ((1 << 22, 8), (1000 * 24, 3), (64, 4)):
        edges = [shard_rows(n, r, world) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == n
        sizes = {b - a for a, b in edges}
        assert len(sizes) == 1 and sizes.pop() % 8 == 0  # equal shards: equal weights in the gradient average
        for (a0, b0), (a1, b1) in zip(edges, edges[1:]):
            assert b0 == a1


def test_shard_rows_rejects_unequal_or_empty_shards():
    """Unequal shards would not give the gradient of the global mean loss, an empty shard would leave one rank
    raising alone while the others wait in the all-reduce: both are refused on every rank before any collective."""
    import pytest

    from tiny_dpcpp_nn.parallel import shard_rows

    for n, world in ((8000, 3), (8, 2), (0, 2), (1 << 22, 7)):
        for r in range(world):
            with pytest.raises(ValueError):
                shard_rows(n, r, world)
