"""Training step for a Network: forward -> L2 loss -> backward -> (gradient all-reduce) -> Adam.

The reference's Trainer<T>::training_step (include/trainer.h:23-46) runs forward_pass and
backward_pass only ("no optimisation as we run benchmarking", trainer.h:39); its Python training
loops add torch's loss and torch.optim.Adam around the module.  This class is the device-resident
equivalent of that whole loop body: nothing leaves the GPU between the kernels, the parameter
vector keeps the packed layout the reference exposes to optimisers (modules.py:169-175), and in
data-parallel runs the only communication is one all-reduce of the fp32 weight-gradient buffer.
"""
import torch

from . import _lib
from .parallel import allreduce_sum_


class Trainer:
    def __init__(self, network, lr=1e-3, betas=(0.9, 0.99), eps=1e-15, loss_scale=1.0, process_group=None,
                 world_size=1):
        """network: a _lib.NetworkModule.  process_group: torch.distributed group for data parallelism
        (None = single GPU); gradients are averaged over world_size ranks."""
        self.net = network
        self.lr, self.betas, self.eps = lr, betas, eps
        self.loss_scale = loss_scale
        self.pg = process_group
        self.world_size = world_size
        n = network.n_params()
        self.master = network.get_params().float().reshape(-1).contiguous()  # fp32 master copy, packed layout
        self.m = torch.zeros(n, dtype=torch.float32, device="cuda")
        self.v = torch.zeros(n, dtype=torch.float32, device="cuda")
        self.grads = torch.zeros(n, dtype=torch.float32, device="cuda")
        self.step = 0
        self._loss = torch.zeros(1, dtype=torch.float32, device="cuda")

    def set_master_params(self, packed_fp32):
        self.master.copy_(packed_fp32.reshape(-1))
        self.net.set_params(self.master, True)

    def forward_backward(self, x, targets):
        """x: batch x width bf16, targets: batch x n_targets fp32.  Leaves the loss sum in self._loss
        and the (packed, transposed) fp32 gradient of the mean loss in self.grads.  One call into the
        library: forward, L2 loss, backward and the weight-gradient reduction are fused."""
        net, lib = self.net, _lib.load()
        _lib.check(lib.tnn_network_train_step(net._h, _lib.dptr(x), _lib.dptr(targets), targets.shape[1], x.shape[0],
                                              float(self.loss_scale), _lib.dptr(self.grads), _lib.DTYPE_FP32, 1,
                                              _lib.dptr(self._loss), _lib.stream_ptr()))
        return self._loss

    def optimizer_step(self):
        if self.world_size > 1:
            allreduce_sum_(self.grads, self.pg)
        self.step += 1
        self.net.adam_step(self.master, self.m, self.v, self.grads, self.step, self.lr, self.betas[0], self.betas[1],
                           self.eps, grad_scale=1.0 / (self.loss_scale * self.world_size))

    def training_step(self, x, targets):
        loss = self.forward_backward(x, targets)
        self.optimizer_step()
        return loss
