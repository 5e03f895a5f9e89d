"""Training step for a Network (optionally behind an input encoding): forward -> L2 loss -> backward ->
(gradient all-reduce) -> Adam, as one call into the library.

The reference's Trainer<T>::training_step (include/trainer.h:23-46) runs forward_pass and
backward_pass only ("no optimisation as we run benchmarking", trainer.h:39); its Python training
loops add torch's loss and torch.optim.Adam around the module.  This class is a thin front end of the
library's tnn_trainer, the device-resident equivalent of that whole loop body: nothing leaves the GPU
between the kernels, the parameter vector keeps the packed layout the reference exposes to optimisers
(modules.py:169-175), and in data-parallel runs the only communication is the sum of the fp32
weight-gradient buffer over the ranks - inside the optimiser kernel through peer windows when the ranks share a
host, else one NCCL all-reduce - plus reduce-scatter / all-gather of a trainable encoding's table.
"""
import ctypes

import torch

from . import _lib
from .parallel import create_dp_comm


class _DevArray:
    """A device buffer owned by the library, exposed through the CUDA array interface."""

    def __init__(self, ptr, n):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (int(ptr), False), "version": 2}


def _wrap(ptr, n):
    return torch.as_tensor(_DevArray(ptr, n), device="cuda")


class Trainer:
    def __init__(self, network, lr=1e-3, betas=(0.9, 0.99), eps=1e-15, loss_scale=1.0, process_group=None,
                 world_size=1, encoding=None):
        """network: a _lib.NetworkModule; encoding: an optional _lib.EncodingModule in front of it (inputs are
        then float32 coordinates).  process_group: torch.distributed group for data parallelism (None = single
        GPU); gradients are averaged over its ranks through a NCCL communicator the library creates."""
        lib = _lib.load()
        self._lib = lib
        self.net = network
        self.encoding = encoding
        self.lr, self.betas, self.eps = lr, betas, eps
        self.loss_scale = loss_scale
        self.world_size = world_size
        h = ctypes.c_void_p()
        _lib.check(lib.tnn_trainer_create(network._h, encoding._h if encoding is not None else None, lr, betas[0],
                                          betas[1], eps, loss_scale, ctypes.byref(h)))
        self._h = h
        self._comm = None
        if process_group is not None and world_size > 1:
            self._comm = create_dp_comm(process_group)
            _lib.check(lib.tnn_trainer_set_dp(self._h, self._comm))
        n = network.n_params()
        # views of the trainer's device state (fp32, packed layout)
        self.master = _wrap(lib.tnn_trainer_master_params(self._h), n)
        self.grads = _wrap(lib.tnn_trainer_grads(self._h), n)
        self._loss = _wrap(lib.tnn_trainer_loss(self._h), 1)
        self.encoding_grads = None
        if encoding is not None and encoding.n_params():
            self.encoding_grads = _wrap(lib.tnn_trainer_encoding_grads(self._h), encoding.n_params())

    def __del__(self):
        try:
            import sys
            if getattr(self, "_h", None) and not sys.is_finalizing():
                self._lib.tnn_trainer_destroy(self._h)
                self._h = None
                if self._comm:
                    self._lib.tnn_dp_comm_destroy(self._comm)
        except Exception:
            pass

    @property
    def peer_window(self):
        """True when the gradient exchange runs inside the optimiser kernel over peer windows (not NCCL)."""
        return bool(self._comm) and bool(self._lib.tnn_dp_peer_window(self._comm))

    def set_peer_window(self, on=True):
        """To be called alike on every rank, between steps."""
        if self._comm:
            _lib.check(self._lib.tnn_dp_set_peer_window(self._comm, int(bool(on))))

    @property
    def step(self):
        return int(self._lib.tnn_trainer_step_count(self._h))

    def set_deterministic_encoding(self, on=True):
        _lib.check(self._lib.tnn_trainer_set_deterministic_encoding(self._h, int(bool(on))))

    def set_master_params(self, packed_fp32):
        src = packed_fp32.reshape(-1).to(torch.float32).contiguous()
        _lib.check(self._lib.tnn_trainer_set_master_params(self._h, _lib.dptr(src), _lib.stream_ptr()))
        src.record_stream(torch.cuda.current_stream())

    def _check(self, x, targets):
        want = torch.float32 if self.encoding is not None else self.net.dtype
        if x.dtype != want or targets.dtype != torch.float32 or x.dim() != 2 or targets.dim() != 2 \
                or targets.shape[0] != x.shape[0]:
            raise _lib.TnnError(f"training inputs must be (batch, n) {want} and targets (batch, n_targets) float32")

    def forward_backward(self, x, targets):
        """x: batch x width bf16 (with an encoding: batch x n_input_dims fp32), targets: batch x n_targets fp32.
        Leaves the loss sum in self._loss and the (packed, transposed) fp32 gradient of the mean loss in self.grads."""
        self._check(x, targets)
        s = _lib.stream_ptr()
        _lib.check(self._lib.tnn_trainer_forward_backward(self._h, _lib.dptr(x), _lib.dptr(targets), targets.shape[1],
                                                          x.shape[0], s))
        _lib.check(self._lib.tnn_trainer_reduce(self._h, s))
        return self._loss

    def optimizer_step(self):
        _lib.check(self._lib.tnn_trainer_optimizer_step(self._h, _lib.stream_ptr()))

    def training_step(self, x, targets):
        """One call: fused forward / loss / backward kernel, then one kernel that finishes the gradient sums,
        applies Adam and refreshes the weights (data parallel: that kernel also exchanges the gradient through the
        peer windows; without them the all-reduce runs between two kernels)."""
        self._check(x, targets)
        _lib.check(self._lib.tnn_trainer_training_step(self._h, _lib.dptr(x), _lib.dptr(targets), targets.shape[1],
                                                       x.shape[0], _lib.stream_ptr()))
        return self._loss
