"""ctypes binding of libtnn_b200.so (the C ABI of include/tnn_b200.h).

Plays the role of the reference's pybind11 module (dpcpp_bindings/tiny_dpcpp_nn/pybind_module.cpp):
same factory names (create_network, create_encoding), same method names on the returned object
(fwd, inference, bwd_no_encoding_grad, bwd_with_encoding_grad, initial_params, set_params,
get_params, n_params, n_output_dims).  torch is used for device memory and streams only.

There is no fallback: if the shared library is missing or no CUDA device is present, loading or
creating a module raises.
"""
import ctypes
import enum
import json
import os
import sys

import torch

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(os.path.dirname(_PKG_DIR), "libtnn_b200.so")

DTYPE_BF16, DTYPE_FP16, DTYPE_FP32 = 0, 1, 2
_c = ctypes
_vp = ctypes.c_void_p

_SIGNATURES = {
    "tnn_last_error": (_c.c_char_p, []),
    "tnn_version": (_c.c_char_p, []),
    "tnn_launch_count": (_c.c_ulonglong, []),
    "tnn_network_create": (_c.c_int, [_c.c_int] * 8 + [_c.POINTER(_vp)]),
    "tnn_network_destroy": (_c.c_int, [_vp]),
    "tnn_network_n_params": (_c.c_size_t, [_vp]),
    "tnn_network_n_output_dims": (_c.c_int, [_vp]),
    "tnn_network_width": (_c.c_int, [_vp]),
    "tnn_network_n_hidden_layers": (_c.c_int, [_vp]),
    "tnn_network_initialize_params": (_c.c_int, [_vp, _c.c_uint64, _vp]),
    "tnn_network_set_params": (_c.c_int, [_vp, _vp, _c.c_int, _c.c_int, _vp]),
    "tnn_network_get_params": (_c.c_int, [_vp, _vp, _vp]),
    "tnn_network_inference": (_c.c_int, [_vp, _vp, _vp, _c.c_size_t, _vp]),
    "tnn_network_forward": (_c.c_int, [_vp, _vp, _vp, _vp, _c.c_size_t, _vp]),
    "tnn_network_backward": (_c.c_int, [_vp, _vp, _vp, _vp, _c.c_int, _c.c_int, _vp, _vp, _c.c_size_t, _vp]),
    "tnn_network_train_step": (_c.c_int, [_vp, _vp, _vp, _c.c_int, _c.c_size_t, _c.c_float, _vp, _c.c_int, _c.c_int,
                                          _vp, _vp]),
    "tnn_network_backward_from_input_supported": (_c.c_int, [_vp]),
    "tnn_network_backward_from_input": (_c.c_int, [_vp, _vp, _vp, _vp, _c.c_int, _c.c_int, _vp, _c.c_size_t, _vp]),
    "tnn_network_workspace_bytes": (_c.c_size_t, [_vp, _c.c_size_t]),
    "tnn_network_set_workspace": (_c.c_int, [_vp, _vp, _c.c_size_t]),
    "tnn_network_with_encoding_workspace_bytes": (_c.c_size_t, [_vp, _c.c_size_t]),
    "tnn_network_with_encoding_inference": (_c.c_int, [_vp, _vp, _vp, _vp, _c.c_size_t, _vp]),
    "tnn_network_with_encoding_forward": (_c.c_int, [_vp, _vp, _vp, _vp, _vp, _c.c_size_t, _vp]),
    "tnn_network_with_encoding_train_step": (_c.c_int, [_vp, _vp, _vp, _vp, _c.c_int, _c.c_size_t, _c.c_float, _vp,
                                                        _c.c_int, _c.c_int, _vp, _c.c_int, _vp, _vp]),
    "tnn_network_sync_status": (_c.c_int, [_vp, _c.POINTER(_c.c_int), _vp]),
    "tnn_network_set_variant": (_c.c_int, [_vp, _c.c_int]),
    "tnn_encoding_create": (_c.c_int, [_c.c_char_p, _c.c_int, _c.POINTER(_vp)]),
    "tnn_encoding_destroy": (_c.c_int, [_vp]),
    "tnn_encoding_n_params": (_c.c_size_t, [_vp]),
    "tnn_encoding_n_output_dims": (_c.c_int, [_vp]),
    "tnn_encoding_n_input_dims": (_c.c_int, [_vp]),
    "tnn_encoding_level_info": (_c.c_int, [_vp, _c.c_int, _c.POINTER(_c.c_uint32), _c.POINTER(_c.c_uint32),
                                           _c.POINTER(_c.c_float), _c.POINTER(_c.c_uint32)]),
    "tnn_encoding_initialize_params": (_c.c_int, [_vp, _c.c_uint64, _vp]),
    "tnn_encoding_set_params": (_c.c_int, [_vp, _vp, _vp]),
    "tnn_encoding_get_params": (_c.c_int, [_vp, _vp, _vp]),
    "tnn_encoding_params_ptr": (_vp, [_vp]),
    "tnn_encoding_bind_params": (ctypes.c_int, [_vp, _vp]),
    "tnn_encoding_forward": (_c.c_int, [_vp, _vp, _vp, _c.c_int, _c.c_size_t, _vp]),
    "tnn_encoding_backward": (_c.c_int, [_vp, _vp, _vp, _c.c_int, _vp, _c.c_size_t, _c.c_int, _vp]),
    "tnn_encoding_backward_input": (_c.c_int, [_vp, _vp, _vp, _c.c_int, _vp, _c.c_size_t, _vp]),
    "tnn_l2_loss": (_c.c_int, [_vp, _vp, _c.c_int, _vp, _vp, _c.c_size_t, _c.c_int, _c.c_float, _vp, _vp]),
    "tnn_l2_loss_dtype": (_c.c_int, [_vp, _c.c_int, _vp, _c.c_int, _vp, _vp, _c.c_size_t, _c.c_int, _c.c_float, _vp, _vp]),
    "tnn_l2_loss_static": (_c.c_int, [_vp, _vp, _c.c_int, _vp, _vp, _c.c_size_t, _c.c_int, _c.c_float, _vp, _vp]),
    "tnn_adam_step": (_c.c_int, [_vp, _vp, _vp, _vp, _c.c_size_t, _c.c_float, _c.c_int, _c.c_float, _c.c_float,
                                 _c.c_float, _c.c_float, _vp]),
    "tnn_network_adam_step": (_c.c_int, [_vp, _vp, _vp, _vp, _vp, _c.c_float, _c.c_int, _c.c_float, _c.c_float,
                                         _c.c_float, _c.c_float, _vp]),
    "tnn_dp_get_unique_id": (_c.c_int, [_vp]),
    "tnn_dp_comm_create": (_c.c_int, [_vp, _c.c_int, _c.c_int, _c.POINTER(_vp)]),
    "tnn_dp_init": (_c.c_int, [_vp, _c.POINTER(_vp)]),
    "tnn_dp_comm_destroy": (_c.c_int, [_vp]),
    "tnn_dp_rank": (_c.c_int, [_vp]),
    "tnn_dp_world_size": (_c.c_int, [_vp]),
    "tnn_dp_peer_window": (_c.c_int, [_vp]),
    "tnn_dp_set_peer_window": (_c.c_int, [_vp, _c.c_int]),
    "tnn_dp_allreduce_sum": (_c.c_int, [_vp, _vp, _c.c_size_t, _vp]),
    "tnn_trainer_create": (_c.c_int, [_vp, _vp, _c.c_float, _c.c_float, _c.c_float, _c.c_float, _c.c_float,
                                      _c.POINTER(_vp)]),
    "tnn_trainer_destroy": (_c.c_int, [_vp]),
    "tnn_trainer_set_dp": (_c.c_int, [_vp, _vp]),
    "tnn_trainer_set_deterministic_encoding": (_c.c_int, [_vp, _c.c_int]),
    "tnn_trainer_set_master_params": (_c.c_int, [_vp, _vp, _vp]),
    "tnn_trainer_master_params": (_vp, [_vp]),
    "tnn_trainer_grads": (_vp, [_vp]),
    "tnn_trainer_encoding_grads": (_vp, [_vp]),
    "tnn_trainer_loss": (_vp, [_vp]),
    "tnn_trainer_step_count": (_c.c_int, [_vp]),
    "tnn_trainer_forward_backward": (_c.c_int, [_vp, _vp, _vp, _c.c_int, _c.c_size_t, _vp]),
    "tnn_trainer_reduce": (_c.c_int, [_vp, _vp]),
    "tnn_trainer_optimizer_step": (_c.c_int, [_vp, _vp]),
    "tnn_trainer_training_step": (_c.c_int, [_vp, _vp, _vp, _c.c_int, _c.c_size_t, _vp]),
}

_lib = None


def exported_symbols():
    """Names of every entry point declared in include/tnn_b200.h."""
    return sorted(_SIGNATURES)


def load():
    """Loads libtnn_b200.so; raises if it has not been built (python tiny-dpcpp-nn_b200/build.py)."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise RuntimeError(f"{_LIB_PATH} not found: build it with `python tiny-dpcpp-nn_b200/build.py`; "
                               "there is no fallback implementation")
        lib = ctypes.CDLL(_LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


class TnnError(RuntimeError):
    pass


def check(rc):
    if rc != 0:
        raise TnnError(load().tnn_last_error().decode())


def stream_ptr():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def dptr(t):
    if t is None:
        return None
    if not t.is_cuda:
        raise TnnError("tensor must be a CUDA tensor")
    if not t.is_contiguous():
        raise TnnError("tensor must be contiguous")
    return ctypes.c_void_p(t.data_ptr())


class Activation(enum.IntEnum):
    """Same values as the reference's Activation enum; `None` is exported as `Linear`
    (pybind_module.cpp:150-160)."""
    ReLU = 0
    LeakyReLU = 1
    Exponential = 2
    Sine = 3
    Sigmoid = 4
    Squareplus = 5
    Softplus = 6
    Tanh = 7
    Linear = 8


def _dtype_code(t):
    if t == torch.bfloat16:
        return DTYPE_BF16
    if t == torch.float16:
        return DTYPE_FP16
    if t == torch.float32:
        return DTYPE_FP32
    raise TnnError(f"unsupported dtype {t}")


class NetworkModule:
    """tnn::NetworkModule<bf16, WIDTH> (include/tnn_api.h:491-697) over the C ABI.

    Stateful like the reference: backward uses the forward workspace of the immediately
    preceding fwd() call of the same batch."""

    def __init__(self, input_width, output_width, n_hidden_layers, activation, output_activation, width, dtype,
                 use_bias, seed=None):
        lib = load()
        if dtype not in ("torch.bfloat16", "torch.float16"):
            raise TnnError("Unsupported dtype: " + str(dtype) + ". Only fp16 and bf16 are supported")
        h = _vp()
        check(lib.tnn_network_create(int(input_width), int(output_width), int(n_hidden_layers), int(activation),
                                     int(output_activation), int(width),
                                     DTYPE_BF16 if dtype == "torch.bfloat16" else DTYPE_FP16, int(bool(use_bias)),
                                     ctypes.byref(h)))
        self._h = h
        self._lib = lib
        self.width = int(width)
        self.dtype = torch.bfloat16 if dtype == "torch.bfloat16" else torch.float16
        self.n_mat = int(n_hidden_layers) + 1
        self._interm_fwd = None
        self._batch = 0
        if seed is None:
            seed = int.from_bytes(os.urandom(4), "little")
        check(lib.tnn_network_initialize_params(self._h, seed, stream_ptr()))

    def __del__(self):
        # at interpreter shutdown the CUDA runtime may already be gone; the process exit frees the memory
        try:
            if getattr(self, "_h", None) and not sys.is_finalizing():
                self._lib.tnn_network_destroy(self._h)
                self._h = None
        except Exception:  # module globals are already torn down
            pass

    def n_params(self):
        return int(self._lib.tnn_network_n_params(self._h))

    def n_output_dims(self):
        return int(self._lib.tnn_network_n_output_dims(self._h))

    def set_variant(self, v):
        check(self._lib.tnn_network_set_variant(self._h, int(v)))

    def status(self):
        st = _c.c_int(0)
        check(self._lib.tnn_network_sync_status(self._h, ctypes.byref(st), stream_ptr()))
        return st.value

    def _check_input(self, x):
        if x.dim() != 2 or x.shape[1] != self.width:
            raise TnnError(f"Input has {tuple(x.shape)} but the network expects (batch, {self.width})")
        if x.dtype != self.dtype:
            raise TnnError(f"network tensors must be {self.dtype}")

    def inference(self, x):
        self._check_input(x)
        y = torch.empty_like(x)
        check(self._lib.tnn_network_inference(self._h, dptr(x), dptr(y), x.shape[0], stream_ptr()))
        return y

    def fwd(self, x):
        self._check_input(x)
        batch = x.shape[0]
        if self._interm_fwd is None or self._interm_fwd.shape[1] != batch:
            self._interm_fwd = torch.empty((self.n_mat + 1, batch, self.width), dtype=self.dtype, device=x.device)
        self._batch = batch
        check(self._lib.tnn_network_forward(self._h, dptr(x), None, dptr(self._interm_fwd), batch, stream_ptr()))
        return self._interm_fwd[self.n_mat].clone()

    def interm_fwd(self):
        return self._interm_fwd

    def bwd_no_encoding_grad(self, grad_output, pack_gradient, get_dl_dinput, want_interm_bwd=False,
                             grads_dtype=None):
        grads_dtype = grads_dtype or self.dtype  # the reference returns gradients in the network's type
        if grad_output.dim() != 2 or grad_output.shape[1] != self.width:
            raise TnnError(f"grad_output.size(1): {grad_output.shape[-1]} is not equal to get_padded_output_width "
                           f"{self.width}")
        batch = grad_output.shape[0]
        if self._interm_fwd is None or batch != self._batch:
            raise TnnError("backward_pass needs the forward pass of the same batch first")
        dev = grad_output.device
        grads = torch.empty((self.n_params(), 1), dtype=grads_dtype, device=dev)
        if grad_output.dtype != self.dtype:
            raise TnnError(f"grad_output must be {self.dtype}")
        dx = torch.empty((batch, self.width), dtype=self.dtype, device=dev) if get_dl_dinput else None
        ibwd = torch.empty((self.n_mat, batch, self.width), dtype=self.dtype, device=dev) if want_interm_bwd else None
        check(self._lib.tnn_network_backward(self._h, dptr(grad_output), dptr(self._interm_fwd), dptr(grads),
                                             _dtype_code(grads_dtype), int(bool(pack_gradient)), dptr(dx), dptr(ibwd),
                                             batch, stream_ptr()))
        self._interm_bwd = ibwd
        return (dx.reshape(-1, 1) if dx is not None else None), grads

    def recompute_supported(self):
        """True when bwd_from_input can serve this network (it fits the fused training kernel)."""
        return bool(self._lib.tnn_network_backward_from_input_supported(self._h))

    def bwd_from_input(self, x, grad_output, pack_gradient, get_dl_dinput, grads_dtype=None):
        """backward_pass given the input of the forward pass instead of stored activations: one fused kernel
        recomputes them on chip.  Returns (dL/dinput or None, grads) like bwd_no_encoding_grad."""
        grads_dtype = grads_dtype or self.dtype
        self._check_input(x)
        if grad_output.shape != x.shape or grad_output.dtype != self.dtype:
            raise TnnError(f"grad_output must be {tuple(x.shape)} {self.dtype}")
        batch = x.shape[0]
        grads = torch.empty((self.n_params(), 1), dtype=grads_dtype, device=x.device)
        dx = torch.empty((batch, self.width), dtype=self.dtype, device=x.device) if get_dl_dinput else None
        check(self._lib.tnn_network_backward_from_input(self._h, dptr(x), dptr(grad_output), dptr(grads),
                                                        _dtype_code(grads_dtype), int(bool(pack_gradient)), dptr(dx),
                                                        batch, stream_ptr()))
        return (dx.reshape(-1, 1) if dx is not None else None), grads

    def bwd_with_encoding_grad(self, grad_output, input_from_fwd, pack_gradient, get_dl_dinput):
        raise TnnError("backward_pass of NetworkModule takes no input_from_fwd")

    def initial_params(self, tensor=None):
        if tensor is not None:
            self.set_params(tensor, False)
        return self.get_params()

    def set_params(self, params, weights_are_packed):
        params = params.contiguous().reshape(-1)
        if params.numel() != self.n_params():
            raise TnnError(f"m_weights_matrices nelements: {self.n_params()} does not match unpacked_weights size: "
                           f"{params.numel()}. Consider padding input and output to have the same amount as "
                           "network_width")
        check(self._lib.tnn_network_set_params(self._h, dptr(params), _dtype_code(params.dtype),
                                               int(bool(weights_are_packed)), stream_ptr()))
        # keep `params` alive until the copy kernel has run on this stream
        params.record_stream(torch.cuda.current_stream())

    def get_params(self):
        out = torch.empty((self.n_params(), 1), dtype=self.dtype, device="cuda")
        check(self._lib.tnn_network_get_params(self._h, dptr(out), stream_ptr()))
        return out

    def adam_step(self, master, m, v, grads, step, lr=1e-3, beta1=0.9, beta2=0.99, eps=1e-15, grad_scale=1.0):
        check(self._lib.tnn_network_adam_step(self._h, dptr(master), dptr(m), dptr(v), dptr(grads), grad_scale, step,
                                              lr, beta1, beta2, eps, stream_ptr()))


class EncodingModule:
    """tnn::EncodingModule<float> (include/tnn_api.h:306-488) over the C ABI."""

    def __init__(self, name, config, padded_output_width=None, seed=None):
        lib = load()
        cfg = dict(config)
        cfg.setdefault("otype", name)
        h = _vp()
        check(lib.tnn_encoding_create(json.dumps(cfg).encode(), int(padded_output_width or 0), ctypes.byref(h)))
        self._h = h
        self._lib = lib
        if self.n_params():
            if seed is None:
                seed = int.from_bytes(os.urandom(4), "little")
            check(lib.tnn_encoding_initialize_params(self._h, seed, stream_ptr()))

    def __del__(self):
        try:
            if getattr(self, "_h", None) and not sys.is_finalizing():
                self._lib.tnn_encoding_destroy(self._h)
                self._h = None
        except Exception:
            pass

    def n_params(self):
        return int(self._lib.tnn_encoding_n_params(self._h))

    def n_output_dims(self):
        return int(self._lib.tnn_encoding_n_output_dims(self._h))

    def n_input_dims(self):
        return int(self._lib.tnn_encoding_n_input_dims(self._h))

    def level_info(self, level):
        off, size, res = _c.c_uint32(), _c.c_uint32(), _c.c_uint32()
        scale = _c.c_float()
        check(self._lib.tnn_encoding_level_info(self._h, level, ctypes.byref(off), ctypes.byref(size),
                                                ctypes.byref(scale), ctypes.byref(res)))
        return off.value, size.value, scale.value, res.value

    def fwd(self, x, out_dtype=torch.float32):
        if x.dim() != 2 or x.shape[1] != self.n_input_dims():
            raise TnnError("Input tensor has incorrect dimensions")
        if x.dtype != torch.float32:
            raise TnnError("encoding input must be torch.float32")
        out = torch.empty((x.shape[0], self.n_output_dims()), dtype=out_dtype, device=x.device)
        check(self._lib.tnn_encoding_forward(self._h, dptr(x), dptr(out), _dtype_code(out_dtype), x.shape[0],
                                             stream_ptr()))
        return out

    inference = fwd

    def bwd_no_encoding_grad(self, grad_output, pack_gradient, get_dl_dinput):
        raise TnnError("backward_pass needs input_from_fwd")

    #: default summation of the table gradient: False = floating-point reductions in memory like the reference's
    #: kernel_grid_backward (grid.h:177-183, order not fixed, fastest); True = 64-bit fixed-point accumulation whose
    #: result repeats bit for bit (about 3x slower at the benchmark grid); 2 = atomic-free segmented reduction in a
    #: fixed order (bit-reproducible as well, slower again)
    deterministic_backward = False

    def bwd_with_encoding_grad(self, grad_output, input_from_fwd, pack_gradient, get_dl_dinput, deterministic=None):
        if deterministic is None:
            deterministic = self.deterministic_backward
        if self.n_params() == 0:
            return None, None
        if pack_gradient:
            raise TnnError("Encoding params are not packed")
        if get_dl_dinput:
            raise TnnError("Encoding get_dl_dinput not implemented")
        batch = grad_output.shape[0]
        if input_from_fwd.dim() != 2 or input_from_fwd.shape[0] != batch or \
                input_from_fwd.shape[1] != self.n_input_dims():
            raise TnnError("Size mismatch for input_from_fwd")
        grads = torch.empty((self.n_params(), 1), dtype=torch.float32, device=grad_output.device)
        check(self._lib.tnn_encoding_backward(self._h, dptr(input_from_fwd), dptr(grad_output),
                                              _dtype_code(grad_output.dtype), dptr(grads), batch,
                                              int(deterministic), stream_ptr()))
        return None, grads

    def bwd_input(self, grad_output, input_from_fwd):
        """dL/dinput (batch x n_input_dims, float32) of the encoding: tnn_encoding_backward_input."""
        batch = grad_output.shape[0]
        if input_from_fwd.dim() != 2 or input_from_fwd.shape[0] != batch or input_from_fwd.shape[1] != self.n_input_dims() \
                or grad_output.shape[1] != self.n_output_dims():
            raise TnnError("Size mismatch for input_from_fwd")
        dx = torch.empty((batch, self.n_input_dims()), dtype=torch.float32, device=grad_output.device)
        check(self._lib.tnn_encoding_backward_input(self._h, dptr(input_from_fwd), dptr(grad_output),
                                                    _dtype_code(grad_output.dtype), dptr(dx), batch, stream_ptr()))
        return dx

    def initial_params(self, tensor=None):
        if tensor is not None:
            self.set_params(tensor, False)
        return self.get_params()

    def set_params(self, params, weights_are_packed=False):
        if self.n_params() == 0:
            raise TnnError("no encoding params to set")
        if weights_are_packed:
            raise TnnError("Packed weights are not supported in api set params")
        params = params.contiguous().reshape(-1)
        if params.dtype != torch.float32 or params.numel() != self.n_params():
            raise TnnError("encoding params must be n_params float32 values")
        check(self._lib.tnn_encoding_set_params(self._h, dptr(params), stream_ptr()))
        params.record_stream(torch.cuda.current_stream())

    def bind_params(self, params):
        """Use `params` (n_params float32 values on the device) in place as the parameter table; the caller keeps
        the tensor alive while it is bound.  None returns to the table owned by the handle."""
        if params is None:
            check(self._lib.tnn_encoding_bind_params(self._h, None))
            self._bound = None
            return
        if params.dtype != torch.float32 or params.numel() != self.n_params() or not params.is_contiguous() \
                or not params.is_cuda:
            raise TnnError("bound encoding params must be n_params contiguous float32 values on the device")
        check(self._lib.tnn_encoding_bind_params(self._h, dptr(params)))
        self._bound = params  # keeps the storage alive

    def get_params(self):
        out = torch.empty((self.n_params(), 1) if self.n_params() else (0,), dtype=torch.float32, device="cuda")
        if self.n_params():
            check(self._lib.tnn_encoding_get_params(self._h, dptr(out), stream_ptr()))
        return out


def create_network(input_width, output_width, n_hidden_layers, activation, output_activation, width, dtype, use_bias,
                   seed=None):
    """pybind_module.cpp:90-139, 175-179."""
    return NetworkModule(input_width, output_width, n_hidden_layers, activation, output_activation, width, dtype,
                         use_bias, seed=seed)


def create_encoding(name, config, padded_output_width=None, seed=None):
    """pybind_module.cpp:141-147, 180."""
    return EncodingModule(name, config, padded_output_width, seed=seed)


def l2_loss(pred, target, loss_scale=1.0, want_values=False):
    """L2Loss::evaluate over the C ABI.  Returns (loss_sum tensor, grads bf16, values or None)."""
    lib = load()
    batch, stride = pred.shape
    grads = torch.empty_like(pred)
    values = torch.empty((batch, stride), dtype=torch.float32, device=pred.device) if want_values else None
    loss_sum = torch.zeros(1, dtype=torch.float32, device=pred.device)
    check(lib.tnn_l2_loss_dtype(dptr(pred), _dtype_code(pred.dtype), dptr(target), target.shape[1], dptr(values),
                                dptr(grads), batch, stride, float(loss_scale), dptr(loss_sum), stream_ptr()))
    return loss_sum, grads, values


def l2_loss_static(pred, target, loss_sum, grads, values=None, loss_scale=1.0):
    """tnn_l2_loss_static: every buffer comes from the caller and the library allocates nothing (its scratch
    is a fixed array inside the library).  Raises TnnError beyond 2^27 elements."""
    lib = load()
    batch, stride = pred.shape
    check(lib.tnn_l2_loss_static(dptr(pred), dptr(target), target.shape[1], dptr(values), dptr(grads), batch, stride,
                                 float(loss_scale), dptr(loss_sum), stream_ptr()))


def nwe_inference(net, enc, x, out=None):
    """tnn_network_with_encoding_inference: y = network(encoding(x)) without the encoded matrix in between where the
    kernels can fold the encoding (identity).  x: batch x n_input_dims float32; returns batch x width bfloat16."""
    lib = load()
    if x.dtype != torch.float32 or x.dim() != 2 or x.shape[1] != enc.n_input_dims():
        raise TnnError("encoding input must be (batch, n_input_dims) float32")
    y = out if out is not None else torch.empty((x.shape[0], net.width), dtype=net.dtype, device=x.device)
    check(lib.tnn_network_with_encoding_inference(net._h, enc._h, dptr(x), dptr(y), x.shape[0], stream_ptr()))
    return y


def nwe_forward(net, enc, x):
    """tnn_network_with_encoding_forward in training mode: stores the activations in the network module (matrix 0 =
    the encoded input) for a following bwd_no_encoding_grad, returns the output rows."""
    lib = load()
    batch = x.shape[0]
    if net._interm_fwd is None or net._interm_fwd.shape[1] != batch:
        net._interm_fwd = torch.empty((net.n_mat + 1, batch, net.width), dtype=net.dtype, device=x.device)
    net._batch = batch
    check(lib.tnn_network_with_encoding_forward(net._h, enc._h, dptr(x), None, dptr(net._interm_fwd), batch,
                                                stream_ptr()))
    return net._interm_fwd[net.n_mat].clone()


def adam_step(params, m, v, grads, step, lr=1e-3, beta1=0.9, beta2=0.99, eps=1e-15, grad_scale=1.0):
    lib = load()
    check(lib.tnn_adam_step(dptr(params), dptr(m), dptr(v), dptr(grads), params.numel(), grad_scale, step, lr, beta1,
                            beta2, eps, stream_ptr()))
