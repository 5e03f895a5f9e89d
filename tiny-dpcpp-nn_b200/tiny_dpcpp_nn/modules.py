"""torch.nn.Module front end: Network, Encoding, NetworkWithInputEncoding.

Mirrors dpcpp_bindings/tiny_dpcpp_nn/modules.py of the reference - same class names, constructor
arguments, padding rules (batch to a multiple of 8, network input columns to `width` with the value
of use_bias), loss scaling, packed parameter vector and autograd contract - with device "cuda" and
the B200 kernels behind it.  Differences that are deliberate:
  * parameters are pushed to the backend with a device-to-device kernel, not through the host
    (reference: tnn_api.h:637-641 copies the tensor to a std::vector on every forward);
  * NetworkWithInputEncoding with an Identity or HashGrid encoding runs its forward pass as ONE kernel: the encoding
    is produced inside the network kernel (identity: folded into the first-layer load; hash grid: gathered by extra
    warps) instead of chaining two modules through a batch x width matrix.
"""
import torch

from ._lib import Activation, TnnError, create_encoding, create_network, nwe_forward, nwe_inference

MIN_BATCH_SIZE = 8  # smallest batch granularity of the network kernels (SwiftNetMLP.h:293-302)


def free_temporary_memory():
    """Kept for compatibility with the reference package (modules.py:17-19)."""


def unpad_tensor_to_input_dim(padded_tensor, output_dim):
    batch_size, current_width = padded_tensor.shape
    if output_dim > current_width:
        raise ValueError("input_dim must be less than or equal to the current width of the tensor")
    return padded_tensor[:, :output_dim]


def get_dpcpp_activation(name):
    """modules.py:33-46 of the reference."""
    lname = name.lower()
    if lname == "relu":
        return Activation.ReLU
    if lname == "tanh":
        return Activation.Tanh
    if lname == "sigmoid":
        return Activation.Sigmoid
    if lname in ("linear", "none"):
        return Activation.Linear
    raise NotImplementedError(f"Activation: {name} not defined")


def to_packed_layout_coord(idx, rows, cols):
    i, j = idx // cols, idx % cols
    return i * cols + 2 * j if (i % 2) == 0 else (i - 1) * cols + 2 * j + 1


def from_packed_layout_coord(idx, rows, cols):
    i, j = idx // (cols * 2), idx % (cols * 2)
    return (i * 2) * cols + j // 2 if (j % 2) == 0 else (i * 2 + 1) * cols + (j - 1) // 2


class _module_function(torch.autograd.Function):
    """modules.py:68-141 of the reference."""

    @staticmethod
    def forward(ctx, native_tnn_module, input, params, info, loss_scale):
        batch_size = input.shape[0]
        if "encoding_out_dtype" in info:
            # an encoding that feeds a network writes the network's dtype directly: no separate cast pass
            output = native_tnn_module.fwd(input, out_dtype=info["encoding_out_dtype"])
        elif info["is_in_eval_mode"]:
            output = native_tnn_module.inference(input)
        elif getattr(native_tnn_module, "recompute_supported", lambda: False)():
            # the backward pass recomputes the activations on chip from `input` (one fused kernel), so the forward
            # pass stores none of them: the (n_hidden_layers + 2) x batch x width block is neither written nor read
            output = native_tnn_module.inference(input)
            ctx.recompute = True
        else:
            output = native_tnn_module.fwd(input)
        if batch_size > 0:
            output = output.reshape(batch_size, -1)
        ctx.save_for_backward(input, output, params)
        ctx.info = info
        ctx.native_tnn_module = native_tnn_module
        ctx.loss_scale = loss_scale
        if "output_dim" in info:
            return output[..., : info["output_dim"]]  # columns after output_dim are padding
        return output

    @staticmethod
    def backward(ctx, doutput):
        input, _, params = ctx.saved_tensors
        loss_scale = ctx.loss_scale
        if "width" in ctx.info and doutput.shape[1] < ctx.info["width"]:
            pad = torch.zeros(doutput.shape[0], ctx.info["width"] - doutput.shape[1], device=doutput.device,
                              dtype=doutput.dtype)
            doutput = torch.hstack((doutput, pad))
        batch_size = input.shape[0]
        doutput = (doutput * loss_scale).contiguous()
        with torch.no_grad():
            if "encoding_config" in ctx.info:
                input_grad = None
                dy = doutput if doutput.dtype in (torch.bfloat16, torch.float16) else doutput.float()
                if batch_size == 0 or params.numel() <= 1:
                    grad = torch.zeros_like(params)
                else:
                    _, grad = ctx.native_tnn_module.bwd_with_encoding_grad(dy, input, False, False)
                if ctx.needs_input_grad[1] and batch_size > 0:
                    # gradient with respect to the encoded positions (the reference's Python layer cannot provide it:
                    # include/tnn_api.h:380-382)
                    input_grad = ctx.native_tnn_module.bwd_input(dy, input)
            else:
                if getattr(ctx, "recompute", False):
                    input_grad, grad = ctx.native_tnn_module.bwd_from_input(
                        input, doutput.to(ctx.native_tnn_module.dtype), True, True, grads_dtype=torch.float32)
                else:
                    input_grad, grad = ctx.native_tnn_module.bwd_no_encoding_grad(
                        doutput.to(ctx.native_tnn_module.dtype), True, True, grads_dtype=torch.float32)
                if input_grad is not None:
                    input_grad = input_grad.reshape(batch_size, -1).to(input.dtype)
        grad = None if grad is None else (grad.reshape(params.shape).to(params.dtype) / loss_scale)
        input_grad = None if input_grad is None else (input_grad / loss_scale)
        return (None, input_grad, grad, None, None)


class _fused_module_function(torch.autograd.Function):
    """Encoding + network as one operator.  Inference is a single library call (identity encoding folded into the
    first-layer load).  Training keeps only the encoded rows between the passes: forward = encoding kernel + inference
    kernel, backward = one fused kernel that recomputes the network's activations on chip and yields the weight
    gradients and dL/d(encoded rows), which an encoding with parameters scatters into its table gradient (networks
    outside the fused kernel's limits store their activations instead).  Same parameter contract as _module_function;
    the positions get no gradient."""

    @staticmethod
    def forward(ctx, native_network, native_encoding, input, net_params, enc_params, info, loss_scale):
        ctx.encoded = None
        if info["is_in_eval_mode"]:
            output = nwe_inference(native_network, native_encoding, input)
        elif native_network.recompute_supported():
            # training forward without stored activations: the encoded rows (128 bytes per sample at width 64) are all
            # the backward pass needs, it recomputes the network's activations on chip
            ctx.encoded = native_encoding.fwd(input, out_dtype=native_network.dtype)
            output = native_network.inference(ctx.encoded)
        else:
            output = nwe_forward(native_network, native_encoding, input)
        ctx.save_for_backward(input, net_params, enc_params)
        ctx.info = info
        ctx.native_network = native_network
        ctx.native_encoding = native_encoding
        ctx.loss_scale = loss_scale
        return output[..., : info["output_dim"]]

    @staticmethod
    def backward(ctx, doutput):
        input, net_params, enc_params = ctx.saved_tensors
        width = ctx.info["width"]
        if doutput.shape[1] < width:
            doutput = torch.nn.functional.pad(doutput, [0, width - doutput.shape[1]])
        doutput = (doutput * ctx.loss_scale).to(ctx.native_network.dtype).contiguous()
        want_enc = ctx.native_encoding.n_params() > 0 and ctx.needs_input_grad[4]
        enc_grad = None
        with torch.no_grad():
            if ctx.encoded is not None:
                dx, grad = ctx.native_network.bwd_from_input(ctx.encoded, doutput, True, want_enc,
                                                             grads_dtype=torch.float32)
                ctx.encoded = None
            else:
                dx, grad = ctx.native_network.bwd_no_encoding_grad(doutput, True, want_enc, grads_dtype=torch.float32)
            if want_enc:
                _, enc_grad = ctx.native_encoding.bwd_with_encoding_grad(dx.reshape(input.shape[0], width), input, False,
                                                                         False)
                enc_grad = enc_grad.reshape(enc_params.shape).to(enc_params.dtype) / ctx.loss_scale
        grad = grad.reshape(net_params.shape).to(net_params.dtype) / ctx.loss_scale
        return (None, None, None, grad, enc_grad, None, None)


class Module(torch.nn.Module):
    """modules.py:144-261 of the reference."""

    def __init__(self, dtype, device="cuda", store_params_as_full_precision=True, use_bias=True, init_module=True):
        super().__init__()
        self.device = device
        self.use_bias = use_bias
        self.dtype = dtype
        self.store_params_as_full_precision = store_params_as_full_precision
        self.loss_scale = 128.0 if dtype == torch.float16 else 1.0
        if not init_module:
            return
        self.tnn_module = self.create_module()
        if self.tnn_module.n_params():
            initial_params = self.tnn_module.initial_params()
            params_dtype = torch.float32 if self.store_params_as_full_precision else self.dtype
            self.params = torch.nn.Parameter(initial_params.clone().detach().to(params_dtype), requires_grad=True)
        else:
            self.params = torch.nn.Parameter(torch.zeros(1, device=self.device), requires_grad=False)

    def set_params(self, params=None):
        if not self.tnn_module.n_params():
            if params is not None:
                raise RuntimeError("Network has no parameters. Cannot set params")
            return
        packed = params is None and self.name != "encoding"  # encoding weights are never packed
        if params is None:
            # (pushed before every forward like modules.py:236 of the reference: an optimiser that writes through
            # `.data` leaves no trace on the tensor's version counter, so the push cannot be skipped safely)
            params = self.params
        assert isinstance(params, torch.Tensor), "Params is not a torch.Tensor"
        src = params.detach()
        if self.name == "encoding" and params is self.params and src.dtype == torch.float32 and src.is_contiguous():
            # the parameter tensor itself is the table the kernels read: no copy per forward pass
            if getattr(self, "_bound_ptr", None) != src.data_ptr():
                self.tnn_module.bind_params(src)
                self._bound_ptr = src.data_ptr()
            return
        if self.name == "encoding":
            src = src.to(torch.float32)
        elif src.dtype not in (torch.float32, torch.bfloat16, torch.float16):
            src = src.to(torch.float32)
        self.tnn_module.set_params(src, packed)
        if not packed and self.name != "encoding":
            self.params.data.copy_(self.get_params().to(self.params.dtype))  # always the packed vector
        elif not packed:
            self.params.data.copy_(self.get_params().to(self.params.dtype).reshape(self.params.shape))

    def get_params(self):
        return self.tnn_module.get_params()

    def forward(self, x):
        batch_size, input_dim = x.shape
        padded_batch_size = (batch_size + MIN_BATCH_SIZE - 1) // MIN_BATCH_SIZE * MIN_BATCH_SIZE
        padded_tensor = (x if batch_size == padded_batch_size
                         else torch.nn.functional.pad(x, [0, 0, 0, padded_batch_size - batch_size])).to(dtype=self.dtype)
        if self.name == "network" and input_dim != self.width:
            padded_tensor = torch.nn.functional.pad(padded_tensor, [0, self.width - input_dim, 0, 0], "constant",
                                                    float(self.use_bias)).to(dtype=self.dtype)
        info = {"is_in_eval_mode": not self.training}
        if hasattr(self, "n_hidden_layers"):
            info.update({"n_hidden_layers": self.n_hidden_layers - 1, "input_dim": self.n_input_dims,
                         "output_dim": self.n_output_dims, "width": self.width})
        if hasattr(self, "encoding_config"):
            info.update({"encoding_config": self.encoding_config})
            if getattr(self, "output_dtype", None) is not None:
                info.update({"encoding_out_dtype": self.output_dtype})
        self.set_params()
        output = _module_function.apply(self.tnn_module, padded_tensor.contiguous(), self.params, info,
                                        self.loss_scale)
        return output[:batch_size, ...]


class Network(Module):
    """modules.py:264-306 of the reference."""

    def __init__(self, n_input_dims, n_output_dims, network_config, store_params_as_full_precision=True,
                 device="cuda", dtype=torch.bfloat16, use_bias=True, seed=None):
        assert dtype in (torch.float16, torch.bfloat16), \
            f"Only torch.float16 or torch.bfloat16 supported, got: {dtype}"
        self.network_config = network_config
        self.width = self.network_config["n_neurons"]
        self.n_input_dims = n_input_dims
        self.n_output_dims = n_output_dims
        self.n_hidden_layers = self.network_config["n_hidden_layers"]
        self.activation = get_dpcpp_activation(self.network_config["activation"])
        self.output_activation = get_dpcpp_activation(self.network_config["output_activation"])
        self.name = "network"
        self._seed = seed
        super().__init__(device=device, dtype=dtype, store_params_as_full_precision=store_params_as_full_precision,
                         use_bias=use_bias)

    def create_module(self):
        return create_network(self.n_input_dims, self.n_output_dims, self.n_hidden_layers, self.activation,
                              self.output_activation, self.width, str(self.dtype), self.use_bias, seed=self._seed)


class Encoding(Module):
    """modules.py:309-354 of the reference."""

    def __init__(self, n_input_dims, encoding_config, n_output_dims=None, device="cuda", dtype=torch.float,
                 store_params_as_full_precision=True, seed=None):
        assert dtype == torch.float, "Only torch.float is currently supported for encoding"
        self.n_input_dims = n_input_dims
        self.encoding_config = dict(encoding_config)
        self.padded_output_dims = n_output_dims
        self.encoding_name = self.encoding_config["otype"]
        self.name = "encoding"
        self._seed = seed
        if "n_dims_to_encode" not in self.encoding_config:
            self.encoding_config["n_dims_to_encode"] = self.n_input_dims
        super().__init__(device=device, dtype=dtype, store_params_as_full_precision=store_params_as_full_precision)
        self.n_output_dims = self.tnn_module.n_output_dims()

    def create_module(self):
        return create_encoding(self.encoding_name, self.encoding_config, self.padded_output_dims, seed=self._seed)


class NetworkWithInputEncoding(Module):
    """modules.py:357-421 of the reference: an Encoding feeding a Network."""

    def __init__(self, n_input_dims, n_output_dims, network_config, encoding_config, device="cuda",
                 store_params_as_full_precision=True, dtype=torch.bfloat16, use_bias=True, seed=None):
        assert dtype in (torch.float16, torch.bfloat16), \
            f"Only torch.float16 or torch.bfloat16 supported, got: {dtype}."
        super().__init__(dtype=dtype, init_module=False)
        self.encoding_config = encoding_config
        self.network_config = network_config
        self.width = self.network_config["n_neurons"]
        self.n_input_dims = n_input_dims
        self.n_output_dims = n_output_dims
        self.n_hidden_layers = self.network_config["n_hidden_layers"]
        self.activation = get_dpcpp_activation(self.network_config["activation"])
        self.output_activation = get_dpcpp_activation(self.network_config["output_activation"])
        self.name = "network_with_encoding"
        self.encoding = Encoding(n_input_dims, encoding_config, device=device, dtype=torch.float,
                                 store_params_as_full_precision=store_params_as_full_precision,
                                 n_output_dims=network_config["n_neurons"], seed=seed)
        assert self.encoding.n_output_dims == network_config["n_neurons"]
        self.encoding.output_dtype = dtype  # the reference casts in Python (modules.py:223); here the kernel does
        self.network = Network(self.encoding.n_output_dims, n_output_dims, network_config, device=device, dtype=dtype,
                               store_params_as_full_precision=store_params_as_full_precision, use_bias=use_bias,
                               seed=seed)
        self.network_with_encoding = torch.nn.Sequential(self.encoding, self.network)

    @property
    def params(self):
        return self.network.params

    def get_params(self):
        raise RuntimeError("Not implemented.")

    def set_params(self, params=None):
        self.network.set_params(params)

    def _fusable(self):
        """One forward kernel for the pair: Identity (up to 16 inputs) or a 2-D / 3-D HashGrid with two features per
        level whose features fit the network width; anything else runs as the two chained modules."""
        cfg = self.encoding.encoding_config
        if self.encoding.encoding_name == "Identity":
            return self.encoding.n_input_dims <= 16
        if self.encoding.encoding_name == "HashGrid":
            return self.encoding.n_input_dims in (2, 3) and int(cfg.get("n_features_per_level", 2)) == 2
        return False

    _foldable = _fusable

    def forward(self, x):
        if not self._fusable() or x.requires_grad:
            return self.network_with_encoding(x)
        batch_size = x.shape[0]
        padded = (batch_size + MIN_BATCH_SIZE - 1) // MIN_BATCH_SIZE * MIN_BATCH_SIZE
        xin = x.to(torch.float32)
        if padded != batch_size:
            xin = torch.nn.functional.pad(xin, [0, 0, 0, padded - batch_size])
        info = {"is_in_eval_mode": not self.training, "output_dim": self.n_output_dims, "width": self.width}
        self.network.set_params()
        self.encoding.set_params()
        out = _fused_module_function.apply(self.network.tnn_module, self.encoding.tnn_module, xin.contiguous(),
                                           self.network.params, self.encoding.params, info, self.network.loss_scale)
        return out[:batch_size, ...]
