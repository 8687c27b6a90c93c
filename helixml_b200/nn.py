"""Python face of the module-level C API (hx_module_* / hx_tensor_*): the reference's
`MambaBlock::new(d_model, d_state, d_conv, expand, &device)`, `S4Block::new(d_model, d_state, &device)`,
`Linear::new`, `RMSNorm::new` and `Module::{forward, parameters}` (crates/nn/src/lib.rs:20-39, 847;
crates/nn/src/ssm.rs:39, 138) on device-resident tensors.  Errors are `HxError`s whose `.variant` is the
TensorError variant the reference would return."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib as L

F32, BF16, U8 = L.HX_F32, L.HX_BF16, L.HX_U8


class Device:
    """tensor_core::Device (crates/tensor-core/src/device.rs:8-60), CUDA variant only."""

    def __init__(self, index: int = 0):
        self.index = index

    @staticmethod
    def cuda(index: int = 0) -> "Device":
        return Device(index)

    def __repr__(self):
        return f"Cuda({self.index})"


class Tensor:
    """A device-resident tensor handle (hx_tensor)."""

    def __init__(self, handle):
        self._h = C.c_void_p(handle) if not isinstance(handle, C.c_void_p) else handle

    @staticmethod
    def from_numpy(a: np.ndarray, dtype: int = F32, device: Device = Device(0)) -> "Tensor":
        out = C.c_void_p()
        if a.dtype == np.uint8:
            a = np.ascontiguousarray(a)
            dims = (C.c_int64 * a.ndim)(*a.shape)
            L.check(L.lib().hx_tensor_from_host_u8(a.ctypes.data_as(C.c_void_p), dims, a.ndim, device.index, C.byref(out)))
        else:
            a = np.ascontiguousarray(a, dtype=np.float32)
            dims = (C.c_int64 * a.ndim)(*a.shape)
            L.check(L.lib().hx_tensor_from_host(a.ctypes.data_as(C.c_void_p), dims, a.ndim, dtype, device.index, C.byref(out)))
        return Tensor(out)

    def _info(self):
        nd, dt, dev = C.c_int32(), C.c_int32(), C.c_int32()
        dims = (C.c_int64 * 8)()
        L.check(L.lib().hx_tensor_info(self._h, C.byref(nd), dims, C.byref(dt), C.byref(dev)))
        return tuple(dims[i] for i in range(nd.value)), dt.value, dev.value

    @property
    def shape(self):
        return self._info()[0]

    @property
    def dtype(self):
        return self._info()[1]

    def numpy(self) -> np.ndarray:
        shape = self.shape
        out = np.empty(shape, dtype=np.float32)
        L.check(L.lib().hx_tensor_to_host(self._h, out.ctypes.data_as(C.c_void_p), out.size))
        return out

    def copy_from(self, a: np.ndarray) -> None:
        a = np.ascontiguousarray(a, dtype=np.float32)
        L.check(L.lib().hx_tensor_copy_from_host(self._h, a.ctypes.data_as(C.c_void_p), a.size))

    def data_ptr(self) -> int:
        return L.lib().hx_tensor_data(self._h) or 0

    # ---- the reference's tensor traits on the device tensor (crates/tensor-core/src/tensor.rs:34-275), same
    # names, same shape rules and error variants as CpuTensor (crates/backend-cpu/src/lib.rs)
    _BINARY = {"add": 0, "sub": 1, "mul": 2, "div": 3, "max": 4, "min": 5, "gt": 6}
    _UNARY = {"sqrt": 16, "exp": 17, "log": 18, "sin": 19, "cos": 20, "tan": 21, "abs": 22, "sign": 23, "neg": 24,
              "relu": 25, "gelu": 26, "silu": 27, "sigmoid": 28, "tanh": 29, "pow": 30, "clamp": 31, "add_scalar": 32,
              "mul_scalar": 33, "gt_scalar": 34, "leaky_relu": 35}

    def _binary(self, name, other: "Tensor") -> "Tensor":
        out = C.c_void_p()
        L.check(L.lib().hx_tensor_binary(self._BINARY[name], self._h, other._h, C.byref(out)))
        return Tensor(out)

    def _unary(self, name, p0=0.0, p1=0.0) -> "Tensor":
        out = C.c_void_p()
        L.check(L.lib().hx_tensor_unary(self._UNARY[name], self._h, p0, p1, C.byref(out)))
        return Tensor(out)

    def add(self, o): return self._binary("add", o)
    def sub(self, o): return self._binary("sub", o)
    def mul(self, o): return self._binary("mul", o)
    def div(self, o): return self._binary("div", o)
    def max(self, o): return self._binary("max", o)
    def min(self, o): return self._binary("min", o)
    def gt(self, o): return self._binary("gt", o)
    def sqrt(self): return self._unary("sqrt")
    def exp(self): return self._unary("exp")
    def log(self): return self._unary("log")
    def sin(self): return self._unary("sin")
    def cos(self): return self._unary("cos")
    def tan(self): return self._unary("tan")
    def abs(self): return self._unary("abs")
    def sign(self): return self._unary("sign")
    def neg(self): return self._unary("neg")
    def relu(self): return self._unary("relu")
    def gelu(self): return self._unary("gelu")
    def silu(self): return self._unary("silu")
    def sigmoid(self): return self._unary("sigmoid")
    def tanh(self): return self._unary("tanh")
    def pow(self, exponent): return self._unary("pow", exponent)
    def clamp(self, lo, hi): return self._unary("clamp", lo, hi)
    def add_scalar(self, v): return self._unary("add_scalar", v)
    def mul_scalar(self, v): return self._unary("mul_scalar", v)
    def gt_scalar(self, v): return self._unary("gt_scalar", v)
    def leaky_relu(self, slope): return self._unary("leaky_relu", slope)

    def matmul(self, other: "Tensor") -> "Tensor":
        out = C.c_void_p()
        L.check(L.lib().hx_tensor_matmul(self._h, other._h, C.byref(out)))
        return Tensor(out)

    def transpose(self, dim0: int, dim1: int) -> "Tensor":
        out = C.c_void_p()
        L.check(L.lib().hx_tensor_transpose(self._h, dim0, dim1, C.byref(out)))
        return Tensor(out)

    def slice(self, start, end) -> "Tensor":
        n = max(len(start), len(end))
        out = C.c_void_p()
        if len(start) != len(end):
            raise L.HxError(1, "slice: start and end differ in length")
        L.check(L.lib().hx_tensor_slice(self._h, (C.c_int64 * n)(*start), (C.c_int64 * n)(*end), n, C.byref(out)))
        return Tensor(out)

    @staticmethod
    def _many(fn, tensors, dim) -> "Tensor":
        arr = (C.c_void_p * len(tensors))(*[t._h.value if isinstance(t._h, C.c_void_p) else t._h for t in tensors])
        out = C.c_void_p()
        L.check(fn(arr, len(tensors), dim, C.byref(out)))
        return Tensor(out)

    @staticmethod
    def cat(tensors, dim: int) -> "Tensor":
        return Tensor._many(L.lib().hx_tensor_cat, tensors, dim)

    @staticmethod
    def stack(tensors, dim: int) -> "Tensor":
        return Tensor._many(L.lib().hx_tensor_stack, tensors, dim)

    def _shaped(self, fn, shape) -> "Tensor":
        out = C.c_void_p()
        L.check(fn(self._h, (C.c_int64 * len(shape))(*shape), len(shape), C.byref(out)))
        return Tensor(out)

    def reshape(self, shape) -> "Tensor":
        return self._shaped(L.lib().hx_tensor_reshape, shape)

    def broadcast_to(self, shape) -> "Tensor":
        return self._shaped(L.lib().hx_tensor_broadcast_to, shape)

    expand = broadcast_to

    def clone(self) -> "Tensor":
        out = C.c_void_p()
        L.check(L.lib().hx_tensor_clone(self._h, C.byref(out)))
        return Tensor(out)

    def cast(self, dtype: int) -> "Tensor":
        out = C.c_void_p()
        L.check(L.lib().hx_tensor_cast(self._h, dtype, C.byref(out)))
        return Tensor(out)

    to_dtype = cast

    def to_scalar(self) -> float:
        v = C.c_float()
        L.check(L.lib().hx_tensor_to_scalar(self._h, C.byref(v)))
        return v.value

    @staticmethod
    def from_scalar(value, shape, dtype: int = F32, device: Device = Device(0)) -> "Tensor":
        out = C.c_void_p()
        L.check(L.lib().hx_tensor_full(value, (C.c_int64 * len(shape))(*shape), len(shape), dtype, device.index, C.byref(out)))
        return Tensor(out)

    @staticmethod
    def zeros(shape, dtype: int = F32, device: Device = Device(0)) -> "Tensor":
        return Tensor.from_scalar(0.0, shape, dtype, device)

    @staticmethod
    def ones(shape, dtype: int = F32, device: Device = Device(0)) -> "Tensor":
        return Tensor.from_scalar(1.0, shape, dtype, device)

    @staticmethod
    def eye(n: int, dtype: int = F32, device: Device = Device(0)) -> "Tensor":
        out = C.c_void_p()
        L.check(L.lib().hx_tensor_eye(n, dtype, device.index, C.byref(out)))
        return Tensor(out)

    @staticmethod
    def arange(start, end, step, dtype: int = F32, device: Device = Device(0)) -> "Tensor":
        out = C.c_void_p()
        L.check(L.lib().hx_tensor_arange(start, end, step, dtype, device.index, C.byref(out)))
        return Tensor(out)

    @staticmethod
    def _random(kind, shape, p0, p1, device) -> "Tensor":
        out = C.c_void_p()
        L.check(L.lib().hx_tensor_random(kind, (C.c_int64 * len(shape))(*shape), len(shape), p0, p1, device.index, C.byref(out)))
        return Tensor(out)

    @staticmethod
    def random_normal(shape, mean, std, device: Device = Device(0)) -> "Tensor":
        return Tensor._random(0, shape, mean, std, device)

    @staticmethod
    def random_uniform(shape, lo, hi, device: Device = Device(0)) -> "Tensor":
        return Tensor._random(1, shape, lo, hi, device)

    @staticmethod
    def random_bernoulli(shape, p, device: Device = Device(0)) -> "Tensor":
        return Tensor._random(2, shape, p, 0.0, device)

    def __del__(self):
        try:
            if self._h:
                L.lib().hx_tensor_free(self._h)
                self._h = None
        except Exception:
            pass


class Module:
    """nn::Module (crates/nn/src/lib.rs:20-39): forward, parameters."""

    def __init__(self, handle):
        self._h = handle

    def forward(self, x: Tensor) -> Tensor:
        out = C.c_void_p()
        L.check(L.lib().hx_module_forward(self._h, x._h, C.byref(out)))
        return Tensor(out)

    __call__ = forward

    def parameters(self):
        n = L.lib().hx_module_num_parameters(self._h)
        ps = []
        for i in range(n):
            out = C.c_void_p()
            L.check(L.lib().hx_module_parameter(self._h, i, C.byref(out)))
            ps.append(Tensor(out))
        return ps

    def load_parameters(self, arrays) -> None:
        """Writes numpy arrays into the parameters, in parameters() order (Module::parameters_mut)."""
        ps = self.parameters()
        if len(arrays) != len(ps):
            raise L.HxError(9, f"expected {len(ps)} parameters, got {len(arrays)}")
        for p, a in zip(ps, arrays):
            p.copy_from(a)
        L.check(L.lib().hx_module_parameters_updated(self._h))

    def save_checkpoint(self, path: str, epoch=0, step=0, training_loss=0.0, validation_loss=0.0, learning_rate=0.0,
                        timestamp_secs=0) -> None:
        """CheckpointableModule::checkpoint + CheckpointManager's file layout (crates/nn/src/lib.rs:50-52,
        crates/training/src/checkpoint.rs:136-170): parameters() as f32 CpuTensors."""
        m = L.CheckpointMeta()
        m.epoch, m.step, m.timestamp_secs = epoch, step, timestamp_secs
        m.training_loss, m.validation_loss, m.learning_rate = training_loss, validation_loss, learning_rate
        L.check(L.lib().hx_module_save_checkpoint(self._h, path.encode(), C.byref(m)))

    def load_checkpoint(self, path: str) -> dict:
        """CheckpointableModule::restore from a file in the reference's layout; returns the metadata."""
        m = L.CheckpointMeta()
        L.check(L.lib().hx_module_load_checkpoint(self._h, path.encode(), C.byref(m)))
        return {k: getattr(m, k) for k, _ in L.CheckpointMeta._fields_}

    @property
    def name(self) -> str:
        return L.lib().hx_module_name(self._h).decode()

    def __del__(self):
        try:
            if self._h:
                L.lib().hx_module_free(self._h)
                self._h = None
        except Exception:
            pass


def manual_seed(seed: int) -> None:
    L.lib().hx_manual_seed(C.c_uint64(seed))


class MambaBlock(Module):
    """MambaBlock::new(d_model, d_state, d_conv, expand, &device) (crates/nn/src/lib.rs:847).
    parameters(): W_in, conv_w, conv_b, W_x, W_dt, b_dt, A, D, W_out."""
    PARAMS = ("W_in", "conv_w", "conv_b", "W_x", "W_dt", "b_dt", "A", "D", "W_out")

    def __init__(self, d_model, d_state, d_conv, expand, device: Device = Device(0), dtype: int = F32):
        h = C.c_void_p()
        L.check(L.lib().hx_mamba_block_new(d_model, d_state, d_conv, expand, dtype, device.index, C.byref(h)))
        super().__init__(h)

    def load_weights(self, w: dict) -> None:
        self.load_parameters([w[k] for k in self.PARAMS])


class S4Block(Module):
    """nn::ssm::S4Block::new(d_model, d_state, &device) (crates/nn/src/ssm.rs:39).  parameters(): A_real,
    A_imag, B, C, D, delta, Lambda (the reference's seven), then A_diag, B_diag, C_diag."""

    def __init__(self, d_model, d_state, device: Device = Device(0)):
        h = C.c_void_p()
        L.check(L.lib().hx_s4_block_new(d_model, d_state, device.index, C.byref(h)))
        super().__init__(h)

    def forward_ssm(self, u: Tensor) -> Tensor:
        out = C.c_void_p()
        L.check(L.lib().hx_s4_block_forward_ssm(self._h, u._h, C.byref(out)))
        return Tensor(out)


class Linear(Module):
    def __init__(self, in_features, out_features, bias=True, device: Device = Device(0), dtype: int = F32):
        h = C.c_void_p()
        L.check(L.lib().hx_linear_new(in_features, out_features, 1 if bias else 0, dtype, device.index, C.byref(h)))
        super().__init__(h)


class RMSNorm(Module):
    def __init__(self, d_model, eps=1e-5, device: Device = Device(0)):
        h = C.c_void_p()
        L.check(L.lib().hx_rmsnorm_new(d_model, C.c_float(eps), device.index, C.byref(h)))
        super().__init__(h)


class Sequential(Module):
    """nn::Sequential (crates/nn/src/lib.rs:577-661): `Sequential::new(&device)`, `add(module)`, `len()`.  add takes
    ownership of the module, as the reference's `Box<dyn Module>` does: the Python object given is emptied."""

    def __init__(self, device: Device = Device(0)):
        h = C.c_void_p()
        L.check(L.lib().hx_sequential_new(device.index, C.byref(h)))
        super().__init__(h)

    def add(self, module: Module) -> None:
        L.check(L.lib().hx_sequential_add(self._h, module._h))
        module._h = None  # consumed

    def __len__(self) -> int:
        return int(L.lib().hx_sequential_len(self._h))


class ByteLM(Module):
    """Byte-level LM: tied embedding, n_layer x (RMSNorm + MambaBlock + residual), final norm, logits.
    parameters(): embedding, then per layer [norm_w, *MambaBlock.PARAMS], then norm_f."""

    def __init__(self, n_layer, d_model, d_state=16, d_conv=4, expand=2, device: Device = Device(0), dtype: int = BF16):
        h = C.c_void_p()
        L.check(L.lib().hx_byte_lm_new(n_layer, d_model, d_state, d_conv, expand, dtype, device.index, C.byref(h)))
        super().__init__(h)
        self.n_layer, self.d_model = n_layer, d_model

    def load_weights(self, emb, layers, norm_f) -> None:
        arrays = [emb]
        for l in layers:
            arrays.append(l["norm_w"])
            arrays.extend(l[k] for k in MambaBlock.PARAMS)
        arrays.append(norm_f)
        self.load_parameters(arrays)

    def weights_numpy(self):
        """(emb, layers, norm_f) as fp32 numpy arrays in the layout load_weights takes: what a CPU check of the
        model's output needs."""
        ps = [p.numpy() for p in self.parameters()]
        per = 1 + len(MambaBlock.PARAMS)
        layers = []
        for l in range(self.n_layer):
            blk = ps[1 + l * per: 1 + (l + 1) * per]
            d = {"norm_w": blk[0]}
            d.update({k: v for k, v in zip(MambaBlock.PARAMS, blk[1:])})
            layers.append(d)
        return ps[0], layers, ps[-1]

    def forward_host(self, tokens_ptr: int, logits_ptr: int, batch: int, seq_len: int, stream: int = 0) -> None:
        L.check(L.lib().hx_byte_lm_forward_host(self._h, C.c_void_p(tokens_ptr), C.c_void_p(logits_ptr), batch, seq_len,
                                                C.c_void_p(stream)))

    def forward_device(self, tokens_ptr: int, logits_ptr: int, batch: int, seq_len: int, stream: int = 0) -> None:
        L.check(L.lib().hx_byte_lm_forward_device(self._h, C.c_void_p(tokens_ptr), C.c_void_p(logits_ptr), batch, seq_len,
                                                  C.c_void_p(stream)))

    def prefill_device(self, tokens_ptr: int, logits_ptr: int, batch: int, seq_len: int, stream: int = 0) -> None:
        """forward_device that also keeps the per-layer state decode_step_device continues from."""
        L.check(L.lib().hx_byte_lm_prefill_device(self._h, C.c_void_p(tokens_ptr), C.c_void_p(logits_ptr), batch, seq_len,
                                                  C.c_void_p(stream)))

    def decode_step_device(self, tokens_ptr: int, logits_ptr: int, batch: int, stream: int = 0) -> None:
        """One token per sequence: tokens [batch] u8 in, logits [batch, 256] out (device pointers)."""
        L.check(L.lib().hx_byte_lm_decode_step_device(self._h, C.c_void_p(tokens_ptr), C.c_void_p(logits_ptr), batch,
                                                      C.c_void_p(stream)))

    def forward_graph(self, enable: bool) -> None:
        """Replay of a captured CUDA graph of the whole forward from the second identical call on (default on)."""
        L.check(L.lib().hx_byte_lm_forward_graph(self._h, 1 if enable else 0))

    def decode_graph(self, enable: bool) -> None:
        L.check(L.lib().hx_byte_lm_decode_graph(self._h, 1 if enable else 0))

    @property
    def launches_per_decode_step(self) -> int:
        return int(L.lib().hx_byte_lm_launches_per_decode_step(self._h))

    @property
    def launches_per_forward(self) -> int:
        return int(L.lib().hx_byte_lm_launches_per_forward(self._h))
