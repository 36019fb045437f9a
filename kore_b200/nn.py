"""Host-side mirror of KORE's ``BitLinear`` / ``QuatLinear`` modules over the C ABI.

Names, argument meaning and error behaviour follow
``crates/kore-nn/src/bit_linear.rs`` / ``quat_linear.rs`` and the Python signatures of
``python/kore/kore.pyi:104-116``.  Inputs may be numpy arrays (host: copied to the
device and back inside one C call) or CUDA ``torch`` tensors (device pointers, work
enqueued on torch's current stream).  All arithmetic runs in the CUDA library; this
file only checks shapes and moves pointers.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _cabi
from ._cabi import KoreError, PATH_AUTO, PATH_GEMM_TC, PATH_GEMV, QUATERNARY, TERNARY  # noqa: F401


def _is_torch(x) -> bool:
    return type(x).__module__.startswith("torch")


def _current_stream_ptr(device_index: int) -> int:
    import torch

    return torch.cuda.current_stream(device_index).cuda_stream


class _QuantLinear:
    """Common body of BitLinear and QuatLinear (the reference duplicates it per type)."""

    KIND = TERNARY
    NAME = "BitLinear"

    def __init__(self):
        self._h = None
        self.in_features = 0
        self.out_features = 0
        self.device = 0
        self._bias = None
        self.training = False

    # ---- construction ------------------------------------------------------------
    def _create_from_f32(self, weight, bias, quantiser, threshold, device):
        w = np.ascontiguousarray(weight, dtype=np.float32)
        if w.ndim != 2:
            # the reference asserts here (bit_linear.rs:50-54)
            raise AssertionError(f"{self.NAME} weight must be 2D, got {list(w.shape)}")
        m, k = w.shape
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32).reshape(m)
        h = C.c_void_p()
        _cabi.check(_cabi.lib().kb_linear_create_from_f32(
            self.KIND, quantiser, w.ctypes.data, None if b is None else b.ctypes.data, m, k,
            C.c_float(threshold), device, C.byref(h)))
        self._adopt(h, m, k, b, device)

    def _create_from_packed(self, packed, scales, bias, out_features, in_features, device):
        p = np.ascontiguousarray(packed, dtype=np.uint8).ravel()
        s = np.ascontiguousarray(scales, dtype=np.float32).ravel()
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32).reshape(out_features)
        h = C.c_void_p()
        _cabi.check(_cabi.lib().kb_linear_create_from_ref_packed(
            self.KIND, p.ctypes.data, p.size, s.ctypes.data, s.size, None if b is None else b.ctypes.data,
            out_features, in_features, device, C.byref(h)))
        self._adopt(h, out_features, in_features, b, device)

    def _adopt(self, h, m, k, bias, device):
        self._h = h
        self.out_features, self.in_features = int(m), int(k)
        self._bias = bias
        self.device = device

    def close(self):
        if self._h is not None:
            _cabi.lib().kb_linear_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def handle(self):
        return self._h

    # ---- accessors (bit_linear.rs:104-167) -----------------------------------------
    def packed_weights(self) -> np.ndarray:
        kp = (self.in_features + 4) // 5 if self.KIND == TERNARY else (self.in_features + 3) // 4
        out = np.zeros(self.out_features * kp, np.uint8)
        _cabi.check(_cabi.lib().kb_linear_packed_weights(self._h, out.ctypes.data, out.size))
        return out

    def scales(self) -> np.ndarray:
        out = np.zeros(self.out_features, np.float32)
        _cabi.check(_cabi.lib().kb_linear_scales(self._h, out.ctypes.data, out.size))
        return out

    def weight_memory_bytes(self) -> int:
        wb = C.c_size_t()
        _cabi.check(_cabi.lib().kb_linear_info(self._h, None, None, None, None, C.byref(wb)))
        return int(wb.value)

    def f32_weight_memory_bytes(self) -> int:
        return self.out_features * self.in_features * 4

    def compression_ratio(self) -> float:
        return float(np.float32(self.f32_weight_memory_bytes()) / np.float32(self.weight_memory_bytes()))

    def dequantize_weights(self) -> np.ndarray:
        out = np.zeros((self.out_features, self.in_features), np.float32)
        _cabi.check(_cabi.lib().kb_linear_dequantize_weights(self._h, out.ctypes.data, out.size))
        return out

    # ---- Module trait (module.rs:9-34) -----------------------------------------------
    def forward(self, input, path: int = PATH_AUTO, return_acc: bool = False):
        """y[..., out] = forward(x[..., in]).  Raises KoreError(ShapeMismatch) when the last
        dimension is not in_features or the input is 0-dimensional (bit_linear.rs:179-184)."""
        if _is_torch(input):
            return self._forward_torch(input, path, return_acc)
        x = np.ascontiguousarray(input, dtype=np.float32)
        if x.ndim == 0:
            raise KoreError(_cabi.ERR_SHAPE, f"shape mismatch: expected [{self.in_features}], got []")
        in_dim = x.shape[-1]
        lead = x.shape[:-1]
        n = int(np.prod(lead)) if x.ndim > 1 else 1
        y = np.zeros((n, self.out_features), np.float32)
        if path == PATH_AUTO and not return_acc:
            _cabi.check(_cabi.lib().kb_linear_forward_host(self._h, x.ctypes.data, n, in_dim, y.ctypes.data))
            return y.reshape(*lead, self.out_features) if x.ndim > 1 else y.reshape(self.out_features)
        import torch

        xt = torch.from_numpy(x.reshape(n, in_dim)).to(f"cuda:{self.device}")
        out = self._forward_torch(xt, path, return_acc)
        if return_acc:
            return out[0].cpu().numpy().reshape(*lead, -1), out[1].cpu().numpy().reshape(*lead, -1)
        return out.cpu().numpy().reshape(*lead, self.out_features) if x.ndim > 1 else out.cpu().numpy().reshape(-1)

    def forward_relu(self, x, path: int = PATH_AUTO):
        """max(forward(x), 0) with the ReLU in the kernel epilogue (CUDA float32 tensor in and out):
        the layer-shaped form of the reference's fused bias + ReLU dequantising matmul
        (crates/kore-kernels/src/cuda/ops.rs:828-878)."""
        import torch

        if not _is_torch(x) or not x.is_cuda or x.dtype != torch.float32:
            raise KoreError(_cabi.ERR_DTYPE, "forward_relu expects a CUDA float32 tensor")
        if x.dim() == 0:
            raise KoreError(_cabi.ERR_SHAPE, f"shape mismatch: expected [{self.in_features}], got []")
        in_dim = x.shape[-1]
        lead = tuple(x.shape[:-1])
        n = int(np.prod(lead)) if x.dim() > 1 else 1
        x2 = x.reshape(n, in_dim).contiguous()
        y = torch.empty((n, self.out_features), dtype=torch.float32, device=x.device)
        _cabi.check(_cabi.lib().kb_linear_forward_act(
            self._h, x2.data_ptr(), n, in_dim, y.data_ptr(), 0, _cabi.ACT_RELU, path, None, 0,
            _current_stream_ptr(x.device.index)))
        return y.reshape(*lead, self.out_features) if x.dim() > 1 else y.reshape(self.out_features)

    def _forward_torch(self, x, path, return_acc):
        import torch

        if not x.is_cuda or x.dtype != torch.float32:
            raise KoreError(_cabi.ERR_DTYPE, f"expected a CUDA float32 tensor, got {x.dtype} on {x.device}")
        if x.dim() == 0:
            raise KoreError(_cabi.ERR_SHAPE, f"shape mismatch: expected [{self.in_features}], got []")
        in_dim = x.shape[-1]
        lead = tuple(x.shape[:-1])
        n = int(np.prod(lead)) if x.dim() > 1 else 1
        x2 = x.reshape(n, in_dim).contiguous()
        y = torch.empty((n, self.out_features), dtype=torch.float32, device=x.device)
        acc = torch.empty((n, self.out_features), dtype=torch.int32, device=x.device) if return_acc else None
        _cabi.check(_cabi.lib().kb_linear_forward_ex(
            self._h, x2.data_ptr(), n, in_dim, y.data_ptr(), 0, None if acc is None else acc.data_ptr(), path,
            None, 0, _current_stream_ptr(x.device.index)))
        y = y.reshape(*lead, self.out_features) if x.dim() > 1 else y.reshape(self.out_features)
        return (y, acc) if return_acc else y

    __call__ = forward

    def parameters(self):
        return [] if self._bias is None else [self._bias]

    def named_parameters(self):
        return [] if self._bias is None else [("bias", self._bias)]

    def train(self, mode: bool = True):
        self.training = mode

    def is_training(self) -> bool:
        return self.training

    def state_dict(self):
        sd = {"weight": self.dequantize_weights()}
        if self._bias is not None:
            sd["bias"] = self._bias.copy()
        return sd


def _xavier(rng, out_features, in_features):
    # Linear::new draws from a Xavier-style uniform range (crates/kore-nn/src/linear.rs:16-22)
    bound = float(np.sqrt(6.0 / (in_features + out_features)))
    return rng.uniform(-bound, bound, size=(out_features, in_features)).astype(np.float32)


class BitLinear(_QuantLinear):
    """1.58-bit linear layer (ternary weights), mirror of kore_nn::BitLinear.

    ``BitLinear(in_features, out_features, bias=False, threshold=0.3)`` follows the Python
    constructor of the reference (random Xavier weights quantised at ``threshold``;
    the reference's RNG is unseeded, here ``seed`` makes it reproducible).  Use
    ``BitLinear.new(weight, bias, threshold)`` / ``from_packed`` for given weights.
    """

    KIND, NAME = TERNARY, "BitLinear"

    def __init__(self, in_features: int, out_features: int, bias: bool = False, threshold: float = 0.3,
                 *, seed: int = 0, device: int = 0):
        super().__init__()
        self.threshold = float(threshold)
        rng = np.random.default_rng(seed)
        w = _xavier(rng, out_features, in_features)
        b = np.zeros(out_features, np.float32) if bias else None
        self._create_from_f32(w, b, _cabi.QUANT_REFERENCE, threshold, device)

    @classmethod
    def new(cls, weight, bias=None, threshold: float = 0.3, *, quantiser: str = "reference", device: int = 0):
        """BitLinear::new (bit_linear.rs:48-77); quantiser="absmean" selects the per-tensor
        absmean ternariser instead of the reference's per-row absmax + threshold."""
        self = cls.__new__(cls)
        _QuantLinear.__init__(self)
        self.threshold = float(threshold)
        q = _cabi.QUANT_ABSMEAN if quantiser == "absmean" else _cabi.QUANT_REFERENCE
        self._create_from_f32(weight, bias, q, threshold, device)
        return self

    @classmethod
    def from_packed(cls, packed_weights, scales, bias, in_features: int, out_features: int, *,
                    threshold: float = 0.3, device: int = 0):
        """Adopt BitLinear::packed_weights()/scales() (base-243 wire format) unchanged."""
        self = cls.__new__(cls)
        _QuantLinear.__init__(self)
        self.threshold = float(threshold)
        self._create_from_packed(packed_weights, scales, bias, out_features, in_features, device)
        return self

    @classmethod
    def random(cls, in_features: int, out_features: int, bias: bool, *, seed: int = 0, device: int = 0):
        """BitLinear::random (bit_linear.rs:87-102): uniform(-1,1) weights, threshold 0.3."""
        rng = np.random.default_rng(seed)
        w = rng.uniform(-1.0, 1.0, size=(out_features, in_features)).astype(np.float32)
        return cls.new(w, np.zeros(out_features, np.float32) if bias else None, 0.3, device=device)

    def __repr__(self):  # Display impl, bit_linear.rs:276-288
        return (f"BitLinear(in={self.in_features}, out={self.out_features}, threshold={self.threshold:g}, "
                f"compression={self.compression_ratio():.1f}x, mem={self.weight_memory_bytes() / 1024.0:.1f}KB)")


class QuatLinear(_QuantLinear):
    """2-bit linear layer (weights in {-3,-1,+1,+3} x per-row scale), mirror of kore_nn::QuatLinear."""

    KIND, NAME = QUATERNARY, "QuatLinear"

    def __init__(self, in_features: int, out_features: int, bias: bool = False, *, seed: int = 0, device: int = 0):
        super().__init__()
        rng = np.random.default_rng(seed)
        w = _xavier(rng, out_features, in_features)
        b = np.zeros(out_features, np.float32) if bias else None
        self._create_from_f32(w, b, _cabi.QUANT_REFERENCE, 0.0, device)

    @classmethod
    def new(cls, weight, bias=None, *, device: int = 0):
        """QuatLinear::new (quat_linear.rs:46-73)."""
        self = cls.__new__(cls)
        _QuantLinear.__init__(self)
        self._create_from_f32(weight, bias, _cabi.QUANT_REFERENCE, 0.0, device)
        return self

    @classmethod
    def from_packed(cls, packed_weights, scales, bias, in_features: int, out_features: int, *, device: int = 0):
        self = cls.__new__(cls)
        _QuantLinear.__init__(self)
        self._create_from_packed(packed_weights, scales, bias, out_features, in_features, device)
        return self

    @classmethod
    def random(cls, in_features: int, out_features: int, bias: bool, *, seed: int = 0, device: int = 0):
        """QuatLinear::random (quat_linear.rs:81-96): uniform(-3,3) weights."""
        rng = np.random.default_rng(seed)
        w = rng.uniform(-3.0, 3.0, size=(out_features, in_features)).astype(np.float32)
        return cls.new(w, np.zeros(out_features, np.float32) if bias else None, device=device)

    def __repr__(self):  # Display impl, quat_linear.rs:227-238
        return (f"QuatLinear(in={self.in_features}, out={self.out_features}, "
                f"bias={'true' if self._bias is not None else 'false'}, compression={self.compression_ratio():.1f}x)")


def lora_a_init(rank: int, in_features: int) -> np.ndarray:
    """The deterministic initial ``lora_a`` of ``QLoraLinear`` (lora.rs:219-225,247-253):
    x_i = ((i * 2654435761 + 1013904223) & 0xFFFFFF) / 0xFFFFFF, a_i = (2 x_i - 1) * sqrt(1 / in)."""
    i = np.arange(rank * in_features, dtype=np.uint64)
    h = (i * np.uint64(2654435761) + np.uint64(1013904223)) & np.uint64(0xFFFFFF)
    x = h.astype(np.float32) / np.float32(0xFFFFFF)
    a_scale = np.sqrt(np.float32(1.0) / np.float32(in_features)).astype(np.float32)
    return ((x * np.float32(2.0) - np.float32(1.0)) * a_scale).astype(np.float32).reshape(rank, in_features)


class QLoraLinear:
    """Quantized base + low-rank adapters (``crates/kore-nn/src/lora.rs:190-357``):

        y = base(x) + ((x @ A^T) @ B^T) * (alpha / rank) (+ bias)

    ``base`` is a BitLinear on the CUDA path; the adapter product (two thin dense f32 matmuls,
    rank columns wide) runs as torch matmuls on the same stream and enters the base
    projection's epilogue as its residual, so the sum is formed in the reference's order
    (base output, then the adapter term, then the bias).  ``lora_a`` [rank, in] starts from the
    reference's deterministic pattern, ``lora_b`` [out, rank] from zero."""

    def __init__(self, base: BitLinear, rank: int, alpha: float, bias=None):
        import torch

        if base._bias is not None:
            raise KoreError(_cabi.ERR_INVALID, "the base layer of QLoraLinear carries no bias; pass it to QLoraLinear")
        self.base, self.rank, self.alpha = base, int(rank), float(alpha)
        self.in_features, self.out_features = base.in_features, base.out_features
        dev = f"cuda:{base.device}"
        self.lora_a = torch.from_numpy(lora_a_init(self.rank, self.in_features)).to(dev)
        self.lora_b = torch.zeros((self.out_features, self.rank), dtype=torch.float32, device=dev)
        self.bias = None if bias is None else torch.as_tensor(np.asarray(bias, np.float32)).to(dev)
        self.training = True

    @classmethod
    def from_linear(cls, weight, bias, rank: int, alpha: float, threshold: float, *, device: int = 0):
        """lora.rs:207-240: quantise a dense layer's weight [out, in] with the reference rule"""
        return cls(BitLinear.new(weight, None, threshold, device=device), rank, alpha, bias)

    @classmethod
    def from_bit_linear(cls, base: BitLinear, rank: int, alpha: float):
        return cls(base, rank, alpha, None)

    def trainable_params(self) -> int:
        return self.rank * self.in_features + self.out_features * self.rank + (0 if self.bias is None else self.bias.numel())

    def base_compression_ratio(self) -> float:
        return self.base.compression_ratio()

    def forward(self, x):
        """x: CUDA float32 tensor [..., in] -> [..., out]"""
        import torch

        if not _is_torch(x) or not x.is_cuda or x.dtype != torch.float32:
            raise KoreError(_cabi.ERR_DTYPE, "QLoraLinear.forward expects a CUDA float32 tensor")
        if x.dim() == 0 or x.shape[-1] != self.in_features:
            raise KoreError(_cabi.ERR_SHAPE, f"shape mismatch: expected [{self.in_features}], got {list(x.shape)}")
        lead = tuple(x.shape[:-1])
        x2 = x.reshape(-1, self.in_features).contiguous()
        n = x2.shape[0]
        scaling = self.alpha / self.rank
        lora_out = ((x2 @ self.lora_a.t()) @ self.lora_b.t()) * scaling
        y = torch.empty((n, self.out_features), dtype=torch.float32, device=x.device)
        lib = _cabi.lib()
        ws_bytes = max(int(lib.kb_linear_workspace_bytes(self.base.handle, n)), 256)
        ws = torch.empty(ws_bytes + 256, dtype=torch.uint8, device=x.device)
        ws_ptr = (ws.data_ptr() + 255) // 256 * 256
        _cabi.check(lib.kb_linear_forward_fused(self.base.handle, x2.data_ptr(), None, 0, None, None, n, lora_out.data_ptr(),
                                                y.data_ptr(), 0, PATH_AUTO, ws_ptr, ws_bytes,
                                                _current_stream_ptr(x.device.index)))
        if self.bias is not None:
            y += self.bias
        return y.reshape(*lead, self.out_features)

    __call__ = forward

    def parameters(self):
        return [self.lora_a, self.lora_b] + ([] if self.bias is None else [self.bias])

    def named_parameters(self):
        return [("lora_a", self.lora_a), ("lora_b", self.lora_b)] + ([] if self.bias is None else [("bias", self.bias)])

    def __repr__(self):  # Display impl, lora.rs:360-372
        return (f"QLoraLinear(in={self.in_features}, out={self.out_features}, rank={self.rank}, alpha={self.alpha:g}, "
                f"base_compression={self.base_compression_ratio():.1f}x, trainable={self.trainable_params()})")


class LinearGroup:
    """Several BitLinear / QuatLinear layers of one shape, each applied to its own single token,
    in one launch (``kb_linear_group_forward_q8``): ``forward(x)[i] == layers[i].forward(x[i])``
    bit for bit.  The counterpart in the reference is a loop of ``forward`` calls over
    independent modules (``crates/kore-nn/src/bit_linear.rs:175-237``)."""

    def __init__(self, layers):
        layers = list(layers)
        if not layers:
            raise KoreError(_cabi.ERR_INVALID, "empty group")
        self.layers = layers  # keeps the members (and their device memory) alive
        self.in_features = layers[0].in_features
        self.out_features = layers[0].out_features
        arr = (C.c_void_p * len(layers))(*[lay.handle for lay in layers])
        h = C.c_void_p()
        _cabi.check(_cabi.lib().kb_linear_group_create(arr, len(layers), C.byref(h)))
        self._h = h

    def __len__(self):
        return len(self.layers)

    @property
    def handle(self):
        if not self._h:
            raise KoreError(_cabi.ERR_BAD_HANDLE, "group was closed")
        return self._h

    def close(self):
        if getattr(self, "_h", None):
            _cabi.lib().kb_linear_group_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def forward_q8(self, xq, sx, sumq, out=None):
        """xq/sx/sumq as returned by ``kernels.quantize_act_i8`` for an input of [len(self), K]."""
        import torch

        if xq.shape[0] != len(self.layers):
            raise KoreError(_cabi.ERR_SHAPE, f"shape mismatch: expected [{len(self.layers)}] rows, got {list(xq.shape)}")
        y = out if out is not None else torch.empty((len(self.layers), self.out_features), dtype=torch.float32, device=xq.device)
        _cabi.check(_cabi.lib().kb_linear_group_forward_q8(self.handle, xq.data_ptr(), xq.stride(0), sx.data_ptr(), sumq.data_ptr(),
                                                           y.data_ptr(), y.stride(0), _current_stream_ptr(xq.device.index)))
        return y

    def forward(self, x, out=None):
        """x: float32 [len(self), K], a CUDA tensor or a numpy array; row i goes through layer i (one
        launch, the per-token quantiser runs in the kernel's prologue)."""
        import torch

        if not _is_torch(x):  # numpy in, numpy out: copies and synchronisation inside one C call
            x = np.ascontiguousarray(x, dtype=np.float32)
            if x.ndim != 2 or x.shape[0] != len(self.layers) or x.shape[1] != self.in_features:
                raise KoreError(_cabi.ERR_SHAPE, f"shape mismatch: expected [{len(self.layers)}, {self.in_features}], got {list(x.shape)}")
            y = np.empty((len(self.layers), self.out_features), np.float32)
            _cabi.check(_cabi.lib().kb_linear_group_forward_host(self.handle, x.ctypes.data, y.ctypes.data))
            return y
        if not x.is_cuda or x.dtype != torch.float32:
            raise KoreError(_cabi.ERR_DTYPE, "expected a CUDA float32 tensor")
        if x.dim() != 2 or x.shape[0] != len(self.layers) or x.shape[1] != self.in_features:
            raise KoreError(_cabi.ERR_SHAPE, f"shape mismatch: expected [{len(self.layers)}, {self.in_features}], got {list(x.shape)}")
        if x.stride(1) != 1:
            x = x.contiguous()
        y = out if out is not None else torch.empty((len(self.layers), self.out_features), dtype=torch.float32, device=x.device)
        _cabi.check(_cabi.lib().kb_linear_group_forward(self.handle, x.data_ptr(), x.stride(0), y.data_ptr(), y.stride(0),
                                                        _current_stream_ptr(x.device.index)))
        return y

    __call__ = forward
