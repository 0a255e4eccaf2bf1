"""Thin Python mirror of Boat's C interface for the attention path.

Every method is one call into ``libboat_b200.so`` through the C ABI; numpy is used only to
hand host bytes in and out.  The class and method names follow the C functions they wrap
(``boat_tensor_*`` -> ``Tensor``, ``boat_attention_*`` -> ``Attention``, ``boat_variable_*``
-> ``Variable``) so that tests read like the reference's own C tests.
"""
import ctypes as C
import numpy as np

from . import capi
from .rng import to_bf16_bits, from_bf16_bits

_NP_OF = {capi.DTYPE_FLOAT32: np.float32, capi.DTYPE_FLOAT64: np.float64}


class BoatError(RuntimeError):
    pass


def _shape_arg(shape):
    return (C.c_int64 * len(shape))(*shape), len(shape)


class Tensor:
    """Owns one reference of a ``boat_tensor_t``."""

    def __init__(self, handle, own=True):
        if not handle:
            raise BoatError("NULL tensor: " + (capi.load().boat_cuda_last_error() or b"").decode())
        self.h = C.c_void_p(handle) if not isinstance(handle, C.c_void_p) else handle
        self.own = own

    # ---- construction -------------------------------------------------------------------
    @classmethod
    def create(cls, shape, dtype=capi.DTYPE_FLOAT32, device=capi.DEVICE_CPU):
        arr, n = _shape_arg(shape)
        return cls(capi.load().boat_tensor_create(arr, n, dtype, device))

    @classmethod
    def from_numpy(cls, a, device=capi.DEVICE_CPU, bf16=False):
        """Host FP32 array -> tensor on `device`; with bf16 the values are rounded to BF16
        storage (dtype BOAT_DTYPE_BFLOAT16)."""
        lib = capi.load()
        a = np.ascontiguousarray(a, dtype=np.float32)
        payload = to_bf16_bits(a) if bf16 else a
        dtype = capi.DTYPE_BFLOAT16 if bf16 else capi.DTYPE_FLOAT32
        arr, n = _shape_arg(a.shape)
        if device == capi.DEVICE_CPU:
            return cls(lib.boat_tensor_from_data(arr, n, dtype, payload.ctypes.data_as(C.c_void_p)))
        t = cls(lib.boat_tensor_create(arr, n, dtype, device))
        lib.boat_memory_copy(lib.boat_tensor_data(t.h), payload.ctypes.data_as(C.c_void_p), payload.nbytes,
                             capi.DEVICE_CUDA, capi.DEVICE_CPU)
        return t

    # ---- properties -----------------------------------------------------------------------
    @property
    def shape(self):
        lib = capi.load()
        p = lib.boat_tensor_shape(self.h)
        return tuple(p[i] for i in range(lib.boat_tensor_ndim(self.h)))

    @property
    def dtype(self):
        return capi.load().boat_tensor_dtype(self.h)

    @property
    def device(self):
        return capi.load().boat_tensor_device(self.h)

    @property
    def data_ptr(self):
        return capi.load().boat_tensor_data(self.h)

    @property
    def nbytes(self):
        return capi.load().boat_tensor_nbytes(self.h)

    def numpy(self):
        """Copy out as a host FP32 (or FP64) array, whatever the device and storage type."""
        lib = capi.load()
        dt = self.dtype
        raw = np.empty(self.nbytes, dtype=np.uint8)
        lib.boat_memory_copy(raw.ctypes.data_as(C.c_void_p), lib.boat_tensor_data(self.h), self.nbytes,
                             capi.DEVICE_CPU, self.device)
        if dt == capi.DTYPE_BFLOAT16:
            return from_bf16_bits(raw.view(np.uint16)).reshape(self.shape)
        return raw.view(_NP_OF[dt]).reshape(self.shape).copy()

    def host_view(self):
        """Writable numpy view of a CPU tensor's own memory (the boat_tensor_data() pointer)."""
        if self.device != capi.DEVICE_CPU:
            raise BoatError("host_view needs a CPU tensor")
        n = int(np.prod(self.shape))
        buf = (C.c_float * n).from_address(self.data_ptr)
        return np.frombuffer(buf, dtype=np.float32).reshape(self.shape)

    def set(self, a):
        """Overwrite the contents from a host FP32 array (H2D copy for CUDA tensors)."""
        lib = capi.load()
        a = np.ascontiguousarray(a, dtype=np.float32)
        payload = to_bf16_bits(a) if self.dtype == capi.DTYPE_BFLOAT16 else a
        assert payload.nbytes == self.nbytes, (payload.nbytes, self.nbytes)
        lib.boat_memory_copy(lib.boat_tensor_data(self.h), payload.ctypes.data_as(C.c_void_p), payload.nbytes,
                             self.device, capi.DEVICE_CPU)

    def free(self):
        if self.own and self.h:
            capi.load().boat_tensor_unref(self.h)
        self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Attention:
    """boat_attention_t."""

    PARAMS = ("weight_q", "weight_k", "weight_v", "weight_o", "bias_q", "bias_k", "bias_v", "bias_o")

    def __init__(self, hidden_size, num_heads, causal=False, use_bias=True, head_size=0, dropout=0.0):
        cfg = capi.AttentionConfig(hidden_size, num_heads, head_size, dropout, causal, use_bias, False, 10000.0)
        self.h = capi.load().boat_attention_create(C.byref(cfg))
        if not self.h:
            raise BoatError("boat_attention_create returned NULL")
        self.h = C.c_void_p(self.h)

    def param(self, name):
        """Borrowed Tensor for "weight_q" ... "grad_bias_o" (None when the layer has none)."""
        h = getattr(capi.load(), "boat_attention_get_" + name)(self.h)
        return Tensor(h, own=False) if h else None

    def set_params(self, **arrays):
        for name, a in arrays.items():
            self.param(name).set(a)

    def to_device(self, device):
        rc = capi.load().boat_attention_to_device(self.h, device)
        if rc:
            raise BoatError("boat_attention_to_device failed (%d)" % rc)

    def set_precision(self, mma):
        if capi.load().boat_attention_set_precision(self.h, mma):
            raise BoatError("boat_attention_set_precision failed")

    def forward(self, q, k=None, v=None):
        k = q if k is None else k
        v = q if v is None else v
        out = capi.load().boat_attention_forward(self.h, q.h, k.h, v.h, None)
        if not out:
            raise BoatError("boat_attention_forward returned NULL: " +
                            (capi.load().boat_cuda_last_error() or b"").decode())
        return Tensor(out)

    def forward_units(self, q, seq_len, k=None, v=None):
        """boat_attention_forward_units: q (k, v) are [R, H] tensors holding the token rows of a
        contiguous range of (batch, head) units of a problem with sequence length seq_len."""
        k = k if k is not None else q
        v = v if v is not None else q
        return Tensor(capi.load().boat_attention_forward_units(self.h, q.h, k.h, v.h, seq_len))

    def backward(self, grad_output):
        gq, gk, gv = C.c_void_p(), C.c_void_p(), C.c_void_p()
        ok = capi.load().boat_attention_backward(self.h, grad_output.h, C.byref(gq), C.byref(gk), C.byref(gv))
        if not ok:
            raise BoatError("boat_attention_backward failed: " +
                            (capi.load().boat_cuda_last_error() or b"").decode())
        return Tensor(gq.value), Tensor(gk.value), Tensor(gv.value)

    def update(self, lr):
        capi.load().boat_attention_update(self.h, lr)

    def load_safetensors(self, image, prefix=None):
        """image: bytes of a safetensors file, or a path.  Returns the library's status code."""
        lib = capi.load()
        pre = prefix.encode() if prefix else None
        if isinstance(image, (bytes, bytearray)):
            buf = (C.c_char * len(image)).from_buffer_copy(image)
            return lib.boat_attention_load_safetensors(self.h, C.cast(buf, C.c_void_p), len(image), pre)
        return lib.boat_attention_load_safetensors_file(self.h, str(image).encode(), pre)

    def set_grad_overlap(self, mode=1):
        if capi.load().boat_attention_set_grad_overlap(self.h, int(mode)):
            raise BoatError("boat_attention_set_grad_overlap failed")

    def allreduce_grads(self):
        rc = capi.load().boat_attention_allreduce_grads(self.h)
        if rc:
            raise BoatError("boat_attention_allreduce_grads failed (%d)" % rc)

    def free(self):
        if self.h:
            capi.load().boat_attention_free(self.h)
        self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Variable:
    """boat_variable_t: a tensor with gradient tracking.  Ops return new Variables; inputs are
    borrowed by the op records, so keep them alive until backward has run (held in _inputs)."""

    def __init__(self, tensor=None, requires_grad=True, handle=None, inputs=()):
        lib = capi.load()
        h = handle if handle is not None else lib.boat_variable_create(tensor.h, requires_grad)
        if not h:
            raise BoatError("NULL variable: " + (lib.boat_cuda_last_error() or b"").decode())
        self.h = C.c_void_p(h)
        self._inputs = tuple(inputs) + ((tensor,) if tensor is not None else ())

    def _op(self, name, other):
        return Variable(handle=getattr(capi.load(), name)(self.h, other.h), inputs=(self, other))

    def __add__(self, other):
        return self._op("boat_var_add", other)

    def __sub__(self, other):
        return self._op("boat_var_sub", other)

    def __mul__(self, other):
        return self._op("boat_var_mul", other)

    def __matmul__(self, other):
        return self._op("boat_var_matmul", other)

    def dense(self, layer):
        return Variable(handle=capi.load().boat_var_dense(self.h, layer.h), inputs=(self, layer))

    def attention(self, layer, key=None, value=None):
        key = self if key is None else key
        value = self if value is None else value
        return Variable(handle=capi.load().boat_var_attention(self.h, key.h, value.h, layer.h, None),
                        inputs=(self, key, value, layer))

    def backward(self, grad=None):
        capi.load().boat_variable_backward(self.h, grad.h if grad is not None else None)

    @property
    def data(self):
        return Tensor(capi.load().boat_variable_data(self.h), own=False)

    @property
    def grad(self):
        h = capi.load().boat_variable_grad(self.h)
        return Tensor(h, own=False) if h else None

    def free(self):
        if self.h:
            capi.load().boat_variable_free(self.h)
        self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Adam:
    """boat_optimizer_t made by boat_adam_optimizer_create.  Registered tensors are borrowed:
    keep them alive while the optimizer is."""

    def __init__(self, lr, beta1=0.9, beta2=0.999, eps=1e-8):
        h = capi.load().boat_adam_optimizer_create(lr, beta1, beta2, eps)
        if not h:
            raise BoatError("boat_adam_optimizer_create refused the hyper-parameters")
        self.h = C.c_void_p(h)
        self._keep = []

    def add(self, param, grad):
        self._keep += [param, grad]
        capi.load().boat_optimizer_add_parameter(self.h, param.h, grad.h)

    def add_attention(self, attention):
        rc = capi.load().boat_attention_add_to_optimizer(attention.h, self.h)
        if rc:
            raise BoatError("boat_attention_add_to_optimizer failed (%d)" % rc)

    def step(self):
        capi.load().boat_optimizer_step(self.h)

    def zero_grad(self):
        capi.load().boat_optimizer_zero_grad(self.h)

    @property
    def lr(self):
        return capi.load().boat_optimizer_get_learning_rate(self.h)

    @lr.setter
    def lr(self, value):
        capi.load().boat_optimizer_set_learning_rate(self.h, value)

    def free(self):
        if self.h:
            capi.load().boat_optimizer_free(self.h)
        self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def check(rc, what="boat_cuda call"):
    if rc != 0:
        raise BoatError("%s failed (%d): %s" % (what, rc, (capi.load().boat_cuda_last_error() or b"").decode()))


class DeviceBuffer:
    """Raw HBM block from boat_cuda_malloc, for tests that call the kernel ABI directly."""

    def __init__(self, nbytes):
        self.p = C.c_void_p()
        self.nbytes = int(nbytes)
        check(capi.load().boat_cuda_malloc(C.byref(self.p), self.nbytes), "boat_cuda_malloc")

    @classmethod
    def from_numpy(cls, a, bf16=False):
        a = np.ascontiguousarray(a, dtype=np.float32)
        payload = to_bf16_bits(a) if bf16 else a
        b = cls(payload.nbytes)
        check(capi.load().boat_cuda_memcpy_h2d(b.p, payload.ctypes.data_as(C.c_void_p), payload.nbytes), "h2d")
        return b

    def numpy(self, shape, bf16=False):
        n = int(np.prod(shape))
        raw = np.empty(n, dtype=np.uint16 if bf16 else np.float32)
        check(capi.load().boat_cuda_memcpy_d2h(raw.ctypes.data_as(C.c_void_p), self.p, raw.nbytes), "d2h")
        return (from_bf16_bits(raw) if bf16 else raw).reshape(shape)

    def free(self):
        if self.p:
            capi.load().boat_cuda_free(self.p)
        self.p = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class LayerNorm:
    """boat_layernorm_t (include/boat/layers/norm.h)."""

    def __init__(self, H, eps=1e-5, weight=None, bias=None, affine=True, device=capi.DEVICE_CPU):
        lib = capi.load()
        has_w = affine or weight is not None
        has_b = has_w and (affine or bias is not None)
        cfg = capi.LayerNormConfig(H, eps, has_w, has_b)
        self.h = C.c_void_p(lib.boat_layernorm_create(C.byref(cfg)))
        if not self.h.value:
            raise BoatError("boat_layernorm_create returned NULL")
        if weight is not None:
            Tensor(lib.boat_layernorm_get_weight(self.h), own=False).set(weight)
        if bias is not None:
            Tensor(lib.boat_layernorm_get_bias(self.h), own=False).set(bias)
        if device == capi.DEVICE_CUDA and lib.boat_layernorm_to_device(self.h, device):
            raise BoatError("boat_layernorm_to_device failed")

    def forward(self, x):
        return Tensor(capi.load().boat_layernorm_forward(self.h, x.h))

    def backward(self, g):
        return Tensor(capi.load().boat_layernorm_backward(self.h, g.h))

    def grads(self):
        lib = capi.load()
        gw, gb = lib.boat_layernorm_get_grad_weight(self.h), lib.boat_layernorm_get_grad_bias(self.h)
        return (Tensor(gw, own=False).numpy() if gw else None, Tensor(gb, own=False).numpy() if gb else None)

    def free(self):
        if self.h:
            capi.load().boat_layernorm_free(self.h)
        self.h = None


class Dense:
    """boat_dense_layer_t (include/boat/layers.h)."""

    def __init__(self, I, O, weight=None, bias=None, use_bias=True, device=capi.DEVICE_CPU):
        lib = capi.load()
        self.h = C.c_void_p(lib.boat_dense_layer_create(I, O, use_bias or bias is not None))
        if not self.h.value:
            raise BoatError("boat_dense_layer_create returned NULL")
        if weight is not None:
            Tensor(lib.boat_dense_layer_get_weight(self.h), own=False).set(weight)
        if bias is not None:
            Tensor(lib.boat_dense_layer_get_bias(self.h), own=False).set(bias)
        if device == capi.DEVICE_CUDA and lib.boat_dense_layer_to_device(self.h, device):
            raise BoatError("boat_dense_layer_to_device failed")

    def forward(self, x):
        return Tensor(capi.load().boat_dense_layer_forward(self.h, x.h))

    def backward(self, g):
        return Tensor(capi.load().boat_dense_layer_backward(self.h, g.h))

    def grads(self):
        lib = capi.load()
        gb = lib.boat_dense_layer_get_grad_bias(self.h)
        return (Tensor(lib.boat_dense_layer_get_grad_weight(self.h), own=False).numpy(),
                Tensor(gb, own=False).numpy() if gb else None)

    def update(self, lr):
        capi.load().boat_dense_layer_update(self.h, C.c_float(lr))

    def free(self):
        if self.h:
            capi.load().boat_dense_layer_free(self.h)
        self.h = None


def reshape(t, shape):
    arr, n = _shape_arg(shape)
    return Tensor(capi.load().boat_tensor_reshape(t.h, arr, n))


def lincomb(a, alpha, b, beta):
    return Tensor(capi.load().boat_lincomb(a.h, C.c_float(alpha), b.h, C.c_float(beta)))


class EncoderBlock:
    """Pre-LN transformer encoder block (boat_encoder_block_t over five layers):
    LN -> attention -> +x -> LN -> dense(4d) -> GELU -> dense(d) -> +, mean-squared-error loss."""

    def __init__(self, d, nh, causal=False, device=capi.DEVICE_CUDA, mma=capi.MMA_BF16, params=None):
        p = params or {}
        self.d = d
        self.ln1 = LayerNorm(d, 1e-5, p.get("g1"), p.get("b1"), device=device)
        self.ln2 = LayerNorm(d, 1e-5, p.get("g2"), p.get("b2"), device=device)
        self.fc1 = Dense(d, 4 * d, p.get("w1"), p.get("c1"), device=device)
        self.fc2 = Dense(4 * d, d, p.get("w2"), p.get("c2"), device=device)
        self.attn = Attention(d, nh, causal=causal)
        if "w" in p:
            for i, q in enumerate("qkvo"):
                self.attn.param("weight_" + q).set(p["w"][i])
                if p.get("b") is not None:
                    self.attn.param("bias_" + q).set(p["b"][i])
        if device == capi.DEVICE_CUDA:
            self.attn.to_device(device)
        self.attn.set_precision(mma)
        self.h = None

    def step(self, x, target):
        """Forward, MSE gradient, backward through boat_encoder_block_forward / _backward.
        Returns (out, dx); parameter gradients stay in the layers."""
        lib = capi.load()
        B, S, d = x.shape
        if self.h is None:
            self.h = C.c_void_p(lib.boat_encoder_block_create(self.ln1.h, self.attn.h, self.ln2.h, self.fc1.h, self.fc2.h))
            if not self.h.value:
                raise BoatError("boat_encoder_block_create returned NULL")
        out = Tensor(lib.boat_encoder_block_forward(self.h, x.h))
        scale = 2.0 / float(B * S * d)
        dout = lincomb(out, scale, target, -scale)
        dx = Tensor(lib.boat_encoder_block_backward(self.h, dout.h))
        return out, dx

    def allreduce_grads(self):
        rc = capi.load().boat_encoder_block_allreduce_grads(self.h)
        if rc:
            raise BoatError("boat_encoder_block_allreduce_grads failed (%d)" % rc)

    def zero_dense_grads(self):
        """Dense gradients accumulate across backward calls (as in the reference); a training loop
        clears them with the update step - lr 0 leaves the weights alone."""
        self.fc1.update(0.0)
        self.fc2.update(0.0)

    def free(self):
        if self.h is not None:
            capi.load().boat_encoder_block_free(self.h)
            self.h = None
        for layer in (self.ln1, self.ln2, self.fc1, self.fc2, self.attn):
            layer.free()
