"""Python access to the CPU checkers.  TEST INFRASTRUCTURE, NOT PRODUCT.

Two checkers, same call shape:

* ``port_step``  - ``liboracle.so``, our plain-C restatement (``attention_oracle.c``).
* ``ref_step``   - ``_ref/libboat_ref.so``, the reference itself compiled from its own
  sources (see ``Makefile``), driven through its public C API exactly as its tests drive it:
  ``boat_attention_create``, weights written through the accessors, ``boat_attention_forward``,
  ``boat_attention_backward``.

Only ``tests/``, the smoke check and the benchmark's CPU-baseline legs import this module.
"""
import contextlib
import ctypes as C
import os
import subprocess
import tempfile

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
PORT_PATH = os.path.join(_HERE, "liboracle.so")
REF_PATH = os.path.join(_HERE, "_ref", "libboat_ref.so")

_port = None
_ref = None

_FP = C.POINTER(C.c_float)
_FP4 = _FP * 4


def reference_tree():
    """Where the reference's sources are: BOAT_REFERENCE_TREE, else a directory named
    "reference" beside the repository; None when neither holds the attention layer."""
    candidates = [os.environ.get("BOAT_REFERENCE_TREE"),
                  os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")]
    for c in candidates:
        if c and os.path.exists(os.path.join(c, "src", "layers", "attention.c")):
            return c
    return None


def build():
    """Compile liboracle.so and, when the reference tree is present, _ref/libboat_ref.so."""
    cmd = ["make", "-C", _HERE]
    tree = reference_tree()
    if tree:
        cmd.append("REF=" + tree)
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError("building the oracle failed:\n" + proc.stdout[-4000:])


def have_ref():
    return os.path.exists(REF_PATH)


def _fp(a):
    return a.ctypes.data_as(_FP) if a is not None else None


def port():
    global _port
    if _port is None:
        if not os.path.exists(PORT_PATH):
            build()
        lib = C.CDLL(PORT_PATH)
        lib.oracle_attention_step.restype = C.c_int
        lib.oracle_attention_step.argtypes = [C.c_int64] * 4 + [C.c_int] + [_FP] * 3 + [C.c_void_p, C.c_void_p] + \
            [_FP] * 5 + [C.c_void_p, C.c_void_p, _FP]
        lib.oracle_attention_core.restype = C.c_int
        lib.oracle_attention_core.argtypes = [C.c_int64] * 3 + [C.c_int, C.c_float] + [_FP] * 8
        lib.oracle_sgd.restype = None
        lib.oracle_sgd.argtypes = [_FP, _FP, C.c_float, C.c_int64]
        lib.oracle_threads.restype = C.c_int
        lib.oracle_set_threads.argtypes = [C.c_int]
        _port = lib
    return _port


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def port_step(q, k, v, w, b, dout, nh, causal, want_lse=False):
    """Forward (+ backward when dout is given) through the C restatement.

    q,k,v,dout: [B,S,H]; w: four [H,H] arrays (Wq,Wk,Wv,Wo, stored [in,out]); b: four [H]
    arrays or None.  Returns a dict with out, and dq,dk,dv,dw (list of 4),db (list of 4 or
    None) after a backward, lse when asked.
    """
    lib = port()
    q, k, v = _f32(q), _f32(k), _f32(v)
    B, S, H = q.shape
    w = [_f32(x) for x in w]
    b = [_f32(x) for x in b] if b is not None else None
    res = {"out": np.empty_like(q)}
    warr = _FP4(*[_fp(x) for x in w])
    barr = _FP4(*[_fp(x) for x in b]) if b is not None else None
    lse = np.empty(B * nh * S, dtype=np.float32) if want_lse else None
    if dout is not None:
        dout = _f32(dout)
        res.update(dq=np.empty_like(q), dk=np.empty_like(q), dv=np.empty_like(q),
                   dw=[np.empty((H, H), np.float32) for _ in range(4)],
                   db=[np.empty(H, np.float32) for _ in range(4)] if b is not None else None)
        dwarr = _FP4(*[_fp(x) for x in res["dw"]])
        dbarr = _FP4(*[_fp(x) for x in res["db"]]) if b is not None else None
        rc = lib.oracle_attention_step(B, S, H, nh, int(causal), _fp(q), _fp(k), _fp(v),
                                       C.cast(warr, C.c_void_p), C.cast(barr, C.c_void_p) if barr else None,
                                       _fp(dout), _fp(res["out"]), _fp(res["dq"]), _fp(res["dk"]), _fp(res["dv"]),
                                       C.cast(dwarr, C.c_void_p), C.cast(dbarr, C.c_void_p) if dbarr else None,
                                       _fp(lse))
    else:
        rc = lib.oracle_attention_step(B, S, H, nh, int(causal), _fp(q), _fp(k), _fp(v),
                                       C.cast(warr, C.c_void_p), C.cast(barr, C.c_void_p) if barr else None,
                                       None, _fp(res["out"]), None, None, None, None, None, _fp(lse))
    if rc != 0:
        raise MemoryError("oracle_attention_step ran out of memory")
    if want_lse:
        res["lse"] = lse.reshape(B * nh, S)
    return res


def port_core(q, k, v, dout, causal, scale):
    """Attention core alone on [units,S,hs] arrays: dict with o (and dq,dk,dv if dout given)."""
    lib = port()
    q, k, v = _f32(q), _f32(k), _f32(v)
    units, S, hs = q.shape
    res = {"o": np.empty_like(q)}
    if dout is not None:
        dout = _f32(dout)
        res.update(dq=np.empty_like(q), dk=np.empty_like(q), dv=np.empty_like(q))
    rc = lib.oracle_attention_core(units, S, hs, int(causal), float(scale), _fp(q), _fp(k), _fp(v), _fp(dout),
                                   _fp(res["o"]), _fp(res.get("dq")), _fp(res.get("dk")), _fp(res.get("dv")))
    if rc != 0:
        raise MemoryError("oracle_attention_core ran out of memory")
    return res


def port_sgd(param, grad, lr):
    p = _f32(param).copy()
    port().oracle_sgd(_fp(p), _fp(_f32(grad)), float(lr), p.size)
    return p


# ---- the reference itself ---------------------------------------------------------------------

class _RefConfig(C.Structure):
    _fields_ = [("hidden_size", C.c_size_t), ("num_heads", C.c_size_t), ("head_size", C.c_size_t),
                ("dropout_prob", C.c_float), ("causal_mask", C.c_bool), ("use_bias", C.c_bool),
                ("use_rotary", C.c_bool), ("rotary_theta", C.c_float)]


def ref():
    """The reference library (its own code), typed for the handful of calls used here."""
    global _ref
    if _ref is None:
        if not have_ref():
            raise FileNotFoundError(REF_PATH + " is not built (needs the reference source tree, see oracle/Makefile)")
        lib = C.CDLL(REF_PATH, mode=os.RTLD_LOCAL | os.RTLD_NOW)
        P = C.c_void_p
        lib.boat_tensor_create.restype = P
        lib.boat_tensor_create.argtypes = [C.POINTER(C.c_int64), C.c_size_t, C.c_int, C.c_int]
        lib.boat_tensor_data.restype = P
        lib.boat_tensor_data.argtypes = [P]
        lib.boat_tensor_nelements.restype = C.c_size_t
        lib.boat_tensor_nelements.argtypes = [P]
        lib.boat_tensor_unref.argtypes = [P]
        lib.boat_attention_create.restype = P
        lib.boat_attention_create.argtypes = [C.POINTER(_RefConfig)]
        lib.boat_attention_free.argtypes = [P]
        lib.boat_attention_forward.restype = P
        lib.boat_attention_forward.argtypes = [P] * 5
        lib.boat_attention_backward.restype = C.c_bool
        lib.boat_attention_backward.argtypes = [P, P, C.POINTER(P), C.POINTER(P), C.POINTER(P)]
        lib.boat_attention_update.argtypes = [P, C.c_float]
        for kind in ("weight", "bias", "grad_weight", "grad_bias"):
            for p in "qkvo":
                fn = getattr(lib, "boat_attention_get_%s_%s" % (kind, p))
                fn.restype = P
                fn.argtypes = [P]
        _ref = lib
    return _ref


@contextlib.contextmanager
def _quiet_scratch_cwd():
    """The reference's backward prints [DEBUG] lines and appends to a file with a Windows
    path name in the current directory (src/layers/attention.c:478-488): run it in a scratch
    directory with stdout pointed at /dev/null."""
    old_cwd = os.getcwd()
    saved = os.dup(1)
    devnull = os.open(os.devnull, os.O_WRONLY)
    with tempfile.TemporaryDirectory() as tmp:
        os.chdir(tmp)
        os.dup2(devnull, 1)
        try:
            yield
        finally:
            C.CDLL(None).fflush(None)
            os.dup2(saved, 1)
            os.close(saved)
            os.close(devnull)
            os.chdir(old_cwd)


class RefTensor:
    def __init__(self, lib, h):
        self.lib, self.h = lib, h

    def view(self, shape=None):
        n = self.lib.boat_tensor_nelements(self.h)
        buf = (C.c_float * n).from_address(self.lib.boat_tensor_data(self.h))
        a = np.frombuffer(buf, dtype=np.float32)
        return a.reshape(shape) if shape is not None else a


def _ref_new(lib, a):
    shape = (C.c_int64 * a.ndim)(*a.shape)
    h = lib.boat_tensor_create(shape, a.ndim, 1, 0)          # FLOAT32, CPU
    RefTensor(lib, h).view()[:] = a.ravel()
    return h


class RefLayer:
    """A reference attention layer with weights written through the accessors."""

    def __init__(self, H, nh, causal, w, b):
        lib = ref()
        self.lib = lib
        cfg = _RefConfig(H, nh, H // nh, 0.0, bool(causal), b is not None, False, 10000.0)
        self.h = lib.boat_attention_create(C.byref(cfg))
        if not self.h:
            raise RuntimeError("reference boat_attention_create returned NULL")
        for i, p in enumerate("qkvo"):
            RefTensor(lib, getattr(lib, "boat_attention_get_weight_" + p)(self.h)).view()[:] = _f32(w[i]).ravel()
            if b is not None:
                RefTensor(lib, getattr(lib, "boat_attention_get_bias_" + p)(self.h)).view()[:] = _f32(b[i]).ravel()

    def step(self, q, k, v, dout):
        lib = self.lib
        q, k, v = _f32(q), _f32(k), _f32(v)
        B, S, H = q.shape
        hq = _ref_new(lib, q)
        hk = hq if k is q else _ref_new(lib, k)
        hv = hq if v is q else _ref_new(lib, v)
        res = {}
        with _quiet_scratch_cwd():
            ho = lib.boat_attention_forward(self.h, hq, hk, hv, None)
            if not ho:
                raise RuntimeError("reference forward returned NULL")
            res["out"] = RefTensor(lib, ho).view((B, S, H)).copy()
            if dout is not None:
                hg = _ref_new(lib, _f32(dout))
                gq, gk, gv = C.c_void_p(), C.c_void_p(), C.c_void_p()
                ok = lib.boat_attention_backward(self.h, hg, C.byref(gq), C.byref(gk), C.byref(gv))
                if not ok:
                    raise RuntimeError("reference backward failed")
                for name, g in (("dq", gq), ("dk", gk), ("dv", gv)):
                    res[name] = RefTensor(lib, g.value).view((B, S, H)).copy()
                    lib.boat_tensor_unref(g)
                res["dw"] = [RefTensor(lib, getattr(lib, "boat_attention_get_grad_weight_" + p)(self.h))
                             .view((H, H)).copy() for p in "qkvo"]
                hb = lib.boat_attention_get_grad_bias_q(self.h)
                res["db"] = [RefTensor(lib, getattr(lib, "boat_attention_get_grad_bias_" + p)(self.h))
                             .view((H,)).copy() for p in "qkvo"] if hb else None
                lib.boat_tensor_unref(hg)
            lib.boat_tensor_unref(ho)
        for h in {hq, hk, hv}:
            lib.boat_tensor_unref(h)
        return res

    def update(self, lr):
        self.lib.boat_attention_update(self.h, lr)

    def weights(self):
        H = None
        out = []
        for p in "qkvo":
            a = RefTensor(self.lib, getattr(self.lib, "boat_attention_get_weight_" + p)(self.h)).view()
            H = int(round(a.size ** 0.5))
            out.append(a.reshape(H, H).copy())
        return out

    def free(self):
        if self.h:
            self.lib.boat_attention_free(self.h)
        self.h = None


def ref_step(q, k, v, w, b, dout, nh, causal):
    """Same contract as port_step, computed by the reference's own code."""
    layer = RefLayer(np.shape(q)[2], nh, causal, w, b)
    try:
        return layer.step(q, k, v, dout)
    finally:
        layer.free()


# ---- layers around attention (block_oracle.c) --------------------------------------------------------

def _block():
    lib = port()
    if not getattr(lib, "_block_typed", False):
        I64, F = C.c_int64, C.c_float
        lib.oracle_layernorm_forward.argtypes = [_FP, I64, I64, _FP, _FP, F, _FP]
        lib.oracle_layernorm_backward.argtypes = [_FP, _FP, I64, I64, _FP, F, _FP, _FP, _FP]
        lib.oracle_gelu_forward.argtypes = [_FP, _FP, I64]
        lib.oracle_gelu_backward.argtypes = [_FP, _FP, _FP, I64]
        lib.oracle_dense_forward.argtypes = [_FP, _FP, _FP, _FP, I64, I64, I64]
        lib.oracle_dense_backward.argtypes = [_FP, _FP, _FP, _FP, _FP, _FP, I64, I64, I64]
        lib.oracle_dense_backward.restype = C.c_int
        lib._block_typed = True
    return lib


def port_layernorm(x, w, b, eps):
    x = _f32(x)
    H = x.shape[-1]
    y = np.empty_like(x)
    w = _f32(w) if w is not None else None
    b = _f32(b) if b is not None else None
    _block().oracle_layernorm_forward(_fp(x), x.size // H, H, _fp(w), _fp(b), float(eps), _fp(y))
    return y


def port_layernorm_backward(dy, x, w, eps):
    dy, x = _f32(dy), _f32(x)
    H = x.shape[-1]
    w = _f32(w) if w is not None else None
    dx, dg, db = np.empty_like(x), np.empty(H, np.float32), np.empty(H, np.float32)
    _block().oracle_layernorm_backward(_fp(dy), _fp(x), x.size // H, H, _fp(w), float(eps), _fp(dx), _fp(dg), _fp(db))
    return dx, dg, db


def port_gelu(x):
    x = _f32(x)
    y = np.empty_like(x)
    _block().oracle_gelu_forward(_fp(x), _fp(y), x.size)
    return y


def port_gelu_backward(dy, x):
    dy, x = _f32(dy), _f32(x)
    dx = np.empty_like(x)
    _block().oracle_gelu_backward(_fp(dy), _fp(x), _fp(dx), x.size)
    return dx


def port_dense(x, w, b):
    x, w = _f32(x), _f32(w)
    b = _f32(b) if b is not None else None
    N, I = x.shape
    O = w.shape[1]
    y = np.empty((N, O), np.float32)
    _block().oracle_dense_forward(_fp(x), _fp(w), _fp(b), _fp(y), N, I, O)
    return y


def port_dense_backward(x, w, dy, dw_acc=None, db_acc=None, bias=True):
    """Returns dx, dw, db where dw/db are the accumulators after adding this call's gradients."""
    x, w, dy = _f32(x), _f32(w), _f32(dy)
    N, I = x.shape
    O = w.shape[1]
    dx = np.empty((N, I), np.float32)
    dw = np.zeros((I, O), np.float32) if dw_acc is None else _f32(dw_acc).copy()
    db = (np.zeros(O, np.float32) if db_acc is None else _f32(db_acc).copy()) if bias else None
    if _block().oracle_dense_backward(_fp(x), _fp(w), _fp(dy), _fp(dx), _fp(dw), _fp(db), N, I, O):
        raise MemoryError
    return dx, dw, db


class _RefLNConfig(C.Structure):
    _fields_ = [("normalized_shape", C.c_size_t), ("eps", C.c_float), ("elementwise_affine", C.c_bool),
                ("use_bias", C.c_bool)]


def ref_layernorm(x, w, b, eps):
    """boat_layernorm_forward of the reference library itself (weights set in place)."""
    lib = ref()
    P = C.c_void_p
    lib.boat_layernorm_create.restype = P
    lib.boat_layernorm_create.argtypes = [C.POINTER(_RefLNConfig)]
    lib.boat_layernorm_forward.restype = P
    lib.boat_layernorm_forward.argtypes = [P, P]
    lib.boat_layernorm_free.argtypes = [P]
    x = _f32(x)
    H = x.shape[-1]
    cfg = _RefLNConfig(H, eps, w is not None, b is not None)
    layer = lib.boat_layernorm_create(C.byref(cfg))
    # the layer struct starts with the config, then weight and bias tensor pointers
    base = C.cast(layer, C.POINTER(C.c_void_p))
    off = (C.sizeof(_RefLNConfig) + 7) // 8
    if w is not None:
        RefTensor(lib, base[off]).view()[:] = _f32(w)
    if b is not None:
        RefTensor(lib, base[off + 1]).view()[:] = _f32(b)
    hx = _ref_new(lib, x)
    hy = lib.boat_layernorm_forward(layer, hx)
    y = RefTensor(lib, hy).view(x.shape).copy()
    lib.boat_tensor_unref(hy)
    lib.boat_tensor_unref(hx)
    lib.boat_layernorm_free(layer)
    return y


def ref_dense_step(x, w, b, dy, repeats=1):
    """Reference dense layer: forward, then `repeats` backward calls (gradients accumulate)."""
    lib = ref()
    P = C.c_void_p
    lib.boat_dense_layer_create.restype = P
    lib.boat_dense_layer_create.argtypes = [C.c_size_t, C.c_size_t, C.c_bool]
    lib.boat_dense_layer_forward.restype = P
    lib.boat_dense_layer_forward.argtypes = [P, P]
    lib.boat_dense_layer_backward.restype = P
    lib.boat_dense_layer_backward.argtypes = [P, P]
    lib.boat_dense_layer_free.argtypes = [P]
    for name in ("weight", "bias", "grad_weight", "grad_bias"):
        fn = getattr(lib, "boat_dense_layer_get_" + name)
        fn.restype = P
        fn.argtypes = [P]
    x, w, dy = _f32(x), _f32(w), _f32(dy)
    N, I = x.shape
    O = w.shape[1]
    layer = lib.boat_dense_layer_create(I, O, b is not None)
    RefTensor(lib, lib.boat_dense_layer_get_weight(layer)).view()[:] = w.ravel()
    if b is not None:
        RefTensor(lib, lib.boat_dense_layer_get_bias(layer)).view()[:] = _f32(b)
    hx, hg = _ref_new(lib, x), _ref_new(lib, dy)
    hy = lib.boat_dense_layer_forward(layer, hx)
    res = {"y": RefTensor(lib, hy).view((N, O)).copy()}
    for _ in range(repeats):
        hdx = lib.boat_dense_layer_backward(layer, hg)
        res["dx"] = RefTensor(lib, hdx).view((N, I)).copy()
        lib.boat_tensor_unref(hdx)
    res["dw"] = RefTensor(lib, lib.boat_dense_layer_get_grad_weight(layer)).view((I, O)).copy()
    res["db"] = RefTensor(lib, lib.boat_dense_layer_get_grad_bias(layer)).view((O,)).copy() if b is not None else None
    for h in (hy, hx, hg):
        lib.boat_tensor_unref(h)
    lib.boat_dense_layer_free(layer)
    return res


# ---- Adam (optimizer_oracle.c) ------------------------------------------------------------------------

def port_adam(params, grads_per_step, lr, beta1, beta2, eps):
    """Runs len(grads_per_step) Adam steps over a list of FP32 arrays with the C restatement.
    grads_per_step[s][i] is the gradient of params[i] at step s.  Returns the final parameters."""
    lib = port()
    lib.oracle_adam_step.argtypes = [_FP, _FP, _FP, _FP, C.c_int64, C.c_float, C.c_float, C.c_float, C.c_float,
                                     C.c_int64]
    ps = [np.ascontiguousarray(p, dtype=np.float32).copy() for p in params]
    ms = [np.zeros(p.size, np.float32) for p in ps]
    vs = [np.zeros(p.size, np.float32) for p in ps]
    for step, grads in enumerate(grads_per_step):
        for p, g, m, v in zip(ps, grads, ms, vs):
            g = _f32(g)
            lib.oracle_adam_step(_fp(p), _fp(g), _fp(m), _fp(v), p.size, lr, beta1, beta2, eps, step)
    return ps


def ref_adam(params, grads_per_step, lr, beta1, beta2, eps):
    """The same through the reference library's own optimizer API (boat_adam_optimizer_create,
    boat_optimizer_add_parameter, boat_optimizer_step)."""
    lib = ref()
    P = C.c_void_p
    lib.boat_adam_optimizer_create.restype = P
    lib.boat_adam_optimizer_create.argtypes = [C.c_float] * 4
    lib.boat_optimizer_add_parameter.argtypes = [P, P, P]
    lib.boat_optimizer_step.argtypes = [P]
    lib.boat_optimizer_free.argtypes = [P]
    opt = lib.boat_adam_optimizer_create(lr, beta1, beta2, eps)
    assert opt, "reference refused the Adam hyper-parameters"
    hp = [_ref_new(lib, _f32(p)) for p in params]
    hg = [_ref_new(lib, np.zeros_like(_f32(p))) for p in params]
    for a, b in zip(hp, hg):
        lib.boat_optimizer_add_parameter(opt, a, b)
    for grads in grads_per_step:
        for h, g in zip(hg, grads):
            RefTensor(lib, h).view()[:] = _f32(g).ravel()
        lib.boat_optimizer_step(opt)
    out = [RefTensor(lib, h).view(np.shape(p)).copy() for h, p in zip(hp, params)]
    lib.boat_optimizer_free(opt)
    for h in hp + hg:
        lib.boat_tensor_unref(h)
    return out


# ---- autodiff graphs through the reference library --------------------------------------------------------

def _ref_autodiff():
    lib = ref()
    if not getattr(lib, "_autodiff_typed", False):
        P = C.c_void_p
        lib.boat_variable_create.restype = P
        lib.boat_variable_create.argtypes = [P, C.c_bool]
        for name in ("boat_variable_data", "boat_variable_grad"):
            getattr(lib, name).restype = P
            getattr(lib, name).argtypes = [P]
        lib.boat_variable_backward.argtypes = [P, P]
        for name in ("boat_var_add", "boat_var_sub", "boat_var_mul", "boat_var_matmul", "boat_var_dense"):
            getattr(lib, name).restype = P
            getattr(lib, name).argtypes = [P, P]
        lib.boat_var_attention.restype = P
        lib.boat_var_attention.argtypes = [P] * 5
        lib.boat_dense_layer_create.restype = P
        lib.boat_dense_layer_create.argtypes = [C.c_size_t, C.c_size_t, C.c_bool]
        for name in ("weight", "bias", "grad_weight", "grad_bias"):
            fn = getattr(lib, "boat_dense_layer_get_" + name)
            fn.restype = P
            fn.argtypes = [P]
        lib._autodiff_typed = True
    return lib


def ref_graph_residual_attention(x, w, b, nh, causal, gout):
    """r = add(attention(x, x, x), x) through the reference's autodiff (boat_var_attention,
    boat_var_add, boat_variable_backward with upstream gradient gout).  Variables and op nodes are
    left to the process: the reference's node destructor frees the layer it points at."""
    lib = _ref_autodiff()
    x = _f32(x)
    layer = RefLayer(x.shape[2], nh, causal, w, b)
    with _quiet_scratch_cwd():
        vx = lib.boat_variable_create(_ref_new(lib, x), True)
        vh = lib.boat_var_attention(vx, vx, vx, layer.h, None)
        vr = lib.boat_var_add(vh, vx)
        res = {"out": RefTensor(lib, lib.boat_variable_data(vr)).view(x.shape).copy()}
        lib.boat_variable_backward(vr, _ref_new(lib, _f32(gout)))
        res["dx"] = RefTensor(lib, lib.boat_variable_grad(vx)).view(x.shape).copy()
        H = x.shape[2]
        res["dw"] = [RefTensor(lib, getattr(lib, "boat_attention_get_grad_weight_" + p)(layer.h)).view((H, H)).copy()
                     for p in "qkvo"]
        res["db"] = [RefTensor(lib, getattr(lib, "boat_attention_get_grad_bias_" + p)(layer.h)).view((H,)).copy()
                     for p in "qkvo"]
    return res


def ref_graph_mlp(a, wm, wd, bd, c, m, gout):
    """z = sub(mul(dense(matmul(a, wm)), m), c) through the reference's autodiff; every leaf
    requires a gradient."""
    lib = _ref_autodiff()
    a, wm, wd, c, m = (_f32(t) for t in (a, wm, wd, c, m))
    with _quiet_scratch_cwd():
        dense = lib.boat_dense_layer_create(wd.shape[0], wd.shape[1], bd is not None)
        RefTensor(lib, lib.boat_dense_layer_get_weight(dense)).view()[:] = wd.ravel()
        if bd is not None:
            RefTensor(lib, lib.boat_dense_layer_get_bias(dense)).view()[:] = _f32(bd)
        va = lib.boat_variable_create(_ref_new(lib, a), True)
        vw = lib.boat_variable_create(_ref_new(lib, wm), True)
        vc = lib.boat_variable_create(_ref_new(lib, c), True)
        vm = lib.boat_variable_create(_ref_new(lib, m), True)
        v1 = lib.boat_var_matmul(va, vw)
        v2 = lib.boat_var_dense(v1, dense)
        v3 = lib.boat_var_mul(v2, vm)
        vz = lib.boat_var_sub(v3, vc)
        res = {"out": RefTensor(lib, lib.boat_variable_data(vz)).view(c.shape).copy()}
        lib.boat_variable_backward(vz, _ref_new(lib, _f32(gout)))
        for name, v, like in (("da", va, a), ("dwm", vw, wm), ("dc", vc, c), ("dm", vm, m)):
            res[name] = RefTensor(lib, lib.boat_variable_grad(v)).view(like.shape).copy()
        res["dwd"] = RefTensor(lib, lib.boat_dense_layer_get_grad_weight(dense)).view(wd.shape).copy()
        if bd is not None:
            res["dbd"] = RefTensor(lib, lib.boat_dense_layer_get_grad_bias(dense)).view((wd.shape[1],)).copy()
    return res


def ref_ops(inp):
    """The reference's generic tensor operations (src/ops/linear.c, src/ops/arithmetic.c) on the operands of
    tests/cases.py::ops_inputs(); returns a dict of FP32 arrays."""
    lib = ref()
    P = C.c_void_p
    lib.boat_transpose.restype = P
    lib.boat_transpose.argtypes = [P, C.c_int, C.c_int]
    for name in ("boat_add", "boat_mul", "boat_matmul"):
        getattr(lib, name).restype = P
        getattr(lib, name).argtypes = [P, P]
    lib.boat_mul_scalar.restype = P
    lib.boat_mul_scalar.argtypes = [P, C.c_double]
    lib.boat_add_.argtypes = [P, P]
    lib.boat_sub_.argtypes = [P, P]
    lib.boat_add_.restype = None
    lib.boat_sub_.restype = None
    out = {}
    made = []

    def new(a):
        h = _ref_new(lib, _f32(a))
        made.append(h)
        return h

    def take(h, shape):
        assert h, "the reference returned NULL"
        made.append(h)
        return RefTensor(lib, h).view(shape).copy()

    with _quiet_scratch_cwd():
        t4, t4r, t2 = inp["t4"], inp["t4_ragged"], inp["t2"]
        out["transpose_t4"] = take(lib.boat_transpose(new(t4), 2, 3), t4.shape[:2] + (t4.shape[3], t4.shape[2]))
        out["transpose_t4_ragged"] = take(lib.boat_transpose(new(t4r), 2, 3), t4r.shape[:2] + (t4r.shape[3], t4r.shape[2]))
        out["transpose_t2"] = take(lib.boat_transpose(new(t2), 0, 1), t2.shape[::-1])
        a, b, bias = inp["a"], inp["b"], inp["bias"]
        out["add"] = take(lib.boat_add(new(a), new(b)), a.shape)
        out["add_bias"] = take(lib.boat_add(new(a), new(bias)), a.shape)
        out["mul"] = take(lib.boat_mul(new(a), new(b)), a.shape)
        out["mul_scalar"] = take(lib.boat_mul_scalar(new(a), float(inp["scalar"])), a.shape)
        ha = new(a)
        lib.boat_add_(ha, new(b))
        out["add_"] = RefTensor(lib, ha).view(a.shape).copy()
        ha = new(a)
        lib.boat_sub_(ha, new(b))
        out["sub_"] = RefTensor(lib, ha).view(a.shape).copy()
        out["matmul3"] = take(lib.boat_matmul(new(inp["m3a"]), new(inp["m3b"])), (3, 9, 11))
        out["matmul4"] = take(lib.boat_matmul(new(inp["m4a"]), new(inp["m4b"])), (2, 3, 8, 6))
        for h in made:
            lib.boat_tensor_unref(h)
    return out
