"""CPU tests of the drop-in boundary: the shared library loads, exports every function the
headers under include/ declare, and the host-only parts of the API (tensor bookkeeping,
memory statistics, layer construction) behave like the reference.  No kernel is launched."""
import ctypes as C
import glob
import os
import re

import numpy as np

from boat_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    names = set()
    for path in glob.glob(os.path.join(ROOT, "include", "**", "*.h"), recursive=True):
        text = open(path).read()
        text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
        text = re.sub(r"//[^\n]*", " ", text)
        text = re.sub(r"^\s*#.*?$", " ", text, flags=re.M)     # macros: the accessor generator is expanded below
        names.update(re.findall(r"\b(boat_[a-z0-9_]+)\s*\(", text))
    names.discard("boat_attention_get_")
    for kind in ("weight", "bias", "grad_weight", "grad_bias"):
        for p in "qkvo":
            names.add("boat_attention_get_%s_%s" % (kind, p))
    # macro names of memory.h, not functions
    return names - {"boat_malloc", "boat_calloc", "boat_realloc", "boat_free"}


def test_library_exports_every_declared_function(lib):
    missing = [n for n in sorted(declared_functions()) if not hasattr(lib, n)]
    assert not missing, missing


def test_python_prototypes_cover_the_headers(lib):
    assert declared_functions() <= set(capi.PROTOTYPES), sorted(declared_functions() - set(capi.PROTOTYPES))


def test_enum_values_match_the_reference(lib):
    assert (capi.DTYPE_FLOAT64, capi.DTYPE_FLOAT32, capi.DEVICE_CPU, capi.DEVICE_CUDA) == (0, 1, 0, 1)
    assert lib.boat_dtype_size(capi.DTYPE_FLOAT32) == 4 and lib.boat_dtype_size(capi.DTYPE_BFLOAT16) == 2
    assert lib.boat_dtype_name(capi.DTYPE_FLOAT32) == b"float32"
    assert lib.boat_dtype_name(capi.DTYPE_BFLOAT16) == b"bfloat16"


def _shape(*dims):
    return (C.c_int64 * len(dims))(*dims), len(dims)


def test_tensor_lifetime_views_and_defaults(lib):
    arr, n = _shape(2, 3, 4)
    t = lib.boat_tensor_create(arr, n, capi.DTYPE_FLOAT32, capi.DEVICE_CPU)
    assert t and lib.boat_tensor_nelements(t) == 24 and lib.boat_tensor_nbytes(t) == 96
    assert lib.boat_tensor_is_contiguous(t)
    data = np.frombuffer((C.c_float * 24).from_address(lib.boat_tensor_data(t)), dtype=np.float32)
    assert not data.any()                                      # create zero-fills
    data[:] = np.arange(24)
    arr2, n2 = _shape(6, 4)
    v = lib.boat_tensor_reshape(t, arr2, n2)
    assert v and lib.boat_tensor_data(v) == lib.boat_tensor_data(t)
    assert not lib.boat_tensor_is_contiguous(v)                # the reference marks views so
    bad, nb = _shape(5, 5)
    assert not lib.boat_tensor_reshape(t, bad, nb)             # element count mismatch
    lib.boat_tensor_free(t)                                    # the view keeps the parent alive
    assert data[5] == 5.0
    lib.boat_tensor_unref(v)
    start, end = (C.c_size_t * 2)(1, 0), (C.c_size_t * 2)(3, 4)
    arr3, n3 = _shape(4, 4)
    u = lib.boat_tensor_create(arr3, n3, capi.DTYPE_FLOAT32, capi.DEVICE_CPU)
    s = lib.boat_tensor_slice(u, start, end, None)
    shp = lib.boat_tensor_shape(s)
    assert (shp[0], shp[1]) == (2, 4) and lib.boat_tensor_data(s) == lib.boat_tensor_data(u) + 16
    assert not lib.boat_tensor_slice(s, start, end, None)      # a slice of a view is refused
    lib.boat_tensor_unref(s)
    lib.boat_tensor_unref(u)
    # NULL handles answer with defaults
    assert lib.boat_tensor_ndim(None) == 0 and lib.boat_tensor_dtype(None) == capi.DTYPE_FLOAT32
    assert lib.boat_tensor_device(None) == capi.DEVICE_CPU and not lib.boat_tensor_data(None)
    empty, ne = _shape(0, 4)
    assert not lib.boat_tensor_create(empty, ne, capi.DTYPE_FLOAT32, capi.DEVICE_CPU)   # 0 bytes -> NULL


def test_memory_statistics(lib):
    lib.boat_memory_reset_stats()
    p = lib.boat_memory_allocate(1000, capi.DEVICE_CPU, None, 0)
    s = lib.boat_memory_get_stats()
    assert s.allocated_bytes == 1000 and s.allocated_blocks == 1 and s.peak_allocated_bytes == 1000
    p = lib.boat_memory_reallocate(p, 4000, capi.DEVICE_CPU, None, 0)
    assert lib.boat_memory_get_stats().allocated_bytes == 4000
    lib.boat_memory_free(p)
    s = lib.boat_memory_get_stats()
    assert s.allocated_bytes == 0 and s.freed_blocks == 2 and s.peak_allocated_bytes == 4000
    assert not lib.boat_memory_allocate(0, capi.DEVICE_CPU, None, 0)


def test_layer_construction_follows_the_reference(lib):
    libc = C.CDLL(None)
    libc.rand.restype = C.c_int
    libc.srand(7)
    cfg = capi.AttentionConfig(16, 4, 0, 0.0, False, True, False, 10000.0)
    layer = lib.boat_attention_create(C.byref(cfg))
    assert layer
    libc.srand(7)
    f32 = np.float32
    bound = f32(np.sqrt(f32(2.0) / f32(32)))
    want = np.array([f32(f32(libc.rand()) / f32(2147483647)) * f32(2.0) * bound - bound for _ in range(256)], f32)
    wq = lib.boat_attention_get_weight_q(layer)
    got = np.frombuffer((C.c_float * 256).from_address(lib.boat_tensor_data(wq)), dtype=np.float32)
    assert np.array_equal(got, want)                           # Xavier-uniform from rand(), same order
    bq = lib.boat_attention_get_bias_q(layer)
    assert not np.frombuffer((C.c_float * 16).from_address(lib.boat_tensor_data(bq)), dtype=np.float32).any()
    assert lib.boat_attention_get_grad_weight_q(layer) is None  # NULL before the first backward
    assert lib.boat_attention_get_precision(layer) == -1
    lib.boat_attention_free(layer)
    for hidden, heads in ((0, 4), (16, 0), (30, 4)):
        bad = capi.AttentionConfig(hidden, heads, 0, 0.0, False, True, False, 10000.0)
        assert not lib.boat_attention_create(C.byref(bad))
    nobias = capi.AttentionConfig(16, 4, 0, 0.0, False, False, False, 10000.0)
    layer = lib.boat_attention_create(C.byref(nobias))
    assert layer and lib.boat_attention_get_bias_o(layer) is None
    lib.boat_attention_free(layer)
    assert not lib.boat_rotary_position_encoding(None, 4, 8, 10000.0)


def test_compute_without_a_gpu_fails_loudly(lib):
    """There is no CPU arithmetic in the product: on a machine without a CUDA device forward
    returns NULL and the runtime explains why."""
    if lib.boat_cuda_device_count() > 0:
        return
    cfg = capi.AttentionConfig(16, 4, 0, 0.0, False, True, False, 10000.0)
    layer = lib.boat_attention_create(C.byref(cfg))
    arr, n = _shape(1, 4, 16)
    x = lib.boat_tensor_create(arr, n, capi.DTYPE_FLOAT32, capi.DEVICE_CPU)
    assert not lib.boat_attention_forward(layer, x, x, x, None)
    assert b"CUDA" in lib.boat_cuda_last_error()
    assert lib.boat_cuda_init(-1) != 0
    lib.boat_tensor_unref(x)
    lib.boat_attention_free(layer)


def test_encoder_block_argument_checks(lib):
    # no layers, no block; NULL blocks are refused without touching a device
    assert lib.boat_encoder_block_create(None, None, None, None, None) is None
    assert lib.boat_encoder_block_forward(None, None) is None
    assert lib.boat_encoder_block_backward(None, None) is None
    lib.boat_encoder_block_free(None)
