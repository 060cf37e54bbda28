"""MemRef descriptors and the per-op external kernels, called exactly the way
buddy-mlir's compiled code calls runtime/external_kernels: host buffers behind
strided descriptors, result descriptor filled (and malloc'ed) by the callee
(frontend/Interfaces/buddy/Core/Container.h:126-138,
runtime/external_kernels/rng/RNGUtils.cpp:87-118).
"""
import ctypes as C

import numpy as np

from . import _lib

_libc = C.CDLL(None)
_libc.free.argtypes = [C.c_void_p]

_CT = {np.dtype(np.float32): C.c_float, np.dtype(np.float16): C.c_uint16,
       np.dtype(np.int8): C.c_int8, np.dtype(np.int64): C.c_longlong,
       np.dtype(np.uint8): C.c_int8, np.dtype(np.uint64): C.c_size_t,
       np.dtype(np.uint16): C.c_uint16}
_cache = {}


def memref_type(dtype, rank):
    key = (np.dtype(dtype), rank)
    if key not in _cache:
        ct = _CT[np.dtype(dtype)]

        class MemRef(C.Structure):
            _fields_ = [("allocated", C.POINTER(ct)), ("aligned", C.POINTER(ct)),
                        ("offset", C.c_ssize_t), ("sizes", C.c_ssize_t * rank),
                        ("strides", C.c_ssize_t * rank)]
        MemRef.__name__ = f"MemRef_{np.dtype(dtype).name}_{rank}"
        _cache[key] = MemRef
    return _cache[key]


def to_memref(a: np.ndarray):
    """Descriptor over a numpy array (any strides that are multiples of the
    item size). The array must outlive the descriptor."""
    T = memref_type(a.dtype, a.ndim)
    ct = _CT[a.dtype]
    m = T()
    ptr = C.cast(a.ctypes.data, C.POINTER(ct))
    m.allocated, m.aligned, m.offset = ptr, ptr, 0
    for i in range(a.ndim):
        m.sizes[i] = a.shape[i]
        m.strides[i] = a.strides[i] // a.itemsize
    return m


def from_result(m, dtype):
    """Copy a callee-allocated result out and free it, as the generated code
    does when it destroys the descriptor (Container.h:378-409)."""
    if not m.aligned:
        raise _lib.B200Error(_lib.load().b200_last_error().decode())
    rank = len(m.sizes)
    shape = tuple(m.sizes[i] for i in range(rank))
    n = int(np.prod(shape))
    buf = np.ctypeslib.as_array(m.aligned, shape=(n,))
    out = np.array(buf, copy=True).view(dtype).reshape(shape)
    _libc.free(C.cast(m.allocated, C.c_void_p))
    return out


def _call(name, result_dtype, result_rank, *arrays):
    lib = _lib.load()
    fn = getattr(lib, name)
    res = memref_type(result_dtype, result_rank)()
    descs = [to_memref(a) for a in arrays]
    fn.restype = None
    fn.argtypes = [C.c_void_p] * (1 + len(descs))
    fn(C.byref(res), *[C.byref(d) for d in descs])
    return from_result(res, result_dtype)


def buddy_matmul_f32(A, B):
    return _call("_mlir_ciface_buddy_matmul_f32", np.float32, 2, A, B)


def buddy_gemv_w8_f32(A, W, scale):
    return _call("_mlir_ciface_buddy_gemv_w8_f32", np.float32, 2, A, W, scale)


def buddy_matmul_w8a8_f32(A, W, scale):
    return _call("_mlir_ciface_buddy_matmul_w8a8_f32", np.float32, 2, A, W, scale)


def buddy_gemv_w4_f16(A, P, scale):
    return _call("_mlir_ciface_buddy_gemv_w4_f16", np.float16, 2, A, P, scale)


def buddy_gemv_w4g_f32(A, P, scale):
    return _call("_mlir_ciface_buddy_gemv_w4g_f32", np.float32, 2, A, P, scale)


def buddy_rmsnorm_f32(x, w, eps):
    return _call("_mlir_ciface_buddy_rmsnorm_f32", np.float32, 2, x, w,
                 np.array([eps], dtype=np.float32))


def buddy_silu_mul_f32(g, u):
    return _call("_mlir_ciface_buddy_silu_mul_f32", np.float32, 2, g, u)


def buddy_rope_f32(x, inv_freq, pos):
    return _call("_mlir_ciface_buddy_rope_f32", np.float32, 4, x, inv_freq,
                 np.array([pos], dtype=np.int64))


def buddy_gqa_decode_f32(q, k_cache, v_cache, pos):
    return _call("_mlir_ciface_buddy_gqa_decode_f32", np.float32, 4, q, k_cache,
                 v_cache, np.array([pos], dtype=np.int64))


def release_cached_weights():
    _lib.load().b200_release_cached_weights()
