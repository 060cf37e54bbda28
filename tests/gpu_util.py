"""Device-memory plumbing for the GPU tests: torch owns the allocations, the
kernels under test are reached only through the C ABI."""
import ctypes as C

import numpy as np
import torch

from buddy_mlir_b200 import _lib


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def ptr(t):
    return C.c_void_p(t.data_ptr())


def stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def sync():
    torch.cuda.synchronize()


def packed_weight(kind, ref_w, K, N, signed=0):
    """Upload a weight in the reference layout and repack it on the device."""
    lib = _lib.load()
    rb = lib.b200_packed_row_bytes(kind, K)
    src = dev(ref_w)
    dst = torch.zeros(N * rb, dtype=torch.uint8, device="cuda")
    _lib.check(lib.b200_pack_weight(kind, ptr(src), K, N, signed, ptr(dst), stream()))
    sync()
    return dst


def packed_scales(scales, dtype, groups, N):
    lib = _lib.load()
    src = dev(scales)
    dst = torch.empty_like(src)
    _lib.check(lib.b200_pack_scales(ptr(src), dtype, groups, N, ptr(dst), stream()))
    sync()
    return dst


def gemv(kind, wbuf, sbuf, K, N, x, *, group=0, scale_dtype=_lib.F32, bias=None,
         residual=None, norm_w=None, eps=1e-6, silu=False, accumulate=False, y0=None,
         x_dtype=_lib.F32, y_dtype=_lib.F32):
    lib = _lib.load()
    M = x.shape[0]
    w = _lib.Weight(kind, group, K, N, wbuf.data_ptr(), sbuf.data_ptr() if sbuf is not None else None,
                    scale_dtype, 0, bias.data_ptr() if bias is not None else None)
    ncol = N // 2 if silu else N
    tdt = torch.float32 if y_dtype == _lib.F32 else torch.float16
    y = torch.zeros((M, ncol), dtype=tdt, device="cuda") if y0 is None else y0
    a = _lib.GemvArgs(x.data_ptr(), x_dtype, y_dtype, 0, 0, y.data_ptr(),
                      residual.data_ptr() if residual is not None else None,
                      norm_w.data_ptr() if norm_w is not None else None, eps, M,
                      int(accumulate), int(silu))
    _lib.check(lib.b200_gemv(C.byref(w), C.byref(a), stream()))
    sync()
    return y


def gemm_w8(wbuf, sbuf, K, N, A, *, bias=None, residual=None, norm_w=None, eps=1e-6, silu=False):
    """C = A * dequant(W)^T through b200_gemm_w8 (the tcgen05 path)."""
    lib = _lib.load()
    M = A.shape[0]
    w = _lib.Weight(_lib.W_I8, 0, K, N, wbuf.data_ptr(), sbuf.data_ptr(), _lib.F32, 0,
                    bias.data_ptr() if bias is not None else None)
    ncol = N // 2 if silu else N
    Cd = torch.zeros((M, ncol), dtype=torch.float32, device="cuda")
    nbytes = lib.b200_gemm_w8_workspace_bytes(M, K)
    ws = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    _lib.check(lib.b200_gemm_w8(C.byref(w), ptr(A), M, A.stride(0), ptr(Cd), ncol,
                                ptr(residual) if residual is not None else None,
                                residual.stride(0) if residual is not None else 0,
                                ptr(norm_w) if norm_w is not None else None, eps, int(silu),
                                ptr(ws), nbytes, stream()))
    _lib.check(lib.b200_gemm_w8_status(ptr(ws), stream()))
    return Cd
