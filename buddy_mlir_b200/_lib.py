"""ctypes binding of libbuddy_b200_kernels.so (the C ABI in include/buddy_b200.h).

The library is the product; there is no Python or CPU fallback.  Importing this
module without the built library raises ImportError with the build command.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libbuddy_b200_kernels.so")

F32, F16, BF16 = 0, 1, 2
W_F32, W_I8, W_U4 = 0, 1, 2

(T_EMBED, T_INV_FREQ, T_FINAL_NORM, T_LM_HEAD, T_IN_NORM, T_POST_NORM, T_Q_NORM,
 T_K_NORM, T_Q, T_K, T_V, T_O, T_GATE, T_UP, T_DOWN, T_Q_BIAS, T_K_BIAS,
 T_V_BIAS) = range(18)


class Weight(C.Structure):
    _fields_ = [("kind", C.c_int32), ("group", C.c_int32), ("K", C.c_int64),
                ("N", C.c_int64), ("w", C.c_void_p), ("scale", C.c_void_p),
                ("scale_dtype", C.c_int32), ("reserved", C.c_int32),
                ("bias", C.c_void_p)]


class GemvArgs(C.Structure):
    _fields_ = [("x", C.c_void_p), ("x_dtype", C.c_int32), ("y_dtype", C.c_int32),
                ("x_ld", C.c_int64), ("y_ld", C.c_int64), ("y", C.c_void_p),
                ("residual", C.c_void_p), ("norm_weight", C.c_void_p),
                ("norm_eps", C.c_float), ("M", C.c_int32),
                ("accumulate", C.c_int32), ("silu_pairs", C.c_int32)]


class ModelConfigC(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                ("hidden", "n_layers", "q_heads", "kv_heads", "head_dim", "ffn",
                 "vocab", "max_len")] + \
               [("eps", C.c_float), ("rope_theta", C.c_float)] + \
               [(n, C.c_int32) for n in ("qkv_bias", "qk_norm", "tp_rank", "tp_size")]


class B200Error(RuntimeError):
    pass


_lib = None


def load():
    """Return the loaded library, loading it on first use."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `make -C {_HERE}/csrc` "
            "(or `python -c 'import __graft_entry__ as g; g.build()'`). "
            "buddy_mlir_b200 has no CPU fallback.")
    lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
    vp, i64, i32, f32 = C.c_void_p, C.c_int64, C.c_int, C.c_float
    sig = {
        "b200_last_error": (C.c_char_p, []),
        "b200_version": (C.c_char_p, []),
        "b200_launch_count": (C.c_uint64, []),
        "b200_packed_k": (i64, [i32, i64]),
        "b200_packed_row_bytes": (i64, [i32, i64]),
        "b200_packed_offset": (i64, [i32, i64, i64, C.POINTER(C.c_int)]),
        "b200_pack_weight": (i32, [i32, vp, i64, i64, i32, vp, vp]),
        "b200_unpack_weight": (i32, [i32, vp, i64, i64, i32, vp, vp]),
        "b200_pack_scales": (i32, [vp, i32, i64, i64, vp, vp]),
        "b200_quantize_per_channel": (i32, [vp, i64, i64, i32, vp, vp, vp]),
        "b200_quantize_w4_group": (i32, [vp, i64, i64, i64, vp, vp, vp]),
        "b200_pack_int4": (i32, [vp, i64, vp, vp]),
        "b200_unpack_int4": (i32, [vp, i64, vp, vp]),
        "b200_gemv": (i32, [C.POINTER(Weight), C.POINTER(GemvArgs), vp]),
        "b200_gemm_w8_workspace_bytes": (i64, [i32, i64]),
        "b200_gemm_w8": (i32, [C.POINTER(Weight), vp, i32, i64, vp, i64, vp, i64, vp, f32, i32,
                               vp, i64, vp]),
        "b200_gemm_w8_status": (i32, [vp, vp]),
        "b200_gemm_w8a8_workspace_bytes": (i64, [i32, i64]),
        "b200_gemm_w8a8": (i32, [vp, vp, i32, i64, vp, i64, vp, i64, vp]),
        "b200_rmsnorm": (i32, [vp, vp, vp, i64, i64, f32, vp]),
        "b200_silu_mul": (i32, [vp, vp, vp, i64, vp]),
        "b200_rope_kv_write": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, f32, i32,
                                     i32, i32, i32, vp, vp]),
        "b200_gqa_scratch_floats": (i64, [i32, i32, i32]),
        "b200_gqa_decode": (i32, [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp]),
        "b200_gqa_decode_static": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp]),
        "b200_embed": (i32, [vp, vp, vp, i64, vp]),
        "b200_argmax_first": (i32, [vp, i64, vp, vp, vp]),
        "b200_kv_overflow": (i32, [vp, i32, i32, i32, i32, i32, i32, f32,
                                   C.POINTER(C.c_int), vp]),
        "b200_model_create": (i32, [C.POINTER(ModelConfigC), C.POINTER(vp)]),
        "b200_model_destroy": (None, [vp]),
        "b200_model_set_vector": (i32, [vp, i32, i32, vp, i64]),
        "b200_model_set_linear": (i32, [vp, i32, i32, i32, vp, vp, i32, i32, i64,
                                        i64, i32, i32]),
        "b200_model_load_blobs": (i32, [vp, C.c_char_p, vp, i64, vp, i64, i32]),
        "b200_model_set_activation_int8": (i32, [vp, i32]),
        "b200_model_activation_int8": (i32, [vp]),
        "b200_model_save_packed": (i32, [vp, C.c_char_p]),
        "b200_model_set_launch_counter": (i32, [vp, C.c_uint32]),
        "b200_model_load_packed": (i32, [vp, C.c_char_p]),
        "b200_blob_elements": (i32, [C.POINTER(ModelConfigC), C.c_char_p,
                                     C.POINTER(i64), C.POINTER(i64)]),
        "b200_model_finalize": (i32, [vp]),
        "b200_model_kv_upload": (i32, [vp, i32, vp, i32, i32]),
        "b200_model_kv_download": (i32, [vp, i32, vp, i32, i32]),
        "b200_model_read_new_kv_rows": (i32, [vp, vp]),
        "b200_model_decode": (i32, [vp, i32, i32, vp, C.POINTER(C.c_int)]),
        "b200_model_generate": (i32, [vp, i32, i32, i32, vp]),
        "b200_model_prefill": (i32, [vp, vp, i32, i32, vp, i32, C.POINTER(C.c_int)]),
        "b200_batch_create": (i32, [vp, i32, i32, i32, i32, C.POINTER(vp)]),
        "b200_batch_destroy": (None, [vp]),
        "b200_batch_add": (i32, [vp, C.POINTER(C.c_int)]),
        "b200_batch_remove": (i32, [vp, i32]),
        "b200_batch_length": (i32, [vp, i32]),
        "b200_batch_free_pages": (i32, [vp]),
        "b200_batch_prefill": (i32, [vp, i32, vp, i32, vp, C.POINTER(C.c_int)]),
        "b200_batch_decode": (i32, [vp, i32, vp, vp, vp, vp]),
        "b200_batch_last_ms": (f32, [vp]),
        "b200_model_last_ms": (f32, [vp]),
        "b200_model_step_bytes": (i64, [vp, i32]),
        "b200_model_kernels_per_step": (i32, [vp]),
        "b200_model_uses_persistent_kernel": (i32, [vp]),
        "b200_model_tp_sum_kind": (i32, [vp]),
        "b200_model_read_trace": (i32, [vp, vp, i64]),
        "b200_model_kv_ptr": (vp, [vp, i32]),
        "b200_model_kv_overflow": (i32, [vp, i32, i32, f32, C.POINTER(C.c_int)]),
        "b200_tp_unique_id": (i32, [vp]),
        "b200_tp_init": (i32, [vp, i32, i32]),
        "b200_tp_shutdown": (None, []),
        "b200_release_cached_weights": (None, []),
        "b200_forward_decode": (i32, [C.POINTER(ModelConfigC), C.c_char_p, i32, vp,
                                      i64, vp, i64, C.c_longlong, C.c_longlong,
                                      C.POINTER(vp), C.POINTER(vp)]),
        "b200_forward_prefill": (i32, [C.POINTER(ModelConfigC), C.c_char_p, i32, vp,
                                       i64, vp, i64, C.POINTER(C.c_longlong), i32,
                                       C.POINTER(vp), vp]),
        "b200_forward_reset": (None, []),
        "b200_forward_status": (i32, []),
        "b200_forward_session_builds": (i32, []),
        "b200_rax_open": (i32, [C.c_char_p, C.POINTER(vp)]),
        "b200_rax_close": (None, [vp]),
        "b200_rax_count": (i32, [vp]),
        "b200_rax_manifest_bytes": (C.c_uint64, [vp]),
        "b200_rax_entry": (i32, [vp, i32, C.c_char_p, i32, C.POINTER(i32), C.POINTER(C.c_uint64),
                                 C.POINTER(C.c_uint64)]),
        "b200_rax_find": (i32, [vp, C.c_char_p]),
        "b200_rax_read": (i32, [vp, i32, vp, C.c_uint64]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(rc):
    """Raise B200Error with the library's message when rc is a failure code."""
    if rc != 0:
        raise B200Error(f"[{rc}] {load().b200_last_error().decode()}")


def exported_symbols():
    """Names every header in include/ declares (used by the load test)."""
    import re
    names = set()
    inc = os.path.join(os.path.dirname(_HERE), "include")
    for h in sorted(os.listdir(inc)):
        text = open(os.path.join(inc, h)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names.update(re.findall(r"\b((?:b200|_mlir_ciface)_[A-Za-z0-9_]+)\s*\(", text))
    return sorted(names)
