"""Host-side checks that need no GPU: the library loads and exports every
declared symbol, the packed-row index map is a bijection, the blob walk
counts match buddy-mlir's specs, and compute entry points refuse to run
without a device instead of falling back."""
import ctypes as C

import numpy as np
import pytest

from buddy_mlir_b200 import DEEPSEEK_R1_1P5B, TINY_QWEN2, _lib, synthetic


def _has_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = _lib.exported_symbols()
    assert len(names) > 40
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


@pytest.mark.parametrize("kind,unit", [(_lib.W_I8, 16), (_lib.W_U4, 32), (_lib.W_F32, 4)])
@pytest.mark.parametrize("K", [8, 16, 100, 512, 1536, 8960, 4096 + 64])
def test_packed_offset_is_a_bijection(kind, unit, K):
    lib = _lib.load()
    Kp = lib.b200_packed_k(kind, K)
    assert Kp % unit == 0 and Kp >= K and Kp - K < unit
    rb = lib.b200_packed_row_bytes(kind, K)
    assert rb == Kp // unit * 16
    seen = set()
    nib = C.c_int(0)
    for k in range(Kp):
        off = lib.b200_packed_offset(kind, K, k, C.byref(nib))
        assert 0 <= off < rb
        if kind == _lib.W_F32:
            assert off % 4 == 0
        seen.add((off, nib.value))
    assert len(seen) == Kp


def test_packed_offset_lane_groups_are_contiguous_across_lanes():
    # group j of lane l covers k = j*(Bs/G) + 4l .. +3: lanes walk x contiguously
    lib = _lib.load()
    K = 1536
    nib = C.c_int(0)
    for k in range(0, 512, 4):
        off = lib.b200_packed_offset(_lib.W_I8, K, k, C.byref(nib))
        j, l = k // 128, (k % 128) // 4
        assert off == l * 16 + j * 4


def test_blob_counts_match_reference_specs():
    # models/deepseek_r1/specs/f32.json and w8a32.json
    lib = _lib.load()
    c = DEEPSEEK_R1_1P5B.to_c()
    nf, ni = C.c_int64(), C.c_int64()
    assert lib.b200_blob_elements(C.byref(c), b"f32", C.byref(nf), C.byref(ni)) == 0
    assert (nf.value, ni.value) == (1777088064, 0)
    assert lib.b200_blob_elements(C.byref(c), b"w8a32", C.byref(nf), C.byref(ni)) == 0
    assert (nf.value, ni.value) == (322338752, 1455489024)
    assert synthetic.blob_elements(DEEPSEEK_R1_1P5B) == 1777088064
    # models/deepseek_r1/specs/w4a16.json: 322338752 f16 elements + 727744512 packed bytes
    assert lib.b200_blob_elements(C.byref(c), b"w4a16", C.byref(nf), C.byref(ni)) == 0
    assert (nf.value, ni.value) == (322338752, 727744512)
    # models/deepseek_r1/specs/w8a16.json: f16_elements 322338752, i8_elements 1455489024
    assert lib.b200_blob_elements(C.byref(c), b"w8a16", C.byref(nf), C.byref(ni)) == 0
    assert (nf.value, ni.value) == (322338752, 1455489024)
    # models/deepseek_r1/specs/f16.json: total 1777088064 (f16 elements)
    assert lib.b200_blob_elements(C.byref(c), b"f16", C.byref(nf), C.byref(ni)) == 0
    assert (nf.value, ni.value) == (1777088064, 0)
    # the bf16 variant: the same walk with bfloat16 elements (tools/buddy-codegen/gen_config.py:54)
    assert lib.b200_blob_elements(C.byref(c), b"bf16", C.byref(nf), C.byref(ni)) == 0
    assert (nf.value, ni.value) == (1777088064, 0)
    # Qwen3 shapes (head norms, no biases): the count of the walk synthetic.tensor_list describes
    from buddy_mlir_b200 import QWEN3_8B, TINY_QWEN3
    for q3 in (TINY_QWEN3, QWEN3_8B):
        c3 = q3.to_c()
        assert lib.b200_blob_elements(C.byref(c3), b"f32", C.byref(nf), C.byref(ni)) == 0
        assert (nf.value, ni.value) == (synthetic.blob_elements(q3), 0)
    # models/deepseek_r1/specs/w8a8.json: linear_elements 1455489024, other_elements 322338752
    assert lib.b200_blob_elements(C.byref(c), b"w8a8", C.byref(nf), C.byref(ni)) == 0
    assert (nf.value, ni.value) == (322338752, 1455489024)
    assert lib.b200_blob_elements(C.byref(c), b"w4a8", C.byref(nf), C.byref(ni)) != 0


def test_w8a32_split_sizes():
    cfg = TINY_QWEN2
    _, views = synthetic.make_f32_blob(cfg, 1)
    fb, ib = synthetic.split_w8a32(
        cfg, views, lambda W: (np.zeros(W.shape, np.int8), np.ones(W.shape[1], np.float32)))
    lib = _lib.load()
    c = cfg.to_c()
    nf, ni = C.c_int64(), C.c_int64()
    lib.b200_blob_elements(C.byref(c), b"w8a32", C.byref(nf), C.byref(ni))
    assert (fb.size, ib.size) == (nf.value, ni.value)


def test_argument_errors_are_reported():
    lib = _lib.load()
    assert lib.b200_pack_int4(None, 3, None, None) == -1
    assert b"pack_int4" in lib.b200_last_error()
    with pytest.raises(_lib.B200Error):
        _lib.check(lib.b200_gemv(None, None, None))


@pytest.mark.skipif(_has_gpu(), reason="only meaningful without a CUDA device")
def test_no_cpu_fallback_without_a_device():
    lib = _lib.load()
    a = np.zeros(16, dtype=np.int8)
    rc = lib.b200_unpack_int4(a.ctypes.data, 8, a.ctypes.data, None)
    assert rc == -3 and b"no CUDA device" in lib.b200_last_error()
    h = C.c_void_p()
    c = TINY_QWEN2.to_c()
    assert lib.b200_model_create(C.byref(c), C.byref(h)) == -3


def test_static_attention_entry_checks_arguments_on_the_host():
    """Every argument check of b200_gqa_decode_static runs before the device is
    touched, so it can be exercised without one: more kv heads than query heads
    at the largest accepted shape, a group size that is not built, a bad head
    size and a null pointer are all B200_EINVAL."""
    lib = _lib.load()
    buf = np.zeros(16, dtype=np.float32)
    p = buf.ctypes.data
    assert lib.b200_gqa_decode_static(p, p, p, p, 64, 128, 128, 64, 32, p, None) == -1
    assert lib.b200_gqa_decode_static(p, p, p, p, 12, 5, 128, 64, 8, p, None) == -1
    assert lib.b200_gqa_decode_static(p, p, p, p, 12, 2, 96, 64, 8, p, None) == -1
    assert lib.b200_gqa_decode_static(None, p, p, p, 12, 2, 128, 64, 8, p, None) == -1
    assert lib.b200_gqa_decode_static(p, p, p, p, 12, 2, 128, 64, 0, p, None) == -1


def test_model_entry_shim_exports_both_symbols():
    """What ModelSession::Impl::loadSo does (tools/buddy-codegen/gen_session.py:1120-1141):
    one dlopen(RTLD_LOCAL) of the model .so, then the prefill and the decode symbol."""
    import os
    from buddy_mlir_b200.gen_model_entry import HERE, build, shim_name
    _lib.load()
    so = os.path.join(HERE, shim_name(TINY_QWEN2, "w8a32"))
    if not os.path.exists(so):
        build(TINY_QWEN2, "w8a32")
    dll = C.CDLL(so, mode=os.RTLD_NOW | os.RTLD_LOCAL)
    assert dll._mlir_ciface_forward_prefill is not None
    assert dll._mlir_ciface_forward_decode is not None


def test_shim_arguments_from_the_reference_variant_specs():
    """gen_model_entry.from_spec reads the two inputs of buddy-mlir's own gen_config.py: every
    spec under models/deepseek_r1/specs/ of a checkout, with the published config of
    DeepSeek-R1-Distill-Qwen-1.5B, gives the 1.5B shapes and the variant, cache sizes and decode
    packing the stock shims are built with."""
    import glob
    import json
    import os
    from buddy_mlir_b200 import gen_model_entry as g
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ref = os.environ.get("BUDDY_MLIR_ROOT") or os.path.join(os.path.dirname(root), "reference")
    specs = sorted(glob.glob(os.path.join(ref, "models", "deepseek_r1", "specs", "*.json")))
    if not specs:
        import pytest
        pytest.skip("needs a buddy-mlir checkout for its spec files")
    hf = {"model_type": "qwen2", "hidden_size": 1536, "intermediate_size": 8960, "num_hidden_layers": 28,
          "num_attention_heads": 12, "num_key_value_heads": 2, "vocab_size": 151936, "rms_norm_eps": 1e-6,
          "rope_theta": 10000, "max_position_embeddings": 131072}
    seen = set()
    for path in specs:
        with open(path) as f:
            spec = json.load(f)
        cfg, kw = g.from_spec(spec, hf)
        assert cfg.with_(name=DEEPSEEK_R1_1P5B.name) == DEEPSEEK_R1_1P5B, path
        assert kw["variant"] == spec["variant"]
        name = os.path.basename(path)
        assert kw.get("tiers") == (g.R1_TIERS if "tiered" in name else None)
        assert kw.get("decode_packed", False) == ("packed_decode" in name)
        seen.add((kw["variant"], "tiers" in kw, kw.get("decode_packed", False)))
        g.source(DEEPSEEK_R1_1P5B, **kw)           # the shim source generates for every spec
    assert {v for v, _, _ in seen} == {"f32", "f16", "w8a32", "w8a8", "w8a16", "w4a16"}
    q3 = dict(hf, model_type="qwen3", head_dim=128, attention_bias=False)
    cfg, _ = g.from_spec({"variant": "f32", "max_token_len": 4096}, q3)
    assert cfg.qk_norm and not cfg.qkv_bias and cfg.head_dim == 128 and cfg.max_len == 4096


def test_reference_manifest_generator_takes_the_shim_and_the_runner_plugin():
    """buddy-mlir's own tools/buddy-codegen/gen_config.py + gen_manifest.py, run on the w8a32
    spec of the 1.5B model with this library's files in place of the compiled model: the
    manifest text names the model-entry shim as the code object, the kernels library as its
    dependency and the runner plugin as the runner library, with the weight files, KV buffers
    and entry arguments the shim serves (what a maintainer packs with rax-pack)."""
    import json
    import os
    import sys
    import pytest
    from buddy_mlir_b200 import gen_model_entry as g
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ref = os.environ.get("BUDDY_MLIR_ROOT") or os.path.join(os.path.dirname(root), "reference")
    tools = os.path.join(ref, "tools", "buddy-codegen")
    spec_path = os.path.join(ref, "models", "deepseek_r1", "specs", "w8a32.json")
    if not os.path.exists(spec_path):
        pytest.skip("needs a buddy-mlir checkout for its generators")
    sys.path.insert(0, tools)
    try:
        import gen_config
        import gen_manifest
    finally:
        sys.path.remove(tools)
    with open(spec_path) as f:
        spec = json.load(f)
    hf = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": 1536, "intermediate_size": 8960,
          "num_hidden_layers": 28, "num_attention_heads": 12, "num_key_value_heads": 2, "vocab_size": 151936,
          "rms_norm_eps": 1e-6, "rope_theta": 10000, "eos_token_id": 151643}
    hf_path = os.path.join(os.environ.get("TMPDIR", "/tmp"), "b200_hf_config_1p5b.json")
    with open(hf_path, "w") as f:
        json.dump(hf, f)
    config = gen_config.gen_config(spec, hf_path)
    cfg, kw = g.from_spec(spec, hf)
    shim = g.shim_name(cfg, kw["variant"])
    config["compilation"]["so_name"] = shim
    text = gen_manifest.gen_manifest(config, dep_shared_libs=["libbuddy_b200_kernels.so"],
                                     runner_library="libbuddy_b200_runner.so")
    assert f'uri = "file:{shim}"' in text and 'rhal.codeobj @model_kernels' in text
    assert 'uri = "file:libbuddy_b200_kernels.so"' in text
    assert 'runner_library = "file:libbuddy_b200_runner.so"' in text
    # the weight files and element counts the shim's loader expects for this variant
    lib = _lib.load()
    nf, ni = C.c_int64(), C.c_int64()
    assert lib.b200_blob_elements(C.byref(cfg.to_c()), b"w8a32", C.byref(nf), C.byref(ni)) == 0
    assert f"tensor<{nf.value}xf32>" in text and 'uri = "file:arg0-w8a32-f32.data"' in text
    assert f"tensor<{ni.value}xi8>" in text and 'uri = "file:arg0-w8a32-i8.data"' in text
    # 56 cache buffers [1, kv_heads, max_len, head_dim] and both entries dispatched to the code object
    assert text.count(f"tensor<1x{cfg.kv_heads}x{cfg.max_len}x{cfg.head_dim}xf32>") == 2 * cfg.n_layers
    assert text.count('dispatch = "model_kernels"') == 2
