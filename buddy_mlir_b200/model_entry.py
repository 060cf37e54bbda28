"""Host harness that drives a model-entry shim the way buddy-mlir's generated
ModelSession does: one dlopen(RTLD_LOCAL) of the model .so, dlsym of
`_mlir_ciface_forward_prefill` and then `_mlir_ciface_forward_decode` (either
one missing is an error, as in ModelSession::Impl::loadSo), the KV cache and
logits owned on the HOST, and the entries called with MemRef descriptors
(tools/buddy-codegen/gen_session.py:1106-1141, 1176-1294, 1345-1373,
1381-1452).  buddy-cli itself cannot be linked here (it needs LLVMSupport and
FlatBuffers), so this is the closest stand-in for the reference's host."""
import ctypes as C
import os

import numpy as np

from . import _lib
from .config import ModelConfig
from .gen_model_entry import HERE, build, shim_name
from .memref import _libc, memref_type, to_memref


class EntrySession:
    def __init__(self, cfg: ModelConfig, variant: str, blobs, all_linear_w8: bool = False, decode_blobs=None):
        """decode_blobs: the weight files the decode entry gets when they differ from the prefill
        entry's (the panel-packed copy of the packed-decode spec, gen_session.py:1393)."""
        _lib.load()
        packed = decode_blobs is not None
        so = os.path.join(HERE, shim_name(cfg, variant, all_linear_w8, packed))
        if not os.path.exists(so):
            build(cfg, variant, all_linear_w8, decode_packed=packed)
        self.dll = C.CDLL(so)          # RTLD_LOCAL, like ModelSession::Impl::loadSo
        # gen_session.py:1127-1141: prefill first, then decode; a missing symbol throws
        self.prefill_fn = self.dll._mlir_ciface_forward_prefill
        self.prefill_fn.restype = None
        self.prefill_fn.argtypes = None
        self.fn = self.dll._mlir_ciface_forward_decode
        self.fn.restype = None
        self.cfg = cfg
        # host element of the cache and the logits: half (as uint16) for the f16-activation variants
        self.half = variant in ("f16", "bf16", "w4a16", "w8a16")
        self.bf16 = variant == "bf16"
        self.ht = np.uint16 if self.half else np.float32
        self.blobs = [np.ascontiguousarray(b) for b in blobs]
        if self.half:   # the f16 blob travels as the uint16 memref the reference's session builds
            self.blobs[0] = self.blobs[0].view(np.uint16)
        self.blob_desc = [to_memref(b) for b in self.blobs]
        self.decode_blobs = [np.ascontiguousarray(b) for b in decode_blobs] if packed else self.blobs
        self.decode_blob_desc = [to_memref(b) for b in self.decode_blobs] if packed else self.blob_desc
        kvs = (1, cfg.kv_heads, cfg.max_len, cfg.head_dim)
        self.kv = [np.zeros(kvs, dtype=self.ht) for _ in range(2 * cfg.n_layers)]
        self.kv_desc = [to_memref(k) for k in self.kv]
        self.token = np.zeros((1, 1), dtype=np.int64)
        self.cache_position = np.zeros(1, dtype=np.int64)
        self.dummies = [np.zeros(1, dtype=np.int64) for _ in range(cfg.n_layers - 1)]
        self.logits = np.zeros(cfg.vocab, dtype=np.float32)
        self.position_ = 0
        # DecodeABI: cache_position_out, kv0, kv1, (dummy_i, kv, kv)*, logits
        I1, K4, L3 = memref_type(np.int64, 1), memref_type(self.ht, 4), memref_type(self.ht, 3)
        fields = [("cache_position_out", I1), ("kv0", K4), ("kv1", K4)]
        for i in range(cfg.n_layers - 1):
            fields += [(f"dummy{i}", I1), (f"kv{2 + 2 * i}", K4), (f"kv{3 + 2 * i}", K4)]
        fields.append(("logits", L3))
        self.ABI = type("DecodeABI", (C.Structure,), {"_fields_": fields})
        # descriptors are built once; decode() only rewrites the scalars
        self._tok_d, self._pos_d = to_memref(self.token), to_memref(self.cache_position)
        self._dum_d = [to_memref(d) for d in self.dummies]
        self._result = self.ABI()
        args = [C.byref(self._result)] + [C.byref(d) for d in self.decode_blob_desc]
        args += [C.byref(self._tok_d), C.byref(self._pos_d), C.byref(self.kv_desc[0]),
                 C.byref(self.kv_desc[1])]
        for i in range(cfg.n_layers - 1):
            args += [C.byref(self._dum_d[i]), C.byref(self.kv_desc[2 + 2 * i]),
                     C.byref(self.kv_desc[3 + 2 * i])]
        self._args = args
        self.fn.argtypes = None

    def prefill(self, prompt, pad_id: int = 0):
        """ModelSession::prefill (gen_session.py:1345-1373): the token container holds
        the prompt padded to max_len; every result is copied into the session's state
        and the callee's buffers are freed; position_ = token count.  Returns the
        logits [max_len, vocab] (the runtime reads row len(prompt) - 1)."""
        cfg = self.cfg
        toks = np.full((1, cfg.max_len), pad_id, dtype=np.uint64)
        toks[0, :len(prompt)] = np.asarray(prompt, dtype=np.uint64)
        tok_d = to_memref(toks)
        K4, L3 = memref_type(self.ht, 4), memref_type(self.ht, 3)
        ABI = type("PrefillABI", (C.Structure,), {"_fields_": [("kv", K4 * (2 * cfg.n_layers)), ("logits", L3)]})
        result = ABI()
        import time
        t0 = time.perf_counter()
        self.prefill_fn(C.byref(result), *[C.byref(d) for d in self.blob_desc], C.byref(tok_d))
        self.last_prefill_call_s = time.perf_counter() - t0     # the entry alone, without this harness's copies
        self._check()
        n = cfg.max_len * cfg.vocab
        logits = self._floats(np.array(np.ctypeslib.as_array(result.logits.aligned, shape=(n,)), copy=True))
        _libc.free(C.cast(result.logits.allocated, C.c_void_p))
        for i, k in enumerate(self.kv):
            src = np.ctypeslib.as_array(result.kv[i].aligned, shape=(k.size,))
            np.copyto(k.reshape(-1), src)
            _libc.free(C.cast(result.kv[i].allocated, C.c_void_p))
        self.position_ = len(prompt)
        self.prefill_logits = logits.reshape(cfg.max_len, cfg.vocab)
        np.copyto(self.logits, self.prefill_logits[len(prompt) - 1])
        return self.prefill_logits

    def decode(self, token_id: int, check_alias: bool = False):
        self.token[0, 0] = token_id
        self.cache_position[0] = self.position_
        for d in self.dummies:
            d[0] = self.position_
        result = self._result
        self.fn(*self._args)
        # gen_session.py:1416-1442: copy the logits out, KV results alias the state
        src = np.ctypeslib.as_array(result.logits.aligned, shape=(self.cfg.vocab,))
        np.copyto(self.logits, self._floats(src))
        _libc.free(C.cast(result.logits.allocated, C.c_void_p))
        # a null descriptor for the next call, as resetDecodeResultABI leaves it (gen_session.py:
        # 1434-1446): a descriptor that still names a buffer would be filled in place
        C.memset(C.byref(result.logits), 0, C.sizeof(result.logits))
        self._check()
        if check_alias:
            for i, k in enumerate(self.kv):
                got = getattr(result, f"kv{i}")
                assert C.addressof(got.aligned.contents) == k.ctypes.data
        self.position_ += 1

    def _floats(self, a):
        """logitsFloat_ of the generated session (gen_session.py:1531: halfToFloat per element)."""
        if self.bf16:   # bfloat16 = the high half of an f32
            return (a.astype(np.uint32) << 16).view(np.float32)
        return a.view(np.float16).astype(np.float32) if self.half else a

    def _check(self):
        """The entries return void; the library keeps the first failure (b200_forward_status)."""
        lib = _lib.load()
        if lib.b200_forward_status() != 0:
            raise _lib.B200Error(lib.b200_last_error().decode())

    def kv_floats(self, i):
        return self._floats(self.kv[i])

    def reset_position(self):
        self.position_ = 0

    def close(self):
        _lib.load().b200_forward_reset()


class TieredEntrySession:
    """The host side of the tiered-cache spec (models/deepseek_r1/specs/f32_tiered_kv_cache.json)
    as gen_session.py:303-800 generates it: one prefill / decode symbol per cache size
    (`_mlir_ciface_forward_prefill_<size>`, `_mlir_ciface_forward_decode_<size>`), the smallest
    tier that holds the sequence is used, and the host cache is copied into the next tier's
    buffers when the sequence outgrows the current one."""

    def __init__(self, cfg: ModelConfig, blob, tiers):
        _lib.load()
        so = os.path.join(HERE, shim_name(cfg, "f32", tiers=tiers))
        if not os.path.exists(so):
            build(cfg, "f32", tiers=tiers)
        self.dll = C.CDLL(so)
        self.cfg, self.tiers = cfg, list(tiers)
        self.prefill_fns = [getattr(self.dll, f"_mlir_ciface_forward_prefill_{t}") for t in tiers]
        self.decode_fns = [getattr(self.dll, f"_mlir_ciface_forward_decode_{t}") for t in tiers]
        for f in self.prefill_fns + self.decode_fns:
            f.restype, f.argtypes = None, None
        self.blob = np.ascontiguousarray(blob, dtype=np.float32)
        self.blob_desc = to_memref(self.blob)
        nl = 2 * cfg.n_layers
        self.kv = [[np.zeros((1, cfg.kv_heads, t, cfg.head_dim), dtype=np.float32) for _ in range(nl)] for t in tiers]
        self.token = np.zeros((1, 1), dtype=np.int64)
        self.cache_position = np.zeros(1, dtype=np.int64)
        self.dummies = [np.zeros(1, dtype=np.int64) for _ in range(cfg.n_layers - 1)]
        self.logits = np.zeros(cfg.vocab, dtype=np.float32)
        self.position_, self.slot = 0, 0
        I1, K4, L3 = memref_type(np.int64, 1), memref_type(np.float32, 4), memref_type(np.float32, 3)
        fields = [("cache_position_out", I1), ("kv0", K4), ("kv1", K4)]
        for i in range(cfg.n_layers - 1):
            fields += [(f"dummy{i}", I1), (f"kv{2 + 2 * i}", K4), (f"kv{3 + 2 * i}", K4)]
        fields.append(("logits", L3))
        self.DecodeABI = type("DecodeABI", (C.Structure,), {"_fields_": fields})
        self.PrefillABI = type("PrefillABI", (C.Structure,), {"_fields_": [("kv", K4 * nl), ("logits", L3)]})

    def _check(self):
        lib = _lib.load()
        if lib.b200_forward_status() != 0:
            raise _lib.B200Error(lib.b200_last_error().decode())

    def prefill(self, prompt, pad_id: int = 0):
        cfg, n = self.cfg, len(prompt)
        self.slot = next(i for i, t in enumerate(self.tiers) if n <= t)        # selectPrefillSize
        S = self.tiers[self.slot]
        toks = np.full((1, S), pad_id, dtype=np.uint64)
        toks[0, :n] = np.asarray(prompt, dtype=np.uint64)
        tok_d = to_memref(toks)
        result = self.PrefillABI()
        self.prefill_fns[self.slot](C.byref(result), C.byref(self.blob_desc), C.byref(tok_d))
        self._check()
        logits = np.array(np.ctypeslib.as_array(result.logits.aligned, shape=(S * cfg.vocab,)), copy=True)
        _libc.free(C.cast(result.logits.allocated, C.c_void_p))
        for i, k in enumerate(self.kv[self.slot]):                             # copyKVCache(prefill -> decode)
            assert tuple(result.kv[i].sizes) == (1, cfg.kv_heads, S, cfg.head_dim)
            src = np.ctypeslib.as_array(result.kv[i].aligned, shape=(k.size,)).reshape(k.shape)
            k[:, :, :n] = src[:, :, :n]
            _libc.free(C.cast(result.kv[i].allocated, C.c_void_p))
        self.position_ = n
        self.prefill_logits = logits.reshape(S, cfg.vocab)
        np.copyto(self.logits, self.prefill_logits[n - 1])
        return self.prefill_logits

    def decode(self, token_id: int):
        cfg = self.cfg
        need = next((i for i, t in enumerate(self.tiers) if self.position_ + 1 < t), len(self.tiers) - 1)  # selectDecodeSize
        if need != self.slot:
            for old, new in zip(self.kv[self.slot], self.kv[need]):            # copyKVCache(tier -> tier)
                new[:, :, :self.position_] = old[:, :, :self.position_]
            self.slot = need
        self.token[0, 0] = token_id
        self.cache_position[0] = self.position_
        for d in self.dummies:
            d[0] = self.position_
        kv = self.kv[self.slot]
        kvd = [to_memref(k) for k in kv]
        result = self.DecodeABI()
        args = [C.byref(result), C.byref(self.blob_desc), C.byref(to_memref(self.token)),
                C.byref(to_memref(self.cache_position)), C.byref(kvd[0]), C.byref(kvd[1])]
        dd = [to_memref(d) for d in self.dummies]
        for i in range(cfg.n_layers - 1):
            args += [C.byref(dd[i]), C.byref(kvd[2 + 2 * i]), C.byref(kvd[3 + 2 * i])]
        self.decode_fns[self.slot](*args)
        np.copyto(self.logits, np.ctypeslib.as_array(result.logits.aligned, shape=(cfg.vocab,)))
        _libc.free(C.cast(result.logits.allocated, C.c_void_p))
        self._check()
        self.position_ += 1

    def close(self):
        _lib.load().b200_forward_reset()
