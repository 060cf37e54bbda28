"""Host-side mirror of buddy-mlir's LLM session interface over the device
session of the C ABI.

ModelSession follows the generated ModelSession / LLMSession
(runtime/include/buddy/runtime/llm/LLMSession.h:41-82,
tools/buddy-codegen/gen_session.py:1345-1541): load weights, decode one token
at the current position, read logits, reset, handle KV overflow.  run_generation
follows runtime/llm/TextGeneration.cpp:157-277 for the greedy case, with token
ids in and out (no tokenizer).
"""
import ctypes as C
import time

import numpy as np

from . import _lib
from .config import ModelConfig
from .synthetic import tensor_list

_SLOT = {"q": _lib.T_Q, "k": _lib.T_K, "v": _lib.T_V, "o": _lib.T_O,
         "gate": _lib.T_GATE, "up": _lib.T_UP, "down": _lib.T_DOWN,
         "lm_head": _lib.T_LM_HEAD, "embed": _lib.T_EMBED,
         "inv_freq": _lib.T_INV_FREQ, "final_norm": _lib.T_FINAL_NORM,
         "in_norm": _lib.T_IN_NORM, "post_norm": _lib.T_POST_NORM,
         "q_norm": _lib.T_Q_NORM, "k_norm": _lib.T_K_NORM,
         "q_bias": _lib.T_Q_BIAS, "k_bias": _lib.T_K_BIAS, "v_bias": _lib.T_V_BIAS}
_LINEAR = ("q", "k", "v", "o", "gate", "up", "down", "lm_head")


def greedy_sample(logits: np.ndarray) -> int:
    """Sampler::greedySample (runtime/include/buddy/runtime/llm/Sampler.h:101-104):
    np.argmax returns the first maximum, like std::max_element."""
    return int(np.argmax(logits))


class ModelSession:
    def __init__(self, cfg: ModelConfig, tp_rank: int = 0, tp_size: int = 1):
        self.cfg = cfg
        self.lib = _lib.load()
        self._h = C.c_void_p()
        self._cfg_c = cfg.to_c(tp_rank, tp_size)
        _lib.check(self.lib.b200_model_create(C.byref(self._cfg_c), C.byref(self._h)))
        self.position_ = 0
        self._logits = np.zeros(cfg.vocab, dtype=np.float32)
        self.tp_rank, self.tp_size = tp_rank, tp_size

    def close(self):
        if self._h:
            self.lib.b200_model_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- loading -----------------------------------------------------------
    def load_blobs(self, variant: str, float_blob: np.ndarray, int_blob=None,
                   all_linear_w8: bool = False, save_packed=None):
        """loadWeights (gen_session.py:1301-1338) for in-memory blobs.
        save_packed: path of a repack-cache file to write before finalising."""
        if variant == "bf16":
            fb = np.ascontiguousarray(float_blob, dtype=np.uint16)     # the high halves of the f32 values
        else:
            fb = np.ascontiguousarray(float_blob, dtype=np.float16 if variant in ("f16", "w4a16", "w8a16") else np.float32)
        ib = None if int_blob is None else np.ascontiguousarray(int_blob, dtype=np.int8)
        _lib.check(self.lib.b200_model_load_blobs(
            self._h, variant.encode(), fb.ctypes.data, fb.size,
            None if ib is None else ib.ctypes.data, 0 if ib is None else ib.size,
            int(all_linear_w8)))
        if save_packed is not None:
            _lib.check(self.lib.b200_model_save_packed(self._h, str(save_packed).encode()))
        self.finalize()

    def set_activation_int8(self, enabled: bool = True):
        """Run this session with the arithmetic of the w8a8 graphs: int8 projections quantise
        their activations, one dynamic scale per activation tensor (load_blobs("w8a8") does it)."""
        _lib.check(self.lib.b200_model_set_activation_int8(self._h, int(enabled)))

    def load_packed(self, path):
        """Fill the model from a repack-cache file (b200_model_save_packed) and finalise."""
        _lib.check(self.lib.b200_model_load_packed(self._h, str(path).encode()))
        self.finalize()

    def load_weights(self, paths, variant: str, all_linear_w8: bool = False):
        """loadWeights from the reference's files (arg0*.data; table in
        tools/buddy-codegen/gen_config.py:51-71)."""
        fb = np.fromfile(paths[0], dtype=np.uint16 if variant == "bf16" else
                         np.float16 if variant in ("f16", "w4a16", "w8a16") else np.float32)
        ib = np.fromfile(paths[1], dtype=np.int8) if len(paths) > 1 else None
        self.load_blobs(variant, fb, ib, all_linear_w8)

    def load_tensors(self, views, quantize_to=None, group=0, save_packed=None):
        """Load from a {(name, layer): array} map of f32 tensors in the
        reference's [K,N] layout; quantize_to in (None, 'w8', 'w4') quantises
        every linear layer on the device.  save_packed: path of a repack-cache
        file to write before finalising."""
        qt = {None: -1, "w8": _lib.W_I8, "w4": _lib.W_U4}[quantize_to]
        for name, layer, shape in tensor_list(self.cfg):
            a = np.ascontiguousarray(views[(name, layer)], dtype=np.float32)
            if name in _LINEAR:
                K, N = shape
                _lib.check(self.lib.b200_model_set_linear(
                    self._h, layer, _SLOT[name], _lib.W_F32, a.ctypes.data, None,
                    _lib.F32, 0, K, N, qt, group))
            elif name.endswith("_bias"):
                continue
            else:
                _lib.check(self.lib.b200_model_set_vector(
                    self._h, layer, _SLOT[name], a.ctypes.data, a.size))
        for name, layer, _ in tensor_list(self.cfg):
            if name.endswith("_bias"):
                a = np.ascontiguousarray(views[(name, layer)], dtype=np.float32)
                _lib.check(self.lib.b200_model_set_vector(
                    self._h, layer, _SLOT[name], a.ctypes.data, a.size))
        if save_packed is not None:
            _lib.check(self.lib.b200_model_save_packed(self._h, str(save_packed).encode()))
        self.finalize()

    def set_linear_quantised(self, layer, name, kind, w, scale, scale_dtype, signed, K, N, group=0):
        w = np.ascontiguousarray(w)
        scale = np.ascontiguousarray(scale)
        _lib.check(self.lib.b200_model_set_linear(
            self._h, layer, _SLOT[name], kind, w.ctypes.data, scale.ctypes.data,
            scale_dtype, int(signed), K, N, -1, group))

    def finalize(self):
        _lib.check(self.lib.b200_model_finalize(self._h))

    # ---- LLMSession interface ----------------------------------------------
    def decode(self, token_id: int):
        _lib.check(self.lib.b200_model_decode(self._h, int(token_id), self.position_,
                                              self._logits.ctypes.data, None))
        self.position_ += 1

    def decode_greedy(self, token_id: int) -> int:
        """decode + device-side argmax; only 4 bytes come back."""
        nxt = C.c_int()
        _lib.check(self.lib.b200_model_decode(self._h, int(token_id), self.position_,
                                              None, C.byref(nxt)))
        self.position_ += 1
        return nxt.value

    def generate(self, token_id: int, steps: int) -> np.ndarray:
        """`steps` greedy steps without leaving the device."""
        out = np.zeros(steps, dtype=np.int32)
        _lib.check(self.lib.b200_model_generate(self._h, int(token_id), self.position_,
                                                steps, out.ctypes.data))
        self.position_ += steps
        return out

    def prefill(self, tokens, dense=None):
        """ModelSession::prefill (gen_session.py:1345-1373): the whole prompt from
        position 0; afterwards logits_data() is the last prompt row's logits.
        dense=True runs all rows at once (tensor-core GEMMs, b200_model_prefill),
        dense=False feeds the prompt through the decode path token by token;
        the default takes the dense path for prompts of 16 tokens or more on
        single-GPU sessions.  Both leave the same KV cache."""
        self.reset_position()
        if dense is None:
            dense = len(tokens) >= 16 and self.tp_size == 1
        if dense:
            self.prefill_rows(tokens, 0, all_rows=False)
            return
        for t in tokens:
            self.decode(int(t))

    def prefill_rows(self, tokens, pos0=None, all_rows=True):
        """Rows at positions pos0.. in one pass; returns the logits ([n, vocab] or the
        last row) and moves the position behind them."""
        toks = np.ascontiguousarray(tokens, dtype=np.int32)
        pos0 = self.position_ if pos0 is None else pos0
        n = toks.size
        out = np.zeros((n, self.cfg.vocab) if all_rows else (self.cfg.vocab,), dtype=np.float32)
        nxt = C.c_int()
        _lib.check(self.lib.b200_model_prefill(self._h, toks.ctypes.data, n, pos0, out.ctypes.data,
                                               int(all_rows), C.byref(nxt)))
        self.position_ = pos0 + n
        np.copyto(self._logits, out[-1] if all_rows else out)
        self.last_next_token = nxt.value
        return out

    def reset_position(self):
        self.position_ = 0

    def position(self) -> int:
        return self.position_

    def logits_data(self) -> np.ndarray:
        return self._logits

    def vocab_size(self) -> int:
        return self.cfg.vocab

    def handle_kv_cache_overflow(self, keep_token_num: int, rope_theta: float = 10000.0) -> bool:
        new_pos = C.c_int(-1)
        _lib.check(self.lib.b200_model_kv_overflow(self._h, self.position_, keep_token_num,
                                                   rope_theta, C.byref(new_pos)))
        if new_pos.value < 0:
            return False
        self.position_ = new_pos.value
        return True

    # ---- extras ---------------------------------------------------------------
    def last_ms(self) -> float:
        return float(self.lib.b200_model_last_ms(self._h))

    def step_bytes(self, ctx: int) -> int:
        return int(self.lib.b200_model_step_bytes(self._h, ctx))

    def kernels_per_step(self) -> int:
        return int(self.lib.b200_model_kernels_per_step(self._h))

    def uses_persistent_kernel(self) -> bool:
        return bool(self.lib.b200_model_uses_persistent_kernel(self._h))

    def tp_sum_kind(self):
        """0: single GPU, 1: NCCL all-reduce, 2: peer stores from the GEMV epilogue."""
        return int(self.lib.b200_model_tp_sum_kind(self._h))

    def kv_upload(self, buffer: int, host: np.ndarray, pos0: int, n_pos: int):
        host = np.ascontiguousarray(host, dtype=np.float32)
        _lib.check(self.lib.b200_model_kv_upload(self._h, buffer, host.ctypes.data, pos0, n_pos))

    def kv_download(self, buffer: int, pos0: int = 0, n_pos=None) -> np.ndarray:
        c = self.cfg
        host = np.zeros((c.kv_heads, c.max_len, c.head_dim), dtype=np.float32)
        n = c.max_len - pos0 if n_pos is None else n_pos
        _lib.check(self.lib.b200_model_kv_download(self._h, buffer, host.ctypes.data, pos0, n))
        return host


def run_generation(session: ModelSession, prompt_tokens, max_new_tokens: int,
                   stop_token_ids=()):
    """runGeneration (runtime/llm/TextGeneration.cpp:157-277), greedy, ids only.
    Returns (generated ids, decode tokens/s measured like TextGeneration.cpp:239-245)."""
    keep = session.cfg.max_len // 4
    session.reset_position()
    session.prefill(prompt_tokens)
    tok = greedy_sample(session.logits_data())
    out = [tok]
    if tok in stop_token_ids:
        return out, 0.0
    max_steps = max_new_tokens - len(prompt_tokens) if max_new_tokens > 0 else 1 << 30
    accum, count = 0.0, 0
    for _ in range(max_steps):
        if session.position() >= session.cfg.max_len:
            session.handle_kv_cache_overflow(keep, 10000.0)
        t0 = time.perf_counter()
        session.decode(tok)
        accum += time.perf_counter() - t0
        count += 1
        tok = greedy_sample(session.logits_data())
        if tok in stop_token_ids:
            break
        out.append(tok)
    return out, (count / accum if accum > 0 else 0.0)


class BatchSession:
    """Many sequences of different lengths over one model and a paged KV cache
    (b200_batch_*): prefill a prompt per sequence, then advance any subset of
    them by one token per step.  Not part of buddy-mlir's interface (its
    sessions are single-sequence); per sequence the results are those of
    ModelSession."""

    def __init__(self, model: ModelSession, max_seqs: int, page_size: int, n_pages: int, max_context: int):
        self.model, self.lib = model, model.lib
        self._h = C.c_void_p()
        _lib.check(self.lib.b200_batch_create(model._h, max_seqs, page_size, n_pages, max_context, C.byref(self._h)))

    def close(self):
        if self._h:
            self.lib.b200_batch_destroy(self._h)
            self._h = C.c_void_p()

    def add(self) -> int:
        s = C.c_int()
        _lib.check(self.lib.b200_batch_add(self._h, C.byref(s)))
        return s.value

    def remove(self, seq: int):
        _lib.check(self.lib.b200_batch_remove(self._h, seq))

    def length(self, seq: int) -> int:
        return int(self.lib.b200_batch_length(self._h, seq))

    def free_pages(self) -> int:
        return int(self.lib.b200_batch_free_pages(self._h))

    def prefill(self, seq: int, tokens, want_logits=True):
        toks = np.ascontiguousarray(tokens, dtype=np.int32)
        out = np.zeros(self.model.cfg.vocab, dtype=np.float32) if want_logits else None
        nxt = C.c_int()
        _lib.check(self.lib.b200_batch_prefill(self._h, seq, toks.ctypes.data, toks.size,
                                               out.ctypes.data if want_logits else None, C.byref(nxt)))
        return out, nxt.value

    def decode(self, seqs, tokens, want_logits=True):
        sq = np.ascontiguousarray(seqs, dtype=np.int32)
        tk = np.ascontiguousarray(tokens, dtype=np.int32)
        n = sq.size
        out = np.zeros((n, self.model.cfg.vocab), dtype=np.float32) if want_logits else None
        nxt = np.zeros(n, dtype=np.int32)
        _lib.check(self.lib.b200_batch_decode(self._h, n, sq.ctypes.data, tk.ctypes.data,
                                              out.ctypes.data if want_logits else None, nxt.ctypes.data))
        return out, nxt

    def last_ms(self) -> float:
        return float(self.lib.b200_batch_last_ms(self._h))
