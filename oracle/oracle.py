"""ctypes front-end of the CPU oracle (oracle/gemma4_oracle.cpp).

Test infrastructure only: imported by tests/, by the smoke check and by the benchmark's
cpu-baseline / reference legs. The product package never imports this module.
"""
import ctypes as C
import os

import numpy as np

from .build import build_oracle

_lib = None

F32, REF_BF16 = 0, 1


def lib():
    global _lib
    if _lib is None:
        path = build_oracle()
        L = C.CDLL(path)
        L.orc_f32_to_bf16.restype = C.c_uint16
        L.orc_f32_to_bf16.argtypes = [C.c_float]
        L.orc_bf16_to_f32.restype = C.c_float
        L.orc_bf16_to_f32.argtypes = [C.c_uint16]
        L.orc_gelu_mul.restype = C.c_float
        L.orc_gelu_mul.argtypes = [C.c_float, C.c_float]
        L.orc_model_create.restype = C.c_void_p
        L.orc_cache_create.restype = C.c_void_p
        L.orc_cache_create.argtypes = [C.c_void_p, C.c_int64]
        L.orc_cache_position.restype = C.c_int64
        L.orc_cache_position.argtypes = [C.c_void_p]
        L.orc_sample_token.restype = C.c_int64
        L.orc_sample_topk_candidates.restype = C.c_int64
        L.orc_generate.restype = C.c_int64
        L.orc_num_threads.restype = C.c_int
        _lib = L
    return _lib


def _fp(a):
    return a.ctypes.data_as(C.c_void_p)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Vectorised restatement of kernel_module.rs:1338-1348 (RNE, no NaN special case)."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    bias = np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))
    return ((bits + bias) >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def rms_norm(x, weight, eps, round_out=False):
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, hidden = x.shape
    out = np.empty_like(x)
    w = None if weight is None else np.ascontiguousarray(weight, dtype=np.float32)
    lib().orc_rms_norm(_fp(x), None if w is None else _fp(w), _fp(out), C.c_int(rows),
                       C.c_int(hidden), C.c_float(eps), C.c_int(int(round_out)))
    return out


def rope(x, heads, head_dim, rotary_dim, theta, factor, position):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty_like(x)
    lib().orc_rope(_fp(x), _fp(out), C.c_int(heads), C.c_int(head_dim), C.c_int(rotary_dim),
                   C.c_float(theta), C.c_float(factor), C.c_int64(position))
    return out


def grouped_query_attention(query, key, value, q_len, kv_len, heads, kv_heads, dim, window=None):
    """crates/oxide-torch/src/nn.rs:684-755. Raises ValueError where the reference returns InvalidShape."""
    q = np.ascontiguousarray(query, dtype=np.float32)
    k = np.ascontiguousarray(key, dtype=np.float32)
    v = np.ascontiguousarray(value, dtype=np.float32)
    if (q.size != q_len * heads * dim or k.size != kv_len * kv_heads * dim or v.size != k.size):
        raise ValueError("invalid grouped-query attention shape")
    out = np.zeros(q.size, dtype=np.float32)
    rc = lib().orc_grouped_query_attention(
        _fp(q), _fp(k), _fp(v), C.c_int64(q_len), C.c_int64(kv_len), C.c_int(heads),
        C.c_int(kv_heads), C.c_int(dim), C.c_int64(window or 0), C.c_int(window is not None), _fp(out))
    if rc != 0:
        raise ValueError("invalid grouped-query attention shape")
    return out


class KvCache:
    """models/gemma4/cache.rs:5-69 (CPU per-layer KV state with sliding truncation)."""

    def __init__(self):
        self._k = np.zeros(0, dtype=np.float32)
        self._v = np.zeros(0, dtype=np.float32)
        self._len = 0
        self._row = 0

    def append(self, key, value, kv_heads, positions, head_dim, window=None):
        key = np.ascontiguousarray(key, dtype=np.float32)
        value = np.ascontiguousarray(value, dtype=np.float32)
        row = kv_heads * head_dim
        if self._len != 0 and self._row != row:
            raise ValueError("KV cache dimensions changed")
        kb = np.zeros((self._len + positions) * max(row, 1), dtype=np.float32)
        vb = np.zeros_like(kb)
        kb[: self._k.size] = self._k
        vb[: self._v.size] = self._v
        n = C.c_int64(self._len)
        rc = lib().orc_kvcache_append(
            _fp(kb), _fp(vb), C.byref(n), _fp(key), _fp(value), C.c_int64(key.size),
            C.c_int64(value.size), C.c_int(kv_heads), C.c_int64(positions), C.c_int(head_dim),
            C.c_int64(window or 0), C.c_int(window is not None))
        if rc != 0:
            raise ValueError("invalid KV cache update")
        self._len = n.value
        self._row = row
        self._k = kb[: self._len * row].copy()
        self._v = vb[: self._len * row].copy()

    def sequence_len(self):
        return self._len

    def key(self):
        return self._k

    def value(self):
        return self._v


def topk(logits, top_k, penalty=1.0, seen=None):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    ids = np.zeros(64, dtype=np.uint32)
    scores = np.zeros(64, dtype=np.float32)
    s = None if seen is None else np.ascontiguousarray(seen, dtype=np.uint8)
    lib().orc_topk(_fp(logits), C.c_int64(logits.size), None if s is None else _fp(s),
                   C.c_int(top_k), C.c_float(penalty), _fp(ids), _fp(scores))
    return ids[:top_k].copy(), scores[:top_k].copy()


def sample_token(logits, temperature, top_k, top_p, random_state):
    """sampling.rs:9-79. `random_state` is a one-element uint64 array updated in place."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    r = lib().orc_sample_token(_fp(logits), C.c_int64(logits.size), C.c_float(temperature),
                               C.c_int64(top_k), C.c_float(top_p), _fp(random_state))
    if r < 0:
        raise ValueError("invalid sampling input")
    return int(r)


def sample_topk_candidates(ids, scores, temperature, top_p, random_state):
    ids = np.ascontiguousarray(ids, dtype=np.uint32)
    scores = np.ascontiguousarray(scores, dtype=np.float32)
    r = lib().orc_sample_topk_candidates(_fp(ids), _fp(scores), C.c_int64(ids.size),
                                         C.c_float(temperature), C.c_float(top_p), _fp(random_state))
    if r < 0:
        raise ValueError("invalid candidate sampling input")
    return int(r)


class _GenCfg(C.Structure):
    _fields_ = [("max_new_tokens", C.c_int64), ("temperature", C.c_float), ("top_k", C.c_int64),
                ("top_p", C.c_float), ("repetition_penalty", C.c_float), ("seed", C.c_uint64)]


class OracleModel:
    """Holds weights and runs the restated decode step on the CPU.

    `cfg` is a dict with the keys of a Gemma4 text config (vocab_size, hidden_size,
    num_hidden_layers, num_attention_heads, num_key_value_heads, head_dim, global_head_dim,
    intermediate_size, sliding_window, rms_norm_eps, layer_types, rope_parameters).
    """

    def __init__(self, cfg: dict, mode: int, kv_bf16: bool = False):
        self.cfg = cfg
        self.mode = mode
        L = cfg["num_hidden_layers"]
        types = cfg["layer_types"]
        sliding = np.array([1 if t == "sliding_attention" else 0 for t in types], dtype=np.int32)
        rot = np.zeros(L, dtype=np.int32)
        theta = np.zeros(L, dtype=np.float32)
        factor = np.zeros(L, dtype=np.float32)
        for l, t in enumerate(types):
            rp = cfg["rope_parameters"][t]
            hd = cfg["head_dim"] if sliding[l] else cfg.get("global_head_dim", cfg["head_dim"])
            # gemma4_cuda/mod.rs:404-405: rotary_dim = (partial_rotary_factor * head_dim) as usize
            rot[l] = int(np.float32(rp.get("partial_rotary_factor", 1.0)) * np.float32(hd))
            theta[l] = rp["rope_theta"]
            factor[l] = rp.get("factor", 1.0)
        ints = np.array([cfg["vocab_size"], cfg["hidden_size"], L, cfg["num_attention_heads"],
                         cfg["num_key_value_heads"], cfg["head_dim"],
                         cfg.get("global_head_dim", cfg["head_dim"]), cfg["intermediate_size"],
                         cfg["sliding_window"], mode, int(kv_bf16),
                         int(cfg.get("num_global_key_value_heads") or 0), int(bool(cfg.get("attention_k_eq_v"))),
                         int(cfg.get("num_kv_shared_layers") or 0), int(cfg.get("hidden_size_per_layer_input") or 0),
                         int(cfg.get("vocab_size_per_layer_input") or 0)], dtype=np.int32)
        h = lib().orc_model_create(_fp(ints), C.c_float(cfg["rms_norm_eps"]), _fp(sliding), _fp(rot), _fp(theta),
                                   _fp(factor))
        if not h:
            raise ValueError("shared layer has no preceding KV source")      # cache.rs:76-80
        self._h = C.c_void_p(h)

    def __del__(self):
        if getattr(self, "_h", None):
            lib().orc_model_destroy(self._h)
            self._h = None

    def set_weight(self, name: str, array: np.ndarray):
        """`array` is float32, or uint16 holding BF16 bits. `name` has no checkpoint prefix."""
        a = np.ascontiguousarray(array)
        if a.dtype == np.uint16:
            dtype = 1
        elif a.dtype == np.float32:
            dtype = 0
        else:
            raise TypeError(a.dtype)
        if a.ndim == 2:
            rows, cols = a.shape
        else:
            rows, cols = 1, a.size
        rc = lib().orc_model_set_weight(self._h, name.encode(), C.c_int(dtype), _fp(a),
                                        C.c_int64(rows), C.c_int64(cols))
        if rc != 0:
            raise KeyError(name)

    def load(self, weights: dict):
        for name, array in weights.items():
            self.set_weight(name, array)

    def new_cache(self, max_sequence: int):
        return OracleCache(self, max_sequence)

    # ---- gemma4_cuda/smoke.rs restated (one token through one block of one layer) ----
    def embedding_logits(self, token: int) -> np.ndarray:
        out = np.empty(self.cfg["vocab_size"], dtype=np.float32)
        if lib().orc_smoke_embedding_logits(self._h, C.c_uint32(token), _fp(out)) != 0:
            raise ValueError("token id exceeds vocabulary")
        return out

    def decoder_mlp_smoke(self, token: int, layer: int) -> np.ndarray:
        out = np.empty(self.cfg["hidden_size"], dtype=np.float32)
        if lib().orc_smoke_decoder_mlp(self._h, C.c_uint32(token), C.c_int(layer), _fp(out)) != 0:
            raise ValueError("invalid token or layer")
        return out

    def decoder_attention_smoke(self, token: int, layer: int) -> np.ndarray:
        out = np.empty(self.cfg["hidden_size"], dtype=np.float32)
        if lib().orc_smoke_decoder_attention(self._h, C.c_uint32(token), C.c_int(layer), _fp(out)) != 0:
            raise ValueError("invalid token or layer")
        return out

    def generate(self, prompt, max_new_tokens, temperature=1.0, top_k=1, top_p=0.95,
                 repetition_penalty=1.0, seed=0x4D595DF4D0F33173, eos=(), want_first_logits=False):
        prompt = np.ascontiguousarray(prompt, dtype=np.uint32)
        g = _GenCfg(max_new_tokens, temperature, top_k, top_p, repetition_penalty, seed)
        eos_a = np.ascontiguousarray(list(eos), dtype=np.uint32)
        out = np.zeros(max(max_new_tokens, 1), dtype=np.uint32)
        fl = np.zeros(self.cfg["vocab_size"], dtype=np.float32) if want_first_logits else None
        n = lib().orc_generate(self._h, _fp(prompt), C.c_int64(prompt.size), C.byref(g), _fp(eos_a),
                               C.c_int64(eos_a.size), _fp(out), None if fl is None else _fp(fl))
        if n < 0:
            raise ValueError("invalid generation input")
        toks = out[:n].copy()
        return (toks, fl) if want_first_logits else toks


class OracleCache:
    def __init__(self, model: OracleModel, max_sequence: int):
        self.model = model
        self._h = C.c_void_p(lib().orc_cache_create(model._h, C.c_int64(max_sequence)))

    def __del__(self):
        if getattr(self, "_h", None):
            lib().orc_cache_destroy(self._h)
            self._h = None

    @property
    def position(self):
        return lib().orc_cache_position(self._h)

    def prefill_token(self, token: int):
        if lib().orc_prefill_token(self.model._h, self._h, C.c_uint32(token)) != 0:
            raise ValueError("token id exceeds vocabulary")

    def _softcap(self, values: np.ndarray):
        """gemma4_cuda/mod.rs:573-579: the reference softcaps the scores it hands back to the host."""
        cap = self.model.cfg.get("final_logit_softcapping")
        if cap:
            lib().orc_softcap(_fp(values), C.c_int64(values.size), C.c_float(cap))
        return values

    def cached_attention_smoke(self, token: int, layer: int) -> np.ndarray:
        """gemma4_cuda/smoke.rs:128-204 on this cache: append the token to the layer's ring, attend, advance."""
        cfg = self.model.cfg
        sliding = cfg["layer_types"][layer] == "sliding_attention"
        d = cfg["head_dim"] if sliding else cfg.get("global_head_dim", cfg["head_dim"])
        out = np.empty(cfg["num_attention_heads"] * d, dtype=np.float32)
        if lib().orc_smoke_cached_attention(self.model._h, self._h, C.c_uint32(token), C.c_int(layer), _fp(out)) != 0:
            raise ValueError("invalid token or layer")
        return out

    def decode_logits(self, token: int) -> np.ndarray:
        logits = np.empty(self.model.cfg["vocab_size"], dtype=np.float32)
        if lib().orc_decode_logits(self.model._h, self._h, C.c_uint32(token), _fp(logits)) != 0:
            raise ValueError("token id exceeds vocabulary")
        return self._softcap(logits)

    def decode_trace(self, token: int, inject=None, want_logits=True):
        """One token; returns (trace [layers + 1, hidden], logits). `inject` [layers, hidden] replaces
        the input hidden state of every layer (layer-wise teacher forcing)."""
        cfg = self.model.cfg
        L, H = cfg["num_hidden_layers"], cfg["hidden_size"]
        trace = np.empty((L + 1, H), dtype=np.float32)
        logits = np.empty(cfg["vocab_size"], dtype=np.float32) if want_logits else None
        inj = None if inject is None else np.ascontiguousarray(inject, dtype=np.float32)
        rc = lib().orc_decode_trace(self.model._h, self._h, C.c_uint32(token), None if inj is None else _fp(inj),
                                    _fp(trace), None if logits is None else _fp(logits))
        if rc != 0:
            raise ValueError("token id exceeds vocabulary")
        return trace, logits

    def decode_topk(self, token: int, top_k=1, penalty=1.0, mark_seen=True, want_logits=False):
        ids = np.zeros(64, dtype=np.uint32)
        scores = np.zeros(64, dtype=np.float32)
        logits = np.empty(self.model.cfg["vocab_size"], dtype=np.float32) if want_logits else None
        k = lib().orc_decode_topk(self.model._h, self._h, C.c_uint32(token), C.c_int(top_k),
                                  C.c_float(penalty), C.c_int(int(mark_seen)), _fp(ids), _fp(scores),
                                  None if logits is None else _fp(logits))
        if k < 0:
            raise ValueError("token id exceeds vocabulary")
        if want_logits:
            return ids[:k].copy(), self._softcap(scores[:k].copy()), self._softcap(logits)
        return ids[:k].copy(), self._softcap(scores[:k].copy())


def set_accum_order(order: int):
    """0: default; 1: eight interleaved partial sums; 2: serial from the last element (test aid)."""
    lib().orc_set_accum_order(C.c_int(order))


def set_num_threads(n: int):
    lib().orc_set_num_threads(C.c_int(n))


def num_threads() -> int:
    return lib().orc_num_threads()
