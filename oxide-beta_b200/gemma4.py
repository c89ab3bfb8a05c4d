"""Host-side mirror of the reference's Gemma4 API over the C ABI (include/oxg4.h).

Names, argument meaning and error behaviour follow the reference so that callers and tests read
like the reference's own:
  Device                    crates/oxide-torch/src/tensor/graph.rs:7-12
  GenerationConfig          crates/oxide-torch-models/src/models/gemma4/config.rs:7-33
  Gemma4TextConfig          .../models/gemma4/config.rs:103-208
  Gemma4ForCausalLM         .../models/gemma4/model.rs:35-254, generation.rs:36-141
  Gemma4CudaState           .../gemma4_cuda/mod.rs:161-175, decode.rs:431-486,666-783
  Gemma4CudaCacheTable      .../gemma4_cuda/mod.rs:119-159, cache.rs:31-95
  sample_token, sample_topk_candidates   .../models/gemma4/sampling.rs:9-158
Every compute call goes to the CUDA library; nothing here computes on the CPU except `embed`
(a CPU helper in the reference as well, model.rs:184-213).
"""
import ctypes as C
import dataclasses
import json
from typing import Callable, Iterable, List, Optional, Sequence

import numpy as np

from . import _native as N
from . import synthetic
from ._native import Oxg4Error


class Device:
    """Device::{Cpu, Cuda(usize)}."""

    def __init__(self, kind: str, index: int = 0):
        self.kind, self.index = kind, index

    @staticmethod
    def Cpu():
        return Device("cpu")

    @staticmethod
    def Cuda(index: int = 0):
        return Device("cuda", index)

    def is_cuda(self):
        return self.kind == "cuda"

    def __repr__(self):
        return "Device::Cpu" if self.kind == "cpu" else f"Device::Cuda({self.index})"


@dataclasses.dataclass
class GenerationConfig:
    max_new_tokens: int = 128
    temperature: float = 1.0
    top_k: int = 64
    top_p: float = 0.95
    eos_token_ids: List[int] = dataclasses.field(default_factory=lambda: [1, 50, 106])
    repetition_penalty: float = 1.1
    stop_token_sequences: List[List[int]] = dataclasses.field(default_factory=list)
    seed: int = 0x4D595DF4D0F33173

    @staticmethod
    def greedy(max_new_tokens: int) -> "GenerationConfig":
        """The reference has no greedy flag; this is the equivalent setting."""
        return GenerationConfig(max_new_tokens=max_new_tokens, top_k=1, repetition_penalty=1.0,
                                eos_token_ids=[], temperature=1.0)


class Gemma4TextConfig:
    """Subset of the Hugging Face text config the decode path reads, with the reference's defaults."""

    def __init__(self, d: dict):
        d = dict(d.get("text_config", d))
        self.vocab_size = d.get("vocab_size", 262144)
        self.hidden_size = d.get("hidden_size", 2304)
        self.intermediate_size = d.get("intermediate_size", 9216)
        self.num_hidden_layers = d.get("num_hidden_layers", 30)
        self.num_attention_heads = d.get("num_attention_heads", 8)
        self.num_key_value_heads = d.get("num_key_value_heads", 4)
        self.head_dim = d.get("head_dim", 256)
        self.global_head_dim = d.get("global_head_dim", 512)
        self.sliding_window = d.get("sliding_window", 512)
        self.rms_norm_eps = d.get("rms_norm_eps", 1e-6)
        self.layer_types = d.get("layer_types")
        self.rope_parameters = d.get("rope_parameters")
        self.final_logit_softcapping = d.get("final_logit_softcapping")
        self.hidden_size_per_layer_input = d.get("hidden_size_per_layer_input", 256)
        self.vocab_size_per_layer_input = d.get("vocab_size_per_layer_input", 262144)
        self.num_kv_shared_layers = d.get("num_kv_shared_layers", 0)
        self.attention_k_eq_v = d.get("attention_k_eq_v", False)
        self.num_global_key_value_heads = d.get("num_global_key_value_heads")
        self.tie_word_embeddings = d.get("tie_word_embeddings", True)
        self.finish()

    def finish(self):
        # config.rs:150-207
        if (self.num_attention_heads == 0 or self.num_key_value_heads == 0
                or self.num_attention_heads % self.num_key_value_heads != 0
                or self.hidden_size == 0 or self.num_hidden_layers == 0):
            raise Oxg4Error(N.OK + 1, "invalid Gemma 4 attention configuration")
        if self.layer_types is None:
            L = self.num_hidden_layers
            self.layer_types = ["full_attention" if ((i + 1) % 6 == 0 or i + 1 == L) else "sliding_attention"
                                for i in range(L)]
        if len(self.layer_types) != self.num_hidden_layers:
            raise Oxg4Error(1, "Gemma 4 layer_types length does not match num_hidden_layers")
        if self.rope_parameters is None:
            self.rope_parameters = {
                "sliding_attention": {"rope_theta": 10000.0, "rope_type": "default",
                                      "partial_rotary_factor": 1.0, "factor": 1.0},
                "full_attention": {"rope_theta": 1000000.0, "rope_type": "proportional",
                                   "partial_rotary_factor": 0.25, "factor": 1.0}}

    def to_dict(self) -> dict:
        return {k: v for k, v in self.__dict__.items()}


def _as_u32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint32)


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _native_config(config: "Gemma4TextConfig", weight_dtype: int, norm_weight_offset: int, tp_rank: int, tp_size: int):
    """oxg4_config for `config` plus the arrays it points into (keep them alive while it is used)."""
    L = config.num_hidden_layers
    sliding = np.array([1 if t == "sliding_attention" else 0 for t in config.layer_types], dtype=np.int32)
    rot = np.zeros(L, dtype=np.int32)
    theta = np.zeros(L, dtype=np.float32)
    factor = np.zeros(L, dtype=np.float32)
    for l, t in enumerate(config.layer_types):
        rp = config.rope_parameters.get(t)
        if rp is None:
            raise Oxg4Error(2, f"RoPE parameters for {t} missing")
        hd = config.head_dim if sliding[l] else config.global_head_dim
        # mod.rs:404-405: rotary_dim = (partial_rotary_factor * head_dim as f32) as usize
        rot[l] = int(np.float32(rp.get("partial_rotary_factor", 1.0)) * np.float32(hd))
        theta[l] = rp.get("rope_theta", 10000.0)
        factor[l] = rp.get("factor", 1.0)
    c = N.Config(
        config.vocab_size, config.hidden_size, L, config.num_attention_heads, config.num_key_value_heads,
        config.head_dim, config.global_head_dim, config.intermediate_size, config.sliding_window,
        config.rms_norm_eps, float(config.final_logit_softcapping or 0.0), weight_dtype, norm_weight_offset,
        sliding.ctypes.data_as(C.POINTER(C.c_int32)), rot.ctypes.data_as(C.POINTER(C.c_int32)),
        theta.ctypes.data_as(C.POINTER(C.c_float)), factor.ctypes.data_as(C.POINTER(C.c_float)),
        tp_rank, tp_size, int(config.num_global_key_value_heads or 0), int(bool(config.attention_k_eq_v)),
        int(config.num_kv_shared_layers or 0), int(config.hidden_size_per_layer_input or 0),
        int(config.vocab_size_per_layer_input or 0))
    return c, (sliding, rot, theta, factor)


class Gemma4CudaCacheTable:
    """Owner of an oxg4_cache handle: KV pages, device decode state and the captured step graphs."""

    def __init__(self, state: "Gemma4CudaState", max_sequence, batch: int = 1, page_tokens: int = 256,
                 kv_dtype: int = N.F32):
        ms = np.ascontiguousarray(np.broadcast_to(np.asarray(max_sequence, dtype=np.int32), (batch,)))
        self._state = state
        self.batch = batch
        self._h = C.c_void_p()
        N.check(N.lib().oxg4_cache_create(state._h, batch, ms.ctypes.data_as(C.POINTER(C.c_int32)),
                                          page_tokens, kv_dtype, C.byref(self._h)))

    def __del__(self):
        self.close()

    def close(self):
        # Finalisers of objects caught in a reference cycle run in no particular order. If the state went first,
        # oxg4_model_destroy has already destroyed this table with it: only forget the handle.
        if getattr(self, "_h", None) and self._h.value:
            st = getattr(self, "_state", None)
            if st is not None and getattr(st, "_h", None) and st._h.value:
                N.lib().oxg4_cache_destroy(self._h)
            self._h = C.c_void_p()

    def _info(self) -> N.CacheInfo:
        info = N.CacheInfo()
        N.check(N.lib().oxg4_cache_info_get(self._h, C.byref(info)))
        return info

    def layer_count(self):
        return self._info().layer_count

    def physical_cache_count(self):
        return self._info().physical_cache_count

    def shared_layer_count(self):
        return self._info().shared_layer_count

    def source_layer(self, layer: int):
        return layer if 0 <= layer < self.layer_count() else None

    def kv_bytes(self):
        return self._info().kv_bytes

    def position(self, b: int = 0):
        return N.lib().oxg4_cache_position(self._h, b)

    def reset(self):
        N.check(N.lib().oxg4_cache_reset(self._h))

    def fill_synthetic(self, lens: Sequence[int]):
        """Measurement aid: marks lens[b] positions per sequence as cached and fills the K/V pools with a fixed
        pseudo-random pattern (timing only; the contents are not the K/V of any prompt)."""
        a = np.ascontiguousarray(lens, dtype=np.int32)
        N.check(N.lib().oxg4_debug_fill_cache(self._state._h, self._h, a.ctypes.data_as(C.POINTER(C.c_int32))))

    def tp_export(self) -> bytes:
        """64-byte CUDA IPC handle of this table's tensor-parallel exchange block."""
        buf = C.create_string_buffer(64)
        N.check(N.lib().oxg4_cache_tp_export(self._h, buf))
        return buf.raw

    def tp_connect(self, handles: Sequence[bytes]):
        """`handles`: every rank's tp_export() result, in rank order."""
        blob = b"".join(handles)
        N.check(N.lib().oxg4_cache_tp_connect(self._h, C.c_char_p(blob)))


class Gemma4CudaState:
    """Owner of an oxg4_model handle (persistent device weights + decode plan)."""

    def __init__(self, config: Gemma4TextConfig, device_index: int = 0, weight_dtype: int = N.BF16,
                 norm_weight_offset: int = 0, tp_rank: int = 0, tp_size: int = 1):
        self.config = config
        c, self._keep = _native_config(config, weight_dtype, norm_weight_offset, tp_rank, tp_size)
        self._h = C.c_void_p()
        self.weight_dtype = weight_dtype
        N.check(N.lib().oxg4_model_create(C.byref(c), device_index, C.byref(self._h)))

    @classmethod
    def load(cls, config: Gemma4TextConfig, weights: Iterable, device_index: int = 0,
             weight_dtype: int = N.BF16, **kw) -> "Gemma4CudaState":
        """Gemma4CudaState::load: upload every tensor, fuse QKV, build the decode plan.
        `weights` yields (name, array); uint16 arrays are BF16 bit patterns."""
        st = cls(config, device_index, weight_dtype, **kw)
        for name, a in weights:
            st.upload(name, a)
        st.finalize()
        return st

    @staticmethod
    def tp_unique_id() -> bytes:
        """128-byte NCCL id created on one rank; the caller distributes it to the others."""
        buf = C.create_string_buffer(128)
        N.check(N.lib().oxg4_tp_unique_id(buf))
        return buf.raw

    def tp_init(self, unique_id: bytes):
        N.check(N.lib().oxg4_model_tp_init(self._h, C.c_char_p(unique_id)))

    def upload(self, name: str, array):
        a = np.ascontiguousarray(array)
        if a.dtype == np.uint16:
            dt = N.BF16
        elif a.dtype == np.float32:
            dt = N.F32
        else:
            raise Oxg4Error(2, f"CUDA tensor `{name}` must be BF16 or F32")
        shape = (C.c_int64 * a.ndim)(*a.shape)
        N.check(N.lib().oxg4_model_upload(self._h, name.encode(), dt, shape, a.ndim, _ptr(a), a.nbytes))

    def finalize(self):
        N.check(N.lib().oxg4_model_finalize(self._h))

    def __del__(self):
        self.close()

    def close(self):
        if getattr(self, "_h", None) and self._h.value:
            N.lib().oxg4_model_destroy(self._h)
            self._h = C.c_void_p()

    def weight_count(self):
        return N.lib().oxg4_weight_count(self._h)

    def weight_bytes(self):
        return N.lib().oxg4_weight_bytes(self._h)

    def synchronize(self):
        N.check(N.lib().oxg4_synchronize(self._h))

    def kernel_launches(self):
        return N.lib().oxg4_kernel_launches(self._h)

    def new_cache_table(self, config=None, max_sequence=None, batch: int = 1, page_tokens: int = 256,
                        kv_dtype: int = N.F32) -> Gemma4CudaCacheTable:
        """The default KV element type is f32, the reference's ring (cache_write_f32_state);
        BF16 pages (half the bytes per step, rounded once at append) are an explicit opt-in."""
        if max_sequence is None:               # allow new_cache_table(max_sequence)
            config, max_sequence = None, config
        return Gemma4CudaCacheTable(self, max_sequence, batch, page_tokens, kv_dtype)

    # ---- steps ------------------------------------------------------------------------------
    def prefill_prompt(self, tokens, table: Gemma4CudaCacheTable, lens=None, want_logits=True):
        """prefill_prompt: returns the final-token logits ([vocab] for batch 1, else [batch, vocab])."""
        t = _as_u32(tokens).reshape(-1)
        if lens is None:
            if table.batch != 1:
                raise Oxg4Error(2, "lens is required for batched prefill")
            lens = [t.size]
        ln = np.ascontiguousarray(lens, dtype=np.int32)
        if t.size == 0 or (ln <= 0).any():
            raise Oxg4Error(2, "batched prefill requires at least one token per sequence")
        V = self.config.vocab_size
        out = np.empty((table.batch, V), dtype=np.float32) if want_logits else None
        N.check(N.lib().oxg4_prefill(self._h, table._h, _ptr(t), _ptr(ln), None if out is None else _ptr(out)))
        if out is None:
            return None
        return out[0] if table.batch == 1 else out

    def prefill_token(self, token, table: Gemma4CudaCacheTable):
        t = _as_u32(np.atleast_1d(token))
        N.check(N.lib().oxg4_prefill_token(self._h, table._h, _ptr(t)))

    def decode_token(self, token, table: Gemma4CudaCacheTable):
        t = _as_u32(np.atleast_1d(token))
        out = np.empty((table.batch, self.config.vocab_size), dtype=np.float32)
        N.check(N.lib().oxg4_decode_logits(self._h, table._h, _ptr(t), _ptr(out)))
        return out[0] if table.batch == 1 else out

    def decode_topk(self, token, table: Gemma4CudaCacheTable, top_k: int, repetition_penalty: float,
                    mark_seen: bool):
        """Returns [(id, score), ...] in descending order for batch 1, else (ids, scores) arrays."""
        t = _as_u32(np.atleast_1d(token))
        k = min(max(int(top_k), 1), 64, self.config.vocab_size)
        ids = np.zeros((table.batch, k), dtype=np.uint32)
        scores = np.zeros((table.batch, k), dtype=np.float32)
        N.check(N.lib().oxg4_decode_topk(self._h, table._h, _ptr(t), k, float(repetition_penalty),
                                         int(bool(mark_seen)), _ptr(ids), _ptr(scores)))
        if table.batch == 1:
            return [(int(i), float(s)) for i, s in zip(ids[0], scores[0])]
        return ids, scores

    def decode_trace(self, token, table: Gemma4CudaCacheTable, inject=None, want_logits=True):
        """One eager step; returns (trace [layers + 1, batch, hidden], logits [batch, vocab] or None).
        `inject` [layers, batch, hidden] replaces the input hidden state of every layer."""
        t = _as_u32(np.atleast_1d(token))
        L, H, B = self.config.num_hidden_layers, self.config.hidden_size, table.batch
        trace = np.empty((L + 1, B, H), dtype=np.float32)
        logits = np.empty((B, self.config.vocab_size), dtype=np.float32) if want_logits else None
        inj = None if inject is None else np.ascontiguousarray(inject, dtype=np.float32).reshape(L, B, H)
        N.check(N.lib().oxg4_decode_trace(self._h, table._h, _ptr(t), None if inj is None else _ptr(inj),
                                          _ptr(trace), None if logits is None else _ptr(logits)))
        return trace, logits

    # ---- the reference's diagnostic entry points (gemma4_cuda/smoke.rs) ----
    def embedding_logits(self, token: int) -> np.ndarray:
        out = np.empty(self.config.vocab_size, dtype=np.float32)
        N.check(N.lib().oxg4_smoke_embedding_logits(self._h, int(token), out.ctypes.data_as(C.c_void_p)))
        return out

    def decoder_mlp_smoke(self, token: int, layer: int) -> np.ndarray:
        out = np.empty(self.config.hidden_size, dtype=np.float32)
        N.check(N.lib().oxg4_smoke_decoder_mlp(self._h, int(token), int(layer), out.ctypes.data_as(C.c_void_p)))
        return out

    def decoder_attention_smoke(self, token: int, layer: int) -> np.ndarray:
        out = np.empty(self.config.hidden_size, dtype=np.float32)
        N.check(N.lib().oxg4_smoke_decoder_attention(self._h, int(token), int(layer), out.ctypes.data_as(C.c_void_p)))
        return out

    def cached_attention_smoke(self, token: int, layer: int, table: Gemma4CudaCacheTable) -> np.ndarray:
        sliding = self.config.layer_types[layer] == "sliding_attention"
        d = self.config.head_dim if sliding else self.config.global_head_dim
        out = np.empty(self.config.num_attention_heads * d, dtype=np.float32)
        N.check(N.lib().oxg4_smoke_cached_attention(self._h, table._h, int(token), int(layer), out.ctypes.data_as(C.c_void_p)))
        return out

    def decode_greedy(self, first_tokens, table: Gemma4CudaCacheTable, steps: int):
        """Device-resident greedy loop: returns (ids [steps, batch], mean device ms per step)."""
        t = _as_u32(np.atleast_1d(first_tokens))
        out = np.zeros((steps, table.batch), dtype=np.uint32)
        ms = C.c_float(0)
        N.check(N.lib().oxg4_decode_greedy(self._h, table._h, _ptr(t), steps, _ptr(out), C.byref(ms)))
        return out, ms.value

    def decode_sampled(self, first_tokens, table: Gemma4CudaCacheTable, steps: int, top_k: int, temperature: float,
                       top_p: float, repetition_penalty: float, seeds):
        """Device-resident sampled loop: returns (ids [steps, batch], generator states after the last
        draw [batch], mean device ms per step). `seeds`: one xorshift64 state per sequence."""
        t = _as_u32(np.atleast_1d(first_tokens))
        s = np.ascontiguousarray(np.atleast_1d(seeds), dtype=np.uint64).copy()
        if s.size != table.batch:
            raise ValueError("one generator state per sequence is required")
        out = np.zeros((steps, table.batch), dtype=np.uint32)
        ms = C.c_float(0)
        N.check(N.lib().oxg4_decode_sampled(self._h, table._h, _ptr(t), steps, top_k, temperature, top_p,
                                            repetition_penalty, _ptr(s), _ptr(out), C.byref(ms)))
        return out, s, ms.value

    PROFILE_KINDS = ["qkv", "qkv_post", "attn", "attn_merge", "o", "gateup", "down", "lmhead", "norm", "geglu", "sum",
                     "topk1", "topk2", "tp_pick", "allreduce", "allgather", "step_begin", "step_end"]

    def profile_step(self, tokens, table: Gemma4CudaCacheTable, totals: bool = False) -> dict:
        """One eager step with CUDA events around every kernel and collective. Returns the mean ms per
        launch of every kind that ran, or with `totals` the ms per STEP of every kind (mean x launches)."""
        t = _as_u32(np.atleast_1d(tokens))
        N.check(N.lib().oxg4_profile_step(self._h, table._h, _ptr(t)))
        out = {}
        for k in self.PROFILE_KINDS:
            n = N.lib().oxg4_profile_count(self._h, k.encode())
            if n > 0:
                ms = N.lib().oxg4_profile_ms(self._h, k.encode())
                out[k] = ms * n if totals else ms
        return out


class Gemma4TpCacheTable:
    """Cache tables of every rank of a Gemma4TpState (oxg4_tp_cache)."""

    def __init__(self, state: "Gemma4TpState", max_sequence, batch: int = 1, page_tokens: int = 256,
                 kv_dtype: int = N.F32):
        ms = np.ascontiguousarray(np.broadcast_to(np.asarray(max_sequence, dtype=np.int32), (batch,)))
        self._state = state
        self.batch = batch
        self._h = C.c_void_p()
        N.check(N.lib().oxg4_tp_cache_create(state._h, batch, ms.ctypes.data_as(C.POINTER(C.c_int32)), page_tokens,
                                             kv_dtype, C.byref(self._h)))

    def __del__(self):
        self.close()

    def close(self):
        if getattr(self, "_h", None) and self._h.value:
            st = getattr(self, "_state", None)
            if st is not None and getattr(st, "_h", None) and st._h.value:
                N.lib().oxg4_tp_cache_destroy(self._h)
            self._h = C.c_void_p()

    def position(self, b: int = 0):
        return N.lib().oxg4_tp_cache_position(self._h, b)


class Gemma4TpState:
    """A tensor-parallel Gemma4CudaState driven by ONE host thread (oxg4_tp_model): one model per device in
    `device_ordinals`, worker threads inside the library. Same calls as Gemma4CudaState."""

    def __init__(self, config: Gemma4TextConfig, device_ordinals: Sequence[int], weight_dtype: int = N.BF16,
                 norm_weight_offset: int = 0):
        self.config = config
        c, self._keep = _native_config(config, weight_dtype, norm_weight_offset, 0, len(device_ordinals))
        dev = np.ascontiguousarray(device_ordinals, dtype=np.int32)
        self._h = C.c_void_p()
        N.check(N.lib().oxg4_tp_model_create(C.byref(c), dev.ctypes.data_as(C.POINTER(C.c_int32)), dev.size,
                                             C.byref(self._h)))

    @classmethod
    def load(cls, config: Gemma4TextConfig, weights: Iterable, device_ordinals: Sequence[int],
             weight_dtype: int = N.BF16, **kw) -> "Gemma4TpState":
        st = cls(config, device_ordinals, weight_dtype, **kw)
        for name, a in weights:
            st.upload(name, a)
        st.finalize()
        return st

    def upload(self, name: str, array):
        a = np.ascontiguousarray(array)
        dt = N.BF16 if a.dtype == np.uint16 else N.F32
        shape = (C.c_int64 * a.ndim)(*a.shape)
        N.check(N.lib().oxg4_tp_model_upload(self._h, name.encode(), dt, shape, a.ndim, _ptr(a), a.nbytes))

    def finalize(self):
        N.check(N.lib().oxg4_tp_model_finalize(self._h))

    def __del__(self):
        self.close()

    def close(self):
        if getattr(self, "_h", None) and self._h.value:
            N.lib().oxg4_tp_model_destroy(self._h)
            self._h = C.c_void_p()

    def weight_bytes(self):
        return N.lib().oxg4_tp_weight_bytes(self._h)

    def new_cache_table(self, max_sequence, batch: int = 1, page_tokens: int = 256, kv_dtype: int = N.F32):
        return Gemma4TpCacheTable(self, max_sequence, batch, page_tokens, kv_dtype)

    def prefill_prompt(self, tokens, table: Gemma4TpCacheTable, lens=None, want_logits=True):
        t = _as_u32(tokens).reshape(-1)
        ln = np.ascontiguousarray([t.size] if lens is None else lens, dtype=np.int32)
        out = np.empty((table.batch, self.config.vocab_size), dtype=np.float32) if want_logits else None
        N.check(N.lib().oxg4_tp_prefill(self._h, table._h, _ptr(t), _ptr(ln), None if out is None else _ptr(out)))
        if out is None:
            return None
        return out[0] if table.batch == 1 else out

    def decode_token(self, token, table: Gemma4TpCacheTable):
        t = _as_u32(np.atleast_1d(token))
        out = np.empty((table.batch, self.config.vocab_size), dtype=np.float32)
        N.check(N.lib().oxg4_tp_decode_logits(self._h, table._h, _ptr(t), _ptr(out)))
        return out[0] if table.batch == 1 else out

    def decode_topk(self, token, table: Gemma4TpCacheTable, top_k: int, repetition_penalty: float, mark_seen: bool):
        t = _as_u32(np.atleast_1d(token))
        k = min(max(int(top_k), 1), 64, self.config.vocab_size)
        ids = np.zeros((table.batch, k), dtype=np.uint32)
        scores = np.zeros((table.batch, k), dtype=np.float32)
        N.check(N.lib().oxg4_tp_decode_topk(self._h, table._h, _ptr(t), k, float(repetition_penalty),
                                            int(bool(mark_seen)), _ptr(ids), _ptr(scores)))
        if table.batch == 1:
            return [(int(i), float(s)) for i, s in zip(ids[0], scores[0])]
        return ids, scores

    def decode_greedy(self, first_tokens, table: Gemma4TpCacheTable, steps: int):
        t = _as_u32(np.atleast_1d(first_tokens))
        out = np.zeros((steps, table.batch), dtype=np.uint32)
        ms = C.c_float(0)
        N.check(N.lib().oxg4_tp_decode_greedy(self._h, table._h, _ptr(t), steps, _ptr(out), C.byref(ms)))
        return out, ms.value


def tp_shard(name: str, rows: int, cols: int, tp_rank: int, tp_size: int, cfg: "Gemma4TextConfig"):
    """(row0, nrows, col0, ncols) of the slice a tensor-parallel rank keeps of a checkpoint tensor."""
    out = (C.c_int64 * 4)()
    N.check(N.lib().oxg4_tp_shard(name.encode(), rows, cols, tp_rank, tp_size, cfg.num_attention_heads,
                                  cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size, out))
    return tuple(out)


def sample_token(logits, config: GenerationConfig, random: np.ndarray) -> int:
    """sampling.rs:9-79; `random` is a one-element uint64 array holding the xorshift state."""
    a = np.ascontiguousarray(logits, dtype=np.float32)
    r = N.lib().oxg4_sample_token(_ptr(a), a.size, config.temperature, config.top_k, config.top_p,
                                  random.ctypes.data_as(C.POINTER(C.c_uint64)))
    if r < 0:
        raise Oxg4Error(2, "invalid sampling input")
    return int(r)


def sample_topk_candidates(candidates: Sequence, config: GenerationConfig, random: np.ndarray) -> int:
    ids = np.ascontiguousarray([c[0] for c in candidates], dtype=np.uint32)
    sc = np.ascontiguousarray([c[1] for c in candidates], dtype=np.float32)
    r = N.lib().oxg4_sample_topk_candidates(_ptr(ids), _ptr(sc), ids.size, config.temperature, config.top_p,
                                            random.ctypes.data_as(C.POINTER(C.c_uint64)))
    if r < 0:
        raise Oxg4Error(2, "invalid candidate sampling input")
    return int(r)


class Gemma4ForCausalLM:
    """Checkpoint adapter + generate loop (model.rs:35-254, generation.rs:36-141)."""

    def __init__(self, config: Gemma4TextConfig, weights: dict, device: Device, weight_dtype: int,
                 checkpoint_directory: Optional[str] = None, kv_dtype: Optional[int] = None):
        self._config = config
        self._weights = weights
        self._device = device
        self._weight_dtype = weight_dtype
        self._kv_dtype = kv_dtype if kv_dtype is not None else N.F32     # the reference's cache is f32
        self._dir = checkpoint_directory
        self._cuda: Optional[Gemma4CudaState] = None
        self._validate_checkpoint()

    @classmethod
    def from_pretrained(cls, directory: str, device: Device, kv_dtype: Optional[int] = None):
        cfg_dict, weights = synthetic.read_checkpoint(directory)
        config = Gemma4TextConfig(cfg_dict)
        first = next(iter(weights.values()))
        dt = N.BF16 if first.dtype == np.uint16 else N.F32
        return cls(config, weights, device, dt, directory, kv_dtype)

    @classmethod
    def from_weights(cls, cfg: dict, weights: dict, device: Device, kv_dtype: Optional[int] = None):
        first = next(iter(weights.values()))
        dt = N.BF16 if first.dtype == np.uint16 else N.F32
        return cls(Gemma4TextConfig(cfg), weights, device, dt, None, kv_dtype)

    def _validate_checkpoint(self):
        # model.rs:215-233
        need = ["embed_tokens.weight", "norm.weight"]
        for l in range(self._config.num_hidden_layers):
            for n in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm",
                      "post_feedforward_layernorm"):
                need.append(f"layers.{l}.{n}.weight")
        for n in need:
            if n not in self._weights:
                raise Oxg4Error(2, f"checkpoint is missing `{n}`")

    def config(self):
        return self._config

    def device(self):
        return self._device

    def checkpoint_directory(self):
        return self._dir

    def weight(self, name: str):
        return self._weights[name]

    def embed(self, input_ids) -> np.ndarray:
        """CPU helper (model.rs:184-213): embedding rows widened to f32, times sqrt(hidden)."""
        ids = np.asarray(input_ids, dtype=np.int64)
        if ids.size and ids.max() >= self._config.vocab_size:
            raise Oxg4Error(2, "token id exceeds embedding vocabulary")
        e = self._weights["embed_tokens.weight"][ids]
        e = synthetic.bf16_bits_to_f32(e) if e.dtype == np.uint16 else np.asarray(e, dtype=np.float32)
        return (e.reshape(ids.size, -1) * np.float32(np.sqrt(np.float32(self._config.hidden_size)))).astype(np.float32)

    def prepare_cuda(self) -> Gemma4CudaState:
        if not self._device.is_cuda():
            raise Oxg4Error(2, "Gemma 4 generate currently requires Device::Cuda")
        return Gemma4CudaState.load(self._config, self._weights.items(), self._device.index, self._weight_dtype)

    def generate(self, input_ids, generation: GenerationConfig) -> List[int]:
        return self._generate_with_callback(input_ids, generation, None)

    def generate_stream(self, input_ids, generation: GenerationConfig, on_token: Callable[[int], None]):
        return self._generate_with_callback(input_ids, generation, on_token)

    def _generate_with_callback(self, input_ids, g: GenerationConfig, on_token):
        if not self._device.is_cuda():
            # generation.rs:82-86 (after validation in the reference; validation happens in the library)
            _validate_generation(g)
            if len(input_ids) == 0:
                raise Oxg4Error(2, "Gemma 4 generation requires at least one input token")
            raise Oxg4Error(2, "Gemma 4 generate currently requires Device::Cuda")
        _validate_generation(g)
        if len(input_ids) == 0:
            raise Oxg4Error(2, "Gemma 4 generation requires at least one input token")
        if self._cuda is None:
            self._cuda = self.prepare_cuda()
        prompt = _as_u32(input_ids)
        eos = _as_u32(g.eos_token_ids)
        flat = _as_u32([t for s in g.stop_token_sequences for t in s])
        lens = np.ascontiguousarray([len(s) for s in g.stop_token_sequences], dtype=np.int64)
        gc = N.GenerationConfigC(
            g.max_new_tokens, g.temperature, g.top_k, g.top_p, g.repetition_penalty, g.seed,
            eos.ctypes.data_as(C.POINTER(C.c_uint32)), eos.size,
            flat.ctypes.data_as(C.POINTER(C.c_uint32)), lens.ctypes.data_as(C.POINTER(C.c_int64)), lens.size)
        failure = []

        def _cb(tok, _user):
            if on_token is None:
                return 0
            try:
                on_token(int(tok))
                return 0
            except Exception as e:      # an Err from on_token aborts generation
                failure.append(e)
                return 1

        cb = N.TOKEN_CALLBACK(_cb)
        out = np.zeros(prompt.size + max(g.max_new_tokens, 0), dtype=np.uint32)
        n_out = C.c_int64(0)
        st = N.lib().oxg4_generate(self._cuda._h, _ptr(prompt), prompt.size, C.byref(gc), self._kv_dtype, cb,
                                   None, _ptr(out), C.byref(n_out))
        if failure:
            raise failure[0]
        N.check(st)
        return [int(t) for t in out[: n_out.value]]


def _validate_generation(g: GenerationConfig):
    # generation.rs:5-34
    if not np.isfinite(g.temperature) or g.temperature <= 0.0:
        raise Oxg4Error(2, "generation temperature must be finite and greater than zero")
    if not np.isfinite(g.top_p) or not (0.0 <= g.top_p <= 1.0):
        raise Oxg4Error(2, "generation top_p must be finite and between zero and one")
    if g.top_k == 0:
        raise Oxg4Error(2, "generation top_k must be greater than zero")
    if not np.isfinite(g.repetition_penalty) or g.repetition_penalty < 1.0:
        raise Oxg4Error(2, "generation repetition_penalty must be finite and at least one")
    if any(len(s) == 0 for s in g.stop_token_sequences):
        raise Oxg4Error(2, "generation stop-token sequences cannot be empty")
