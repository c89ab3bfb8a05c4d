"""ctypes binding of liboxg4.so — the same symbols a Rust `-sys` crate would bind (include/oxg4.h).

There is no fallback: if the shared object is missing it is built with nvcc; if that fails, or a
compute call is made without a CUDA device, an exception is raised.
"""
import ctypes as C
import os

from .build import build_library

OK = 0
F32, BF16 = 0, 1
INACTIVE = 0xFFFFFFFF

STATUS_NAMES = {0: "OK", 1: "INVALID_SHAPE", 2: "INVALID_ARGUMENT", 3: "CUDA", 4: "NCCL", 5: "OOM",
                6: "TIMEOUT", 7: "UNSUPPORTED"}


class Config(C.Structure):
    _fields_ = [
        ("vocab_size", C.c_int32), ("hidden_size", C.c_int32), ("num_hidden_layers", C.c_int32),
        ("num_attention_heads", C.c_int32), ("num_key_value_heads", C.c_int32), ("head_dim", C.c_int32),
        ("global_head_dim", C.c_int32), ("intermediate_size", C.c_int32), ("sliding_window", C.c_int32),
        ("rms_norm_eps", C.c_float), ("final_logit_softcapping", C.c_float), ("weight_dtype", C.c_int32),
        ("norm_weight_offset", C.c_int32), ("layer_is_sliding", C.POINTER(C.c_int32)),
        ("rotary_dim", C.POINTER(C.c_int32)), ("rope_theta", C.POINTER(C.c_float)),
        ("rope_factor", C.POINTER(C.c_float)), ("tp_rank", C.c_int32), ("tp_size", C.c_int32),
        ("num_global_key_value_heads", C.c_int32), ("attention_k_eq_v", C.c_int32),
        ("num_kv_shared_layers", C.c_int32), ("hidden_size_per_layer_input", C.c_int32),
        ("vocab_size_per_layer_input", C.c_int32)]


class CacheInfo(C.Structure):
    _fields_ = [("batch", C.c_int32), ("layer_count", C.c_int32), ("physical_cache_count", C.c_int32),
                ("shared_layer_count", C.c_int32), ("page_tokens", C.c_int32), ("kv_dtype", C.c_int32),
                ("kv_bytes", C.c_int64)]


class GenerationConfigC(C.Structure):
    _fields_ = [("max_new_tokens", C.c_int64), ("temperature", C.c_float), ("top_k", C.c_int64),
                ("top_p", C.c_float), ("repetition_penalty", C.c_float), ("seed", C.c_uint64),
                ("eos_token_ids", C.POINTER(C.c_uint32)), ("n_eos", C.c_int64),
                ("stop_sequences", C.POINTER(C.c_uint32)), ("stop_sequence_lens", C.POINTER(C.c_int64)),
                ("n_stop_sequences", C.c_int64)]


TOKEN_CALLBACK = C.CFUNCTYPE(C.c_int32, C.c_uint32, C.c_void_p)

# every symbol include/oxg4.h declares: name -> (restype, argtypes)
SYMBOLS = {
    "oxg4_last_error": (C.c_char_p, []),
    "oxg4_model_create": (C.c_int32, [C.POINTER(Config), C.c_int32, C.POINTER(C.c_void_p)]),
    "oxg4_model_upload": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_int32, C.POINTER(C.c_int64), C.c_int32,
                                      C.c_void_p, C.c_size_t]),
    "oxg4_model_finalize": (C.c_int32, [C.c_void_p]),
    "oxg4_model_destroy": (None, [C.c_void_p]),
    "oxg4_weight_count": (C.c_int64, [C.c_void_p]),
    "oxg4_weight_bytes": (C.c_int64, [C.c_void_p]),
    "oxg4_synchronize": (C.c_int32, [C.c_void_p]),
    "oxg4_tp_unique_id": (C.c_int32, [C.c_void_p]),
    "oxg4_tp_shard": (C.c_int32, [C.c_char_p, C.c_int64, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                  C.c_int32, C.POINTER(C.c_int64)]),
    "oxg4_model_tp_init": (C.c_int32, [C.c_void_p, C.c_void_p]),
    "oxg4_tp_model_create": (C.c_int32, [C.POINTER(Config), C.POINTER(C.c_int32), C.c_int32, C.POINTER(C.c_void_p)]),
    "oxg4_tp_model_upload": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_int32, C.POINTER(C.c_int64), C.c_int32,
                                         C.c_void_p, C.c_size_t]),
    "oxg4_tp_model_finalize": (C.c_int32, [C.c_void_p]),
    "oxg4_tp_model_destroy": (None, [C.c_void_p]),
    "oxg4_tp_weight_bytes": (C.c_int64, [C.c_void_p]),
    "oxg4_tp_cache_create": (C.c_int32, [C.c_void_p, C.c_int32, C.POINTER(C.c_int32), C.c_int32, C.c_int32,
                                         C.POINTER(C.c_void_p)]),
    "oxg4_tp_cache_destroy": (None, [C.c_void_p]),
    "oxg4_tp_cache_position": (C.c_int32, [C.c_void_p, C.c_int32]),
    "oxg4_tp_prefill": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "oxg4_tp_decode_logits": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "oxg4_tp_decode_topk": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_float, C.c_int32,
                                        C.c_void_p, C.c_void_p]),
    "oxg4_tp_decode_greedy": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p,
                                          C.POINTER(C.c_float)]),
    "oxg4_cache_tp_export": (C.c_int32, [C.c_void_p, C.c_void_p]),
    "oxg4_cache_tp_connect": (C.c_int32, [C.c_void_p, C.c_void_p]),
    "oxg4_cache_create": (C.c_int32, [C.c_void_p, C.c_int32, C.POINTER(C.c_int32), C.c_int32, C.c_int32,
                                      C.POINTER(C.c_void_p)]),
    "oxg4_cache_destroy": (None, [C.c_void_p]),
    "oxg4_cache_info_get": (C.c_int32, [C.c_void_p, C.POINTER(CacheInfo)]),
    "oxg4_cache_position": (C.c_int32, [C.c_void_p, C.c_int32]),
    "oxg4_cache_reset": (C.c_int32, [C.c_void_p]),
    "oxg4_prefill": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "oxg4_prefill_token": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "oxg4_decode_logits": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "oxg4_decode_topk": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_float, C.c_int32,
                                     C.c_void_p, C.c_void_p]),
    "oxg4_decode_sampled": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_float,
                                        C.c_float, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p]),
    "oxg4_decode_greedy": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p,
                                       C.POINTER(C.c_float)]),
    "oxg4_kernel_launches": (C.c_int64, [C.c_void_p]),
    "oxg4_profile_step": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "oxg4_profile_ms": (C.c_float, [C.c_void_p, C.c_char_p]),
    "oxg4_profile_count": (C.c_int32, [C.c_void_p, C.c_char_p]),
    "oxg4_debug_wait_timeout": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_uint32]),
    "oxg4_debug_fail_alloc_after": (None, [C.c_int32]),
    "oxg4_smoke_embedding_logits": (C.c_int32, [C.c_void_p, C.c_uint32, C.c_void_p]),
    "oxg4_smoke_decoder_mlp": (C.c_int32, [C.c_void_p, C.c_uint32, C.c_int32, C.c_void_p]),
    "oxg4_smoke_decoder_attention": (C.c_int32, [C.c_void_p, C.c_uint32, C.c_int32, C.c_void_p]),
    "oxg4_smoke_cached_attention": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_int32, C.c_void_p]),
    "oxg4_debug_fill_cache": (C.c_int32, [C.c_void_p, C.c_void_p, C.POINTER(C.c_int32)]),
    "oxg4_topk_noalloc": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_float, C.c_int32, C.c_void_p,
                                      C.c_void_p, C.c_void_p]),
    "oxg4_decode_trace": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "oxg4_debug_tc_gemm": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                                       C.POINTER(C.c_float)]),
    "oxg4_debug_timeline": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32]),
    "oxg4_generate": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int64, C.POINTER(GenerationConfigC), C.c_int32,
                                  TOKEN_CALLBACK, C.c_void_p, C.c_void_p, C.POINTER(C.c_int64)]),
    "oxg4_sample_token": (C.c_int64, [C.c_void_p, C.c_int64, C.c_float, C.c_int64, C.c_float,
                                      C.POINTER(C.c_uint64)]),
    "oxg4_sample_topk_candidates": (C.c_int64, [C.c_void_p, C.c_void_p, C.c_int64, C.c_float, C.c_float,
                                                C.POINTER(C.c_uint64)]),
}

_lib = None


def library_path() -> str:
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "liboxg4.so")


def lib():
    global _lib
    if _lib is None:
        path = build_library()
        L = C.CDLL(path)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(L, name)          # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


class Oxg4Error(RuntimeError):
    """Mirror of oxide_torch::Error: `.kind` is the status name (InvalidShape / Execution ...)."""

    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status
        self.kind = STATUS_NAMES.get(status, str(status))
        self.message = message


def check(status: int):
    if status != OK:
        raise Oxg4Error(status, lib().oxg4_last_error().decode(errors="replace"))
