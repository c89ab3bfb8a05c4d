"""B200-native Gemma4 token generation behind the reference's Gemma4 API (see gemma4.py).

The directory name carries a hyphen, so import it with
    importlib.import_module("oxide-beta_b200")
from the repository root.
"""
from . import _native, synthetic
from ._native import BF16, F32, INACTIVE, Oxg4Error, library_path
from .gemma4 import (Device, Gemma4CudaCacheTable, Gemma4CudaState, Gemma4ForCausalLM, Gemma4TextConfig,
                     Gemma4TpCacheTable, Gemma4TpState, GenerationConfig, sample_token, sample_topk_candidates,
                     tp_shard)

__all__ = ["BF16", "F32", "INACTIVE", "Oxg4Error", "Device", "Gemma4CudaCacheTable", "Gemma4CudaState",
           "Gemma4ForCausalLM", "Gemma4TextConfig", "Gemma4TpCacheTable", "Gemma4TpState", "GenerationConfig", "sample_token",
           "sample_topk_candidates", "synthetic", "library_path", "tp_shard"]
