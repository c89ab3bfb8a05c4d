"""Shared helpers of the parity tests: build the CUDA model and the CPU oracle from one set of
seeded weights and compare them step by step."""
import importlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

pkg = importlib.import_module("oxide-beta_b200")
syn = pkg.synthetic
from oracle import oracle as orc  # noqa: E402


def small_cfg(hidden=256, layers=2, heads=4, kv_heads=1, head_dim=64, inter=512, vocab=1024, window=16,
              layer_types=None):
    c = syn._cfg(vocab, hidden, layers, heads, kv_heads, head_dim, inter, window, layer_types)
    return c


def build_pair(cfg, dtype, kv_bf16, seed=0, norm_jitter=0.0, want_gpu=True, want_oracle=True):
    """Returns (Gemma4CudaState | None, OracleModel | None) holding identical weights."""
    weights = list(syn.generate_weights(cfg, seed=seed, dtype=dtype, norm_jitter=norm_jitter))
    gpu = oracle = None
    if want_oracle:
        oracle = orc.OracleModel(cfg, orc.F32 if dtype == "f32" else orc.REF_BF16, kv_bf16=kv_bf16)
        oracle.load(dict(weights))
    if want_gpu:
        gpu = pkg.Gemma4CudaState.load(pkg.Gemma4TextConfig(cfg), weights, 0,
                                       pkg.F32 if dtype == "f32" else pkg.BF16)
    return gpu, oracle


def margin(logits):
    top = np.sort(logits)[-2:]
    return float(top[1] - top[0])
