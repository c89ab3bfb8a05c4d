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


def layerwise_compare(gpu, oracle, cfg, prompts, kv_dtype, page_tokens, logits_every=1):
    """Layer-wise teacher forcing over a batch of ragged prompts: one oracle per sequence runs freely, the CUDA path
    gets the oracle's input of every layer injected (oxg4_decode_trace). Returns (worst layer-output difference,
    worst logits difference, largest hidden magnitude, cache table)."""
    L, H = cfg["num_hidden_layers"], cfg["hidden_size"]
    batch = len(prompts)
    lens = [len(p) for p in prompts]
    table = gpu.new_cache_table([n + 2 for n in lens], batch=batch, page_tokens=page_tokens, kv_dtype=kv_dtype)
    caches = [oracle.new_cache(n + 2) for n in lens]
    worst_h = worst_logit = scale = 0.0
    for t in range(max(lens)):
        toks = np.full(batch, pkg.INACTIVE, dtype=np.uint32)
        inject = np.zeros((L, batch, H), dtype=np.float32)
        refs = {}
        for b in range(batch):
            if t >= lens[b]:
                continue
            toks[b] = prompts[b][t]
            tr_o, lg_o = caches[b].decode_trace(int(prompts[b][t]), want_logits=(t % logits_every == 0 or t >= lens[b] - 2))
            inject[:, b] = tr_o[:L]
            refs[b] = (tr_o, lg_o)
        tr_g, lg_g = gpu.decode_trace(toks, table, inject=inject)
        for b, (tr_o, lg_o) in refs.items():
            worst_h = max(worst_h, float(np.abs(tr_g[:, b] - tr_o).max()))
            scale = max(scale, float(np.abs(tr_o).max()))
            if lg_o is not None:
                worst_logit = max(worst_logit, float(np.abs(lg_g[b] - lg_o).max()))
    return worst_h, worst_logit, scale, table
