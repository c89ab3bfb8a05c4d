"""The reference's diagnostic entry points (crates/oxide-torch-models/src/gemma4_cuda/smoke.rs:8-204:
embedding_logits, decoder_mlp_smoke, decoder_attention_smoke, cached_attention_smoke over new_kv_cache) through
the C ABI (oxg4_smoke_*), against the oracle's restatement of the same functions."""
import importlib

import numpy as np
import pytest

from tests.util import build_pair, small_cfg

pkg = importlib.import_module("oxide-beta_b200")

pytestmark = pytest.mark.gpu

CFG = dict(hidden=256, layers=3, heads=4, kv_heads=2, head_dim=64, inter=640, vocab=1500, window=12,
           layer_types=["sliding_attention", "full_attention", "sliding_attention"])


@pytest.mark.parametrize("dtype,tol", [("f32", 1e-3), ("bf16", 2e-2)])
def test_embedding_mlp_and_attention_smoke_match_the_oracle(dtype, tol):
    cfg = small_cfg(**CFG)
    gpu, oracle = build_pair(cfg, dtype, kv_bf16=False, norm_jitter=0.1)
    for token in (0, 7, 1499):
        a, b = gpu.embedding_logits(token), oracle.embedding_logits(token)
        assert a.shape == (cfg["vocab_size"],)
        assert np.abs(a - b).max() <= tol * max(1.0, np.abs(b).max())
        for layer in range(cfg["num_hidden_layers"]):
            a, b = gpu.decoder_mlp_smoke(token, layer), oracle.decoder_mlp_smoke(token, layer)
            assert np.abs(a - b).max() <= tol * max(1.0, np.abs(b).max())
            a, b = gpu.decoder_attention_smoke(token, layer), oracle.decoder_attention_smoke(token, layer)
            assert np.abs(a - b).max() <= tol * max(1.0, np.abs(b).max())


@pytest.mark.parametrize("dtype,kv,tol", [("f32", "f32", 1e-3), ("bf16", "bf16", 2e-2)])
def test_cached_attention_smoke_over_a_wrapping_ring(dtype, kv, tol):
    """30 tokens through one layer's ring: the sliding layer (window 12) wraps, the global layer keeps all."""
    cfg = small_cfg(**CFG)
    gpu, oracle = build_pair(cfg, dtype, kv_bf16=(kv == "bf16"), norm_jitter=0.1)
    rng = np.random.default_rng(5)
    for layer in (0, 1):
        table = gpu.new_cache_table(40, kv_dtype=pkg.BF16 if kv == "bf16" else pkg.F32)
        cache = oracle.new_cache(40)
        for step, token in enumerate(rng.integers(0, cfg["vocab_size"], size=30)):
            a = gpu.cached_attention_smoke(int(token), layer, table)
            b = cache.cached_attention_smoke(int(token), layer)
            assert a.shape == b.shape
            assert np.abs(a - b).max() <= tol, (layer, step)
            assert table.position(0) == step + 1


def test_smoke_entry_points_reject_bad_input():
    cfg = small_cfg(**CFG)
    gpu, _ = build_pair(cfg, "f32", kv_bf16=False, want_oracle=False)
    with pytest.raises(pkg.Oxg4Error, match="exceeds CUDA embedding table"):       # attention.rs:13-17
        gpu.embedding_logits(cfg["vocab_size"])
    with pytest.raises(pkg.Oxg4Error, match="layer out of range"):
        gpu.decoder_mlp_smoke(1, 3)
    two = gpu.new_cache_table([8, 8], batch=2, kv_dtype=pkg.F32)
    with pytest.raises(pkg.Oxg4Error, match="one-sequence"):
        gpu.cached_attention_smoke(1, 0, two)
    full = gpu.new_cache_table(2, kv_dtype=pkg.F32)
    gpu.cached_attention_smoke(1, 0, full)
    gpu.cached_attention_smoke(2, 0, full)
    with pytest.raises(pkg.Oxg4Error, match="max_sequence"):
        gpu.cached_attention_smoke(3, 0, full)
