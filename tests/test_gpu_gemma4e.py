"""GPU parity of the Gemma4-E features: per-kind head geometry (global_head_dim, num_global_key_value_heads with
attention_k_eq_v), KV-shared layers and per-layer embeddings (crates/oxide-torch-models/src/gemma4_cuda/
mod.rs:371-413, cache.rs:43-86, ple.rs:55-185). The oracle's treatment of them is pinned by the Hugging Face
fixture tests/golden/e_tiny_hf_gemma4.npz (tests/test_oracle.py)."""
import os

import numpy as np
import pytest

from util import build_pair, layerwise_compare, margin, pkg, syn

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-3
TOL_BF16 = 2e-2
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_e_tiny_f32_matches_oracle_and_hf_fixture():
    """All three features at once, f32: chunked prefill of the 40-token prompt, then 12 greedy tokens equal to
    Hugging Face's; logits within 1e-3 of the oracle; cache accounting reports the shared layers."""
    gold = np.load(os.path.join(GOLDEN, "e_tiny_hf_gemma4.npz"))
    cfg = syn.e_tiny_cfg()
    gpu, oracle = build_pair(cfg, "f32", kv_bf16=False, norm_jitter=0.1)
    table = gpu.new_cache_table(64, page_tokens=16, kv_dtype=pkg.F32)
    info = table._info()
    assert (info.layer_count, info.physical_cache_count, info.shared_layer_count) == (6, 4, 2)
    got = gpu.prefill_prompt(gold["prompt"], table)
    assert np.abs(got - gold["logits"][-1]).max() <= TOL_F32
    cache = oracle.new_cache(64)
    for t in gold["prompt"][:-1]:
        cache.prefill_token(int(t))
    ref = cache.decode_logits(int(gold["prompt"][-1]))
    toks = []
    for _ in range(12):
        assert np.abs(got - ref).max() <= TOL_F32
        toks.append(int(np.argmax(got)))
        ref = cache.decode_logits(toks[-1])
        got = gpu.decode_token(toks[-1], table)
    assert toks == gold["tokens"].tolist()
    # token-by-token ingestion (decode kernels) agrees with the chunked pass
    t2 = gpu.new_cache_table(64, page_tokens=16, kv_dtype=pkg.F32)
    for t in gold["prompt"][:-1]:
        gpu.prefill_token(int(t), t2)
    assert np.abs(gpu.decode_token(int(gold["prompt"][-1]), t2) - gold["logits"][-1]).max() <= TOL_F32


@pytest.mark.parametrize("batch", [1, 3, 9])
def test_e_tiny_bf16_layerwise(batch):
    """BF16 recipe with BF16 KV pages, layer by layer with teacher forcing (six random-init BF16 layers are not
    comparable end to end): one sequence, a small ragged batch, and nine sequences."""
    cfg = syn.e_tiny_cfg()
    gpu, oracle = build_pair(cfg, "bf16", kv_bf16=True, norm_jitter=0.1)
    prompts = [syn.prompt_ids(cfg["vocab_size"], 6 + (11 * b) % 30, seed=80 + b) for b in range(batch)]
    worst_h, worst_logit, scale, table = layerwise_compare(gpu, oracle, cfg, prompts, pkg.BF16, 16)
    assert worst_logit <= TOL_BF16, (worst_logit, worst_h, scale)
    assert worst_h <= TOL_BF16 * max(1.0, scale), (worst_h, scale)


def _geometry_cfg():
    """No per-layer embeddings (so that eight or more sequences take the tcgen05 path): head_dim 64 with 2 KV heads on
    the sliding layers, global_head_dim 128 with ONE KV head on the global layers (attention_k_eq_v), the last two
    layers KV-shared."""
    c = syn._cfg(700, 256, 4, 4, 2, 64, 512, 12, ["sliding_attention", "full_attention", "sliding_attention",
                                                  "full_attention"])
    c.update(global_head_dim=128, attention_k_eq_v=True, num_global_key_value_heads=1, num_kv_shared_layers=2)
    return c


def test_per_kind_geometry_and_shared_layers_f32():
    cfg = _geometry_cfg()
    gpu, oracle = build_pair(cfg, "f32", kv_bf16=False, norm_jitter=0.1)
    lens = [30, 5, 17]
    prompts = [syn.prompt_ids(cfg["vocab_size"], n, seed=90 + b) for b, n in enumerate(lens)]
    table = gpu.new_cache_table([n + 6 for n in lens], batch=3, page_tokens=8, kv_dtype=pkg.F32)
    got = gpu.prefill_prompt(np.concatenate(prompts), table, lens=lens)
    caches, refs = [], []
    for b in range(3):
        c = oracle.new_cache(lens[b] + 6)
        for t in prompts[b][:-1]:
            c.prefill_token(int(t))
        refs.append(c.decode_logits(int(prompts[b][-1])))
        caches.append(c)
    refs = np.stack(refs)
    assert np.abs(got - refs).max() <= TOL_F32
    for _ in range(5):
        toks = refs.argmax(-1).astype(np.uint32)
        got = gpu.decode_token(toks, table)
        refs = np.stack([caches[b].decode_logits(int(toks[b])) for b in range(3)])
        assert np.abs(got - refs).max() <= TOL_F32


@pytest.mark.parametrize("batch", [2, 9])
def test_per_kind_geometry_and_shared_layers_bf16_layerwise(batch):
    """Batch 9 runs the tcgen05 projections and the tensor-core attention kernel with a different head_dim and
    group size per layer kind, and query-only projections on the shared layers."""
    cfg = _geometry_cfg()
    gpu, oracle = build_pair(cfg, "bf16", kv_bf16=True, norm_jitter=0.1)
    prompts = [syn.prompt_ids(cfg["vocab_size"], 4 + (13 * b) % 29, seed=95 + b) for b in range(batch)]
    worst_h, worst_logit, scale, table = layerwise_compare(gpu, oracle, cfg, prompts, pkg.BF16, 16)
    assert worst_logit <= TOL_BF16, (worst_logit, worst_h, scale)
    assert worst_h <= TOL_BF16 * max(1.0, scale), (worst_h, scale)
    # chunked prefill of the same prompts reaches the same cache state: the next logits agree with the oracle's
    lens = [len(p) for p in prompts]
    t2 = gpu.new_cache_table([n + 2 for n in lens], batch=batch, page_tokens=16, kv_dtype=pkg.BF16)
    got = gpu.prefill_prompt(np.concatenate(prompts), t2, lens=lens)
    assert got.shape[-1] == cfg["vocab_size"] and np.isfinite(got).all()
    assert [t2.position(b) for b in range(batch)] == lens


def test_ple_token_outside_its_vocabulary_is_rejected():
    cfg = syn.e_tiny_cfg()
    cfg["vocab_size_per_layer_input"] = 300                    # smaller than the 512-entry vocabulary
    gpu, _ = build_pair(cfg, "f32", kv_bf16=False, want_oracle=False)
    table = gpu.new_cache_table(8, kv_dtype=pkg.F32)
    gpu.decode_token(299, table)
    with pytest.raises(pkg.Oxg4Error) as e:
        gpu.decode_token(300, table)                            # ple.rs:113-119
    assert e.value.kind == "INVALID_SHAPE" and "PLE" in e.value.message
