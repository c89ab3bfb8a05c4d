"""GPU parity of chunked batched prompt ingestion (oxg4_prefill): prompts go through the layers in chunks
of up to 256 tokens with matrix-shaped projections and causal / sliding paged attention, in place of the
reference's prefill_prompt (crates/oxide-torch-models/src/gemma4_cuda/decode.rs:386-459, 176-325;
kernel_module.rs:1896-1974). Checked against the token-by-token path of this library (prefill_token +
decode_token, the reference's own sequential alternative, decode.rs:464-472) and against the CPU oracle,
which ingests prompts token by token."""
import numpy as np
import pytest

from util import build_pair, margin, pkg, small_cfg, syn

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-3
TOL_BF16 = 2e-2


def _oracle_prompt(oracle, prompt, max_seq):
    cache = oracle.new_cache(max_seq)
    for t in prompt[:-1]:
        cache.prefill_token(int(t))
    return cache, cache.decode_logits(int(prompt[-1]))


def _by_token(gpu, prompt, table):
    for t in prompt[:-1]:
        gpu.prefill_token(int(t), table)
    return gpu.decode_token(int(prompt[-1]), table)


@pytest.mark.parametrize("n_prompt,page_tokens", [(1, 16), (255, 16), (256, 4), (257, 16), (700, 64)])
def test_chunked_prefill_equals_token_by_token_f32(n_prompt, page_tokens):
    """f32 recipe: last-token logits of the chunked path against the token-by-token path and the oracle
    (<= 1e-3), across chunk boundaries, with the sliding ring (window 40) wrapped many times, and the
    decode steps that follow read the cache the chunks wrote."""
    cfg = small_cfg(hidden=128, layers=3, heads=4, kv_heads=2, head_dim=64, inter=256, vocab=900, window=40,
                    layer_types=["sliding_attention", "full_attention", "sliding_attention"])
    gpu, oracle = build_pair(cfg, "f32", kv_bf16=False, norm_jitter=0.1)
    prompt = syn.prompt_ids(cfg["vocab_size"], n_prompt, seed=50 + n_prompt)
    max_seq = n_prompt + 6
    t_chunk = gpu.new_cache_table(max_seq, page_tokens=page_tokens, kv_dtype=pkg.F32)
    t_token = gpu.new_cache_table(max_seq, page_tokens=page_tokens, kv_dtype=pkg.F32)
    got = gpu.prefill_prompt(prompt, t_chunk)
    ref_gpu = _by_token(gpu, prompt, t_token)
    cache, ref = _oracle_prompt(oracle, prompt, max_seq)
    assert np.abs(got - ref_gpu).max() <= TOL_F32
    assert np.abs(got - ref).max() <= TOL_F32
    assert t_chunk.position() == n_prompt
    for _ in range(5):
        tok = int(np.argmax(ref))
        ref = cache.decode_logits(tok)
        got = gpu.decode_token(tok, t_chunk)
        assert np.abs(got - ref).max() <= TOL_F32


@pytest.mark.parametrize("head_dim,heads,kv_heads", [(64, 8, 1), (64, 4, 2), (128, 4, 2), (128, 4, 4), (256, 4, 2), (256, 8, 2)])
def test_chunked_prefill_tensor_core_attention_bf16(head_dim, heads, kv_heads):
    """BF16 weights and BF16 KV pages: tcgen05 projections over the chunk's rows and the tensor-core,
    TMA-fed attention kernel (every head_dim and 1 / 2 / 4 / 8 query heads per KV head), against the
    oracle within the BF16 tolerance; 330 tokens = two chunks, window 48."""
    cfg = small_cfg(hidden=256, layers=2, heads=heads, kv_heads=kv_heads, head_dim=head_dim, inter=512, vocab=1200,
                    window=48, layer_types=["sliding_attention", "full_attention"])
    gpu, oracle = build_pair(cfg, "bf16", kv_bf16=True, norm_jitter=0.1)
    prompt = syn.prompt_ids(cfg["vocab_size"], 330, seed=7)
    table = gpu.new_cache_table(340, page_tokens=64, kv_dtype=pkg.BF16)
    got = gpu.prefill_prompt(prompt, table)
    cache, ref = _oracle_prompt(oracle, prompt, 340)
    worst = float(np.abs(got - ref).max())
    for _ in range(6):
        tok = int(np.argmax(ref))
        ref = cache.decode_logits(tok)
        got = gpu.decode_token(tok, table)
        worst = max(worst, float(np.abs(got - ref).max()))
    assert worst <= TOL_BF16, worst


@pytest.mark.parametrize("dtype,batch", [("f32", 3), ("bf16", 5), ("bf16", 11)])
def test_batched_ragged_chunked_prefill(dtype, batch):
    """Several sequences of ragged lengths packed into shared chunks (a chunk holds the tail of one
    sequence and the head of the next); batch 11 then decodes on the tcgen05 path with the
    tensor-core attention kernel. One oracle per sequence."""
    cfg = small_cfg(hidden=128, layers=2, heads=4, kv_heads=2, head_dim=64, inter=256, vocab=700, window=24,
                    layer_types=["sliding_attention", "full_attention"])
    kv = pkg.F32 if dtype == "f32" else pkg.BF16
    tol = TOL_F32 if dtype == "f32" else TOL_BF16
    gpu, oracle = build_pair(cfg, dtype, kv_bf16=(dtype == "bf16"), norm_jitter=0.1)
    lens = [(37 * (b + 3)) % 301 + 1 for b in range(batch)]
    lens[1] = 270
    prompts = [syn.prompt_ids(cfg["vocab_size"], n, seed=60 + b) for b, n in enumerate(lens)]
    table = gpu.new_cache_table([n + 4 for n in lens], batch=batch, page_tokens=16, kv_dtype=kv)
    got = gpu.prefill_prompt(np.concatenate(prompts), table, lens=lens)
    caches, refs = [], []
    for b in range(batch):
        c, r = _oracle_prompt(oracle, prompts[b], lens[b] + 4)
        caches.append(c)
        refs.append(r)
    refs = np.stack(refs)
    assert np.abs(got - refs).max() <= tol
    assert [table.position(b) for b in range(batch)] == lens
    for _ in range(3):
        toks = refs.argmax(-1).astype(np.uint32)
        ids, scores = gpu.decode_topk(toks, table, 1, 1.0, False)
        refs = np.stack([caches[b].decode_logits(int(toks[b])) for b in range(batch)])
        assert np.abs(scores[:, 0] - refs.max(-1)).max() <= tol
        for b in range(batch):
            assert ids[b, 0] == refs[b].argmax() or margin(refs[b]) < 2 * tol


def test_chunked_prefill_at_benchmark_widths():
    """The ~4B widths (hidden 2560, 8 / 4 heads of 256, MLP 10240), one layer, 600-token prompt over 256-token
    pages: tcgen05 row blocks, tensor-core attention with a 128-position window, against the oracle."""
    cfg = syn.scaled_down(syn.workload("c3")["cfg"], layers=1, vocab=8192)
    cfg["sliding_window"] = 128
    gpu, oracle = build_pair(cfg, "bf16", kv_bf16=True)
    prompt = syn.prompt_ids(cfg["vocab_size"], 600, seed=3)
    table = gpu.new_cache_table(608, page_tokens=256, kv_dtype=pkg.BF16)
    got = gpu.prefill_prompt(prompt, table)
    cache, ref = _oracle_prompt(oracle, prompt, 608)
    worst = float(np.abs(got - ref).max())
    for _ in range(4):
        tok = int(np.argmax(ref))
        ref = cache.decode_logits(tok)
        got = gpu.decode_token(tok, table)
        worst = max(worst, float(np.abs(got - ref).max()))
    assert worst <= TOL_BF16, worst


def test_prefill_rejects_what_the_reference_rejects():
    cfg = small_cfg(hidden=64, layers=1, heads=2, kv_heads=1, head_dim=64, inter=128, vocab=300, window=8,
                    layer_types=["full_attention"])
    gpu, _ = build_pair(cfg, "f32", kv_bf16=False, want_oracle=False)
    table = gpu.new_cache_table(8, kv_dtype=pkg.F32)
    with pytest.raises(pkg.Oxg4Error) as e:
        gpu.prefill_prompt([1, 2, 300], table)                  # decode.rs:675-679
    assert "token id exceeds" in e.value.message
    with pytest.raises(pkg.Oxg4Error) as e:
        gpu.prefill_prompt(list(range(9)), table)
    assert e.value.kind == "INVALID_SHAPE"
    gpu.prefill_prompt([1, 2, 3], table, want_logits=False)
    assert table.position() == 3
    with pytest.raises(pkg.Oxg4Error) as e:
        gpu.prefill_prompt([4], table)                          # decode.rs:392-396
    assert "empty cache table" in e.value.message
