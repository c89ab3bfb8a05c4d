"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle on identical
seeded weights and prompts.

Tolerances (from the benchmark specification): greedy token ids bit-exact over the first 32
generated tokens; logits max-abs <= 1e-3 in f32 mode and <= 2e-2 in BF16 mode.
"""
import os

import numpy as np
import pytest

from util import build_pair, margin, orc, pkg, small_cfg, syn

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-3
TOL_BF16 = 2e-2
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def run_both(gpu, oracle, prompt, n_decode, kv_dtype, page_tokens=256, max_seq=None):
    """Teacher-forced comparison: both sides consume the oracle's greedy tokens; returns
    (max logits diff, gpu greedy ids, oracle greedy ids, min oracle margin)."""
    max_seq = max_seq or (len(prompt) + n_decode)
    table = gpu.new_cache_table(max_seq, page_tokens=page_tokens, kv_dtype=kv_dtype)
    cache = oracle.new_cache(max_seq)
    for t in prompt[:-1]:
        cache.prefill_token(int(t))
    ref = cache.decode_logits(int(prompt[-1]))
    got = gpu.prefill_prompt(prompt, table)
    worst = float(np.abs(got - ref).max())
    g_ids, o_ids, margins = [], [], []
    for _ in range(n_decode):
        o_tok = int(np.argmax(ref))
        g_ids.append(int(np.argmax(got)))
        o_ids.append(o_tok)
        margins.append(margin(ref))
        ref = cache.decode_logits(o_tok)
        got = gpu.decode_token(o_tok, table)
        worst = max(worst, float(np.abs(got - ref).max()))
    return worst, g_ids, o_ids, min(margins)


# ---- configuration 1: tiny f32 model ------------------------------------------------------------

@pytest.fixture(scope="module")
def c1():
    cfg = syn.workload("c1")["cfg"]
    gpu, oracle = build_pair(cfg, "f32", kv_bf16=False)
    return cfg, gpu, oracle


def test_c1_greedy_tokens_bit_exact_and_logits(c1):
    cfg, gpu, oracle = c1
    prompt = syn.prompt_ids(cfg["vocab_size"], 16, seed=1)
    worst, g_ids, o_ids, mm = run_both(gpu, oracle, prompt, 32, pkg.F32)
    assert g_ids == o_ids, f"first divergence margin {mm}"
    assert worst <= TOL_F32, worst
    gold = np.load(os.path.join(GOLDEN, "c1_hf_gemma4.npz"))
    assert o_ids == gold["tokens"].tolist()


def test_c1_generate_api_matches_fixture_and_oracle(c1):
    cfg, gpu, oracle = c1
    gold = np.load(os.path.join(GOLDEN, "c1_hf_gemma4.npz"))
    weights = dict(syn.generate_weights(cfg, 0, "f32"))
    model = pkg.Gemma4ForCausalLM.from_weights(cfg, weights, pkg.Device.Cuda(0), kv_dtype=pkg.F32)
    streamed = []
    out = model.generate_stream(gold["prompt"], pkg.GenerationConfig.greedy(32), streamed.append)
    assert out[:16] == gold["prompt"].tolist()
    assert out[16:] == gold["tokens"].tolist() == streamed
    assert out[16:] == oracle.generate(gold["prompt"], 32, top_k=1).tolist()


def test_c1_long_prompt_crosses_sliding_window(c1):
    cfg, gpu, oracle = c1
    gold = np.load(os.path.join(GOLDEN, "c1_hf_gemma4.npz"))
    table = gpu.new_cache_table(208, kv_dtype=pkg.F32)
    logits = gpu.prefill_prompt(gold["long_prompt"], table)
    assert np.abs(logits - gold["long_logits"]).max() <= TOL_F32
    assert table.position() == 200


def test_c1_sampled_generation_matches_oracle(c1):
    """Non-greedy path: top-k 8 candidates with repetition penalty, xorshift sampling on the host."""
    cfg, gpu, oracle = c1
    prompt = syn.prompt_ids(cfg["vocab_size"], 12, seed=4)
    weights = dict(syn.generate_weights(cfg, 0, "f32"))
    model = pkg.Gemma4ForCausalLM.from_weights(cfg, weights, pkg.Device.Cuda(0), kv_dtype=pkg.F32)
    g = pkg.GenerationConfig(max_new_tokens=24, temperature=0.9, top_k=8, top_p=0.9, repetition_penalty=1.3,
                             eos_token_ids=[], seed=1234)
    ours = model.generate(prompt, g)[12:]
    ref = oracle.generate(prompt, 24, temperature=0.9, top_k=8, top_p=0.9, repetition_penalty=1.3, seed=1234)
    assert ours == ref.tolist()


def test_c1_decode_topk_lists_match_oracle(c1):
    cfg, gpu, oracle = c1
    table = gpu.new_cache_table(16, kv_dtype=pkg.F32)
    cache = oracle.new_cache(16)
    tok = 7
    for step, (k, pen) in enumerate([(1, 1.0), (5, 1.0), (64, 1.5), (64, 1.5), (3, 2.0)]):
        got = gpu.decode_topk(tok, table, k, pen, True)
        ids, scores = cache.decode_topk(tok, k, pen, True)
        assert [g[0] for g in got] == ids.tolist(), (step, k)
        np.testing.assert_allclose([g[1] for g in got], scores, atol=TOL_F32)
        tok = int(ids[0])


def test_c1_graph_replay_equals_eager(c1):
    cfg, gpu, oracle = c1
    prompt = syn.prompt_ids(cfg["vocab_size"], 10, seed=9)
    outs = []
    for disable in (False, True):
        if disable:
            os.environ["GEMMA4_DISABLE_CUDA_GRAPH"] = "1"
        try:
            table = gpu.new_cache_table(32, kv_dtype=pkg.F32)
            logits = [gpu.prefill_prompt(prompt, table)]
            tok = int(np.argmax(logits[0]))
            for _ in range(6):
                logits.append(gpu.decode_token(tok, table))
                tok = int(np.argmax(logits[-1]))
            outs.append(np.stack(logits))
        finally:
            os.environ.pop("GEMMA4_DISABLE_CUDA_GRAPH", None)
    assert np.array_equal(outs[0], outs[1])           # same kernels, same order: identical bits


def test_c1_device_greedy_loop_equals_host_loop(c1):
    cfg, gpu, oracle = c1
    prompt = syn.prompt_ids(cfg["vocab_size"], 16, seed=1)
    table = gpu.new_cache_table(64, kv_dtype=pkg.F32)
    first = int(np.argmax(gpu.prefill_prompt(prompt, table)))
    ids, ms = gpu.decode_greedy(first, table, 20)
    table2 = gpu.new_cache_table(64, kv_dtype=pkg.F32)
    tok = int(np.argmax(gpu.prefill_prompt(prompt, table2)))
    host = []
    for _ in range(20):
        tok = gpu.decode_topk(tok, table2, 1, 1.0, False)[0][0]
        host.append(tok)
    assert ids[:, 0].tolist() == host
    assert ms > 0 and table.position() == 36


def test_error_paths_on_device(c1):
    cfg, gpu, oracle = c1
    table = gpu.new_cache_table(4, kv_dtype=pkg.F32)
    with pytest.raises(pkg.Oxg4Error) as e:
        gpu.decode_topk(cfg["vocab_size"], table, 1, 1.0, True)       # decode.rs:675-679
    assert "token id exceeds" in e.value.message
    with pytest.raises(pkg.Oxg4Error):
        gpu.prefill_prompt([], table)
    with pytest.raises(pkg.Oxg4Error):
        gpu.new_cache_table(0)                                         # cache.rs:36-38
    gpu.prefill_prompt([1, 2, 3, 4], table, want_logits=False)
    with pytest.raises(pkg.Oxg4Error) as e:
        gpu.decode_token(5, table)                                     # cache is full
    assert e.value.kind == "INVALID_SHAPE"
    with pytest.raises(pkg.Oxg4Error) as e:
        gpu.prefill_prompt([1, 2], table)                              # decode.rs:392-396
    assert "empty cache table" in e.value.message
    table.reset()
    assert table.position() == 0
    info = table._info()
    assert info.layer_count == 2 and info.physical_cache_count == 2 and info.shared_layer_count == 0
    assert gpu.weight_count() == 2 + 2 * 12 and gpu.weight_bytes() > 0


# ---- BF16 recipe on small shapes: every head_dim / group size / cache type ------------------------

@pytest.mark.parametrize("head_dim,heads,kv_heads,kv", [
    (64, 4, 1, "bf16"), (64, 8, 1, "f32"), (128, 4, 2, "bf16"), (128, 2, 2, "f32"), (256, 4, 2, "bf16"),
    (256, 4, 1, "f32")])
def test_bf16_small_models(head_dim, heads, kv_heads, kv):
    # two layers: deeper random-init BF16 stacks amplify single rounding flips beyond the tolerance
    # for any two implementations (see test_layerwise_*), so end-to-end BF16 cases stay shallow
    cfg = small_cfg(hidden=192, layers=2, heads=heads, kv_heads=kv_heads, head_dim=head_dim, inter=448,
                    vocab=1000, window=12, layer_types=["sliding_attention", "full_attention"])
    gpu, oracle = build_pair(cfg, "bf16", kv_bf16=(kv == "bf16"), norm_jitter=0.1)
    prompt = syn.prompt_ids(cfg["vocab_size"], 20, seed=11)          # longer than the window
    worst, g_ids, o_ids, mm = run_both(gpu, oracle, prompt, 16, pkg.BF16 if kv == "bf16" else pkg.F32,
                                       page_tokens=8)
    assert worst <= TOL_BF16, worst
    if g_ids != o_ids:
        assert mm < 2 * worst, f"token mismatch with margin {mm}, logits diff {worst}"


def test_partial_rotary_and_rope_factor():
    cfg = small_cfg(hidden=128, layers=2, heads=2, kv_heads=1, head_dim=64, inter=256, vocab=512, window=8,
                    layer_types=["sliding_attention", "full_attention"])
    cfg["rope_parameters"]["full_attention"].update(partial_rotary_factor=0.25, factor=8.0)
    gpu, oracle = build_pair(cfg, "f32", kv_bf16=False, norm_jitter=0.1)
    prompt = syn.prompt_ids(cfg["vocab_size"], 14, seed=12)
    worst, g_ids, o_ids, _ = run_both(gpu, oracle, prompt, 8, pkg.F32, page_tokens=4)
    assert worst <= TOL_F32 and g_ids == o_ids


def test_ragged_shapes_odd_sizes():
    """Hidden / intermediate sizes that are not multiples of the 512-byte chunk, vocabulary that is
    odd, context of one token."""
    cfg = small_cfg(hidden=136, layers=2, heads=2, kv_heads=2, head_dim=64, inter=200, vocab=777, window=5)
    gpu, oracle = build_pair(cfg, "bf16", kv_bf16=True, norm_jitter=0.1)
    worst, g_ids, o_ids, mm = run_both(gpu, oracle, np.array([3], dtype=np.uint32), 12, pkg.BF16, page_tokens=2)
    assert worst <= TOL_BF16
    if g_ids != o_ids:
        assert mm < 2 * worst


# ---- batches ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("batch", [2, 3, 5])
def test_batched_ragged_decode_matches_per_sequence_oracle(batch):
    cfg = small_cfg(hidden=128, layers=2, heads=4, kv_heads=2, head_dim=64, inter=256, vocab=600, window=10,
                    layer_types=["sliding_attention", "full_attention"])
    gpu, oracle = build_pair(cfg, "bf16", kv_bf16=True, norm_jitter=0.1)
    lens = [3 + 4 * b for b in range(batch)]
    prompts = [syn.prompt_ids(cfg["vocab_size"], n, seed=20 + b) for b, n in enumerate(lens)]
    max_seq = [n + 6 for n in lens]
    table = gpu.new_cache_table(max_seq, batch=batch, page_tokens=4, kv_dtype=pkg.BF16)
    got = gpu.prefill_prompt(np.concatenate(prompts), table, lens=lens)
    caches, refs = [], []
    for b in range(batch):
        c = oracle.new_cache(max_seq[b])
        for t in prompts[b][:-1]:
            c.prefill_token(int(t))
        refs.append(c.decode_logits(int(prompts[b][-1])))
        caches.append(c)
    refs = np.stack(refs)
    assert np.abs(got - refs).max() <= TOL_BF16
    for _ in range(5):
        toks = refs.argmax(-1).astype(np.uint32)
        ids, scores = gpu.decode_topk(toks, table, 1, 1.0, True)
        refs = np.stack([caches[b].decode_logits(int(toks[b])) for b in range(batch)])
        for b in range(batch):
            assert abs(scores[b, 0] - refs[b].max()) <= TOL_BF16
            assert ids[b, 0] == refs[b].argmax() or margin(refs[b]) < 2 * TOL_BF16
    assert [table.position(b) for b in range(batch)] == [n + 5 for n in lens]


def test_batch_rows_are_independent():
    """The same sequence placed in different rows of a batch, next to different neighbours, yields
    bit-identical logits (no cross-row leakage; fixed reduction order)."""
    cfg = small_cfg(hidden=128, layers=2, heads=4, kv_heads=2, head_dim=64, inter=256, vocab=600, window=10)
    gpu, _ = build_pair(cfg, "bf16", kv_bf16=True, want_oracle=False)
    a = syn.prompt_ids(cfg["vocab_size"], 9, seed=30)
    b = syn.prompt_ids(cfg["vocab_size"], 5, seed=31)
    t1 = gpu.new_cache_table([16, 16], batch=2, page_tokens=4, kv_dtype=pkg.BF16)
    l1 = gpu.prefill_prompt(np.concatenate([a, b]), t1, lens=[9, 5])
    t2 = gpu.new_cache_table([16, 16, 16], batch=3, page_tokens=4, kv_dtype=pkg.BF16)
    l2 = gpu.prefill_prompt(np.concatenate([b, b, a]), t2, lens=[5, 5, 9])
    assert np.array_equal(l1[0], l2[2]) and np.array_equal(l1[1], l2[0]) and np.array_equal(l2[0], l2[1])


# ---- benchmark architectures at reduced depth / context (full widths, full vocabulary) -------------------------

@pytest.mark.parametrize("name,layers", [("c2", 7), ("c3", 6)])
def test_benchmark_architecture_reduced_depth_f32(name, layers):
    """Full widths and vocabulary of the ~1B / ~4B workloads at reduced depth, f32 recipe, so that the
    end-to-end comparison is well conditioned (tests/test_oracle.py::test_summation_order_spread_grows_with_depth
    shows why the BF16 recipe is not, at depth)."""
    w = syn.workload(name)
    cfg = syn.scaled_down(w["cfg"], layers=layers)
    gpu, oracle = build_pair(cfg, "f32", kv_bf16=False)
    prompt = syn.prompt_ids(cfg["vocab_size"], 24, seed=1)
    worst, g_ids, o_ids, mm = run_both(gpu, oracle, prompt, 8, pkg.F32)
    assert worst <= TOL_F32, worst
    assert g_ids == o_ids, (mm, worst)


@pytest.mark.parametrize("name", ["c2", "c3"])
def test_benchmark_architecture_one_layer_bf16(name):
    """BF16 recipe at the full widths of the ~1B / ~4B workloads, one layer deep."""
    cfg = syn.scaled_down(syn.workload(name)["cfg"], layers=1, vocab=32768)
    gpu, oracle = build_pair(cfg, "bf16", kv_bf16=True)
    prompt = syn.prompt_ids(cfg["vocab_size"], 24, seed=1)
    worst, g_ids, o_ids, mm = run_both(gpu, oracle, prompt, 8, pkg.BF16)
    assert worst <= TOL_BF16, worst
    assert g_ids == o_ids or mm < 2 * worst, (mm, worst)


def test_determinism_two_runs_identical():
    cfg = syn.scaled_down(syn.workload("c2")["cfg"], layers=3, vocab=8192)
    gpu, _ = build_pair(cfg, "bf16", kv_bf16=True, want_oracle=False)
    prompt = syn.prompt_ids(cfg["vocab_size"], 40, seed=5)
    runs = []
    for _ in range(2):
        table = gpu.new_cache_table(64, kv_dtype=pkg.BF16)
        first = int(np.argmax(gpu.prefill_prompt(prompt, table)))
        ids, _ = gpu.decode_greedy(first, table, 16)
        runs.append((ids.copy(), gpu.decode_token(int(ids[-1, 0]), table)))
    assert np.array_equal(runs[0][0], runs[1][0]) and np.array_equal(runs[0][1], runs[1][1])


# ---- layer-wise teacher forcing: BF16 recipe at depth ------------------------------------------------------------

@pytest.mark.parametrize("name,layers", [("c2", 7), ("c3", 6)])
def test_layerwise_bf16_parity_at_depth(name, layers):
    """End-to-end BF16 logits of a deep random-init stack are ill-conditioned (one rounding flip is
    amplified ~6x per layer for ANY two implementations), so depth is checked layer by layer: the
    oracle runs freely, the CUDA path gets the oracle's input of every layer injected, and each
    layer's output (= next layer's input before injection), the final hidden state and the logits
    must agree. Both KV caches are filled by their own side from identical layer inputs."""
    cfg = syn.scaled_down(syn.workload(name)["cfg"], layers=layers, vocab=8192)
    gpu, oracle = build_pair(cfg, "bf16", kv_bf16=True)
    L = layers
    prompt = syn.prompt_ids(cfg["vocab_size"], 20, seed=1)
    table = gpu.new_cache_table(32, kv_dtype=pkg.BF16)
    cache = oracle.new_cache(32)
    worst_h, worst_logit, scale = 0.0, 0.0, 0.0
    for t in prompt:
        tr_o, lg_o = cache.decode_trace(int(t))
        tr_g, lg_g = gpu.decode_trace(int(t), table, inject=tr_o[:L][:, None, :])
        # tr_g[l] is the CUDA path's own output of layer l-1, computed from the oracle's input of layer l-1
        worst_h = max(worst_h, float(np.abs(tr_g[:, 0] - tr_o).max()))
        scale = max(scale, float(np.abs(tr_o).max()))
        worst_logit = max(worst_logit, float(np.abs(lg_g[0] - lg_o).max()))
    assert worst_logit <= TOL_BF16, (worst_logit, worst_h, scale)
    assert worst_h <= TOL_BF16 * max(1.0, scale), (worst_h, scale)


def test_layerwise_trace_without_injection_matches_oracle_f32():
    """The trace itself (no injection) reproduces the oracle's hidden state after every layer in f32."""
    cfg = small_cfg(hidden=256, layers=4, heads=4, kv_heads=2, head_dim=64, inter=512, vocab=1024, window=8,
                    layer_types=["sliding_attention", "full_attention", "sliding_attention", "full_attention"])
    gpu, oracle = build_pair(cfg, "f32", kv_bf16=False, norm_jitter=0.1)
    table = gpu.new_cache_table(16, kv_dtype=pkg.F32)
    cache = oracle.new_cache(16)
    for t in syn.prompt_ids(cfg["vocab_size"], 12, seed=2):
        tr_o, lg_o = cache.decode_trace(int(t))
        tr_g, lg_g = gpu.decode_trace(int(t), table)
        assert np.abs(tr_g[:, 0] - tr_o).max() <= TOL_F32
        assert np.abs(lg_g[0] - lg_o).max() <= TOL_F32
    assert table.position() == 12


# ---- tensor-core projection kernel: 2..16 rows per pass, several passes --------------------------------------------

@pytest.mark.parametrize("batch", [8, 16, 21, 80, 130])
def test_large_batches_tensor_core_path(batch):
    cfg = small_cfg(hidden=256, layers=2, heads=4, kv_heads=2, head_dim=64, inter=520, vocab=1000, window=10,
                    layer_types=["sliding_attention", "full_attention"])
    gpu, oracle = build_pair(cfg, "bf16", kv_bf16=True, norm_jitter=0.1)
    lens = [2 + (3 * b) % 11 for b in range(batch)]
    prompts = [syn.prompt_ids(cfg["vocab_size"], n, seed=100 + b) for b, n in enumerate(lens)]
    table = gpu.new_cache_table([n + 4 for n in lens], batch=batch, page_tokens=4, kv_dtype=pkg.BF16)
    got = gpu.prefill_prompt(np.concatenate(prompts), table, lens=lens)
    refs, caches = [], []
    for b in range(batch):
        c = oracle.new_cache(lens[b] + 4)
        for t in prompts[b][:-1]:
            c.prefill_token(int(t))
        refs.append(c.decode_logits(int(prompts[b][-1])))
        caches.append(c)
    refs = np.stack(refs)
    assert np.abs(got - refs).max() <= TOL_BF16
    toks = refs.argmax(-1).astype(np.uint32)
    ids, scores = gpu.decode_topk(toks, table, 1, 1.0, False)
    refs = np.stack([caches[b].decode_logits(int(toks[b])) for b in range(batch)])
    assert np.abs(scores[:, 0] - refs.max(-1)).max() <= TOL_BF16


# ---- device-side sampling ---------------------------------------------------------------------------

@pytest.mark.parametrize("seed,top_k,top_p,penalty", [(1234, 8, 0.9, 1.3), (7, 64, 1.0, 1.0), (99, 4, 0.5, 1.1)])
def test_device_sampled_loop_equals_host_sampling(c1, seed, top_k, top_p, penalty):
    """oxg4_decode_sampled (draw on the device, no per-token round trip) against the host loop that calls
    decode_topk + sample_topk_candidates per token: same tokens, same generator state afterwards."""
    cfg, gpu, oracle = c1
    prompt = syn.prompt_ids(cfg["vocab_size"], 12, seed=4)
    steps, temperature = 20, 0.9
    gcfg = pkg.GenerationConfig(max_new_tokens=steps, temperature=temperature, top_k=top_k, top_p=top_p,
                                repetition_penalty=penalty, eos_token_ids=[], seed=seed)
    first = int(np.argmax(gpu.prefill_prompt(prompt, gpu.new_cache_table(64, kv_dtype=pkg.F32))))
    # host loop
    t_host = gpu.new_cache_table(64, kv_dtype=pkg.F32)
    gpu.prefill_prompt(prompt, t_host)
    rnd = np.array([seed], dtype=np.uint64)
    tok, host_ids = first, []
    for _ in range(steps):
        cand = gpu.decode_topk(tok, t_host, top_k, penalty, True)
        tok = pkg.sample_topk_candidates(cand, gcfg, rnd)
        host_ids.append(tok)
    # device loop
    t_dev = gpu.new_cache_table(64, kv_dtype=pkg.F32)
    gpu.prefill_prompt(prompt, t_dev)
    dev_ids, state, _ = gpu.decode_sampled(first, t_dev, steps, top_k, temperature, top_p, penalty, [seed])
    assert dev_ids.ravel().tolist() == host_ids
    assert int(state[0]) == int(rnd[0])
    assert t_dev.position(0) == t_host.position(0)


def test_device_sampled_loop_argument_checks(c1):
    cfg, gpu, _ = c1
    t = gpu.new_cache_table(32, kv_dtype=pkg.F32)
    gpu.prefill_prompt(syn.prompt_ids(cfg["vocab_size"], 4, seed=1), t)
    with pytest.raises(pkg.Oxg4Error):
        gpu.decode_sampled(1, t, 4, 1, 1.0, 1.0, 1.0, [1])          # one candidate: greedy, not sampling
    with pytest.raises(pkg.Oxg4Error):
        gpu.decode_sampled(1, t, 4, 8, 0.0, 1.0, 1.0, [1])          # temperature must be positive
    with pytest.raises(pkg.Oxg4Error):
        gpu.decode_sampled(1, t, 400, 8, 1.0, 1.0, 1.0, [1])        # would outgrow the table


# ---- final_logit_softcapping ----------------------------------------------------------------------------

@pytest.fixture(scope="module")
def capped():
    cfg = small_cfg(hidden=128, layers=2, heads=2, kv_heads=1, head_dim=64, inter=256, vocab=1500, window=8,
                    layer_types=["sliding_attention", "full_attention"])
    cfg["final_logit_softcapping"] = 0.75          # small enough to bend the seeded model's logits (|x| up to ~1.5)
    gpu, oracle = build_pair(cfg, "f32", kv_bf16=False, norm_jitter=0.1)
    return cfg, gpu, oracle


def test_softcap_logits_and_topk_match_oracle(capped):
    """gemma4_cuda/mod.rs:573-579: tanh(x / cap) * cap on every score handed back to the host."""
    cfg, gpu, oracle = capped
    prompt = syn.prompt_ids(cfg["vocab_size"], 10, seed=3)
    worst, g_ids, o_ids, _ = run_both(gpu, oracle, prompt, 6, pkg.F32, page_tokens=4)
    assert worst <= TOL_F32 and g_ids == o_ids
    table = gpu.new_cache_table(8, kv_dtype=pkg.F32)
    cache = oracle.new_cache(8)
    tok = 3
    for k, pen in [(4, 1.0), (16, 1.4)]:
        got = gpu.decode_topk(tok, table, k, pen, True)
        ids, scores = cache.decode_topk(tok, k, pen, True)
        assert [g[0] for g in got] == ids.tolist()
        np.testing.assert_allclose([g[1] for g in got], scores, atol=TOL_F32)
        assert max(abs(g[1]) for g in got) < 0.75
        tok = int(ids[0])


@pytest.mark.parametrize("seed,top_k,top_p,penalty", [(1234, 8, 0.9, 1.3), (5, 32, 1.0, 1.0)])
def test_device_sampled_loop_equals_host_sampling_with_softcap(capped, seed, top_k, top_p, penalty):
    """The device sampler softcaps the candidate scores before the draw, like the host loop
    (decode_topk -> softcap -> sample_topk_candidates): same tokens, same generator state."""
    cfg, gpu, _ = capped
    prompt = syn.prompt_ids(cfg["vocab_size"], 9, seed=4)
    steps, temperature = 16, 0.7
    gcfg = pkg.GenerationConfig(max_new_tokens=steps, temperature=temperature, top_k=top_k, top_p=top_p,
                                repetition_penalty=penalty, eos_token_ids=[], seed=seed)
    t_host = gpu.new_cache_table(40, kv_dtype=pkg.F32)
    first = int(np.argmax(gpu.prefill_prompt(prompt, t_host)))
    rnd = np.array([seed], dtype=np.uint64)
    tok, host_ids = first, []
    for _ in range(steps):
        cand = gpu.decode_topk(tok, t_host, top_k, penalty, True)
        tok = pkg.sample_topk_candidates(cand, gcfg, rnd)
        host_ids.append(tok)
    t_dev = gpu.new_cache_table(40, kv_dtype=pkg.F32)
    gpu.prefill_prompt(prompt, t_dev)
    dev_ids, state, _ = gpu.decode_sampled(first, t_dev, steps, top_k, temperature, top_p, penalty, [seed])
    assert dev_ids.ravel().tolist() == host_ids
    assert int(state[0]) == int(rnd[0])


# ---- failure paths, made on the host: no GPU fault, trap or hang ------------------------------------------

@pytest.mark.parametrize("kind", [1, 2])
def test_bounded_wait_runs_out_and_reports_timeout(c1, kind):
    """A device-side wait on something nobody signals (kind 1: an mbarrier phase, the wait of the TMA /
    tcgen05 / attention pipelines; kind 2: a tensor-parallel peer flag) with a small polling budget: the
    kernel returns, the status word is raised, the call returns OXG4_TIMEOUT, and the next calls work."""
    cfg, gpu, oracle = c1
    N = pkg._native
    table = gpu.new_cache_table(16, kv_dtype=pkg.F32)
    before = gpu.decode_token(5, table)
    st = N.lib().oxg4_debug_wait_timeout(gpu._h, table._h, kind, 2000)
    assert N.STATUS_NAMES[st] == "TIMEOUT"
    assert b"bounded wait ran out" in N.lib().oxg4_last_error()
    table.reset()
    after = gpu.decode_token(5, table)                    # the context and the table are still usable
    assert np.array_equal(before, after)
    assert N.lib().oxg4_debug_wait_timeout(gpu._h, table._h, 3, 2000) == 2      # INVALID_ARGUMENT


def test_synthetic_cache_fill_sets_positions_and_decodes(c1):
    """The measurement aid behind `bench.py --cache-fill synthetic`: positions advance to the given lengths, the
    pools hold finite values (decode steps return finite logits, twice the same on two tables), and a table
    that already holds tokens is refused."""
    cfg, gpu, oracle = c1
    outs = []
    for kv in (pkg.F32, pkg.BF16):
        for _ in range(2):
            table = gpu.new_cache_table([40, 24], batch=2, kv_dtype=kv)
            table.fill_synthetic([33, 7])
            assert [table.position(0), table.position(1)] == [33, 7]
            logits = gpu.decode_token(np.array([3, 9], dtype=np.uint32), table)
            assert np.isfinite(logits).all()
            assert [table.position(0), table.position(1)] == [34, 8]
            outs.append(logits)
        assert np.array_equal(outs[-1], outs[-2])
    with pytest.raises(pkg.Oxg4Error, match="empty cache table"):
        table.fill_synthetic([1, 1])
    fresh = gpu.new_cache_table([8, 8], batch=2, kv_dtype=pkg.F32)
    with pytest.raises(pkg.Oxg4Error, match="does not fit"):
        fresh.fill_synthetic([9, 1])


def test_cache_create_out_of_memory_leaks_nothing(c1):
    """An allocation that fails in the middle of oxg4_cache_create (injected on the host): OXG4_OOM comes
    back, no handle is produced and the driver's free-memory figure returns to what it was."""
    import torch
    cfg, gpu, oracle = c1
    N = pkg._native
    gpu.new_cache_table(16, kv_dtype=pkg.F32).close()     # warm: kernels loaded, pools of the driver settled
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    for nth in (1, 7, 23):
        N.lib().oxg4_debug_fail_alloc_after(nth)
        with pytest.raises(pkg.Oxg4Error) as e:
            gpu.new_cache_table(16, kv_dtype=pkg.F32)
        assert e.value.kind == "OOM"
        N.lib().oxg4_debug_fail_alloc_after(0)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free0, nth
    t = gpu.new_cache_table(16, kv_dtype=pkg.F32)         # and creation works again
    assert t.position() == 0


def test_state_closed_before_its_table_does_not_crash():
    """Finalisers of objects in a reference cycle run in no particular order: a model that goes first takes
    its live cache tables with it, and the table's own close then only forgets the handle."""
    cfg = small_cfg(hidden=64, layers=1, heads=2, kv_heads=1, head_dim=64, inter=128, vocab=300, window=8,
                    layer_types=["full_attention"])
    gpu, _ = build_pair(cfg, "f32", kv_bf16=False, want_oracle=False)
    t1 = gpu.new_cache_table(8, kv_dtype=pkg.F32)
    t2 = gpu.new_cache_table(8, kv_dtype=pkg.BF16)
    gpu.decode_token(3, t1)
    t2.close()
    gpu.close()
    t1.close()
    t1.close()
