"""GPU parity at the sizes that are benchmarked: full depth, full widths, full vocabulary.

End-to-end BF16 logits of a deep random-init stack are ill-conditioned for ANY two implementations
(tests/test_oracle.py::test_summation_order_spread_grows_with_depth), so depth in the BF16 recipe is
checked layer by layer with teacher forcing, which is depth-independent by construction: the oracle
runs freely, the CUDA path receives the oracle's input of every layer (oxg4_decode_trace), and every
layer's output, the final hidden state and the logits must agree. Both sides fill their own KV caches.
The prompt is kept affordable for the CPU oracle by shrinking only `sliding_window`; widths, depth,
head counts and vocabulary are the workload's.
"""
import numpy as np
import pytest

from util import build_pair, margin, pkg, syn

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-3
TOL_BF16 = 2e-2


@pytest.mark.parametrize("name", ["c2", "c3"])
def test_layerwise_bf16_parity_full_depth_full_vocabulary(name):
    """All 26 / 34 layers and the 262144-row LM head of the ~1B / ~4B workloads, BF16 weights and BF16
    KV pages of 32 tokens, sliding window 64, 104 tokens: the sliding ring wraps and page boundaries
    are crossed on both layer kinds."""
    cfg = syn.workload(name)["cfg"]
    cfg["sliding_window"] = 64
    gpu, oracle = build_pair(cfg, "bf16", kv_bf16=True)
    L = cfg["num_hidden_layers"]
    n_tokens = cfg["sliding_window"] + 40
    prompt = syn.prompt_ids(cfg["vocab_size"], n_tokens, seed=1)
    table = gpu.new_cache_table(n_tokens, page_tokens=32, kv_dtype=pkg.BF16)
    cache = oracle.new_cache(n_tokens)
    worst_h, worst_logit, scale = 0.0, 0.0, 0.0
    for i, t in enumerate(prompt):
        want_logits = i % 8 == 7 or i >= n_tokens - 8          # the 1.3 GB LM head on the CPU: not every token
        tr_o, lg_o = cache.decode_trace(int(t), want_logits=want_logits)
        tr_g, lg_g = gpu.decode_trace(int(t), table, inject=tr_o[:L][:, None, :], want_logits=want_logits)
        worst_h = max(worst_h, float(np.abs(tr_g[:, 0] - tr_o).max()))
        scale = max(scale, float(np.abs(tr_o).max()))
        if want_logits:
            worst_logit = max(worst_logit, float(np.abs(lg_g[0] - lg_o).max()))
    assert table.position() == n_tokens
    assert worst_logit <= TOL_BF16, (worst_logit, worst_h, scale)
    assert worst_h <= TOL_BF16 * max(1.0, scale), (worst_h, scale)


def test_c2_full_depth_f32_layerwise_and_greedy_tokens():
    """The ~1B workload at its full depth (26 layers), widths and vocabulary in the f32 recipe.

    Layer by layer with teacher forcing every layer output and the logits agree to 1e-3. Free-running,
    26 random-init layers with attention scale 1.0 are ill-conditioned even in f32: the oracle run
    against ITSELF with only the summation order of the projections changed differs by ~1e-2 in logits
    at this depth (measured below, in the same test). The free-running comparison therefore asks that
    the CUDA path is no farther from the oracle than three times that spread, and that the 32 greedy
    tokens are identical wherever the oracle's own top-2 margin exceeds the difference observed."""
    from util import orc
    cfg = syn.workload("c2")["cfg"]
    cfg["sliding_window"] = 24                                   # the 24-token prompt fills the ring; decoding wraps it
    gpu, oracle = build_pair(cfg, "f32", kv_bf16=False)
    L = cfg["num_hidden_layers"]
    prompt = syn.prompt_ids(cfg["vocab_size"], 24, seed=1)
    # (1) layer-wise teacher forcing, strict f32 tolerance
    table = gpu.new_cache_table(24 + 32, page_tokens=16, kv_dtype=pkg.F32)
    cache = oracle.new_cache(24 + 32)
    worst_h, worst_logit, scale = 0.0, 0.0, 0.0
    for i, t in enumerate(prompt):
        tr_o, lg_o = cache.decode_trace(int(t), want_logits=(i >= 20))
        tr_g, lg_g = gpu.decode_trace(int(t), table, inject=tr_o[:L][:, None, :], want_logits=(i >= 20))
        worst_h = max(worst_h, float(np.abs(tr_g[:, 0] - tr_o).max()))
        scale = max(scale, float(np.abs(tr_o).max()))
        if lg_o is not None:
            worst_logit = max(worst_logit, float(np.abs(lg_g[0] - lg_o).max()))
    assert worst_logit <= TOL_F32, (worst_logit, worst_h, scale)
    assert worst_h <= TOL_F32 * max(1.0, scale), (worst_h, scale)

    # (2) free-running: oracle vs oracle under two summation orders gives the conditioning of this stack
    def oracle_run(order, forced=None):
        orc.set_accum_order(order)
        try:
            c = oracle.new_cache(24 + 32)
            for t in prompt[:-1]:
                c.prefill_token(int(t))
            lg = [c.decode_logits(int(prompt[-1]))]
            toks = []
            for i in range(8):
                toks.append(int(np.argmax(lg[-1])) if forced is None else forced[i])
                lg.append(c.decode_logits(toks[-1]))
            return np.stack(lg), toks
        finally:
            orc.set_accum_order(0)
    a, toks = oracle_run(1)
    b, _ = oracle_run(2, forced=toks)
    spread = float(np.abs(a - b).max())
    print(f"f32, 26 layers, oracle vs oracle (summation order only): logits spread {spread:.4g}")

    table = gpu.new_cache_table(24 + 32, page_tokens=16, kv_dtype=pkg.F32)
    cache = oracle.new_cache(24 + 32)
    for t in prompt[:-1]:
        cache.prefill_token(int(t))
    ref = cache.decode_logits(int(prompt[-1]))
    got = gpu.prefill_prompt(prompt, table)
    worst = float(np.abs(got - ref).max())
    for step in range(32):
        o_tok = int(np.argmax(ref))
        diff = float(np.abs(got - ref).max())
        worst = max(worst, diff)
        assert int(np.argmax(got)) == o_tok or margin(ref) <= 2 * diff, (step, margin(ref), diff)
        ref = cache.decode_logits(o_tok)
        got = gpu.decode_token(o_tok, table)
    assert worst <= max(TOL_F32, 3 * spread), (worst, spread)


def _ragged_lens(batch, long_lens, seed):
    rng = np.random.default_rng(seed)
    lens = rng.integers(3, 41, size=batch).tolist()
    for i, n in enumerate(long_lens):
        lens[(i * 7 + 1) % batch] = n
    return lens


@pytest.mark.parametrize("name,batch,layers", [("c3", 16, 2), ("c4", 32, 1), ("c5", 64, 1)])
def test_tcgen05_step_at_benchmark_widths(name, batch, layers):
    """The step used for eight or more sequences (tcgen05 projections fed by TMA, per-row norm / GeGLU
    kernels, K-split summation, batch attention) at the real widths of the ~4B / ~12B / ~27B workloads
    with their batch sizes, against one oracle per sequence: ragged contexts, two of which cross a
    256-token page. Layer-wise teacher forcing; logits and every layer output within the BF16 tolerance."""
    cfg = syn.scaled_down(syn.workload(name)["cfg"], layers=layers, vocab=8192)
    gpu, oracle = build_pair(cfg, "bf16", kv_bf16=True)
    L, H = layers, cfg["hidden_size"]
    lens = _ragged_lens(batch, [262, 275], seed=batch)
    prompts = [syn.prompt_ids(cfg["vocab_size"], n, seed=300 + b) for b, n in enumerate(lens)]
    table = gpu.new_cache_table([n + 2 for n in lens], batch=batch, page_tokens=256, kv_dtype=pkg.BF16)
    caches = [oracle.new_cache(n + 2) for n in lens]
    worst_h, worst_logit, scale = 0.0, 0.0, 0.0
    for t in range(max(lens)):
        active = [b for b in range(batch) if t < lens[b]]
        toks = np.full(batch, pkg.INACTIVE, dtype=np.uint32)
        inject = np.zeros((L, batch, H), dtype=np.float32)
        refs = {}
        for b in active:
            toks[b] = prompts[b][t]
            # logits where they are cheap to compare: the last tokens of every sequence and the page crossing
            tr_o, lg_o = caches[b].decode_trace(int(prompts[b][t]), want_logits=(t >= lens[b] - 3 or t in (255, 256, 257)))
            inject[:, b] = tr_o[:L]
            refs[b] = (tr_o, lg_o)
        tr_g, lg_g = gpu.decode_trace(toks, table, inject=inject)
        for b in active:
            tr_o, lg_o = refs[b]
            worst_h = max(worst_h, float(np.abs(tr_g[:, b] - tr_o).max()))
            scale = max(scale, float(np.abs(tr_o).max()))
            if lg_o is not None:
                worst_logit = max(worst_logit, float(np.abs(lg_g[b] - lg_o).max()))
    assert [table.position(b) for b in range(batch)] == lens
    assert worst_logit <= TOL_BF16, (worst_logit, worst_h, scale)
    assert worst_h <= TOL_BF16 * max(1.0, scale), (worst_h, scale)
