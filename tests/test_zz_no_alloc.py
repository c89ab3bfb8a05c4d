"""GPU test of oxg4_topk_noalloc, the top-k entry point for callers that may not allocate device
memory (stream capture in progress, fixed-budget serving loops, hosts with their own arena).

It must return exactly what the usual path returns. The usual path is oxg4_decode_topk, whose
candidate lists live in buffers of the cache table; here the same logits (obtained from a second
cache table with oxg4_decode_logits on the same token history) go through the allocation-free entry
point, twice in a row, because the second call finds the first call's leftovers in the shared array.
This file sorts last so that a run stopping at the first failure has already run everything else.
"""
import ctypes as C

import numpy as np
import pytest

from util import build_pair, pkg, syn

pytestmark = pytest.mark.gpu


def _numpy_topk(logits, seen, penalty, k):
    """Descending score, lowest index first among equal scores; repetition penalty on seen ids."""
    s = logits.astype(np.float32).copy()
    if seen is not None and penalty > 1.0:
        hit = seen != 0
        s[hit] = np.where(s[hit] >= 0, s[hit] / np.float32(penalty), s[hit] * np.float32(penalty))
    order = np.lexsort((np.arange(s.size), -s))[:k]
    return order.astype(np.uint32), s[order]


def test_topk_noalloc_large_vocabulary_four_rows_against_numpy():
    """Four rows of a 262144-entry vocabulary, top-k 64 then 5, with and without the repetition penalty.
    Run alone in a fresh process this is the entry point's very first call on the device, so its own
    set-up (symbol address, shared-memory opt-in of the merge kernel, which needs 64 KiB here) is what
    runs. The driver's free-memory figure (cudaMemGetInfo), which also sees allocations made inside the
    library, must not move across a call."""
    import torch
    N = pkg._native
    rows, V = 4, 262144
    rng = np.random.default_rng(7)
    logits = rng.standard_normal((rows, V)).astype(np.float32)
    logits[:, 1000] = logits[:, 5]                                # exact ties: the lower id must come first
    logits[1, 77] = np.nan                                        # NaN is never selected
    seen = (rng.random((rows, V)) < 0.01).astype(np.uint8)
    d_logits = torch.from_numpy(logits).cuda()
    d_seen = torch.from_numpy(seen).cuda()
    for call, (k, penalty, use_seen) in enumerate([(64, 1.0, False), (5, 1.7, True), (64, 1.2, True)]):
        d_ids = torch.zeros((rows, k), dtype=torch.int32, device="cuda")
        d_scores = torch.zeros((rows, k), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        N.check(N.lib().oxg4_topk_noalloc(C.c_void_p(d_logits.data_ptr()), rows, V,
                                          C.c_void_p(d_seen.data_ptr()) if use_seen else None, penalty, k,
                                          C.c_void_p(d_ids.data_ptr()), C.c_void_p(d_scores.data_ptr()), None))
        torch.cuda.synchronize()
        if call > 0:                 # the first call may load the kernels' module; later calls change nothing
            assert torch.cuda.mem_get_info()[0] == free_before
        ids = d_ids.cpu().numpy().view(np.uint32)
        scores = d_scores.cpu().numpy()
        for r in range(rows):
            row = np.where(np.isnan(logits[r]), -np.inf, logits[r])
            want_ids, want_scores = _numpy_topk(row, seen[r] if use_seen else None, penalty, k)
            assert ids[r].tolist() == want_ids.tolist(), (call, r)
            np.testing.assert_array_equal(scores[r], want_scores)


def test_topk_noalloc_matches_decode_topk_twice():
    import torch
    N = pkg._native
    cfg = syn.workload("c1")["cfg"]
    gpu, _ = build_pair(cfg, "f32", kv_bf16=False, want_oracle=False)
    V = cfg["vocab_size"]
    prompt = syn.prompt_ids(V, 9, seed=21)
    t_topk = gpu.new_cache_table(32, kv_dtype=pkg.F32)
    t_logits = gpu.new_cache_table(32, kv_dtype=pkg.F32)
    gpu.prefill_prompt(prompt, t_topk, want_logits=False)
    gpu.prefill_prompt(prompt, t_logits, want_logits=False)
    seen = np.zeros((1, V), dtype=np.uint8)
    tok = 11
    for call, (k, penalty) in enumerate([(64, 1.0), (7, 1.5)]):
        seen[0, tok] = 1                                        # decode_topk(mark_seen=True) marks the fed token
        want = gpu.decode_topk(tok, t_topk, k, penalty, True)   # existing entry point
        logits = gpu.decode_token(tok, t_logits)                # same history, full logits
        d_logits = torch.from_numpy(np.ascontiguousarray(logits[None])).cuda()
        d_seen = torch.from_numpy(seen).cuda()
        d_ids = torch.zeros((1, k), dtype=torch.int32, device="cuda")
        d_scores = torch.zeros((1, k), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        # free device memory as the driver reports it: unlike torch's own counter it would also show a
        # cudaMalloc made inside the library
        free_before = torch.cuda.mem_get_info()[0]
        N.check(N.lib().oxg4_topk_noalloc(C.c_void_p(d_logits.data_ptr()), 1, V, C.c_void_p(d_seen.data_ptr()),
                                          penalty, k, C.c_void_p(d_ids.data_ptr()),
                                          C.c_void_p(d_scores.data_ptr()), None))
        torch.cuda.synchronize()
        if call > 0:
            assert torch.cuda.mem_get_info()[0] == free_before
        ids = d_ids.cpu().numpy().view(np.uint32)[0]
        scores = d_scores.cpu().numpy()[0]
        assert ids.tolist() == [w[0] for w in want], call
        # same kernels on the same logits: the parity tests' f32 tolerance is met with room to spare
        np.testing.assert_allclose(scores, [w[1] for w in want], rtol=0, atol=1e-3)
        tok = int(ids[0])


def test_topk_noalloc_rejects_sizes_beyond_its_array():
    N = pkg._native
    dummy = C.c_void_p(16)
    assert N.lib().oxg4_topk_noalloc(dummy, 5, 1024, None, 1.0, 4, dummy, dummy, None) == 1
    assert b"rows" in N.lib().oxg4_last_error()
    assert N.lib().oxg4_topk_noalloc(dummy, 1, 524289, None, 1.0, 4, dummy, dummy, None) == 1
    assert b"vocabulary" in N.lib().oxg4_last_error()
    assert N.lib().oxg4_topk_noalloc(None, 1, 1024, None, 1.0, 4, dummy, dummy, None) == 2
