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
        before = torch.cuda.memory_allocated()
        N.check(N.lib().oxg4_topk_noalloc(C.c_void_p(d_logits.data_ptr()), 1, V, C.c_void_p(d_seen.data_ptr()),
                                          penalty, k, C.c_void_p(d_ids.data_ptr()),
                                          C.c_void_p(d_scores.data_ptr()), None))
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
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
