"""CPU tests of the C-ABI boundary and the host-side logic. No compute call needs a GPU here."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from util import ROOT, orc, pkg, syn

N = pkg._native


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "oxg4.h")).read()
    declared = set(re.findall(r"\b(oxg4_[a-z0-9_]+)\s*\(", header))
    declared -= {"oxg4_token_callback"}
    assert declared, "no declarations found"
    lib = C.CDLL(pkg.library_path())
    for name in sorted(declared):
        assert hasattr(lib, name), f"liboxg4.so does not export {name}"
    assert declared == set(N.SYMBOLS), declared ^ set(N.SYMBOLS)


def test_struct_layouts_match_header():
    # field order and count of the ctypes mirrors follow the header's structs
    header = open(os.path.join(ROOT, "include", "oxg4.h")).read()
    body = re.search(r"typedef struct \{([^}]*)\} oxg4_config;", header, re.S).group(1)
    names = re.findall(r"(\w+);", re.sub(r"/\*.*?\*/", "", body, flags=re.S))
    assert names == [f[0] for f in N.Config._fields_]
    body = re.search(r"typedef struct \{([^}]*)\} oxg4_generation_config;", header, re.S).group(1)
    names = re.findall(r"(\w+);", re.sub(r"/\*.*?\*/", "", body, flags=re.S))
    assert names == [f[0] for f in N.GenerationConfigC._fields_]


def test_invalid_configuration_is_rejected_before_cuda():
    cfg = syn.workload("c1")["cfg"]
    bad = dict(cfg, num_key_value_heads=3)
    with pytest.raises(pkg.Oxg4Error) as e:
        pkg.Gemma4TextConfig(bad)
    assert e.value.kind == "INVALID_SHAPE"
    c = pkg.Gemma4TextConfig(cfg)
    c.num_key_value_heads = 3                         # bypass the Python check: the library re-checks
    with pytest.raises(pkg.Oxg4Error) as e:
        pkg.Gemma4CudaState(c, 0, pkg.F32)
    assert e.value.kind == "INVALID_SHAPE"
    c = pkg.Gemma4TextConfig(dict(cfg, global_head_dim=512))
    with pytest.raises(pkg.Oxg4Error) as e:
        pkg.Gemma4CudaState(c, 0, pkg.F32)
    assert e.value.kind == "UNSUPPORTED"


def test_null_handles_return_status_not_crash():
    lib = N.lib()
    assert lib.oxg4_model_finalize(None) == 2
    assert lib.oxg4_decode_topk(None, None, None, 1, 1.0, 0, None, None) == 2
    assert lib.oxg4_cache_reset(None) == 2
    assert b"null" in lib.oxg4_last_error()
    assert lib.oxg4_weight_count(None) == 0
    lib.oxg4_model_destroy(None)
    lib.oxg4_cache_destroy(None)


def test_no_cpu_fallback_without_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    c = pkg.Gemma4TextConfig(syn.workload("c1")["cfg"])
    with pytest.raises(pkg.Oxg4Error) as e:
        pkg.Gemma4CudaState(c, 0, pkg.F32)
    assert e.value.kind == "CUDA" and "no CPU path" in e.value.message


def test_text_config_defaults_follow_reference():
    # config.rs:162-205: every 6th and the last layer are global; default rope parameters
    c = pkg.Gemma4TextConfig({"num_hidden_layers": 8, "num_attention_heads": 8, "num_key_value_heads": 4,
                              "hidden_size": 64})
    assert c.layer_types == ["sliding_attention"] * 5 + ["full_attention", "sliding_attention", "full_attention"]
    assert c.rope_parameters["sliding_attention"]["rope_theta"] == 10000.0
    assert c.rope_parameters["full_attention"]["partial_rotary_factor"] == 0.25
    with pytest.raises(pkg.Oxg4Error):
        pkg.Gemma4TextConfig({"num_hidden_layers": 2, "layer_types": ["full_attention"]})
    nested = pkg.Gemma4TextConfig({"text_config": {"num_hidden_layers": 3, "hidden_size": 32}})
    assert nested.num_hidden_layers == 3


def test_generation_config_validation_messages():
    m = pkg.Gemma4ForCausalLM.from_weights(syn.workload("c1")["cfg"],
                                           dict(syn.generate_weights(syn.workload("c1")["cfg"], 0, "f32")),
                                           pkg.Device.Cpu())
    G = pkg.GenerationConfig
    for g, msg in [(G(temperature=0.0), "temperature"), (G(top_p=1.5), "top_p"), (G(top_k=0), "top_k"),
                   (G(repetition_penalty=0.5), "repetition_penalty"),
                   (G(stop_token_sequences=[[]]), "stop-token")]:
        with pytest.raises(pkg.Oxg4Error) as e:
            m.generate([1, 2, 3], g)
        assert msg in e.value.message
    with pytest.raises(pkg.Oxg4Error) as e:
        m.generate([], G())
    assert "at least one input token" in e.value.message
    with pytest.raises(pkg.Oxg4Error) as e:
        m.generate([1], G())
    assert "requires Device::Cuda" in e.value.message       # generation.rs:82-86


def test_generation_config_defaults():
    g = pkg.GenerationConfig()
    assert (g.max_new_tokens, g.temperature, g.top_k, g.top_p, g.repetition_penalty) == (128, 1.0, 64, 0.95, 1.1)
    assert g.eos_token_ids == [1, 50, 106] and g.seed == 0x4D595DF4D0F33173


def test_host_sampling_matches_oracle():
    rng = np.random.default_rng(5)
    logits = (rng.standard_normal(2000) * 2).astype(np.float32)
    logits[17] = np.nan
    for temp, k, p in [(1.0, 64, 0.95), (0.7, 8, 1.0), (1.3, 1, 0.5), (1.0, 5000, 0.9)]:
        g = pkg.GenerationConfig(temperature=temp, top_k=k, top_p=p)
        r1 = np.array([g.seed], dtype=np.uint64)
        r2 = np.array([g.seed], dtype=np.uint64)
        ours = [pkg.sample_token(logits, g, r1) for _ in range(40)]
        ref = [orc.sample_token(logits, temp, k, p, r2) for _ in range(40)]
        assert ours == ref and r1[0] == r2[0]
        ids, scores = orc.topk(logits, min(k, 64))
        r1[0] = r2[0] = 99
        ours = [pkg.sample_topk_candidates(list(zip(ids, scores)), g, r1) for _ in range(40)]
        ref = [orc.sample_topk_candidates(ids, scores, temp, p, r2) for _ in range(40)]
        assert ours == ref
    r = np.array([0], dtype=np.uint64)                  # zero state is re-seeded (sampling.rs:57-59)
    pkg.sample_token([0.0, 1.0], pkg.GenerationConfig(), r)
    assert r[0] != 0
    with pytest.raises(pkg.Oxg4Error):
        pkg.sample_token([], pkg.GenerationConfig(), r)
    with pytest.raises(pkg.Oxg4Error):
        pkg.sample_token([np.nan, np.inf], pkg.GenerationConfig(), r)


def test_checkpoint_round_trip(tmp_path):
    cfg = syn.workload("c1")["cfg"]
    for dtype in ("f32", "bf16"):
        d = str(tmp_path / dtype)
        w = dict(syn.generate_weights(cfg, 0, dtype))
        syn.write_checkpoint(d, cfg, w.items(), dtype)
        cfg2, w2 = syn.read_checkpoint(d)
        assert cfg2["hidden_size"] == cfg["hidden_size"]
        assert set(w2) == set(w)
        for k in w:
            assert np.array_equal(np.asarray(w2[k]), w[k])
        m = pkg.Gemma4ForCausalLM.from_pretrained(d, pkg.Device.Cpu())
        assert m.config().num_hidden_layers == 2
        e = m.embed([3, 7])
        assert e.shape == (2, cfg["hidden_size"])
        raw = w["embed_tokens.weight"][3]
        raw = syn.bf16_bits_to_f32(raw) if dtype == "bf16" else raw
        np.testing.assert_array_equal(e[0], raw * np.float32(16.0))     # sqrt(256)


def test_workload_table_matches_specification():
    c2, c3, c5 = (syn.workload(n)["cfg"] for n in ("c2", "c3", "c5"))
    assert c2["layer_types"].count("full_attention") == 4 and len(c2["layer_types"]) == 26
    assert c3["layer_types"].count("full_attention") == 5 and c3["layer_types"][5] == "full_attention"
    assert c5["num_attention_heads"] // c5["num_key_value_heads"] == 2 and c5["head_dim"] == 128
    names = [n for n, _, _ in syn.weight_names(c2)]
    assert names[0] == "embed_tokens.weight" and names[-1] == "norm.weight"
    assert len(names) == 2 + 14 * 26
    lens = syn.ragged_lengths(64, 1024, 32768, seed=2)
    assert lens.min() >= 1024 and lens.max() <= 32768


def test_tp_group_create_fails_loudly_without_a_device_or_on_bad_arguments():
    """The single-process tensor-parallel handle reports its workers' failures to the calling thread."""
    import ctypes as C
    import torch
    N = pkg._native
    cfg = pkg.Gemma4TextConfig(syn.workload("c1")["cfg"])
    from importlib import import_module
    g4 = import_module("oxide-beta_b200.gemma4")
    c, keep = g4._native_config(cfg, pkg.F32, 0, 0, 2)
    h = C.c_void_p()
    dev = (C.c_int32 * 2)(0, 0)
    assert N.lib().oxg4_tp_model_create(C.byref(c), dev, 2, C.byref(h)) == 2          # same device twice
    assert b"own device" in N.lib().oxg4_last_error()
    dev = (C.c_int32 * 3)(0, 1, 2)
    assert N.lib().oxg4_tp_model_create(C.byref(c), dev, 3, C.byref(h)) == 2          # tp must be 1, 2, 4 or 8
    if not torch.cuda.is_available():
        dev = (C.c_int32 * 1)(0)
        st = N.lib().oxg4_tp_model_create(C.byref(c), dev, 1, C.byref(h))
        assert N.STATUS_NAMES[st] == "CUDA" and not h.value
        assert b"rank 0" in N.lib().oxg4_last_error() and b"no CPU path" in N.lib().oxg4_last_error()
