"""A C program (tests/c_driver.c) that calls the C ABI the way the reference's Rust side would through a
`-sys` crate: create -> upload -> finalize -> cache -> prefill -> decode_topk -> destroy on the tiny f32
configuration. Without a CUDA device the library must refuse loudly (OXG4_CUDA, no CPU path); on a GPU the
32 greedy tokens must equal the committed Hugging Face fixture."""
import os
import struct
import subprocess

import numpy as np
import pytest

from util import ROOT, pkg, syn

GOLDEN = os.path.join(ROOT, "tests", "golden", "c1_hf_gemma4.npz")


def _build(tmp_path):
    exe = os.path.join(str(tmp_path), "c_driver")
    libdir = os.path.dirname(pkg.library_path())
    pkg._native.lib()                                  # makes sure liboxg4.so exists
    subprocess.check_call(["gcc", "-O1", "-Wall", "-Werror", "-std=c99", os.path.join(ROOT, "tests", "c_driver.c"),
                           "-I", os.path.join(ROOT, "include"), "-L", libdir, "-l:liboxg4.so",
                           "-Wl,-rpath," + libdir, "-o", exe])
    return exe


def _write_case(path, cfg, prompt, n_decode, weights, weight_dtype, kv_dtype):
    tc = pkg.Gemma4TextConfig(cfg)
    L = tc.num_hidden_layers
    with open(path, "wb") as f:
        f.write(b"OXG4TEST")
        f.write(struct.pack("<10i", tc.vocab_size, tc.hidden_size, L, tc.num_attention_heads, tc.num_key_value_heads,
                            tc.head_dim, tc.intermediate_size, tc.sliding_window, weight_dtype, kv_dtype))
        f.write(struct.pack("<f", tc.rms_norm_eps))
        sliding = [1 if t == "sliding_attention" else 0 for t in tc.layer_types]
        rp = [tc.rope_parameters[t] for t in tc.layer_types]
        f.write(np.asarray(sliding, dtype=np.int32).tobytes())
        f.write(np.asarray([int(np.float32(r.get("partial_rotary_factor", 1.0)) * np.float32(tc.head_dim)) for r in rp],
                           dtype=np.int32).tobytes())
        f.write(np.asarray([r["rope_theta"] for r in rp], dtype=np.float32).tobytes())
        f.write(np.asarray([r.get("factor", 1.0) for r in rp], dtype=np.float32).tobytes())
        p = np.ascontiguousarray(prompt, dtype=np.uint32)
        f.write(struct.pack("<I", p.size))
        f.write(p.tobytes())
        f.write(struct.pack("<I", n_decode))
        f.write(struct.pack("<I", len(weights)))
        for name, a in weights:
            a = np.ascontiguousarray(a)
            nm = ("model.language_model." + name).encode()        # the checkpoint's own names, prefix included
            f.write(struct.pack("<I", len(nm)))
            f.write(nm)
            f.write(struct.pack("<II", pkg.BF16 if a.dtype == np.uint16 else pkg.F32, a.ndim))
            f.write(np.asarray(a.shape, dtype=np.int64).tobytes())
            f.write(struct.pack("<Q", a.nbytes))
            f.write(a.tobytes())


def _case(tmp_path):
    gold = np.load(GOLDEN)
    cfg = syn.workload("c1")["cfg"]
    weights = list(syn.generate_weights(cfg, 0, "f32"))
    path = os.path.join(str(tmp_path), "c1.bin")
    _write_case(path, cfg, gold["prompt"], 32, weights, pkg.F32, pkg.F32)
    return path, gold


def test_c_driver_refuses_without_a_device_or_matches_fixture(tmp_path):
    """Runs everywhere: on a box without a GPU the driver must see OXG4_CUDA from oxg4_model_create."""
    import torch
    exe = _build(tmp_path)
    path, gold = _case(tmp_path)
    r = subprocess.run([exe, path], capture_output=True, text=True, timeout=300)
    if torch.cuda.is_available():
        assert r.returncode == 0, r.stderr
        assert [int(t) for t in r.stdout.split(":")[1].split()] == gold["tokens"].tolist()
    else:
        assert r.returncode == 3, (r.returncode, r.stdout, r.stderr)
        assert r.stdout.startswith("NO_DEVICE:") and "no CPU path" in r.stdout


@pytest.mark.gpu
def test_c_driver_greedy_tokens_equal_fixture(tmp_path):
    exe = _build(tmp_path)
    path, gold = _case(tmp_path)
    r = subprocess.run([exe, path], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert [int(t) for t in r.stdout.split(":")[1].split()] == gold["tokens"].tolist()
