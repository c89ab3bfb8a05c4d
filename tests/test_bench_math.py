"""Host-side arithmetic behind the benchmark's roofline figures and the binding table (no GPU)."""
import importlib
import os
import re
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402

pkg = importlib.import_module("oxide-beta_b200")
syn = pkg.synthetic


def test_algorithmic_bytes_of_the_4b_workload_by_hand():
    """bytes per decode step = weights of every projection + tied LM head + visible K/V of every layer
    (sliding layers see min(context, window) positions), BF16 everywhere."""
    cfg = syn.workload("c3")["cfg"]
    H, D, Nq, Nkv, I, V, L = 2560, 256, 8, 4, 10240, 262144, 34
    assert (cfg["hidden_size"], cfg["head_dim"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
            cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]) == (H, D, Nq, Nkv, I, V, L)
    per_layer = (H * (Nq + 2 * Nkv) * D + Nq * D * H + 3 * H * I) * 2
    weights = L * per_layer + V * H * 2
    n_global = sum(t == "full_attention" for t in cfg["layer_types"])
    ctx = 2579
    kv = (n_global * ctx + (L - n_global) * min(ctx, cfg["sliding_window"])) * 2 * Nkv * D * 2
    total, parts = bench.algorithmic_bytes(cfg, 1, [ctx])
    assert parts["weights"] == weights and parts["kv"] == kv and total == weights + kv
    assert parts["gateup_launch"] == 2 * I * H * 2 == 104857600
    assert total == 7933915136                       # the figure the bench line reports as step_bytes


def test_algorithmic_bytes_sum_over_ragged_contexts():
    cfg = syn.workload("c5")["cfg"]
    lens = syn.ragged_lengths(64, 1024, 32768, seed=2).tolist()
    assert len(lens) == 64 and min(lens) >= 1024 and max(lens) <= 32768
    total, parts = bench.algorithmic_bytes(cfg, 64, lens)
    one_by_one = sum(bench.algorithmic_bytes(cfg, 1, [n])[1]["kv"] for n in lens)
    assert parts["kv"] == one_by_one                  # K/V bytes add up over the sequences, weights are read once
    assert total == parts["weights"] + one_by_one


def test_every_declared_entry_point_has_a_ctypes_prototype():
    header = open(os.path.join(ROOT, "include", "oxg4.h")).read()
    declared = set(re.findall(r"\b(oxg4_[a-z0-9_]+)\s*\(", header))
    table = open(os.path.join(ROOT, "oxide-beta_b200", "_native.py")).read()
    bound = set(re.findall(r'"(oxg4_[a-z0-9_]+)"\s*:', table))
    assert declared - bound == set(), sorted(declared - bound)


def test_peaks_prefers_the_measured_file():
    peak, kind = bench.peaks()
    assert peak > 0 and kind in ("measured", "fallback")
    if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")):
        assert kind == "measured"
    else:
        assert (peak, kind) == (6650.0, "fallback")
