"""Generates tests/golden/c1_hf_gemma4.npz: an independent f32 cross-check of the CPU oracle.

Hugging Face Transformers' Gemma4ForCausalLM is the model the reference's own validation script
(scripts/reference_gemma4.py:8,43-46) treats as ground truth. This script instantiates it on the
CPU in f32 with the tiny two-layer configuration, loads the seeded synthetic weights produced by
the package's generator, and records
  - the 16-token prompt (seed 1), the 32 greedy token ids, the logits of the first and the last
    decode step;
  - the final-position logits of a 200-token prompt (longer than the 128-token sliding window).
The fixture is consumed by tests/test_oracle.py on machines without transformers or the reference.

Run from the repository root:  python tests/golden/make_hf_fixture.py
"""
import importlib
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
synthetic = importlib.import_module("oxide-beta_b200.synthetic")


def build_hf(cfg, weights):
    from transformers import Gemma4ForCausalLM, Gemma4TextConfig
    keys = ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
            "num_attention_heads", "num_key_value_heads", "head_dim", "global_head_dim",
            "rms_norm_eps", "sliding_window", "layer_types", "rope_parameters",
            "hidden_size_per_layer_input", "vocab_size_per_layer_input", "num_kv_shared_layers", "attention_k_eq_v",
            "final_logit_softcapping", "tie_word_embeddings", "hidden_activation"]
    hf_cfg = Gemma4TextConfig(**{k: cfg[k] for k in keys if k in cfg}, attn_implementation="eager")
    model = Gemma4ForCausalLM(hf_cfg).to(torch.float32).eval()
    sd = model.state_dict()
    seen = set()
    for name, a in weights.items():
        key = "model." + name
        if key not in sd:
            raise KeyError(key)
        t = torch.from_numpy(np.array(a, dtype=np.float32)).reshape(sd[key].shape)
        sd[key].copy_(t)
        seen.add(key)
    # HF keeps (unused) k/v projections and k norms on KV-shared layers; the reference's loader and this
    # package's checkpoints have a q projection only there (gemma4_cuda/mod.rs:287, 420-424)
    shared_from = cfg["num_hidden_layers"] - int(cfg.get("num_kv_shared_layers") or 0)
    unused = {f"model.layers.{l}.self_attn.{n}.weight" for l in range(shared_from, cfg["num_hidden_layers"])
              for n in ("k_proj", "v_proj", "k_norm")}
    missing = [k for k in sd if k not in seen and k not in unused and "lm_head" not in k and "rotary" not in k]
    if missing:
        raise RuntimeError(f"HF tensors without a synthetic counterpart: {missing}")
    return model


@torch.no_grad()
def main():
    w = synthetic.workload("c1")
    cfg = w["cfg"]
    weights = dict(synthetic.generate_weights(cfg, seed=0, dtype="f32"))
    model = build_hf(cfg, weights)
    prompt = synthetic.prompt_ids(cfg["vocab_size"], 16, seed=1)
    ids = torch.from_numpy(prompt.astype(np.int64))[None]
    out = model(ids, use_cache=True)
    past = out.past_key_values
    logits = out.logits[0, -1].float().numpy()
    first_logits = logits.copy()
    tokens, margins = [], []
    last_logits = None
    for step in range(32):
        order = np.argsort(-logits, kind="stable")
        tokens.append(int(order[0]))
        margins.append(float(logits[order[0]] - logits[order[1]]))
        out = model(torch.tensor([[tokens[-1]]]), past_key_values=past, use_cache=True)
        past = out.past_key_values
        logits = out.logits[0, -1].float().numpy()
        if step == 30:
            last_logits = logits.copy()     # logits that select token 31
    long_prompt = synthetic.prompt_ids(cfg["vocab_size"], 200, seed=3)
    long_logits = model(torch.from_numpy(long_prompt.astype(np.int64))[None]).logits[0, -1].float().numpy()
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "c1_hf_gemma4.npz")
    np.savez_compressed(path, prompt=prompt, tokens=np.array(tokens, dtype=np.uint32),
                        first_logits=first_logits, last_logits=last_logits,
                        margins=np.array(margins, dtype=np.float32),
                        long_prompt=long_prompt, long_logits=long_logits)
    print("wrote", path, "min top1-top2 margin", min(margins))
    e_fixture()


@torch.no_grad()
def e_fixture():
    """tests/golden/e_tiny_hf_gemma4.npz: the Gemma4-E features on a tiny configuration (see
    synthetic.e_tiny_cfg): global_head_dim != head_dim with proportional partial RoPE on the global
    layers, two KV-shared layers, per-layer embeddings. Logits at every position of a 40-token prompt
    and 12 greedy tokens."""
    cfg = synthetic.e_tiny_cfg()
    weights = dict(synthetic.generate_weights(cfg, seed=0, dtype="f32", norm_jitter=0.1))
    model = build_hf(cfg, weights)
    prompt = synthetic.prompt_ids(cfg["vocab_size"], 40, seed=5)
    out = model(torch.from_numpy(prompt.astype(np.int64))[None], use_cache=True)
    logits = out.logits[0].float().numpy()
    past = out.past_key_values
    tokens, cur = [], logits[-1]
    for _ in range(12):
        tokens.append(int(np.argsort(-cur, kind="stable")[0]))
        out = model(torch.tensor([[tokens[-1]]]), past_key_values=past, use_cache=True)
        past = out.past_key_values
        cur = out.logits[0, -1].float().numpy()
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "e_tiny_hf_gemma4.npz")
    np.savez_compressed(path, prompt=prompt, logits=logits.astype(np.float32), tokens=np.array(tokens, dtype=np.uint32))
    print("wrote", path)


if __name__ == "__main__":
    main()
