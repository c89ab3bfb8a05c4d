"""Synthetic Gemma4 text configurations and seeded random-init checkpoints.

The five workloads are the ones the benchmark specification names; no public checkpoint or
dataset is involved. Tensor names and shapes follow what the reference's loader expects
(crates/oxide-torch-models/src/gemma4_cuda/mod.rs:236-350, 414-447): every name lives under
"model.language_model."; this module yields the canonical names with that prefix removed and
`write_checkpoint` adds it back.

Every projection matrix is N(0, 0.02) from `numpy.random.default_rng(seed)`, drawn in the fixed
order of `weight_names`. RMSNorm weights and `layer_scalar` are 1.0: the reference multiplies by
the stored weight directly (kernel_module.rs:1163-1168), so 1.0 is the "(1 + w), w = 0" of the
workload description.
"""
import json
import os
import struct

import numpy as np

PREFIX = "model.language_model."


def _layer_types(n_layers: int, period: int = 6):
    # "5 sliding-window layers then 1 global layer, repeating"
    return ["full_attention" if (i + 1) % period == 0 else "sliding_attention" for i in range(n_layers)]


def _cfg(vocab, hidden, layers, heads, kv_heads, head_dim, inter, window, layer_types=None):
    return {
        "model_type": "gemma4_text",
        "vocab_size": vocab,
        "hidden_size": hidden,
        "num_hidden_layers": layers,
        "num_attention_heads": heads,
        "num_key_value_heads": kv_heads,
        "head_dim": head_dim,
        "global_head_dim": head_dim,
        "intermediate_size": inter,
        "sliding_window": window,
        "rms_norm_eps": 1e-6,
        "layer_types": layer_types or _layer_types(layers),
        "rope_parameters": {
            "sliding_attention": {"rope_theta": 10000.0, "rope_type": "default",
                                  "partial_rotary_factor": 1.0, "factor": 1.0},
            "full_attention": {"rope_theta": 1000000.0, "rope_type": "default",
                               "partial_rotary_factor": 1.0, "factor": 1.0},
        },
        "hidden_size_per_layer_input": 0,
        "num_kv_shared_layers": 0,
        "attention_k_eq_v": False,
        "final_logit_softcapping": None,
        "tie_word_embeddings": True,
        "hidden_activation": "gelu_pytorch_tanh",
    }


CONFIGS = {
    # tiny f32 case: layer 0 sliding-window 128 (theta 1e4), layer 1 global (theta 1e6)
    "c1": dict(cfg=_cfg(4096, 256, 2, 4, 1, 64, 1024, 128,
                        ["sliding_attention", "full_attention"]),
               dtype="f32", batch=1, prompt=16, decode=32),
    "c2": dict(cfg=_cfg(262144, 1152, 26, 4, 1, 256, 6912, 512), dtype="bf16", batch=1,
               prompt=512, decode=256),
    "c3": dict(cfg=_cfg(262144, 2560, 34, 8, 4, 256, 10240, 1024), dtype="bf16", batch=1,
               prompt=2048, decode=512),
    "c3b16": dict(cfg=_cfg(262144, 2560, 34, 8, 4, 256, 10240, 1024), dtype="bf16", batch=16,
                  prompt=2048, decode=512),
    "c4": dict(cfg=_cfg(262144, 3840, 48, 16, 8, 256, 15360, 1024), dtype="bf16", batch=32,
               prompt=8192, decode=256),
    "c5": dict(cfg=_cfg(262144, 5376, 62, 32, 16, 128, 21504, 1024), dtype="bf16", batch=64,
               prompt=(1024, 32768), decode=128),
}


def e_tiny_cfg() -> dict:
    """A tiny configuration with the Gemma4-E features switched on (parity tests and the HF fixture): six layers
    (s, s, g, s, s, g), head_dim 64 / global_head_dim 128 with proportional RoPE at a quarter of the dimensions on
    the global layers, the last two layers KV-shared (layer 4 reads layer 3's cache, layer 5 reads layer 2's),
    per-layer embeddings of width 32."""
    c = _cfg(512, 128, 6, 4, 2, 64, 256, 16, ["sliding_attention", "sliding_attention", "full_attention",
                                             "sliding_attention", "sliding_attention", "full_attention"])
    c.update(global_head_dim=128, num_kv_shared_layers=2, hidden_size_per_layer_input=32,
             vocab_size_per_layer_input=512)
    c["rope_parameters"]["full_attention"].update(rope_type="proportional", partial_rotary_factor=0.25)
    return c


def workload(name: str) -> dict:
    w = CONFIGS[name]
    return dict(w, cfg=json.loads(json.dumps(w["cfg"])))


def scaled_down(cfg: dict, layers=None, vocab=None) -> dict:
    """Same architecture with fewer layers / a smaller vocabulary (for CPU-checkable parity cases)."""
    c = json.loads(json.dumps(cfg))
    if layers is not None:
        c["num_hidden_layers"] = layers
        c["layer_types"] = c["layer_types"][:layers]
    if vocab is not None:
        c["vocab_size"] = vocab
    return c


def layer_geometry(cfg: dict, l: int):
    """(head_dim, kv_heads, shares_kv) of layer l: global layers use global_head_dim and, with
    attention_k_eq_v, num_global_key_value_heads (gemma4_cuda/mod.rs:391-395, cache.rs:63-68); the last
    num_kv_shared_layers layers read an earlier layer's cache and have a q projection only (cache.rs:43-86)."""
    sliding = cfg["layer_types"][l] == "sliding_attention"
    D = cfg["head_dim"] if sliding else cfg.get("global_head_dim", cfg["head_dim"])
    kvh = cfg["num_key_value_heads"]
    if not sliding and cfg.get("attention_k_eq_v") and cfg.get("num_global_key_value_heads"):
        kvh = cfg["num_global_key_value_heads"]
    shared = l >= cfg["num_hidden_layers"] - int(cfg.get("num_kv_shared_layers") or 0)
    return D, kvh, shared


def weight_names(cfg: dict):
    """(name, shape, kind) in generation order. kind: 'matrix' | 'ones'."""
    H = cfg["hidden_size"]
    Nq, I, L = cfg["num_attention_heads"], cfg["intermediate_size"], cfg["num_hidden_layers"]
    P = int(cfg.get("hidden_size_per_layer_input") or 0)
    out = [("embed_tokens.weight", (cfg["vocab_size"], H), "matrix")]
    if P:
        out += [("embed_tokens_per_layer.weight", (cfg["vocab_size_per_layer_input"], L * P), "matrix"),
                ("per_layer_model_projection.weight", (L * P, H), "matrix"),
                ("per_layer_projection_norm.weight", (P,), "ones")]
    for l in range(L):
        p = f"layers.{l}."
        D, Nkv, shared = layer_geometry(cfg, l)
        out += [(p + "input_layernorm.weight", (H,), "ones"),
                (p + "self_attn.q_proj.weight", (Nq * D, H), "matrix")]
        if not shared:
            out += [(p + "self_attn.k_proj.weight", (Nkv * D, H), "matrix"),
                    (p + "self_attn.v_proj.weight", (Nkv * D, H), "matrix")]
        out.append((p + "self_attn.q_norm.weight", (D,), "ones"))
        if not shared:
            out.append((p + "self_attn.k_norm.weight", (D,), "ones"))
        out += [
            (p + "self_attn.o_proj.weight", (H, Nq * D), "matrix"),
            (p + "post_attention_layernorm.weight", (H,), "ones"),
            (p + "pre_feedforward_layernorm.weight", (H,), "ones"),
            (p + "mlp.gate_proj.weight", (I, H), "matrix"),
            (p + "mlp.up_proj.weight", (I, H), "matrix"),
            (p + "mlp.down_proj.weight", (H, I), "matrix"),
            (p + "post_feedforward_layernorm.weight", (H,), "ones"),
        ]
        if P:
            out += [(p + "per_layer_input_gate.weight", (P, H), "matrix"),
                    (p + "per_layer_projection.weight", (H, P), "matrix"),
                    (p + "post_per_layer_input_norm.weight", (H,), "ones")]
        out.append((p + "layer_scalar", (1,), "ones"))
    out.append(("norm.weight", (H,), "ones"))
    return out


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> BF16 bit pattern (uint16)."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    bias = np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))
    return ((bits + bias) >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def generate_weights(cfg: dict, seed: int = 0, dtype: str = "bf16", std: float = 0.02,
                     norm_jitter: float = 0.0):
    """Yields (name, array). dtype 'f32' -> float32 arrays, 'bf16' -> uint16 BF16 bit patterns.

    `norm_jitter` > 0 perturbs the norm weights and layer_scalar around 1.0 (used by parity tests
    so that a kernel which ignored a norm weight would be caught); the benchmark workloads use 0.
    """
    rng = np.random.default_rng(seed)
    for name, shape, kind in weight_names(cfg):
        if kind == "matrix":
            a = rng.standard_normal(shape, dtype=np.float32)
            a *= np.float32(std)
        else:
            a = np.ones(shape, dtype=np.float32)
            if norm_jitter:
                a += (rng.standard_normal(shape, dtype=np.float32) * np.float32(norm_jitter))
        yield name, (f32_to_bf16_bits(a).reshape(shape) if dtype == "bf16" else a)


def prompt_ids(vocab: int, length: int, seed: int = 1) -> np.ndarray:
    return np.random.default_rng(seed).integers(0, vocab, size=length, dtype=np.int64).astype(np.uint32)


def ragged_lengths(batch: int, lo: int, hi: int, seed: int = 2) -> np.ndarray:
    return np.random.default_rng(seed).integers(lo, hi + 1, size=batch, dtype=np.int64).astype(np.int32)


# ---- minimal safetensors reader / writer (single file; F32 and BF16) --------------------------

_ST_DTYPE = {"F32": (np.float32, 4), "BF16": (np.uint16, 2)}


def write_checkpoint(directory: str, cfg: dict, weights, dtype: str):
    """Writes config.json and model.safetensors in the layout the reference loads
    (crates/oxide-torch/src/safetensors.rs:58-123; names under "model.language_model.")."""
    os.makedirs(directory, exist_ok=True)
    with open(os.path.join(directory, "config.json"), "w") as f:
        json.dump({"model_type": "gemma4", "text_config": cfg}, f, indent=1)
    tag = "BF16" if dtype == "bf16" else "F32"
    header, blobs, off = {}, [], 0
    for name, a in weights:
        a = np.ascontiguousarray(a)
        n = a.nbytes
        header[PREFIX + name] = {"dtype": tag, "shape": list(a.shape), "data_offsets": [off, off + n]}
        blobs.append(a.tobytes())
        off += n
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(os.path.join(directory, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def read_checkpoint(directory: str):
    """Returns (text_config, {canonical name: memory-mapped array}). BF16 comes back as uint16."""
    with open(os.path.join(directory, "config.json")) as f:
        cfg = json.load(f)
    cfg = cfg.get("text_config", cfg)
    path = os.path.join(directory, "model.safetensors")
    with open(path, "rb") as f:
        (hl,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(hl))
    mm = np.memmap(path, dtype=np.uint8, mode="r", offset=8 + hl)
    out = {}
    for name, meta in header.items():
        if name == "__metadata__" or not name.startswith(PREFIX):
            continue   # gemma4_cuda/mod.rs:236-243: only the language-model tensors are taken
        np_dtype, _ = _ST_DTYPE[meta["dtype"]]
        a, b = meta["data_offsets"]
        out[name[len(PREFIX):]] = mm[a:b].view(np_dtype).reshape(meta["shape"])
    return cfg, out
