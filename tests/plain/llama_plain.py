"""A plain, slow implementation of the Llama-family decoder that Glassbox runs.

It rests on the formulas of the reference's Rust sources (each function cites file:line): the
reference itself is Rust with no toolchain on this machine, so it cannot be imported or compiled
here and no golden outputs of it exist; what stands in is this restatement, written from
crates/glassbox-core/src/model.rs. It shares no code with the ``glassbox_b200`` package: it
reads config.json with ``json``, the weights with the ``safetensors`` library, and computes whole
sequences with no cache, one function per part, in float64 NumPy (except where the reference
deliberately rounds to float32: the rotary angles).

``forward_logits(model_dir, tokens)`` -> float64 [len(tokens), vocab].
"""
from __future__ import annotations

import json
import os

import numpy as np


# --------------------------------------------------------------------------------------- loading
def read_config(model_dir):
    """Keys and defaults of crates/glassbox-core/src/model.rs:7-55."""
    with open(os.path.join(model_dir, "config.json")) as f:
        raw = json.load(f)
    theta = raw.get("rope_theta")
    if theta is None:
        theta = (raw.get("rope_parameters") or {}).get("rope_theta", 10000.0)  # model.rs:39-47
    heads = raw["num_attention_heads"]
    return {
        "d": raw["hidden_size"], "inter": raw["intermediate_size"], "layers": raw["num_hidden_layers"],
        "nh": heads, "nkv": raw["num_key_value_heads"], "vocab": raw["vocab_size"],
        "eps": float(np.float32(raw.get("rms_norm_eps", 1e-5))),          # f32 field, model.rs:16
        "theta": float(np.float32(theta)),                                # f32 field, model.rs:18
        "tie": bool(raw.get("tie_word_embeddings", False)),               # model.rs:19-20
        "hd": raw.get("head_dim") or raw["hidden_size"] // heads,         # model.rs:49-51
        "max_pos": raw.get("max_position_embeddings", 2048),
    }


def read_weights(model_dir):
    """Tensor names of crates/glassbox-core/src/load.rs:50-78, widened to float64."""
    from safetensors import safe_open
    out = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            out[name] = f.get_tensor(name).double().numpy()
    return out


# ----------------------------------------------------------------------------------------- parts
def rms_norm(x, w, eps):
    """model.rs:94-100: ms = mean(x^2); out = w * (x / sqrt(ms + eps))."""
    ms = np.mean(x * x, axis=-1, keepdims=True)
    return w * (x * (1.0 / np.sqrt(ms + eps)))


def rope_angles(positions, hd, theta):
    """model.rs:104-109: inv = (1 / theta^(2i/hd)) rounded to f32; angle = f32(pos) * inv in f32;
    sin and cos of the angle evaluated in f64 and rounded to f32."""
    i = np.arange(hd // 2, dtype=np.float64)
    inv = (1.0 / np.power(np.float64(theta), 2.0 * i / hd)).astype(np.float32)
    ang = (np.asarray(positions, dtype=np.float32)[:, None] * inv[None, :]).astype(np.float32)
    a64 = ang.astype(np.float64)
    return np.cos(a64).astype(np.float32).astype(np.float64), np.sin(a64).astype(np.float32).astype(np.float64)


def rope(x, cos, sin):
    """model.rs:110-114, half-split pairs (i, i + hd/2): x[T, heads, hd]."""
    half = x.shape[-1] // 2
    x0, x1 = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return np.concatenate([x0 * c - x1 * s, x1 * c + x0 * s], axis=-1)


def attention(q, k, v, scale, window=None):
    """model.rs:285-312: per head, scores over positions 0..=pos, softmax with the maximum
    subtracted, probabilities normalised, then the weighted sum of values. q [T, nh, hd];
    k, v [T, nkv, hd]; query head h reads kv head h // (nh // nkv) (model.rs:287)."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    out = np.zeros_like(q)
    for h in range(nh):
        kh, vh = k[:, h // group, :], v[:, h // group, :]
        scores = (q[:, h, :] @ kh.T) * scale
        idx = np.arange(T)
        visible = idx[None, :] <= idx[:, None]
        if window is not None:
            visible &= idx[None, :] > idx[:, None] - window
        scores = np.where(visible, scores, -np.inf)
        scores = scores - scores.max(axis=-1, keepdims=True)
        e = np.exp(scores)
        p = e / e.sum(axis=-1, keepdims=True)
        out[:, h, :] = p @ vh
    return out


def swiglu(g, u):
    """model.rs:336-340: act = g / (1 + exp(-g)) * u."""
    return g / (1.0 + np.exp(-g)) * u


# ---------------------------------------------------------------------------------------- model
_LOADED = {}


def _load(model_dir):
    key = (os.path.realpath(model_dir), os.path.getmtime(os.path.join(model_dir, "model.safetensors")))
    if key not in _LOADED:
        _LOADED[key] = (read_config(model_dir), read_weights(model_dir))
    return _LOADED[key]


def forward_logits(model_dir, tokens, window=None, rows=None):
    """Whole sequence, no cache: model.rs:207-362 with every row wanted, or (``rows``: a list of positions) with
    only those rows taken through the final norm and the head (model.rs:350-361 does the same with ``want``)."""
    c, w = _load(model_dir)
    tokens = np.asarray(tokens, dtype=np.int64)
    T = tokens.shape[0]
    d, nh, nkv, hd = c["d"], c["nh"], c["nkv"], c["hd"]
    x = w["model.embed_tokens.weight"][tokens]                                  # model.rs:228-231
    cos, sin = rope_angles(np.arange(T), hd, c["theta"])
    scale = float(np.float32(1.0) / np.sqrt(np.float32(hd)))                    # model.rs:244 (f32)
    for li in range(c["layers"]):
        p = f"model.layers.{li}"
        h = rms_norm(x, w[f"{p}.input_layernorm.weight"], c["eps"])             # model.rs:252-259
        q = (h @ w[f"{p}.self_attn.q_proj.weight"].T).reshape(T, nh, hd)        # model.rs:260-265
        k = (h @ w[f"{p}.self_attn.k_proj.weight"].T).reshape(T, nkv, hd)
        v = (h @ w[f"{p}.self_attn.v_proj.weight"].T).reshape(T, nkv, hd)
        q, k = rope(q, cos, sin), rope(k, cos, sin)                             # model.rs:266-272
        att = attention(q, k, v, scale, window).reshape(T, nh * hd)             # model.rs:278-317
        x = x + att @ w[f"{p}.self_attn.o_proj.weight"].T                       # model.rs:322-325
        h = rms_norm(x, w[f"{p}.post_attention_layernorm.weight"], c["eps"])    # model.rs:327-334
        g = h @ w[f"{p}.mlp.gate_proj.weight"].T                                # model.rs:335
        u = h @ w[f"{p}.mlp.up_proj.weight"].T
        x = x + swiglu(g, u) @ w[f"{p}.mlp.down_proj.weight"].T                 # model.rs:336-344
    if rows is not None:
        x = x[np.asarray(rows, dtype=np.int64)]
    hs = rms_norm(x, w["model.norm.weight"], c["eps"])                          # model.rs:350-358
    head = w["model.embed_tokens.weight"] if c["tie"] or "lm_head.weight" not in w else w["lm_head.weight"]
    return hs @ head.T                                                          # model.rs:359-361, 190-192


def argmax_first(x):
    """crates/glassbox-core/src/sampler.rs:49-57: the first maximum wins."""
    return int(np.argmax(x))


def greedy(model_dir, prompt, n):
    """crates/glassbox-core/src/lib.rs:64-74, recomputing the whole sequence for every token."""
    tokens = list(prompt)
    out = []
    for _ in range(n):
        t = argmax_first(forward_logits(model_dir, tokens)[-1])
        out.append(t)
        tokens.append(t)
    return out
