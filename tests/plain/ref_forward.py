"""Python face of ``ref_forward.cpp``, the second plain implementation (C++, float32): builds it with the C++
compiler into a temporary folder, loads it with ctypes, and feeds it a model folder's tensors. It reads config.json
and the safetensors file by itself and shares no code with the ``glassbox_b200`` package.

``RefModel(model_dir).forward(tokens, pos0=0, want=None)`` -> float32 [wanted, vocab]; the model keeps a contiguous
cache for one sequence, so a prompt can be followed by single tokens. ``pp_tg`` times it the way the reference's
benchmark does (crates/glassbox-bench/src/main.rs:72-96).
"""
from __future__ import annotations

import ctypes
import hashlib
import json
import os
import shutil
import subprocess
import tempfile
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_lib = None


def _build() -> str:
    src = os.path.join(HERE, "ref_forward.cpp")
    with open(src, "rb") as f:
        tag = hashlib.sha256(f.read()).hexdigest()[:16]
    out_dir = os.path.join(tempfile.gettempdir(), f"glassbox_b200_ref_{os.getuid()}")
    os.makedirs(out_dir, exist_ok=True)
    lib = os.path.join(out_dir, f"libref_forward_{tag}.so")
    if not os.path.exists(lib):
        cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
        if cxx is None:
            raise RuntimeError("no C++ compiler for the plain C++ implementation")
        tmp = lib + f".{os.getpid()}.tmp"
        # no -ffast-math: the sums keep the order the source gives them
        subprocess.run([cxx, "-O3", "-march=native", "-pthread", "-std=c++17", "-fPIC", "-shared", "-o", tmp, src], check=True)
        os.replace(tmp, lib)
    return lib


def lib():
    global _lib
    if _lib is None:
        h = ctypes.CDLL(_build())
        h.ref_new.restype = ctypes.c_void_p
        h.ref_new.argtypes = [ctypes.c_void_p, ctypes.c_float, ctypes.c_float]
        h.ref_set.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        h.ref_set.restype = None
        h.ref_free.argtypes = [ctypes.c_void_p]
        h.ref_free.restype = None
        h.ref_forward.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
                                  ctypes.c_void_p]
        h.ref_forward.restype = ctypes.c_int
        _lib = h
    return _lib


class RefModel:
    """Keys and defaults of crates/glassbox-core/src/model.rs:7-55; tensor names of crates/glassbox-core/src/load.rs:50-78."""

    def __init__(self, model_dir: str, max_pos: int = 0):
        from safetensors import safe_open
        with open(os.path.join(model_dir, "config.json")) as f:
            raw = json.load(f)
        theta = raw.get("rope_theta")
        if theta is None:
            theta = (raw.get("rope_parameters") or {}).get("rope_theta", 10000.0)
        nh = raw["num_attention_heads"]
        self.vocab = raw["vocab_size"]
        self.max_pos = max_pos or raw.get("max_position_embeddings", 2048)
        sizes = np.array([raw["hidden_size"], raw["intermediate_size"], raw["num_hidden_layers"], nh, raw["num_key_value_heads"],
                          raw.get("head_dim") or raw["hidden_size"] // nh, self.vocab, self.max_pos], dtype=np.int32)
        self._h = lib().ref_new(sizes.ctypes.data, float(raw.get("rms_norm_eps", 1e-5)), float(theta))
        self._keep = []
        with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
            names = set(f.keys())

            def put(layer, which, name):
                a = np.ascontiguousarray(f.get_tensor(name).float().numpy())
                self._keep.append(a)
                lib().ref_set(self._h, layer, which, a.ctypes.data)
                return a
            embed = put(-1, 0, "model.embed_tokens.weight")
            put(-1, 1, "model.norm.weight")
            if raw.get("tie_word_embeddings", False) or "lm_head.weight" not in names:       # load.rs:70-75
                lib().ref_set(self._h, -1, 2, embed.ctypes.data)
            else:
                put(-1, 2, "lm_head.weight")
            for i in range(raw["num_hidden_layers"]):
                p = f"model.layers.{i}."
                for which, name in enumerate(("input_layernorm", "self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj",
                                              "self_attn.o_proj", "post_attention_layernorm", "mlp.gate_proj", "mlp.up_proj",
                                              "mlp.down_proj")):
                    put(i, which, p + name + ".weight")

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and _lib is not None:
            _lib.ref_free(h)

    def forward(self, tokens, pos0: int = 0, want=None) -> np.ndarray:
        toks = np.ascontiguousarray(tokens, dtype=np.int32)
        want = np.arange(toks.size, dtype=np.int32) if want is None else np.ascontiguousarray(want, dtype=np.int32)
        out = np.empty((max(want.size, 1), self.vocab), dtype=np.float32)
        rc = lib().ref_forward(self._h, toks.ctypes.data, toks.size, int(pos0), want.ctypes.data, want.size, out.ctypes.data)
        if rc:
            raise ValueError("positions run past the model's cache")
        return out[:want.size]


def pp_tg(model_dir: str, pp: int = 512, tg: int = 128, reps: int = 2):
    """(prefill tokens/s, decode tokens/s) as crates/glassbox-bench/src/main.rs:72-96 measures them: a synthetic prompt
    (i * 7919 + 13) % vocab in one forward pass; then, on a fresh cache, ``tg`` greedy tokens one at a time from token 1
    (near-empty context); the first repetition is a warm-up and is discarded."""
    m = RefModel(model_dir, max_pos=max(pp, tg + 1))
    prompt = [(i * 7919 + 13) % m.vocab for i in range(pp)]
    pre, dec = [], []
    for rep in range(reps + 1):
        t0 = time.perf_counter()
        m.forward(prompt, 0, [pp - 1])
        t1 = time.perf_counter()
        tok = 1
        for i in range(tg):
            tok = int(np.argmax(m.forward([tok], i, [0])[0]))
        t2 = time.perf_counter()
        if rep:
            pre.append(pp / (t1 - t0))
            dec.append(tg / (t2 - t1))
    return float(np.mean(pre)), float(np.mean(dec))
