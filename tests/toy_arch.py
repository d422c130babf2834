"""Toy parts and architectures that exist only in the tests. They are registered from here, through
the same public calls a user would make, without touching the framework's files:

* ``ProbeForCausalLM``: one attention layer between an identity "norm" and a feed-forward that adds
  nothing, with every matrix given by the test. With 0/1-structured weights each logit says which
  keys a row read, so a misread key, page or window edge shows at full size in any precision.
* ``ToyStateForCausalLM``: layer 0 mixes with a decaying running sum kept in a per-request state
  slot (no keys, no pages); layer 1 is ordinary attention. Its schedule may run a layer twice or
  let a run read another run's cache.
* ``ToyRoutedForCausalLM``: layer 0 is attention whose position encoding is a learned table added to
  queries and keys (not a rotation) followed by a feed-forward that routes each token to its top-k of a
  few small experts; layer 1 is rotary attention with the dense gated feed-forward.

These are test fixtures for the framework's interfaces, not models of anything.
"""
from dataclasses import dataclass

import numpy as np
import torch

from glassbox_b200.config import (GqaAttentionSpec, LayerSpec, ModelConfig, NoPositionSpec, RmsNormSpec, RopeSpec,
                                  RunSpec, SwiGluSpec)
from glassbox_b200.config.registry import Architecture, register_architecture
from glassbox_b200.parts import FeedForward, Mixer, Norm, OutputHead, Position, StateSpec, TokenEmbedding, register_part
from glassbox_b200.weights.binding import ParamSpec, Stacked


# ------------------------------------------------------------------------------------ toy parts
@dataclass(frozen=True)
class IdentityNormSpec:
    kind: str = "test_identity_norm"


class IdentityNorm(Norm):
    def __init__(self, spec, *, hidden_size):
        super().__init__(spec)

    def forward(self, ctx, x, out, rows=None):
        out.copy_(x if rows is None else x[rows.long()])


@dataclass(frozen=True)
class ZeroFfnSpec:
    kind: str = "test_zero_ffn"


class ZeroFfn(FeedForward):
    def __init__(self, spec, *, hidden_size):
        super().__init__(spec)

    def forward(self, ctx, h, residual):
        return None


@dataclass(frozen=True)
class RunningStateSpec:
    """out_t = W s_t with s_t = decay * s_{t-1} + h_t, s kept per request between steps."""
    decay: float
    kind: str = "test_running_state"


class RunningState(Mixer):
    def __init__(self, spec, *, hidden_size):
        super().__init__(spec)
        self.d = hidden_size

    def param_specs(self):
        return {"w": ParamSpec((self.d, self.d))}

    def cache_spec(self):
        return StateSpec((self.d,), torch.float32)

    def recordable(self, decode_only):
        return decode_only                         # prompt portions walk the host's list of sequences (below)

    def forward(self, ctx, h, residual, cache, writes_cache):
        w = self.params["w"].float()
        if ctx.decode_only:
            # one row per request: everything from the device, so that the step can be replayed as a graph. Padding
            # requests of a graph's fixed shape (start position -1) must leave every slot as it is.
            n = h.shape[0]
            live = (ctx.seq_start_pos[:n] >= 0).unsqueeze(1)
            idx = ctx.seq_slots[:n].clamp(min=0).long()
            old = cache.state.index_select(0, idx)
            new = self.spec.decay * old + h.float()
            residual += torch.where(live, new @ w.T, torch.zeros_like(new))
            if writes_cache:
                cache.state.index_add_(0, idx, torch.where(live, new - old, torch.zeros_like(new)))
            return
        for seq in ctx.seqs:                       # rows of one request are consecutive and in order
            s = cache.state[seq.slot].clone()
            for r in range(seq.first_row, seq.first_row + seq.n_rows):
                s = self.spec.decay * s + h[r].float()
                residual[r] += w @ s
            if writes_cache:
                cache.state[seq.slot].copy_(s)


@dataclass(frozen=True)
class ZeroMixerSpec:
    kind: str = "test_zero_mixer"


class ZeroMixer(Mixer):
    def __init__(self, spec, *, hidden_size):
        super().__init__(spec)

    def forward(self, ctx, h, residual, cache, writes_cache):
        return None


@dataclass(frozen=True)
class RoutedFfnSpec:
    """Each token goes to the ``top_k`` experts with the largest router logits; their outputs are mixed
    with the softmax of those logits. Every expert is a small gated feed-forward."""
    num_experts: int
    top_k: int
    intermediate_size: int
    kind: str = "test_routed_ffn"


class RoutedFfn(FeedForward):
    def __init__(self, spec, *, hidden_size):
        super().__init__(spec)
        self.d = hidden_size

    def param_specs(self):
        e, i = self.spec.num_experts, self.spec.intermediate_size
        return {"router": ParamSpec((e, self.d)), "w_gate_up": ParamSpec((e, 2 * i, self.d)),
                "w_down": ParamSpec((e, self.d, i))}

    def forward(self, ctx, h, residual):
        # router logits and mixing weights in float32; every expert runs on every row and rows it was
        # not chosen for get weight zero (static shapes: the step can be recorded as a CUDA graph)
        x = h.float()
        logits = x @ self.params["router"].float().T
        top = logits.topk(self.spec.top_k, dim=-1)
        mix = torch.zeros_like(logits).scatter_(1, top.indices, torch.softmax(top.values, dim=-1))
        i = self.spec.intermediate_size
        for e in range(self.spec.num_experts):
            gu = x @ self.params["w_gate_up"][e].float().T
            act = torch.nn.functional.silu(gu[:, :i]) * gu[:, i:]
            residual += mix[:, e:e + 1] * (act @ self.params["w_down"][e].float().T)


@dataclass(frozen=True)
class LearnedOffsetPositionSpec:
    """q and k of the token at position p get a learned vector table[p] added, per head."""
    head_dim: int
    max_position: int
    kind: str = "test_learned_offset"


class LearnedOffsetPosition(Position):
    rotary_dim = 0

    def param_specs(self):
        return {"table": ParamSpec((self.spec.max_position, self.spec.head_dim))}

    def apply_qk(self, ctx, qkv, num_heads, num_kv_heads, head_dim):
        live = (ctx.positions >= 0).unsqueeze(-1).unsqueeze(-1)            # padding rows carry position -1
        add = self.params["table"][ctx.positions.clamp(min=0).long()].to(qkv.dtype).unsqueeze(1) * live
        heads = qkv[:, :(num_heads + num_kv_heads) * head_dim].unflatten(1, (num_heads + num_kv_heads, head_dim))
        heads += add


@dataclass(frozen=True)
class ScaledEmbeddingSpec:
    """The residual row of a token is its table row times a constant."""
    scale: float
    kind: str = "test_scaled_embedding"


class ScaledEmbedding(TokenEmbedding):
    def __init__(self, spec, *, vocab_size, hidden_size):
        super().__init__(spec)
        self.vocab_size, self.hidden_size = vocab_size, hidden_size

    def param_specs(self):
        return {"weight": ParamSpec((self.vocab_size, self.hidden_size))}

    def forward(self, ctx, tokens, x):
        from glassbox_b200 import kernels
        kernels.embed(self.params["weight"], tokens, x, ctx.status)
        x.mul_(self.spec.scale)


@dataclass(frozen=True)
class BiasedHeadSpec:
    """logits = hs H^T + b."""
    kind: str = "test_biased_head"


class BiasedHead(OutputHead):
    def __init__(self, spec, *, vocab_size, hidden_size):
        super().__init__(spec)
        self.vocab_size, self.hidden_size = vocab_size, hidden_size

    def param_specs(self):
        return {"weight": ParamSpec((self.vocab_size, self.hidden_size)), "bias": ParamSpec((self.vocab_size,), role="gain")}

    def forward(self, ctx, hs, logits):
        from glassbox_b200.parts.linear import linear
        linear(ctx, hs, self.params["weight"], logits)
        logits += self.params["bias"]


register_part("embedding", "test_scaled_embedding", ScaledEmbedding, replace=True)
register_part("head", "test_biased_head", BiasedHead, replace=True)
register_part("ffn", "test_routed_ffn", RoutedFfn, replace=True)
register_part("position", "test_learned_offset", LearnedOffsetPosition, replace=True)
register_part("mixer", "test_zero_mixer", ZeroMixer, replace=True)
register_part("norm", "test_identity_norm", IdentityNorm, replace=True)
register_part("ffn", "test_zero_ffn", ZeroFfn, replace=True)
register_part("mixer", "test_running_state", RunningState, replace=True)


# -------------------------------------------------------------------------------- architectures
def _parse_probe(raw):
    hd = raw["head_dim"]
    position = NoPositionSpec() if raw.get("rope_theta") is None else \
        RopeSpec(theta=float(raw["rope_theta"]), rotary_dim=raw.get("rotary_dim", hd), max_position=raw["max_position"])
    attn = GqaAttentionSpec(num_heads=raw["num_heads"], num_kv_heads=raw["num_kv_heads"], head_dim=hd,
                            scale=float(raw.get("scale", 1.0)), position=position, window=raw.get("window"))
    layer = LayerSpec(mixer=attn, ffn=ZeroFfnSpec(), mixer_norm=IdentityNormSpec(), ffn_norm=IdentityNormSpec())
    return ModelConfig(architecture="ProbeForCausalLM", vocab_size=raw["vocab_size"], hidden_size=raw["hidden_size"],
                       max_position=raw["max_position"], tie_word_embeddings=False, layers=(layer,),
                       schedule=(RunSpec(0, 0),), final_norm=IdentityNormSpec(), raw=dict(raw))


def _bind_probe(config):
    return {"embed.weight": Stacked(("embed",)), "layers.0.mixer.wqkv": Stacked(("wq", "wk", "wv")),
            "layers.0.mixer.wo": Stacked(("wo",)), "head.weight": Stacked(("head",))}


register_architecture(Architecture("ProbeForCausalLM", _parse_probe, _bind_probe), replace=True)


def _parse_toy_state(raw):
    d, hd = raw["hidden_size"], raw["head_dim"]
    norm = RmsNormSpec(eps=raw["eps"])
    ffn = SwiGluSpec(intermediate_size=raw["intermediate_size"])
    rope = RopeSpec(theta=raw["rope_theta"], rotary_dim=hd, max_position=raw["max_position"])
    attn = GqaAttentionSpec(num_heads=raw["num_heads"], num_kv_heads=raw["num_kv_heads"], head_dim=hd,
                            scale=hd ** -0.5, position=rope, window=raw.get("window"))
    layers = (LayerSpec(RunningStateSpec(decay=raw["decay"]), ffn, norm, norm), LayerSpec(attn, ffn, norm, norm))
    schedule = tuple(RunSpec(*r) for r in raw.get("schedule", [(0, 0, True), (1, 1, True)]))
    return ModelConfig(architecture="ToyStateForCausalLM", vocab_size=raw["vocab_size"], hidden_size=d,
                       max_position=raw["max_position"], tie_word_embeddings=True, layers=layers, schedule=schedule,
                       final_norm=norm, raw=dict(raw))


def _bind_toy_state(config):
    from glassbox_b200.weights.binding import Tied
    b = {"embed.weight": Stacked(("embed",)), "head.weight": Tied("embed.weight"),
         "final_norm.weight": Stacked(("final_norm",)), "layers.0.mixer.w": Stacked(("state_w",)),
         "layers.1.mixer.wqkv": Stacked(("wq", "wk", "wv")), "layers.1.mixer.wo": Stacked(("wo",))}
    for i in (0, 1):
        b[f"layers.{i}.mixer_norm.weight"] = Stacked((f"norm{i}a",))
        b[f"layers.{i}.ffn_norm.weight"] = Stacked((f"norm{i}b",))
        b[f"layers.{i}.ffn.w_gate_up"] = Stacked((f"gate{i}", f"up{i}"))
        b[f"layers.{i}.ffn.w_down"] = Stacked((f"down{i}",))
    return b


register_architecture(Architecture("ToyStateForCausalLM", _parse_toy_state, _bind_toy_state), replace=True)


def _parse_toy_routed(raw):
    d, hd = raw["hidden_size"], raw["head_dim"]
    norm = RmsNormSpec(eps=raw["eps"])
    learned = LearnedOffsetPositionSpec(head_dim=hd, max_position=raw["max_position"])
    rope = RopeSpec(theta=raw["rope_theta"], rotary_dim=hd, max_position=raw["max_position"])
    attn = lambda position: GqaAttentionSpec(num_heads=raw["num_heads"], num_kv_heads=raw["num_kv_heads"], head_dim=hd,
                                             scale=hd ** -0.5, position=position)
    routed = RoutedFfnSpec(num_experts=raw["num_experts"], top_k=raw["top_k"], intermediate_size=raw["expert_size"])
    layers = (LayerSpec(attn(learned), routed, norm, norm),
              LayerSpec(attn(rope), SwiGluSpec(intermediate_size=raw["intermediate_size"]), norm, norm))
    return ModelConfig(architecture="ToyRoutedForCausalLM", vocab_size=raw["vocab_size"], hidden_size=d,
                       max_position=raw["max_position"], tie_word_embeddings=True, layers=layers,
                       schedule=(RunSpec(0, 0), RunSpec(1, 1)), final_norm=norm, raw=dict(raw))


def _bind_toy_routed(config):
    from glassbox_b200.weights.binding import Tied
    b = {"embed.weight": Stacked(("embed",)), "head.weight": Tied("embed.weight"),
         "final_norm.weight": Stacked(("final_norm",)),
         "layers.0.mixer.position.table": Stacked(("offsets",)),
         "layers.0.ffn.router": Stacked(("router",)), "layers.0.ffn.w_gate_up": Stacked(("experts_gate_up",)),
         "layers.0.ffn.w_down": Stacked(("experts_down",)),
         "layers.1.ffn.w_gate_up": Stacked(("gate", "up")), "layers.1.ffn.w_down": Stacked(("down",))}
    for i in (0, 1):
        b[f"layers.{i}.mixer.wqkv"] = Stacked((f"wq{i}", f"wk{i}", f"wv{i}"))
        b[f"layers.{i}.mixer.wo"] = Stacked((f"wo{i}",))
        b[f"layers.{i}.mixer_norm.weight"] = Stacked((f"norm{i}a",))
        b[f"layers.{i}.ffn_norm.weight"] = Stacked((f"norm{i}b",))
    return b


register_architecture(Architecture("ToyRoutedForCausalLM", _parse_toy_routed, _bind_toy_routed), replace=True)


def _parse_toy_scaled(raw):
    """``ToyScaledForCausalLM``: the stock Llama layers between an embedding that scales its rows and a head with a bias;
    both are parts that exist only here."""
    import dataclasses
    from glassbox_b200.models.llama import parse_llama_config
    cfg = parse_llama_config(raw)
    return dataclasses.replace(cfg, architecture="ToyScaledForCausalLM", embedding=ScaledEmbeddingSpec(scale=float(raw["embedding_scale"])),
                               head=BiasedHeadSpec())


def _bind_toy_scaled(config):
    from glassbox_b200.models.llama import bind_llama_weights
    b = bind_llama_weights(config)
    b["head.bias"] = Stacked(("lm_head.bias",))
    return b


register_architecture(Architecture("ToyScaledForCausalLM", _parse_toy_scaled, _bind_toy_scaled), replace=True)


def _parse_one_part(raw):
    """``OnePartForCausalLM``: a single layer in which exactly one part is real and every other part
    is an identity or adds nothing; the embedding table holds the test's input vectors (token i is
    input i) and the head is the identity, so the logits ARE the part's output (plus its input, the
    residual). raw["part"] is "norm" | "ffn" | "mixer" | "block"."""
    d, hd = raw["hidden_size"], raw.get("head_dim", 16)
    part = raw["part"]
    ident, real_norm = IdentityNormSpec(), RmsNormSpec(eps=raw.get("eps", 1e-5))
    position = NoPositionSpec() if raw.get("rope_theta") is None else \
        RopeSpec(theta=float(raw["rope_theta"]), rotary_dim=hd, max_position=raw["max_position"])
    attn = GqaAttentionSpec(num_heads=raw.get("num_heads", 1), num_kv_heads=raw.get("num_kv_heads", 1), head_dim=hd,
                            scale=float(raw.get("scale", hd ** -0.5)), position=position, window=raw.get("window"))
    ffn = SwiGluSpec(intermediate_size=raw.get("intermediate_size", 16))
    layer = LayerSpec(mixer=attn if part in ("mixer", "block") else ZeroMixerSpec(),
                      ffn=ffn if part in ("ffn", "block") else ZeroFfnSpec(),
                      mixer_norm=real_norm if part == "block" else ident,
                      ffn_norm=real_norm if part == "block" else ident)
    return ModelConfig(architecture="OnePartForCausalLM", vocab_size=raw["vocab_size"], hidden_size=d,
                       max_position=raw["max_position"], tie_word_embeddings=False, layers=(layer,),
                       schedule=(RunSpec(0, 0),), final_norm=real_norm if part == "norm" else ident, raw=dict(raw))


def _bind_one_part(config):
    b = {"embed.weight": Stacked(("embed",)), "head.weight": Stacked(("head",))}
    part = config.raw["part"]
    if part in ("mixer", "block"):
        b["layers.0.mixer.wqkv"] = Stacked(("wq", "wk", "wv"))
        b["layers.0.mixer.wo"] = Stacked(("wo",))
    if part in ("ffn", "block"):
        b["layers.0.ffn.w_gate_up"] = Stacked(("gate", "up"))
        b["layers.0.ffn.w_down"] = Stacked(("down",))
    if part == "block":
        b["layers.0.mixer_norm.weight"] = Stacked(("norm_a",))
        b["layers.0.ffn_norm.weight"] = Stacked(("norm_b",))
    if part == "norm":
        b["final_norm.weight"] = Stacked(("norm",))
    return b


register_architecture(Architecture("OnePartForCausalLM", _parse_one_part, _bind_one_part), replace=True)


# ----------------------------------------------------------------- the probe model, and its truth
ROOT = 1.25     # q and k are +-1 vectors times this: a matching pair scores ROOT^2 * head_dim, exactly


def write_probe_model(folder, *, vocab=400, hd=32, nh=2, nkv=1, window=None, max_position=512, seed=0,
                      store=torch.float32):
    """Token t carries, per query head, a query direction; a key direction; and a value vector. A row
    scores ROOT^2 * hd (50 at hd 32) against keys whose direction equals its query direction and
    exactly 0 against all others: directions are rows of a Hadamard matrix with entries +-1, and
    every weight is exact in bfloat16, so the softmax is the same in every precision. Logit
    j < nh*hd is channel j of (query direction + attention output). Returns the per-token tables
    from which ``probe_truth`` states what the logits must be."""
    import json
    import os
    from glassbox_b200.weights import write_safetensors
    rng = np.random.default_rng(seed)
    had = np.array([[1.0]])
    while had.shape[0] < hd:
        had = np.block([[had, had], [had, -had]])
    qdir = rng.integers(0, hd, size=(vocab, nh))
    kdir = rng.integers(0, hd, size=(vocab, nkv))
    # values: small integers / 8 are exact in bfloat16
    val = rng.integers(-16, 17, size=(vocab, nkv, hd)).astype(np.float64) / 8.0
    d = (nh + 2 * nkv) * hd
    embed = np.zeros((vocab, d))
    for h in range(nh):
        embed[:, h * hd:(h + 1) * hd] = had[qdir[:, h]]
    for g in range(nkv):
        embed[:, (nh + g) * hd:(nh + g + 1) * hd] = had[kdir[:, g]]
        embed[:, (nh + nkv + g) * hd:(nh + nkv + g + 1) * hd] = val[:, g]
    root = ROOT
    wq = np.zeros((nh * hd, d)); wq[:, :nh * hd] = np.eye(nh * hd) * root
    wk = np.zeros((nkv * hd, d)); wk[:, nh * hd:(nh + nkv) * hd] = np.eye(nkv * hd) * root
    wv = np.zeros((nkv * hd, d)); wv[:, (nh + nkv) * hd:] = np.eye(nkv * hd)
    # the output projection adds the attention output onto the channels that hold the query
    # directions; the head reads those channels back
    wo = np.zeros((d, nh * hd)); wo[:nh * hd, :] = np.eye(nh * hd)
    head = np.zeros((vocab, d)); head[:nh * hd, :nh * hd] = np.eye(nh * hd)
    assert vocab >= nh * hd
    os.makedirs(folder, exist_ok=True)
    raw = {"architectures": ["ProbeForCausalLM"], "vocab_size": vocab, "hidden_size": d, "num_heads": nh,
           "num_kv_heads": nkv, "head_dim": hd, "window": window, "scale": 1.0, "max_position": max_position,
           "rope_theta": None}
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(raw, f)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(store)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      {"embed": t(embed), "wq": t(wq), "wk": t(wk), "wv": t(wv), "wo": t(wo), "head": t(head)})
    return {"qdir": qdir, "kdir": kdir, "val": val, "had": had, "nh": nh, "nkv": nkv, "hd": hd, "window": window,
            "vocab": vocab}


def probe_truth(info, tokens):
    """Expected logits[:, :nh*hd] for a whole sequence, from the plain attention part."""
    from plain.llama_plain import attention
    nh, nkv, hd = info["nh"], info["nkv"], info["hd"]
    toks = np.asarray(tokens)
    root = ROOT
    q = np.stack([info["had"][info["qdir"][toks, h]] for h in range(nh)], axis=1) * root
    k = np.stack([info["had"][info["kdir"][toks, g]] for g in range(nkv)], axis=1) * root
    v = info["val"][toks]
    att = attention(q, k, v, 1.0, info["window"]).reshape(len(toks), nh * hd)
    return att + (q / root).reshape(len(toks), nh * hd)          # the residual carried the query part
