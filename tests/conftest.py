"""Shared fixtures: tiny random-weight model folders made in temporary directories.

Tests marked ``gpu`` need a CUDA device (they drive the real kernels); everything else runs on
the CPU. The two tiny configurations differ in every size and option.
"""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import torch  # noqa: E402

import glassbox_b200  # noqa: E402
from glassbox_b200.models.llama import make_llama_raw_config  # noqa: E402

# fp32: the plain implementation is float64, the engine true float32: absolute bound.
FP32_ATOL = 1e-4
# bf16: weights are identical (bf16 on disk); activations are rounded to 8 mantissa bits (2^-9
# relative) after each of ~10 operations per layer, so the bound is relative to the spread of the
# logits: worst element within 5 % of their standard deviation, mean error within 0.8 %. (The largest seen over the
# whole suite, printed at the end of a run: 3.8 % and 0.55 %, both at SmolLM2-1.7B widths, where K reaches 8,192; the tiny
# models stay near 1.5 %.) A model
# whose attention is sharpened (see ``sharpen``) is compared in float32 only: peaked softmax
# amplifies bfloat16 rounding of the scores until the comparison with a float64 computation says
# nothing. In bfloat16, faults that hide below this bound are caught by the crafted-model tests, in
# which every score is either a large constant or zero, so that rounding cannot move the softmax.
BF16_REL_MAX = 0.05
BF16_REL_MEAN = 0.008

TINY = {
    # GQA, tied head, power-of-two-free intermediate size
    "A": dict(hidden_size=64, intermediate_size=176, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-5,
              tie_word_embeddings=True, max_position_embeddings=128),
    # MQA, untied head, other theta and eps, three heads
    "B": dict(hidden_size=96, intermediate_size=256, num_hidden_layers=3, num_attention_heads=3,
              num_key_value_heads=1, vocab_size=512, rope_theta=100000.0, rms_norm_eps=1e-6,
              tie_word_embeddings=False, max_position_embeddings=256),
    # MHA, explicit head_dim that is not hidden/heads, nothing a power of two
    "C": dict(hidden_size=80, intermediate_size=136, num_hidden_layers=1, num_attention_heads=5,
              num_key_value_heads=5, head_dim=48, vocab_size=301, rope_theta=500000.0, rms_norm_eps=3e-6,
              tie_word_embeddings=False, max_position_embeddings=320),
    # head size 64, the size the tensor-core attention kernels are built for, so that whole-model
    # tests run them too (the other configurations take the float32-FMA kernels of any head size)
    "D": dict(hidden_size=128, intermediate_size=208, num_hidden_layers=2, num_attention_heads=2,
              num_key_value_heads=1, vocab_size=300, rope_theta=100000.0, rms_norm_eps=1e-5,
              tie_word_embeddings=True, max_position_embeddings=320),
}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (runs the real kernels)")


def tiny_raw(name):
    return make_llama_raw_config(**TINY[name])


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """{(name, 'float32'|'bfloat16'): folder} made on demand."""
    made = {}

    def get(name, dtype="float32", seed=11):
        key = (name, dtype, seed)
        if key not in made:
            d = tmp_path_factory.mktemp(f"tiny{name}_{dtype}_{seed}")
            store = torch.float32 if dtype == "float32" else torch.bfloat16
            glassbox_b200.write_random_model(str(d), tiny_raw(name), seed, store)
            made[key] = str(d)
        return made[key]

    return get


def sharpen(folder, out, qk=12.0, vo=4.0):
    """Copy a model folder with q/k projections scaled so that attention is peaked (about ten keys
    carry the softmax, the best one a fifth of it, instead of hundreds averaging out) and v/o scaled
    so that attention dominates the logits. A fault in which key a row reads, or from which page,
    then moves the logits by far more than any tolerance. Scaling further (24) makes the softmax so
    steep that float32 rounding of the scores alone moves logits by more than 1e-4, which would
    test the conditioning of the crafted model and not the engine."""
    import shutil
    from safetensors.torch import load_file, save_file
    os.makedirs(out, exist_ok=True)
    shutil.copy(os.path.join(folder, "config.json"), os.path.join(out, "config.json"))
    tensors = load_file(os.path.join(folder, "model.safetensors"))
    for name in list(tensors):
        t = tensors[name]
        if "q_proj" in name or "k_proj" in name:
            tensors[name] = (t.float() * qk).to(t.dtype)
        elif "v_proj" in name or "o_proj" in name:
            tensors[name] = (t.float() * vo).to(t.dtype)
    save_file(tensors, os.path.join(out, "model.safetensors"))
    return out


@pytest.fixture(scope="session")
def sharp_dirs(model_dirs, tmp_path_factory):
    made = {}

    def get(name, dtype="float32", seed=11):
        key = (name, dtype, seed)
        if key not in made:
            made[key] = sharpen(model_dirs(name, dtype, seed), str(tmp_path_factory.mktemp(f"sharp{name}_{dtype}")))
        return made[key]

    return get


#: the largest bfloat16 errors seen in this session, as fractions of the logits' spread (printed at the end of the run)
WORST_BF16 = {"max": 0.0, "mean": 0.0, "where": ""}


def pytest_terminal_summary(terminalreporter):
    if WORST_BF16["max"] > 0:
        terminalreporter.write_line(f"bfloat16 logits: worst max error {WORST_BF16['max']:.4f} and worst mean error "
                                    f"{WORST_BF16['mean']:.4f} of the spread (bounds {BF16_REL_MAX}, {BF16_REL_MEAN}); "
                                    f"worst at: {WORST_BF16['where']}")


def assert_logits_close(got, want, dtype, what=""):
    import numpy as np
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} != {want.shape}"
    diff = np.abs(got - want)
    worst = np.unravel_index(np.argmax(diff), diff.shape)
    if dtype == "float32":
        assert diff.max() <= FP32_ATOL, f"{what}: max abs diff {diff.max():.3e} > {FP32_ATOL} at {worst} (float32)"
    else:
        spread = want.std()
        if spread > 0:
            if diff.max() / spread > WORST_BF16["max"]:
                WORST_BF16["max"], WORST_BF16["where"] = float(diff.max() / spread), what
            WORST_BF16["mean"] = max(WORST_BF16["mean"], float(diff.mean() / spread))
        assert diff.max() <= BF16_REL_MAX * spread, \
            f"{what}: max abs diff {diff.max():.3e} > {BF16_REL_MAX} x spread {spread:.3e} at {worst} (bfloat16)"
        assert diff.mean() <= BF16_REL_MEAN * spread, \
            f"{what}: mean abs diff {diff.mean():.3e} > {BF16_REL_MEAN} x spread {spread:.3e} (bfloat16)"
