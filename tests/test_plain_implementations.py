"""The two plain implementations against each other: float64 NumPy (tests/plain/llama_plain.py) and float32 C++
(tests/plain/ref_forward.cpp), written separately from the reference's formulas. They must agree before either is
used to judge the engine. Whole sequences, and the C++ one also cut into a prompt and single tokens (its cache)."""
import random

import numpy as np
import pytest

from conftest import TINY
from plain.llama_plain import forward_logits
from plain.ref_forward import RefModel


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_the_two_plain_implementations_agree(model_dirs, name):
    folder = model_dirs(name, "float32")
    rng = random.Random(5)
    n = min(TINY[name]["max_position_embeddings"], 150)
    toks = [rng.randrange(TINY[name]["vocab_size"]) for _ in range(n)]
    want = forward_logits(folder, toks)
    m = RefModel(folder)
    whole = m.forward(toks)
    assert np.abs(whole - want).max() <= 1e-5, f"whole sequence: {np.abs(whole - want).max():.3e}"
    m2 = RefModel(folder)
    head = n - 20
    rows = [m2.forward(toks[:head], 0, [0, head - 1])]
    rows += [m2.forward([toks[i]], i, [0]) for i in range(head, n)]
    cut = np.concatenate(rows)
    assert np.abs(cut - want[[0, head - 1] + list(range(head, n))]).max() <= 1e-5
    assert (whole.argmax(axis=1) == want.argmax(axis=1)).all()


def test_the_two_plain_implementations_agree_on_a_sharpened_model(sharp_dirs):
    folder = sharp_dirs("B", "float32")
    rng = random.Random(6)
    toks = [rng.randrange(512) for _ in range(120)]
    diff = np.abs(RefModel(folder).forward(toks) - forward_logits(folder, toks)).max()
    assert diff <= 1e-4, f"{diff:.3e}"
