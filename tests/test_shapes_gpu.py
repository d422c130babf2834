"""The engine at SmolLM2 widths (few layers, so that the float64 plain implementation stays quick): real head
counts, head size 64, hidden sizes 576 and 2048, the 49,152-token vocabulary. A prompt portion long enough for
the tile kernels (tcgen05 GEMM with the rotation and cache write in its epilogue, tcgen05 attention over more
than one key tile), a second portion that takes the few-row kernels, then single decoded tokens."""
import random

import numpy as np
import pytest
import torch

import glassbox_b200
from conftest import assert_logits_close
from glassbox_b200.models.llama import make_llama_raw_config
from plain.llama_plain import forward_logits

pytestmark = pytest.mark.gpu

SHAPES = {
    "135m": dict(num_hidden_layers=2, hidden_size=576, num_attention_heads=9, num_key_value_heads=3,
                 intermediate_size=1536, vocab_size=49152, rope_theta=100000.0, rms_norm_eps=1e-5,
                 tie_word_embeddings=True, max_position_embeddings=8192),
    "1.7b": dict(num_hidden_layers=1, hidden_size=2048, num_attention_heads=32, num_key_value_heads=32,
                 intermediate_size=8192, vocab_size=49152, rope_theta=130000.0, rms_norm_eps=1e-5,
                 tie_word_embeddings=True, max_position_embeddings=8192),
}


@pytest.mark.parametrize("shape, dtype", [("135m", "float32"), ("135m", "bfloat16"), ("1.7b", "bfloat16")])
def test_smollm2_widths_portions_and_decoding(tmp_path, shape, dtype):
    from glassbox_b200.engine.engine import Engine, StepEntry
    folder = str(tmp_path / "m")
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    glassbox_b200.write_random_model(folder, make_llama_raw_config(**SHAPES[shape]), 5, store)
    rng = random.Random(2)
    T, first, second = 330, 270, 40
    toks = [rng.randrange(SHAPES[shape]["vocab_size"]) for _ in range(T)]
    ref = forward_logits(folder, toks)
    eng = Engine(folder, dtype, cache_tokens=1024, max_batch_tokens=512, max_requests=4)
    eng.add_request("a")
    want_first = [0, 1, 127, 128, 129, first - 1]
    rows = [eng.step([StepEntry("a", toks[:first], want_first)]).cpu().numpy()]
    want_second = [0, 17, second - 1]
    rows.append(eng.step([StepEntry("a", toks[first:first + second], want_second)]).cpu().numpy())
    for i in range(first + second, T):
        rows.append(eng.step([StepEntry("a", [toks[i]], [0])]).cpu().numpy())
    eng.check()
    got = np.concatenate(rows)
    places = want_first + [first + w for w in want_second] + list(range(first + second, T))
    assert_logits_close(got, ref[places], dtype, f"{shape} widths: portions of {first} and {second} tokens, then decoding")
