"""Safetensors reading/writing, name binding and the loader's error report (CPU)."""
import json
import os

import pytest
import torch

import glassbox_b200
from glassbox_b200.config.registry import get_architecture
from glassbox_b200.engine.model import DecoderModel
from glassbox_b200.weights import SafetensorsFile, WeightsError, load_parameters, random_tensors, write_safetensors

from conftest import tiny_raw


def _load(folder, dtype):
    cfg = glassbox_b200.load_config(folder)
    model = DecoderModel(cfg)
    with SafetensorsFile(os.path.join(folder, "model.safetensors")) as st:
        return model, load_parameters(model.param_specs(), get_architecture(cfg.architecture).bind(cfg), st, dtype,
                                      "cpu")


def test_round_trip_matches_the_safetensors_library(tmp_path):
    from safetensors.torch import load_file
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32),
               "d": torch.randn(2, 2).to(torch.float16)}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, tensors)
    theirs = load_file(path)
    with SafetensorsFile(path) as st:
        assert set(st.names()) == set(tensors)
        for k, v in tensors.items():
            assert torch.equal(st.tensor(k), v) and torch.equal(theirs[k], v)


def test_random_model_folder_loads_and_stacks(model_dirs):
    folder = model_dirs("B", "bfloat16")
    model, params = _load(folder, torch.bfloat16)
    assert params["layers.0.mixer.wqkv"].shape == (3 * 32 + 2 * 32, 96)
    assert params["layers.0.mixer.wqkv"].dtype == torch.bfloat16
    assert params["layers.1.mixer_norm.weight"].dtype == torch.float32      # gains are always float32
    assert params["head.weight"].data_ptr() != params["embed.weight"].data_ptr()
    with SafetensorsFile(os.path.join(folder, "model.safetensors")) as st:
        q = st.tensor("model.layers.2.self_attn.q_proj.weight")
        v = st.tensor("model.layers.2.self_attn.v_proj.weight")
        assert torch.equal(params["layers.2.mixer.wqkv"][:96], q) and torch.equal(params["layers.2.mixer.wqkv"][128:], v)
        up = st.tensor("model.layers.0.mlp.up_proj.weight")
        assert torch.equal(params["layers.0.ffn.w_gate_up"][256:], up)
    # gains are not exactly one, so a mistake in applying them shows
    assert (params["final_norm.weight"] - 1).abs().max() > 1e-3


def test_tied_head_shares_storage_and_tolerates_a_stored_head(model_dirs, tmp_path):
    folder = model_dirs("A", "float32")
    _, params = _load(folder, torch.float32)
    assert params["head.weight"].data_ptr() == params["embed.weight"].data_ptr()
    tensors = random_tensors(tiny_raw("A"), 5, torch.float32)
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    (tmp_path / "config.json").write_text(json.dumps(tiny_raw("A")))
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    _load(str(tmp_path), torch.float32)


def test_precision_rule(model_dirs, tmp_path):
    # float32 mode widens everything
    _, p32 = _load(model_dirs("A", "bfloat16"), torch.float32)
    assert all(t.dtype == torch.float32 for t in p32.values())
    # bfloat16 mode keeps a matrix that the file stores in 32-bit
    tensors = random_tensors(tiny_raw("A"), 5, torch.bfloat16)
    name = "model.layers.0.self_attn.o_proj.weight"
    tensors[name] = tensors[name].float()
    (tmp_path / "config.json").write_text(json.dumps(tiny_raw("A")))
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    _, p = _load(str(tmp_path), torch.bfloat16)
    assert p["layers.0.mixer.wo"].dtype == torch.float32 and p["layers.1.mixer.wo"].dtype == torch.bfloat16


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    raw = tiny_raw("B")
    tensors = random_tensors(raw, 1, torch.float32)
    del tensors["model.layers.1.mlp.down_proj.weight"]
    del tensors["lm_head.weight"]                                   # untied config must bring its head
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 96)
    tensors["model.layers.7.extra.weight"] = torch.zeros(2)
    tensors["model.norm.weight"] = torch.zeros(96, dtype=torch.int32)
    (tmp_path / "config.json").write_text(json.dumps(raw))
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    with pytest.raises(WeightsError) as e:
        _load(str(tmp_path), torch.float32)
    msg = str(e.value)
    for needle in ("model.layers.1.mlp.down_proj.weight", "lm_head.weight", "model.layers.7.extra.weight",
                   "model.layers.0.self_attn.k_proj.weight", "[16, 96]", "[32, 96]", "model.norm.weight",
                   "missing", "unexpected", "wrong"):
        assert needle in msg, needle


def test_broken_files_are_refused(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x01")
    with pytest.raises(WeightsError):
        SafetensorsFile(str(p))
    p.write_bytes((10 ** 9).to_bytes(8, "little") + b"{}")
    with pytest.raises(WeightsError):
        SafetensorsFile(str(p))
    header = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 64]}}).encode()
    p.write_bytes(len(header).to_bytes(8, "little") + header + b"\0" * 16)
    with pytest.raises(WeightsError):
        SafetensorsFile(str(p))
    with pytest.raises(WeightsError):
        SafetensorsFile(str(tmp_path / "nothing.safetensors"))


def test_random_weights_depend_on_seed_only(tmp_path):
    a = random_tensors(tiny_raw("A"), 3, torch.float32)
    b = random_tensors(tiny_raw("A"), 3, torch.float32)
    c = random_tensors(tiny_raw("A"), 4, torch.float32)
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    w = a["model.layers.0.mlp.gate_proj.weight"]
    assert abs(float(w.std()) - 0.02) < 2e-3
