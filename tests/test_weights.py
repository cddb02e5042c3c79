"""The weight loader's errors, dtypes and the random-weights mode (no GPU)."""
import json
import os

import numpy as np
import pytest
import torch

import helpers
from hk_b200.config import config_from_dict, resolve_architecture
from hk_b200.parts import Precision
from hk_b200.weights import (SafetensorsError, WeightError, load_tensors, open_model_files, save_file,
                             write_random_model)


def specs_of(raw):
    cfg = config_from_dict(raw)
    return resolve_architecture(cfg.architecture)[1](cfg, 16).param_specs()


def cpu(dtype):
    return Precision(dtype, torch.device("cpu"))


def test_random_model_folder_loads_and_is_seeded(tmp_path):
    d = helpers.make_model_dir(tmp_path, "B", torch.bfloat16)
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    t = load_tensors(d, specs_of(helpers.TINY_B), cpu(torch.bfloat16))
    assert t["model.layers.2.mlp.down_proj.weight"].dtype == torch.bfloat16      # matrices: compute type
    assert t["model.norm.weight"].dtype == torch.float32                         # vectors: float32
    assert t["lm_head.weight"].shape == (512, 96)
    w = t["model.layers.0.self_attn.q_proj.weight"].float()
    assert abs(w.std().item() - 0.03) < 0.003 and abs(w.mean().item()) < 0.002
    n = t["model.layers.1.input_layernorm.weight"]
    assert abs(n.mean().item() - 1.0) < 0.05 and 0.05 < n.std().item() < 0.15
    # same seed, same bytes; other seed, other bytes; and the independent reader agrees
    d2 = os.path.join(str(tmp_path), "again")
    write_random_model(d2, config_from_dict(helpers.TINY_B), 1, std=0.03, norm_std=0.1, dtype=torch.bfloat16)
    a = open(os.path.join(d, "model.safetensors"), "rb").read()
    assert a == open(os.path.join(d2, "model.safetensors"), "rb").read()
    write_random_model(d2, config_from_dict(helpers.TINY_B), 2, std=0.03, norm_std=0.1, dtype=torch.bfloat16)
    assert a != open(os.path.join(d2, "model.safetensors"), "rb").read()
    plain = helpers.read_safetensors(os.path.join(d, "model.safetensors"))
    assert np.array_equal(plain["model.layers.0.self_attn.q_proj.weight"], w.double().numpy())


def test_float32_file_stays_float32_on_the_32_bit_path(tmp_path):
    d = helpers.make_model_dir(tmp_path, "A", torch.float32)
    t = load_tensors(d, specs_of(helpers.TINY_A), cpu(torch.float32))
    assert all(v.dtype == torch.float32 for v in t.values())
    assert "lm_head.weight" not in t          # tied: optional and absent
    raw = helpers.read_safetensors(os.path.join(d, "model.safetensors"))
    assert np.array_equal(raw["model.embed_tokens.weight"], t["model.embed_tokens.weight"].double().numpy())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = helpers.make_model_dir(tmp_path, "A", torch.float32)
    path = os.path.join(d, "model.safetensors")
    f = open_model_files(d)[0]
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64)
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)     # skipped, not an error
    save_file(tensors, path)
    with pytest.raises(WeightError) as e:
        load_tensors(d, specs_of(helpers.TINY_A), cpu(torch.float32))
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert err.wrong_shape == {"model.layers.0.self_attn.k_proj.weight": ((16, 64), (32, 64))}
    msg = str(err)
    for needle in ("missing (2)", "unexpected (1)", "model.norm.weight", "q_proj.bias", "is [16, 64], expected [32, 64]"):
        assert needle in msg


def test_untied_model_without_head_is_an_error_and_tied_head_may_be_present(tmp_path):
    d = helpers.make_model_dir(tmp_path, "B", torch.float32)
    f = open_model_files(d)[0]
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    head = tensors.pop("lm_head.weight")
    save_file(tensors, os.path.join(d, "model.safetensors"))
    with pytest.raises(WeightError) as e:
        load_tensors(d, specs_of(helpers.TINY_B), cpu(torch.float32))
    assert e.value.missing == ["lm_head.weight"]
    tied = dict(helpers.TINY_B, tie_word_embeddings=True)
    assert "lm_head.weight" not in load_tensors(d, specs_of(tied), cpu(torch.float32))
    tensors["lm_head.weight"] = head
    save_file(tensors, os.path.join(d, "model.safetensors"))
    assert "lm_head.weight" in load_tensors(d, specs_of(tied), cpu(torch.float32))


def test_integer_tensor_where_floats_are_expected(tmp_path):
    d = helpers.make_model_dir(tmp_path, "A", torch.float32)
    f = open_model_files(d)[0]
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    tensors["model.norm.weight"] = torch.ones(64, dtype=torch.int32)
    save_file(tensors, os.path.join(d, "model.safetensors"))
    with pytest.raises(WeightError) as e:
        load_tensors(d, specs_of(helpers.TINY_A), cpu(torch.float32))
    assert "model.norm.weight" in e.value.wrong_dtype


def test_malformed_files(tmp_path):
    d = tmp_path / "m"
    d.mkdir()
    with pytest.raises(SafetensorsError):
        open_model_files(str(d))
    (d / "model.safetensors").write_bytes(b"\x05\x00\x00")
    with pytest.raises(SafetensorsError):
        open_model_files(str(d))
    hdr = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    (d / "model.safetensors").write_bytes(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError) as e:
        open_model_files(str(d))
    assert "'x'" in str(e.value) and "16" in str(e.value)
    hdr = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    (d / "model.safetensors").write_bytes(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError):
        open_model_files(str(d))


def test_sharded_folder_follows_the_index(tmp_path):
    d = helpers.make_model_dir(tmp_path, "A", torch.float32)
    f = open_model_files(d)[0]
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    names = sorted(tensors)
    half = len(names) // 2
    save_file({n: tensors[n] for n in names[:half]}, os.path.join(d, "model-00001-of-00002.safetensors"))
    save_file({n: tensors[n] for n in names[half:]}, os.path.join(d, "model-00002-of-00002.safetensors"))
    os.unlink(os.path.join(d, "model.safetensors"))
    wm = {n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors") for i, n in enumerate(names)}
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as fh:
        json.dump({"weight_map": wm}, fh)
    t = load_tensors(d, specs_of(helpers.TINY_A), cpu(torch.float32))
    assert torch.equal(t["model.embed_tokens.weight"], tensors["model.embed_tokens.weight"])


def test_a_tensor_stored_in_32_bit_stays_so_on_the_bfloat16_path(tmp_path):
    from hk_b200.weights.safetensors_io import save_file
    d = helpers.make_model_dir(tmp_path, "A", torch.bfloat16)
    path = os.path.join(d, "model.safetensors")
    t0 = load_tensors(d, specs_of(helpers.TINY_A), cpu(torch.float32))      # everything, widened
    names32 = ["model.layers.0.self_attn.q_proj.weight", "model.layers.1.mlp.down_proj.weight", "model.norm.weight"]
    out = {}
    g = torch.Generator().manual_seed(3)
    for k, v in t0.items():
        if k in names32:
            out[k] = (v + 1e-4 * torch.randn(v.shape, generator=g)).float()      # not representable in bfloat16
        else:
            out[k] = v.to(torch.bfloat16)
    save_file(out, path)
    t = load_tensors(d, specs_of(helpers.TINY_A), cpu(torch.bfloat16))
    for k, v in t.items():
        if k in names32 or k.endswith("norm.weight") or k.endswith("layernorm.weight"):
            assert v.dtype == torch.float32, k
        else:
            assert v.dtype == torch.bfloat16, k
    assert torch.equal(t[names32[0]], out[names32[0]])
