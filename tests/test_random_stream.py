"""Seeded random weights: one counter-based stream, the same bits whoever draws them."""
import math

import numpy as np
import pytest
import torch

import plain_random


def test_numpy_stream_equals_the_plain_restatement_element_by_element():
    from hk_b200.weights import random_stream as rs
    for seed, name in ((0, "model.embed_tokens.weight"), (2, "model.layers.35.mlp.down_proj.weight"), (7, "x")):
        key = rs.tensor_key(seed, name)
        assert key == plain_random.key_of(seed, name)
        for start in (0, 1 << 20, (1 << 33) + 5):               # also far into a tensor larger than 2^32 elements
            got = rs.standard_normal(key, start, 300)
            want = np.array([plain_random.normal(key, start + i) for i in range(300)], dtype=np.float32)
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_ln_and_cos_of_the_stream_are_the_functions_they_stand_for():
    # the fixed operation sequences are ln and cos to the last bits of a double: compare with the math library
    from hk_b200.weights import random_stream as rs
    key = rs.tensor_key(1, "t")
    r = rs._bits(key, 0, 20000)
    a = (r >> np.uint64(40)).astype(np.int64)
    b = ((r >> np.uint64(16)) & np.uint64(0xFFFFFF)).astype(np.int64)
    want = np.sqrt(-2.0 * np.log((2 * a + 1) / 2.0 ** 25)) * np.cos(2 * math.pi * b / 2.0 ** 24)
    got = rs.standard_normal(key, 0, 20000).astype(np.float64)
    assert np.abs(got - want).max() < 1e-6


def test_stream_is_standard_normal_and_tensors_are_independent():
    from hk_b200.weights import random_stream as rs
    z = rs.fill(rs.tensor_key(3, "a"), 400000, 1.0, 0.0).astype(np.float64)
    assert abs(z.mean()) < 0.01 and abs(z.var() - 1) < 0.01
    assert abs(((z - z.mean()) ** 4).mean() / z.var() ** 2 - 3) < 0.05          # the tails of a normal
    assert abs((np.abs(z) > 1.959964).mean() - 0.05) < 0.003
    y = rs.fill(rs.tensor_key(3, "b"), 400000, 1.0, 0.0).astype(np.float64)
    assert abs(np.corrcoef(z, y)[0, 1]) < 0.01 and abs(np.corrcoef(z[:-1], z[1:])[0, 1]) < 0.01


def test_random_tensors_scale_and_offset_in_float32():
    from hk_b200.parts import ParamSpec, VECTOR
    from hk_b200.weights import random_tensors
    specs = {"w": ParamSpec((5, 7)), "n": ParamSpec((9,), VECTOR, "one_plus_normal")}
    t = random_tensors(specs, 4, 0.03, 0.1, "cpu")
    for i in range(35):
        assert float(t["w"].reshape(-1)[i]) == plain_random.value(4, "w", i, 0.03)
    for i in range(9):
        assert float(t["n"][i]) == plain_random.value(4, "n", i, 0.1, 1.0)
    # another tensor beside them changes neither
    t2 = random_tensors({"zzz": ParamSpec((3,)), **specs}, 4, 0.03, 0.1, "cpu")
    assert torch.equal(t["w"], t2["w"]) and torch.equal(t["n"], t2["n"])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_the_gpu_draws_the_same_bits_as_the_cpu(dtype):
    from hk_b200.parts import ParamSpec, VECTOR
    from hk_b200.weights import random_tensors
    specs = {"model.embed_tokens.weight": ParamSpec((1031, 997)), "model.norm.weight": ParamSpec((4099,), VECTOR, "one_plus_normal")}
    cpu = random_tensors(specs, 2, 0.02, 0.05, "cpu", dtype_of=lambda s: dtype)
    gpu = random_tensors(specs, 2, 0.02, 0.05, "cuda", dtype_of=lambda s: dtype)
    for k in specs:
        assert gpu[k].dtype == dtype and torch.equal(gpu[k].cpu(), cpu[k]), k
    for i in (0, 1, 12345, 1031 * 997 - 1):
        assert float(gpu["model.embed_tokens.weight"].float().reshape(-1)[i]) == \
            float(torch.tensor(plain_random.value(2, "model.embed_tokens.weight", i, 0.02)).to(dtype).float())


@pytest.mark.gpu
def test_an_engine_with_a_seed_and_a_written_model_folder_hold_the_same_weights(tmp_path):
    import helpers
    from hk_b200.config import config_from_dict
    from hk_b200.engine import Engine
    from hk_b200.weights import write_random_model
    from hk_b200.weights.safetensors_io import open_model_files
    cfg = config_from_dict(helpers.TINY_B)
    folder = str(tmp_path / "m")
    write_random_model(folder, cfg, seed=2, std=0.03, norm_std=0.1, dtype=torch.bfloat16)
    from_seed = Engine(config=cfg, random_seed=2, random_std=0.03, random_norm_std=0.1, dtype="bfloat16", max_tokens=64, max_requests=1)
    from_file = Engine(folder, dtype="bfloat16", max_tokens=64, max_requests=1)
    _same_weights(from_seed.model, from_file.model)
    # the same folder under a 32-bit engine: the seed's values rounded to bfloat16, held in 32-bit
    wide_seed = Engine(config=cfg, random_seed=2, random_std=0.03, random_norm_std=0.1, random_dtype="bfloat16", dtype="float32",
                       max_tokens=64, max_requests=1)
    wide_file = Engine(folder, dtype="float32", max_tokens=64, max_requests=1)
    assert wide_seed.model.embedding.table.dtype == torch.float32
    _same_weights(wide_seed.model, wide_file.model)
    assert torch.equal(wide_seed.model.embedding.table, from_seed.model.embedding.table.float())


def _same_weights(a, b):
    assert torch.equal(a.embedding.table, b.embedding.table) and torch.equal(a.head.weight, b.head.weight)
    for la, lb in zip(a.layers, b.layers):
        assert torch.equal(la.mixer.w_qkv, lb.mixer.w_qkv) and torch.equal(la.feed_forward.w_down, lb.feed_forward.w_down)
        assert torch.equal(la.mixer.q_norm, lb.mixer.q_norm) and torch.equal(la.mixer_norm.weight, lb.mixer_norm.weight)
