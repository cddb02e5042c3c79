"""The two serving workloads of `hk_b200.workloads`, at a tiny shape: every request gets all its tokens, prompt
portions run beside decoded tokens, the cache's books close without a lost page."""
import types

import pytest

pytestmark = pytest.mark.gpu

TINY = dict(hidden_size=96, num_hidden_layers=2, intermediate_size=320, num_attention_heads=6, num_key_value_heads=2,
            head_dim=32, vocab_size=515)


@pytest.fixture
def tiny_shapes(monkeypatch):
    from hk_b200 import workloads
    monkeypatch.setitem(workloads.SHAPES, "serve14b", dict(TINY))
    monkeypatch.setitem(workloads.SHAPES, "mixed32b", dict(TINY))
    return workloads


def test_many_requests_with_portions_beside_decoding(tiny_shapes):
    r = tiny_shapes.serve14b(types.SimpleNamespace(layers=0))
    assert r["generated_tokens"] == 32 * 128
    assert r["mixed_steps"] > 0 and r["preemptions"] == 0
    assert r["steps"] >= 128 and r["ahead_steps"] > 0
    assert r["layers"] == TINY["num_hidden_layers"]


def test_new_prompts_arrive_beside_long_decoding_requests(tiny_shapes):
    r = tiny_shapes.mixed32b(types.SimpleNamespace(layers=1))
    assert r["generated_tokens"] == 16 * 64
    assert r["mixed_steps"] > 0 and r["preemptions"] == 0
    assert r["layers"] == 1 and r["layers_full"] == TINY["num_hidden_layers"]


def _plain_model(cfg, seed):
    """config.json keys and float64 weights of the engine `workloads._engine` builds with `seed` in float32."""
    import torch
    from hk_b200.config import resolve_architecture
    from hk_b200.weights import random_tensors
    _, build_model = resolve_architecture(cfg.architecture)
    specs = build_model(cfg, 8).param_specs()
    w = random_tensors(specs, seed, 0.02, 0.05, "cuda")
    return cfg.to_dict(), {k: v.double().cpu().numpy() for k, v in w.items()}


def _plain_greedy(cfg, w, prompt, n):
    import plain_qwen3 as P
    ids = list(prompt)
    for _ in range(n):
        ids.append(P.greedy(P.forward(cfg, w, ids)[-1]))
    return ids[len(prompt):]


def test_tokens_of_the_serving_workload_are_the_plain_greedy_tokens(tiny_shapes):
    """The workload made greedy, small and 32-bit: 32 requests in portions of 24 beside decoding; the tokens of the
    shortest, the longest and a middle request against plain greedy decoding (no cache, whole sequence every token)."""
    args = types.SimpleNamespace(layers=0, temperature=0.0, dtype="float32", prompt_range=(20, 150), new_tokens=10, portion=24,
                                 keep_tokens=True)
    r = tiny_shapes.serve14b(args)
    assert r["generated_tokens"] == 32 * 10 and r["mixed_steps"] > 0
    cfg, prompts, outputs = args.kept
    raw, w = _plain_model(cfg, 3)
    order = sorted(range(32), key=lambda i: len(prompts[i]))
    for i in (order[0], order[15], order[31], 0):
        assert outputs[i] == _plain_greedy(raw, w, prompts[i], 10), f"request {i} ({len(prompts[i])} prompt tokens)"


def test_tokens_of_the_mixed_workload_are_the_plain_greedy_tokens(tiny_shapes):
    """Eight requests far into their decoding when eight prompts arrive; old and new requests against plain greedy."""
    args = types.SimpleNamespace(layers=0, dtype="float32", context=150, new_prompt=60, new_tokens=6, portion=32, keep_tokens=True)
    r = tiny_shapes.mixed32b(args)
    assert r["generated_tokens"] == 16 * 6 and r["mixed_steps"] > 0
    cfg, prompts, outputs = args.kept
    raw, w = _plain_model(cfg, 4)
    for i in (0, 7, 8, 15):
        n = 7 if i < 8 else 6
        assert outputs[i] == _plain_greedy(raw, w, prompts[i], n), f"request {i}"
