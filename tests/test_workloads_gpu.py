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
