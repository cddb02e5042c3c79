"""The serving kernels at a serving model's layer sizes (two layers of the 8B shape, a vocabulary that is no
multiple of 16): the bfloat16 engine against the float32 engine of the same seed, through prompt steps of more than
a thousand rows (tcgen05 products and attention), a 2,048-token portion, a mixed step and replayed decode graphs
(streaming and small-M products, TMA-fed decode attention).  The tiny configurations of the other tests never reach
these kernels' large-shape paths."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPE = dict(architectures=["Qwen3ForCausalLM"], hidden_size=4096, num_hidden_layers=2, intermediate_size=12288,
             num_attention_heads=32, num_key_value_heads=8, head_dim=128, vocab_size=32003, rope_theta=1000000.0,
             rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=4096, initializer_range=0.02)


def test_bfloat16_engine_follows_the_float32_engine_at_serving_sizes():
    from hk_b200.config import config_from_dict
    from hk_b200.engine import Engine, StepEntry
    cfg = config_from_dict(SHAPE)
    rng = np.random.default_rng(0)
    v = SHAPE["vocab_size"]
    prompts = {"a": rng.integers(0, v, 700).tolist(), "b": rng.integers(0, v, 333).tolist(), "c": rng.integers(0, v, 2100).tolist()}
    outs = {}
    for dt in ("float32", "bfloat16"):
        e = Engine(config=cfg, random_seed=7, dtype=dt, max_tokens=4096, page_tokens=64, max_requests=3, max_context=4096,
                   max_batch_tokens=4096)
        for k in prompts:
            e.open_request(k)
        res = [e.step([StepEntry("a", prompts["a"], [0, 350, 699]), StepEntry("b", prompts["b"], [332])]).float().cpu(),
               e.step([StepEntry("c", prompts["c"][:2048], [2047])]).float().cpu(),
               e.step([StepEntry("c", prompts["c"][2048:], [51]), StepEntry("a", [5], [0])]).float().cpu()]
        for s in range(5):
            res.append(e.step([StepEntry(k, [100 + s], [0]) for k in prompts]).float().cpu())
        outs[dt] = torch.cat(res)
        if dt == "bfloat16":
            assert 3 in e._graphs                      # the last steps replayed a captured graph
            from hk_b200.csrc import gemm_fast
            gemm_fast.check_status(e.device)
        del e
        torch.cuda.empty_cache()
    a, b = outs["float32"], outs["bfloat16"]
    scale = a.abs().max().item()
    err = (a - b).abs().max(dim=1).values / scale
    # the float32 engine computes with weights that were not rounded to bfloat16, so this bound also holds that rounding
    assert err.max().item() <= 2e-2, err.tolist()
    top2 = a.topk(2, dim=1).values
    clear = (top2[:, 0] - top2[:, 1]) / scale > 2e-2
    assert torch.equal(a.argmax(1)[clear], b.argmax(1)[clear])


def test_decode_batch_of_twenty_at_serving_sizes():
    """Twenty requests decoding together: the graph of 24 rows (filled up with repeats), tcgen05 products with K
    slices for 24 rows, decode attention without key splits; against the float32 engine."""
    from hk_b200.config import config_from_dict
    from hk_b200.engine import Engine, StepEntry
    cfg = config_from_dict(SHAPE)
    rng = np.random.default_rng(1)
    v = SHAPE["vocab_size"]
    prompts = [rng.integers(0, v, int(n)).tolist() for n in rng.integers(90, 330, 20)]
    outs = {}
    for dt in ("float32", "bfloat16"):
        e = Engine(config=cfg, random_seed=9, dtype=dt, max_tokens=20 * 384, page_tokens=64, max_requests=20, max_context=384,
                   max_batch_tokens=4096)
        for i in range(20):
            e.open_request(i)
        for lo in (0, 10):
            e.step([StepEntry(i, prompts[i], []) for i in range(lo, lo + 10)])
        res = [e.step([StepEntry(i, [7 + s + i], [0]) for i in range(20)]).float().cpu() for s in range(3)]
        outs[dt] = torch.cat(res)
        if dt == "bfloat16":
            assert 24 in e._graphs
            from hk_b200.csrc import gemm_fast
            gemm_fast.check_status(e.device)
        del e
        torch.cuda.empty_cache()
    a, b = outs["float32"], outs["bfloat16"]
    scale = a.abs().max().item()
    assert ((a - b).abs().max(dim=1).values / scale).max().item() <= 2e-2


WIDER = {
    # one layer each of the two larger serving shapes: a hidden width that is no power of two, 40 and 64 query heads
    # (query width equal to and larger than the hidden width), feed-forward widths of 17,408 and 25,600
    "hidden5120_heads40": dict(hidden_size=5120, num_attention_heads=40, intermediate_size=17408, vocab_size=20011),
    "hidden5120_heads64": dict(hidden_size=5120, num_attention_heads=64, intermediate_size=25600, vocab_size=16001),
}


@pytest.mark.parametrize("name", sorted(WIDER))
def test_wider_serving_shapes(name):
    """Prompt steps (one of more than a thousand rows, one mixed with a decoded token) and replayed decode graphs at
    the layer sizes of the larger models of the family; the bfloat16 engine against the float32 engine."""
    from hk_b200.config import config_from_dict
    from hk_b200.engine import Engine, StepEntry
    cfg = config_from_dict(dict(SHAPE, num_hidden_layers=1, max_position_embeddings=2048, **WIDER[name]))
    rng = np.random.default_rng(2)
    v = cfg.vocab_size
    prompts = {"a": rng.integers(0, v, 1100).tolist(), "b": rng.integers(0, v, 150).tolist(), "c": rng.integers(0, v, 77).tolist()}
    outs = {}
    for dt in ("float32", "bfloat16"):
        e = Engine(config=cfg, random_seed=11, dtype=dt, max_tokens=2048, page_tokens=64, max_requests=3, max_context=1280,
                   max_batch_tokens=2048)
        for k in prompts:
            e.open_request(k)
        res = [e.step([StepEntry("a", prompts["a"], [0, 1099])]).float().cpu(),
               e.step([StepEntry("b", prompts["b"], [149]), StepEntry("a", [3], [0]), StepEntry("c", prompts["c"], [76])]).float().cpu()]
        for s in range(4):
            res.append(e.step([StepEntry(k, [50 + s], [0]) for k in prompts]).float().cpu())
        outs[dt] = torch.cat(res)
        if dt == "bfloat16":
            assert 3 in e._graphs
            from hk_b200.csrc import gemm_fast
            gemm_fast.check_status(e.device)
        del e
        torch.cuda.empty_cache()
    a, b = outs["float32"], outs["bfloat16"]
    scale = a.abs().max().item()
    assert ((a - b).abs().max(dim=1).values / scale).max().item() <= 2e-2
