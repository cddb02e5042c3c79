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


def plain_weights(cfg, seed, std, norm_std, dtype):
    """The tensors an engine of this seed computes with, by their Hugging Face names, as float64 numpy arrays: drawn
    again from the seeded stream (the same bits on every device; tests/test_random_stream.py) in the working types."""
    from hk_b200.config import resolve_architecture
    from hk_b200.parts import Precision
    from hk_b200.weights import random_tensors
    _, build_model = resolve_architecture(cfg.architecture)
    prec = Precision(dtype, torch.device("cuda"))
    specs = build_model(cfg, 8).param_specs()
    out = {}
    for name, spec in specs.items():        # one tensor at a time: the float64 copies are what takes the memory
        t = random_tensors({name: spec}, seed, std, norm_std, "cuda", dtype_of=lambda s: prec.working_dtype(s.kind))
        out[name] = t[name].double().cpu().numpy()
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_serving_sizes_against_the_plain_implementation(dtype):
    """Two layers of the 8B shape against the plain implementation (not against another path of the engine): a
    prompt of 150 tokens whole, in portions down to two tokens, with its tail token by token, and mixed with a second
    request.  Rows of 4,096 and 12,288 elements, 32 heads of 128, block tables of 64-token and 16-token pages."""
    import helpers
    import plain_qwen3
    from hk_b200.config import config_from_dict
    from hk_b200.engine import Engine
    cfg = config_from_dict(SHAPE)
    rng = np.random.default_rng(5)
    seqs = {"a": rng.integers(0, SHAPE["vocab_size"], 150).tolist(), "b": rng.integers(0, SHAPE["vocab_size"], 70).tolist()}
    weights = plain_weights(cfg, 13, 0.02, 0.05, dtype)
    ref = {k: plain_qwen3.forward(SHAPE, weights, ids) for k, ids in seqs.items()}
    del weights
    scale = max(np.abs(r).max() for r in ref.values())
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for page_tokens, family in ((64, "whole"), (16, "portions"), (64, "tail"), (16, "mixed")):
        steps = {"whole": helpers.trace_whole, "portions": helpers.trace_portions, "tail": helpers.trace_tail_decode,
                 "mixed": lambda s: helpers.trace_mixed(s, np.random.default_rng(2), max_live=2)}[family](seqs)
        e = Engine(config=cfg, random_seed=13, dtype=dtype, max_tokens=512, page_tokens=page_tokens, max_requests=2, max_context=256,
                   max_batch_tokens=512)
        got = helpers.run_trace_on_engine(e, steps)
        e.check_kernel_status()
        assert len(got) == 220
        for (rid, p), v in sorted(got.items()):
            d = np.abs(v.astype(np.float64) - ref[rid][p]).max()
            assert d <= tol * scale, f"{family}: first wrong position: request {rid} position {p}: |diff| {d:.3g} > {tol * scale:.3g}"
        del e
        torch.cuda.empty_cache()


def test_full_depth_parity_at_the_8b_shape():
    """All 36 layers of the 8B shape: the float32 engine gives the same logits whole, in portions and mixed with a second
    request (within 2e-5 of the largest logit), and the bfloat16 engine stays within 2e-2 of it.  Both compute with the
    same matrices (the seed's values rounded to bfloat16, as a bfloat16 model folder stores them), so the second bound
    is on the arithmetic alone."""
    import gc

    import helpers
    from hk_b200.config import config_from_dict
    from hk_b200.engine import Engine
    shape = dict(SHAPE, num_hidden_layers=36, vocab_size=151936)
    cfg = config_from_dict(shape)
    rng = np.random.default_rng(6)
    seqs = {"a": rng.integers(0, shape["vocab_size"], 96).tolist(), "b": rng.integers(0, shape["vocab_size"], 41).tolist()}
    want_rows = {"a": [0, 1, 17, 50, 94, 95], "b": [0, 40]}

    def run(dtype, family):
        steps = {"whole": helpers.trace_whole, "portions": helpers.trace_portions,
                 "mixed": lambda s: helpers.trace_mixed(s, np.random.default_rng(2), max_live=2)}[family](seqs)
        # logits only at a few places of each request: a row of 151,936 floats for every token is not needed
        pos, thin = {k: 0 for k in seqs}, []
        for st in steps:
            entries = []
            for rid, toks, _ in st["entries"]:
                entries.append((rid, toks, [w - pos[rid] for w in want_rows[rid] if pos[rid] <= w < pos[rid] + len(toks)]))
                pos[rid] += len(toks)
            thin.append({"entries": entries, "end": st["end"]})
        e = Engine(config=cfg, random_seed=2, random_dtype="bfloat16", dtype=dtype, max_tokens=256, page_tokens=16, max_requests=2,
                   max_context=128, max_batch_tokens=256)
        got = helpers.run_trace_on_engine(e, thin)
        e.check_kernel_status()
        del e
        gc.collect()
        torch.cuda.empty_cache()
        return got

    whole = run(torch.float32, "whole")
    assert sorted(whole) == sorted((k, w) for k, ws in want_rows.items() for w in ws)
    scale = max(np.abs(v).max() for v in whole.values())
    for family in ("portions", "mixed"):
        got = run(torch.float32, family)
        for key, v in whole.items():
            assert np.abs(got[key] - v).max() <= 2e-5 * scale, (family, key)
    # bfloat16 against it: every layer rounds the inputs of its four products and its cache entries to 8 bits, the
    # residual sum stays in 32-bit, so the layers' errors are independent and add in quadrature.  The bound of the
    # tiny configurations (2e-2 of the largest logit at up to 4 layers) therefore scales with the square root of the
    # depth: 6e-2 at 36 layers (measured: 0.84e-2, 1.1e-2, 1.7e-2, 2.1e-2, 3.2e-2 at 2, 4, 9, 18, 36 layers).
    bound = 2e-2 * (36 / 4) ** 0.5
    for family in ("whole", "mixed"):
        got = run(torch.bfloat16, family)
        diffs = np.stack([np.abs(got[key] - v) for key, v in whole.items()])
        assert diffs.max() / scale <= bound, (family, diffs.max() / scale)
        assert diffs.mean() / scale <= 3e-3 * (36 / 4) ** 0.5, (family, diffs.mean() / scale)


def test_bfloat16_error_grows_with_the_square_root_of_the_depth():
    """The rounding model behind the bounds above, measured: the same prompt through 4 and 36 layers of the 8B shape in
    bfloat16 against 32-bit with the same matrices.  Nine times the depth gives three times the error (within a
    factor 1.6 either way); a fault in some layer or at some depth would break the law."""
    import gc

    from hk_b200.config import config_from_dict
    from hk_b200.engine import Engine, StepEntry
    rng = np.random.default_rng(6)
    ids = rng.integers(0, 151936, 96).tolist()
    worst = {}
    for layers in (4, 36):
        cfg = config_from_dict(dict(SHAPE, num_hidden_layers=layers, vocab_size=151936))
        outs = {}
        for dt in ("float32", "bfloat16"):
            e = Engine(config=cfg, random_seed=2, random_dtype="bfloat16", dtype=dt, max_tokens=256, page_tokens=16, max_requests=2,
                       max_context=128, max_batch_tokens=256)
            e.open_request("a")
            outs[dt] = e.step([StepEntry("a", ids, [0, 1, 17, 50, 94, 95])]).float().cpu().numpy()
            e.check_kernel_status()
            del e
            gc.collect()
            torch.cuda.empty_cache()
        worst[layers] = np.abs(outs["float32"] - outs["bfloat16"]).max() / np.abs(outs["float32"]).max()
    assert worst[4] <= 2e-2
    assert 3 / 1.6 <= worst[36] / worst[4] <= 3 * 1.6, worst
