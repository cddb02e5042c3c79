"""Generation through the entry points, long decoding, the first tokens of a sequence, and the
device sampler against the plain restatement of the reference's chain."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers
import plain_qwen3 as P

pytestmark = pytest.mark.gpu
ROOT = os.path.join(os.path.dirname(os.path.abspath(__file__)), os.pardir)


def plain_greedy(cfg, w, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        ids.append(P.greedy(P.forward(cfg, w, ids)[-1]))
    return ids[len(prompt):]


@pytest.fixture(scope="module")
def model_b(tmp_path_factory):
    d = helpers.make_model_dir(tmp_path_factory.mktemp("gen"), "B", torch.float32)
    return (d,) + helpers.load_plain(d)


def test_greedy_generation_through_the_entry_point(model_b):
    import hk_b200
    d, cfg, w = model_b
    prompts = helpers.prompts_for("B", np.random.default_rng(5), [5, 19, 64, 33])
    want = [plain_greedy(cfg, w, p, 8) for p in prompts]
    got = hk_b200.generate(d, prompts, max_new_tokens=8, temperature=0, dtype="float32")
    assert got == want
    # a tight pool and few slots: requests wait, portions are short, pages are reused; same tokens
    from hk_b200.api import GenerationStats, generate_with_engine
    eng = hk_b200.Engine(d, dtype="float32", max_tokens=192, page_tokens=8, max_requests=2, max_context=128, max_batch_tokens=24)
    st = GenerationStats()
    assert generate_with_engine(eng, prompts, 8, temperature=0, prefill_chunk=13, stats=st) == want
    assert st.generated_tokens == 32 and st.prompt_tokens == 121 and eng.free_pages() == [24]
    # the reference's class and signature: input followed by new tokens, tensor in, tensor out
    model = hk_b200.HKForCausalLM(eng)
    out = model.generate(torch.tensor([prompts[0]]), max_new_tokens=8, temperature=0)
    assert out.shape == (1, 13) and out[0].tolist() == prompts[0] + want[0]


def test_bfloat16_greedy_generation_agrees_where_the_margin_is_clear(tmp_path):
    import hk_b200
    d = helpers.make_model_dir(tmp_path, "A", torch.bfloat16)
    cfg, w = helpers.load_plain(d)
    prompts = helpers.prompts_for("A", np.random.default_rng(6), [7, 16, 33])
    got = hk_b200.generate(d, prompts, max_new_tokens=8, temperature=0, dtype="bfloat16")
    for p, g in zip(prompts, got):
        ids = list(p)
        for tok in g:                      # follow the engine's own tokens; check each choice against the oracle
            logits = P.forward(cfg, w, ids)[-1]
            top = np.sort(logits)[-2:]
            assert logits[tok] >= top[1] - 0.02 * np.abs(logits).max(), "the engine chose a token the oracle ranks clearly lower"
            ids.append(tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_run_ahead_decoding_gives_the_same_tokens(tmp_path, dtype):
    """Decode steps launched before the earlier tokens are read (ids handed over on the device) against
    the step-by-step order: greedy and seeded sampling, an end token in the middle, a tight pool."""
    import hk_b200
    from hk_b200.api import GenerationStats, generate_with_engine
    d = helpers.make_model_dir(tmp_path, "A", torch.float32 if dtype == "float32" else torch.bfloat16)
    prompts = helpers.prompts_for("A", np.random.default_rng(8), [3, 21, 40, 9])
    eng = hk_b200.Engine(d, dtype=dtype, max_tokens=384, max_requests=4, max_context=96)
    for kw in (dict(temperature=0), dict(temperature=0.9, top_k=20, top_p=0.9, seed=11)):
        base = generate_with_engine(eng, prompts, 40, run_ahead=False, eos_token_ids=(), **kw)
        st = GenerationStats()
        assert generate_with_engine(eng, prompts, 40, run_ahead=True, eos_token_ids=(), stats=st, **kw) == base
        assert st.decode_steps >= 39
        # an end token taken from the middle of one request's output: that request stops there, the others go on
        eos = base[1][17]
        cut = [o[:o.index(eos)] if eos in o else o for o in base]
        assert generate_with_engine(eng, prompts, 40, run_ahead=True, eos_token_ids=(eos,), **kw) == cut
    assert eng.free_pages() == [eng.cache.books.groups[0].pool.num_pages] * len(eng.cache.books.groups)


@pytest.mark.parametrize("run_ahead", [False, True])
def test_decode_graphs_are_shared_by_batch_sizes_that_round_to_the_same(model_b, run_ahead):
    """Eleven requests of different lengths: the decode batch shrinks from 11 to 1 as they finish.  Sizes above 8
    replay the graph of the next multiple of 8, filled up with repeats of the last row; the tokens are the plain
    implementation's."""
    import hk_b200
    from hk_b200.api import generate_with_engine
    d, cfg, w = model_b
    prompts = helpers.prompts_for("B", np.random.default_rng(12), [3, 9, 4, 17, 6, 5, 11, 8, 2, 7, 10])
    eng = hk_b200.Engine(d, dtype="float32", max_tokens=11 * 64, max_requests=11, max_context=64)
    from hk_b200.engine.scheduler import Scheduler
    from hk_b200.sampling import GREEDY
    sched = Scheduler(eng, prefill_chunk=64, eos_token_ids=(), run_ahead=run_ahead)
    ids = [sched.submit(p, 3 + i, GREEDY) for i, p in enumerate(prompts)]
    done = sched.run()
    for i, (rid, p) in enumerate(zip(ids, prompts)):
        assert done[rid].output == plain_greedy(cfg, w, p, 3 + i)
    assert set(eng._graphs) <= {16, 8, 7, 6, 5, 4, 3, 2, 1} and 16 in eng._graphs
    assert eng.free_pages() == [eng.cache.num_pages]


def test_matrices_stored_in_32_bit_run_in_32_bit_on_the_bfloat16_path(tmp_path):
    """A bfloat16 model folder in which a few matrices (and the embedding) are stored as float32 with values that
    bfloat16 cannot hold: the engine keeps them so, runs their products in 32-bit, and the logits follow the plain
    implementation of exactly the stored values, whole and cut."""
    from hk_b200.engine import Engine, StepEntry
    from hk_b200.weights import load_tensors
    from hk_b200.weights.safetensors_io import save_file
    d = helpers.make_model_dir(tmp_path, "A", torch.bfloat16)
    path = os.path.join(d, "model.safetensors")
    stored = {k: torch.from_numpy(v).float() for k, v in helpers.read_safetensors(path).items()}
    names32 = ["model.embed_tokens.weight", "model.layers.0.self_attn.k_proj.weight", "model.layers.0.mlp.gate_proj.weight",
               "model.layers.1.self_attn.o_proj.weight", "model.layers.1.mlp.down_proj.weight"]
    g = torch.Generator().manual_seed(4)
    out = {k: (v + 2e-4 * torch.randn(v.shape, generator=g)).float() if k in names32 else v.to(torch.bfloat16) for k, v in stored.items()}
    save_file(out, path)
    cfg, w = helpers.load_plain(d)
    eng = Engine(d, dtype="bfloat16", max_tokens=128, page_tokens=16, max_requests=2)
    blk0, blk1 = eng.model.layers[0], eng.model.layers[1]
    assert eng.model.embedding.table.dtype == torch.float32
    assert blk0.mixer.w_qkv.dtype == torch.float32 and blk0.mixer.w_o.dtype == torch.bfloat16
    assert blk0.feed_forward.w_gate_up.dtype == torch.float32 and blk0.feed_forward.w_down.dtype == torch.bfloat16
    assert blk1.mixer.w_qkv.dtype == torch.bfloat16 and blk1.mixer.w_o.dtype == torch.float32
    assert blk1.feed_forward.w_down.dtype == torch.float32
    ids = helpers.prompts_for("A", np.random.default_rng(3), [45])[0]
    ref = P.forward(cfg, w, ids)
    scale = np.abs(ref).max()
    eng.open_request("w")
    whole = eng.step([StepEntry("w", ids, list(range(45)))]).double().cpu().numpy()
    eng.open_request("c")
    parts = [eng.step([StepEntry("c", ids[a:b], list(range(b - a)))]).double().cpu().numpy() for a, b in ((0, 17), (17, 19), (19, 44), (44, 45))]
    assert np.abs(whole - ref).max() <= 2e-2 * scale
    assert np.abs(np.concatenate(parts) - ref).max() <= 2e-2 * scale


@pytest.mark.parametrize("which,page_tokens,max_tokens", [("C", 16, 256), ("D", 16, 384), ("B", 8, 104)])
def test_scheduler_under_pressure_follows_the_plain_implementation(tmp_path, which, page_tokens, max_tokens):
    """Twelve requests arrive while others run, over three slots and a pool so small that requests wait, prompt
    portions are shortened, pages are reused and the newest request is preempted and recomputed; windowed
    configurations give pages back as they go.  Every request's greedy tokens are the plain implementation's."""
    from hk_b200.engine import Engine
    from hk_b200.engine.scheduler import Scheduler
    from hk_b200.sampling import GREEDY
    d = helpers.make_model_dir(tmp_path, which, torch.float32)
    cfg, w = helpers.load_plain(d)
    rng = np.random.default_rng(21)
    lengths = [int(x) for x in rng.integers(3, 70, 12)]
    news = [int(x) for x in rng.integers(2, 14, 12)]
    prompts = helpers.prompts_for(which, rng, lengths)
    eng = Engine(d, dtype="float32", max_tokens=max_tokens, page_tokens=page_tokens, max_requests=3, max_context=96, max_batch_tokens=40)
    sched = Scheduler(eng, prefill_chunk=24, eos_token_ids=(), run_ahead=True)
    ids, k = [], 0
    for step in range(2000):
        if k < 12 and step % 3 == 0:
            ids.append(sched.submit(prompts[k], news[k], GREEDY))
            k += 1
        if not sched.has_work() and k == 12:
            break
        sched.step()
        eng.cache.books.audit()
    assert k == 12 and not sched.has_work()
    for rid, p, n in zip(ids, prompts, news):
        assert sched.finished[rid].output == plain_greedy(cfg, w, p, n), f"request {rid}"
    assert eng.free_pages() == [eng.cache.num_pages] * len(eng.cache.books.groups)
    if which == "B":
        assert sched.stats.preemptions >= 1


def test_native_engine_forward_and_rewind(model_b):
    import hk_b200
    d, cfg, w = model_b
    ids = helpers.prompts_for("B", np.random.default_rng(8), [20])[0]
    ref = P.forward(cfg, w, ids)
    with hk_b200.NativeHKEngine(d, dtype="float32") as eng:
        assert eng.vocab_size == 512 and eng.context_size == 256
        a = eng.forward(ids[:12], 0)
        b = eng.forward_step(ids[12], 12)
        c = eng.forward(ids[5:], 5)          # rewinds to position 5 and feeds the rest again
        eng.reset_cache()
        e = eng.forward(ids, 0)
    scale = np.abs(ref).max()
    for got, want in ((a, ref[11]), (b, ref[12]), (c, ref[19]), (e, ref[19])):
        assert np.abs(got - want).max() < 2e-5 * scale


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_long_decoding_and_first_tokens(tmp_path, dtype):
    """A 3-token prompt given token by token from position 0, then 300 more single-token steps
    (twenty pages of 16), every step compared with the plain implementation."""
    from hk_b200.engine import Engine, StepEntry
    d = helpers.make_model_dir(tmp_path, "C", dtype)
    cfg, w = helpers.load_plain(d)
    ids = helpers.prompts_for("C", np.random.default_rng(9), [303])[0]
    ref = P.forward(cfg, w, ids)
    eng = Engine(d, dtype=dtype, max_tokens=320, page_tokens=16, max_requests=1, max_context=320)
    eng.open_request("r")
    tol_max = 2e-5 if dtype == torch.float32 else 2e-2
    scale = np.abs(ref).max()
    for p, tok in enumerate(ids):
        got = eng.step([StepEntry("r", [tok], [0])])[0].double().cpu().numpy()
        err = np.abs(got - ref[p]).max()
        assert err <= tol_max * scale, f"first wrong position {p}: {err:.3g}"
    eng.close_request("r")


def test_step_errors_leave_the_engine_usable(model_b):
    # cf. tests/test_engine.zig:189-203 of the reference
    from hk_b200.cache import ContextFull, OutOfPages
    from hk_b200.engine import BatchTooLarge, Engine, EngineError, StepEntry, TokenOutOfRange
    d, cfg, w = model_b
    eng = Engine(d, dtype="float32", max_tokens=64, page_tokens=8, max_requests=2, max_context=48, max_batch_tokens=40)
    eng.open_request("a")
    eng.open_request("b")
    ids = helpers.prompts_for("B", np.random.default_rng(10), [30])[0]
    with pytest.raises(TokenOutOfRange):
        eng.step([StepEntry("a", [1, 512], [1])])
    with pytest.raises(BatchTooLarge):
        eng.step([StepEntry("a", ids[:30], []), StepEntry("b", ids[:11], [])])
    with pytest.raises(ContextFull):
        eng.step([StepEntry("a", ids + ids[:19], [])])
    with pytest.raises(EngineError):
        eng.step([StepEntry("a", ids[:3], [3])])
    with pytest.raises(EngineError):
        eng.step([StepEntry("zz", ids[:3], [])])
    eng.step([StepEntry("a", ids[:30], [])])          # 4 of 8 pages
    eng.step([StepEntry("b", ids[:30], [])])          # the other 4
    with pytest.raises(OutOfPages):
        eng.step([StepEntry("a", ids[:3], [])])
    assert eng.request_length("a") == 30 and eng.free_pages() == [0]
    eng.cache.books.audit()
    eng.close_request("b")
    got = eng.step([StepEntry("a", ids[:3], [2])])[0].double().cpu().numpy()
    ref = P.forward(cfg, w, ids + ids[:3])[-1]
    assert np.abs(got - ref).max() < 2e-5 * np.abs(ref).max()


def test_a_recorded_kernel_timeout_is_raised_at_the_next_step_and_cleared(tmp_path):
    """The status word that a timed-out barrier wait would set is written from the host here (no kernel is
    made to wait): the engine raises at the step after the one that carried it, then works again."""
    from hk_b200.csrc import gemm_fast
    from hk_b200.engine import Engine, KernelTimeout, StepEntry
    d = helpers.make_model_dir(tmp_path, "A", torch.bfloat16)
    eng = Engine(d, dtype="bfloat16", max_tokens=128)
    eng.open_request("a")
    first = eng.step([StepEntry("a", [1, 2, 3], [2])]).clone()
    gemm_fast.status_flag(eng.device).fill_(1)
    eng.step([StepEntry("a", [4], [0])])
    torch.cuda.synchronize()
    with pytest.raises(KernelTimeout):
        eng.step([StepEntry("a", [5], [0])])
    assert eng.request_length("a") == 4              # the refused step changed nothing
    eng.close_request("a")
    eng.open_request("a")
    assert torch.equal(eng.step([StepEntry("a", [1, 2, 3], [2])]), first)
    gemm_fast.check_status(eng.device)


# ---- the sampler -------------------------------------------------------------------------------


def sample_many(logits_row, params, draws):
    from hk_b200.sampling import Sampler, SamplingState
    s = Sampler(torch.device("cuda"))
    logits = torch.tensor(logits_row, dtype=torch.float32, device="cuda").repeat(draws, 1)
    states = [SamplingState(params, seed=1234, drawn=i) for i in range(draws)]
    return s.sample(logits, states).cpu().numpy()


def test_argmax_first_maximum_and_nan():
    from hk_b200.csrc import ops
    v = 151936 + 3
    x = torch.full((3, v), -1.0, device="cuda")
    x[0, 77] = x[0, 150000] = 5.0           # a tie: the first wins (src/sampler.zig:128-135)
    x[1, v - 1] = 2.0
    x[1, 5] = float("nan")
    x[2, :] = float("-inf")
    out = torch.empty(3, dtype=torch.int32, device="cuda")
    ops.argmax(x, out)
    assert out.tolist() == [77, v - 1, 0]


def test_sampler_frequencies_follow_the_chain():
    # cf. "empirical frequencies ≈ softmax over 20 000 draws", src/sampler.zig:220-299
    from hk_b200.sampling import SamplingParams
    rng = np.random.default_rng(0)
    logits = rng.standard_normal(1000) * 2
    for params in (SamplingParams(temperature=1.0, top_k=0, top_p=1.0, min_p=0.0),
                   SamplingParams(temperature=0.7, top_k=12, top_p=1.0, min_p=0.0),
                   SamplingParams(temperature=1.3, top_k=50, top_p=0.8, min_p=0.0),
                   SamplingParams(temperature=0.8, top_k=40, top_p=0.95, min_p=0.05)):
        ids, probs = P.candidate_distribution(logits, params.temperature, params.top_k, params.top_p, params.min_p)
        draws = sample_many(logits, params, 20000)
        assert set(draws.tolist()) <= set(ids.tolist()), "a token outside the surviving candidates was drawn"
        freq = np.array([(draws == i).mean() for i in ids])
        assert np.abs(freq - probs).max() < 0.015


def test_sampler_top_k_one_is_argmax_and_ties_keep_the_smaller_id():
    from hk_b200.sampling import SamplingParams
    logits = np.zeros(5000)
    logits[[40, 4000]] = 3.0
    draws = sample_many(logits, SamplingParams(temperature=1.0, top_k=1, top_p=1.0, min_p=0.0), 64)
    assert (draws == 40).all()
    draws = sample_many(logits, SamplingParams(temperature=1.0, top_k=2, top_p=1.0, min_p=0.0), 512)
    assert set(draws.tolist()) == {40, 4000}
    logits[:] = 1.0                              # all equal, k = 3: the three smallest ids survive
    draws = sample_many(logits, SamplingParams(temperature=1.0, top_k=3, top_p=1.0, min_p=0.0), 512)
    assert set(draws.tolist()) == {0, 1, 2}
    logits[7] = float("-inf")
    logits[9] = float("nan")
    draws = sample_many(logits, SamplingParams(temperature=5.0, top_k=0, top_p=1.0, min_p=0.0), 8192)
    assert 7 not in draws and 9 not in draws and draws.max() <= 4097   # capped at 4096 finite candidates


def test_sampler_is_seeded_and_independent_of_the_batch():
    from hk_b200.sampling import Sampler, SamplingParams, SamplingState
    rng = np.random.default_rng(1)
    rows = torch.tensor(rng.standard_normal((6, 3000)) * 3, dtype=torch.float32, device="cuda")
    s = Sampler(torch.device("cuda"))
    p = SamplingParams(temperature=0.9, top_k=100, top_p=0.9, min_p=0.01)
    mk = lambda seed: [SamplingState(p, seed=seed + i, drawn=3) for i in range(6)]
    a = s.sample(rows.clone(), mk(50)).tolist()
    assert a == s.sample(rows.clone(), mk(50)).tolist()
    assert a != s.sample(rows.clone(), mk(51)).tolist()
    alone = [s.sample(rows[i:i + 1].clone(), [SamplingState(p, seed=50 + i, drawn=3)]).item() for i in range(6)]
    assert alone == a
    greedy_mixed = [SamplingState(SamplingParams(temperature=0.0), seed=1) if i % 2 else st for i, st in enumerate(mk(50))]
    mixed = s.sample(rows.clone(), greedy_mixed).tolist()
    assert mixed[1::2] == rows.argmax(1).tolist()[1::2] and mixed[0::2] == a[0::2]


def test_penalties_and_bias_follow_the_reference():
    # src/sampler.zig:82-111 and its test "temperature zero is argmax and honours penalties"
    from hk_b200.sampling import Sampler, SamplingParams, SamplingState
    s = Sampler(torch.device("cuda"))
    base = torch.tensor([[1.0, 4.0, 3.5, -2.0, 3.9]], device="cuda")
    st = SamplingState(SamplingParams(temperature=0.0, repeat_penalty=2.0), seed=1, history=[1, 1, 3])
    lg = base.clone()
    assert s.sample(lg, [st]).item() == 4                    # 4.0 / 2 = 2.0 loses to 3.9
    assert torch.allclose(lg.cpu(), torch.tensor([[1.0, 2.0, 3.5, -4.0, 3.9]]))
    st = SamplingState(SamplingParams(temperature=0.0, frequency_penalty=0.3, presence_penalty=0.1), seed=1, history=[1, 1, 4])
    lg = base.clone()
    assert s.sample(lg, [st]).item() == 2                    # 4.0 - 0.7 = 3.3 ; 3.9 - 0.4 = 3.5 ; 3.5 wins by index
    st = SamplingState(SamplingParams(temperature=0.0, logit_bias=[(3, 10.0)]), seed=1)
    assert s.sample(base.clone(), [st]).item() == 3
    st = SamplingState(SamplingParams(temperature=0.0, repeat_penalty=2.0, repeat_last_n=1), seed=1, history=[1, 0])
    assert s.sample(base.clone(), [st]).item() == 1          # only the last token is looked at


# ---- the command line ----------------------------------------------------------------------------


def run_cli(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bin", "hk"), "run", *args], capture_output=True, text=True, timeout=600)


def test_command_line_greedy_and_seeds(model_b):
    # cf. tests/cli_tests.zig:88-165 of the reference: greedy repeats exactly; a seed repeats, another differs
    d, cfg, w = model_b
    prompt = helpers.prompts_for("B", np.random.default_rng(12), [9])[0]
    text = ",".join(map(str, prompt))
    a = run_cli(d, text, "-n", "6", "--temp", "0", "--dtype", "float32")
    assert a.returncode == 0, a.stderr
    assert [int(t) for t in a.stdout.split()] == plain_greedy(cfg, w, prompt, 6)
    assert "[prompt 9 tok (0 cached)," in a.stderr and "generated 6 tok" in a.stderr
    s1 = run_cli(d, "-p", text, "-n", "12", "--temp", "1.5", "--seed", "7", "--dtype", "float32")
    s2 = run_cli(d, "-p", text, "-n", "12", "--temp", "1.5", "--seed", "7", "--dtype", "float32")
    s3 = run_cli(d, "-p", text, "-n", "12", "--temp", "1.5", "--seed", "8", "--dtype", "float32")
    assert s1.returncode == 0 and s1.stdout == s2.stdout and s1.stdout != s3.stdout
    bad = run_cli(d, text, "--tmp", "0")
    assert bad.returncode == 2 and "unknown argument" in bad.stderr
    missing = run_cli(os.path.join(d, "nope"), text)
    assert missing.returncode == 1 and "config.json" in missing.stderr


def test_command_line_random_model_and_drawn_prompt(tmp_path):
    """`hk random` writes a model folder from a config.json; `hk run --prompt-len` draws the prompt with the seed; the
    greedy continuation is the plain implementation's, with 8-token pages as with the default ones."""
    cfg_json = os.path.join(str(tmp_path), "c.json")
    with open(cfg_json, "w") as f:
        json.dump(helpers.TINY_A, f)
    out = os.path.join(str(tmp_path), "m")
    made = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "hk"), "random", cfg_json, out, "--seed", "3", "--dtype", "float32"],
                          capture_output=True, text=True, timeout=600)
    assert made.returncode == 0, made.stderr
    cfg, w = helpers.load_plain(out)
    prompt = np.random.default_rng(5).integers(0, cfg["vocab_size"], 11).tolist()
    for extra in ([], ["--page-tokens", "8"]):
        r = run_cli(out, "--prompt-len", "11", "--seed", "5", "-n", "5", "--temp", "0", "--dtype", "float32", *extra)
        assert r.returncode == 0, r.stderr
        assert [int(t) for t in r.stdout.split()] == plain_greedy(cfg, w, prompt, 5)
        assert "[prompt 11 tok" in r.stderr
