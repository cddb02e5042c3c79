"""The scheduler's decisions on a fake engine: budget, portions, finishing, and what happens
when pages run out (no GPU).  The fake engine keeps real cache books and returns logits that
make the greedy continuation a known function of the tokens fed so far."""
import pytest
import torch

from hk_b200.cache import CacheBooks
from hk_b200.engine import DeviceToken
from hk_b200.engine.scheduler import RequestRefused, Scheduler
from hk_b200.sampling import GREEDY, SamplingParams

VOCAB = 50


class FakeCache:
    def __init__(self, books):
        self.books = books


class FakeEngine:
    """Next token = (sum of all tokens fed so far + their count) % VOCAB."""

    def __init__(self, num_pages=16, page_tokens=4, max_requests=4, max_context=64, max_batch_tokens=16, windows=(None,)):
        self.cache = FakeCache(CacheBooks(list(windows), page_tokens, num_pages, max_requests, max_context))
        self.max_context, self.max_batch_tokens, self.vocab = max_context, max_batch_tokens, VOCAB
        self.device = torch.device("cpu")
        self.slots, self.fed, self.log = {}, {}, []

    def open_request(self, rid):
        self.slots[rid] = self.cache.books.open()
        self.fed[rid] = []

    def close_request(self, rid):
        self.cache.books.close(self.slots.pop(rid))
        del self.fed[rid]

    def slot_of(self, rid):
        return self.slots[rid]

    def step(self, entries):
        assert sum(len(e.tokens) for e in entries) <= self.max_batch_tokens
        rows = []
        for e in entries:
            self.cache.books.extend(self.slots[e.request], len(e.tokens))
            toks = [int(e.tokens.tensor[e.tokens.index])] if isinstance(e.tokens, DeviceToken) else e.tokens
            for i, t in enumerate(toks):
                self.fed[e.request].append(int(t))
                if i in e.want:
                    row = torch.zeros(VOCAB)
                    row[(sum(self.fed[e.request]) + len(self.fed[e.request])) % VOCAB] = 1.0
                    rows.append(row)
        self.cache.books.audit()
        self.log.append([(e.request, len(e.tokens), list(e.want)) for e in entries])
        return torch.stack(rows) if rows else None


class CpuSampler:
    def sample(self, logits, states):
        return torch.argmax(logits, dim=1)

    @staticmethod
    def accept(state, token):
        state.history.append(int(token))
        state.drawn += 1


def expected(prompt, n):
    fed, out = list(prompt), []
    for _ in range(n):
        t = (sum(fed) + len(fed)) % VOCAB
        out.append(t)
        fed.append(t)
    return out


def make(prefill_chunk=8, run_ahead=True, **kw):
    eng = FakeEngine(**kw)
    return eng, Scheduler(eng, sampler=CpuSampler(), prefill_chunk=prefill_chunk, run_ahead=run_ahead)


def test_decodes_first_then_prompt_portions_within_the_budget():
    eng, s = make(max_batch_tokens=10, num_pages=32)
    a = s.submit([1, 2, 3], 4, GREEDY)
    s.step()                                       # whole prompt of a, wants its last place
    assert eng.log[-1] == [(a, 3, [2])]
    b = s.submit(list(range(20)), 2, GREEDY)
    c = s.submit(list(range(30, 47)), 2, GREEDY)
    s.step()
    # a decodes one token first; the other 9 tokens are shared: 4 each (9 // 2)
    assert eng.log[-1] == [(a, 1, [0]), (b, 4, []), (c, 4, [])]
    s.step()
    assert eng.log[-1] == [(a, 1, [0]), (b, 4, []), (c, 4, [])]
    done = s.run()
    assert done[a].output == expected([1, 2, 3], 4) and done[a].finish_reason == "length"
    assert done[b].output == expected(list(range(20)), 2)
    assert done[c].output == expected(list(range(30, 47)), 2)
    # a prompt's last portion, and only it, asks for logits
    for step in eng.log:
        for rid, n, want in step:
            assert want in ([], [n - 1])
    assert eng.cache.books.free_pages() == [32]


def test_prefill_chunk_caps_a_portion():
    eng, s = make(max_batch_tokens=16, num_pages=32)
    s.prefill_chunk = 5
    a = s.submit(list(range(12)), 1, GREEDY)
    s.run()
    assert [st[0][1] for st in eng.log] == [5, 5, 2]


def test_finish_reasons_stop_length_context_cancel():
    eng, s = make(max_context=8, num_pages=32)
    s.eos = {expected([4, 4], 1)[0]}
    a = s.submit([4, 4], 5, GREEDY)
    b = s.submit([1, 2, 3, 4, 5, 6], 10, GREEDY)      # context of 8 fills first
    c = s.submit([20], 3, GREEDY)
    d = s.submit([7, 7], 50, GREEDY)
    s.step()
    s.cancel(d)
    done = s.run()
    assert done[a].finish_reason == "stop" and done[a].output == []
    assert done[b].finish_reason == "context" and done[b].output == expected([1, 2, 3, 4, 5, 6], 3)
    assert done[c].finish_reason == "length" and len(done[c].output) == 3
    assert done[d].finish_reason == "cancelled"
    assert eng.cache.books.free_pages() == [32] and not eng.slots


def test_refusals_at_submit():
    eng, s = make(num_pages=4, page_tokens=4, max_context=64)
    with pytest.raises(RequestRefused):
        s.submit([], 4)
    with pytest.raises(RequestRefused):
        s.submit([VOCAB], 4)
    with pytest.raises(RequestRefused):
        s.submit([1] * 65, 1)                      # longer than the context
    with pytest.raises(RequestRefused):
        s.submit([1] * 10, 8)                      # 17 tokens = 5 pages > 4: could never finish alone
    s.submit([1] * 10, 7)                          # 16 tokens = 4 pages: fits alone


def test_pages_run_out_newest_request_is_preempted_and_recomputed():
    # 6 pages of 4 tokens.  Two requests of 9 prompt tokens (3 pages each) fill the pool; their
    # decodes need a 4th page each after 3 more tokens: the newer one is preempted, the older
    # finishes, then the newer is recomputed from prompt + what it had produced.
    eng, s = make(num_pages=6, page_tokens=4, max_context=32, max_batch_tokens=32, prefill_chunk=32)
    s.prefill_chunk = 32
    p1, p2 = list(range(1, 10)), list(range(11, 20))
    a = s.submit(p1, 10, GREEDY)
    b = s.submit(p2, 10, GREEDY)
    done = s.run()
    assert s.stats.preemptions >= 1 and done[b].preemptions >= 1 and done[a].preemptions == 0
    assert done[a].output == expected(p1, 10)
    assert done[b].output == expected(p2, 10)       # recomputation changes nothing
    assert eng.cache.books.free_pages() == [6] and not eng.slots
    # after the preemption b was fed again from position 0 with its prompt and its outputs so far
    refeeds = [n for st in eng.log for rid, n, _ in st if rid == b and n > 1]
    assert len(refeeds) >= 2 and refeeds[-1] > len(p2)


def test_a_prompt_portion_is_shortened_to_the_free_pages():
    eng, s = make(num_pages=5, page_tokens=4, max_context=32, max_batch_tokens=32)
    s.prefill_chunk = 32
    a = s.submit([1] * 11, 2, GREEDY)               # 3 pages
    s.step()
    b = s.submit([2] * 14, 1, GREEDY)               # would need 4 pages; 2 are free
    s.step()
    assert eng.log[-1][0][:2] == (a, 1)
    # one page stays reserved for a's decode, b gets what is left and never starves a
    assert all(n <= 8 for rid, n, _ in eng.log[-1] if rid == b)
    done = s.run()
    assert done[a].output == expected([1] * 11, 2) and done[b].output == expected([2] * 14, 1)


def test_many_requests_over_few_slots_all_finish_in_order_of_arrival():
    eng, s = make(num_pages=12, page_tokens=4, max_requests=3, max_context=40, max_batch_tokens=12)
    prompts = [[(7 * i + j) % VOCAB for j in range(3 + (5 * i) % 11)] for i in range(9)]
    ids = [s.submit(p, 3 + i % 4, GREEDY) for i, p in enumerate(prompts)]
    done = s.run()
    for i, (rid, p) in enumerate(zip(ids, prompts)):
        assert done[rid].output == expected(p, 3 + i % 4)
    assert max(len(st) for st in eng.log) <= 3
    assert eng.cache.books.free_pages() == [12]


def test_run_ahead_launches_the_next_decode_before_reading_and_drops_the_token_after_an_end():
    eng, s = make(num_pages=32, max_context=64)
    p = [3, 1, 4]
    want = expected(p, 12)
    s.eos = {want[6]}
    a = s.submit(p, 12, GREEDY)
    done = s.run()
    assert done[a].finish_reason == "stop" and done[a].output == want[:6]
    # the end token (the 7th) is read one step late: one more decode step ran with it and its result is dropped
    decodes = [st for st in eng.log if st == [(a, 1, [0])]]
    assert len(decodes) == 7
    assert eng.cache.books.free_pages() == [32] and not eng.slots and not s.has_work()
    # without run-ahead: same output, one step fewer
    eng2, s2 = make(num_pages=32, max_context=64, run_ahead=False)
    s2.eos = {want[6]}
    a2 = s2.submit(p, 12, GREEDY)
    assert s2.run()[a2].output == want[:6]
    assert len([st for st in eng2.log if st == [(a2, 1, [0])]]) == 6


@pytest.mark.parametrize("seed", range(6))
def test_run_ahead_changes_no_output_under_random_arrivals_tight_pages_and_limits(seed):
    import random
    outs = []
    for ahead in (False, True):
        rnd = random.Random(seed)
        eng, s = make(num_pages=10, page_tokens=4, max_requests=3, max_context=24, max_batch_tokens=12, run_ahead=ahead,
                      windows=(None, 6) if seed % 2 else (None,))
        s.eos = {7, 23}
        ids, prompts = [], {}
        for step in range(200):
            if rnd.random() < 0.25 and len(ids) < 14:
                pr = [rnd.randrange(VOCAB) for _ in range(rnd.randint(1, 14))]
                rid = s.submit(pr, rnd.randint(1, 12), GREEDY)
                ids.append(rid)
                prompts[rid] = pr
            if rnd.random() < 0.03 and ids:
                s.cancel(rnd.choice(ids))
            s.step()
            eng.cache.books.audit()
        done = s.run()
        assert (s.stats.ahead_steps > 0) == ahead
        assert not eng.slots and all(f == 10 for f in eng.cache.books.free_pages())
        outs.append({rid: (done[rid].output, done[rid].finish_reason) for rid in ids})
        for rid in ids:
            out, why = outs[-1][rid]
            if why != "cancelled":
                full = expected(prompts[rid], len(out) + 1)
                assert out == full[:len(out)]
                if why == "stop":
                    assert full[len(out)] in s.eos
    # cancellations land at different moments of a request's life in the two modes; everything else is equal
    for rid, (out, why) in outs[0].items():
        out2, why2 = outs[1][rid]
        if "cancelled" not in (why, why2):
            assert (out, why) == (out2, why2)


def test_sampling_params_defaults_are_the_references():
    p = SamplingParams()
    assert (p.temperature, p.top_k, p.top_p, p.min_p, p.repeat_penalty, p.repeat_last_n, p.seed) == \
        (0.8, 40, 0.95, 0.05, 1.0, 64, 0)
    with pytest.raises(ValueError):
        SamplingParams(top_p=1.5).validate()
