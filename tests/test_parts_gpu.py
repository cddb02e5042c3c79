"""Each part alone against the plain implementation's function for it, and a toy mixer with
state of its own that is registered, built and stepped without touching the package."""
import math
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
IDS = ["f32", "bf16"]


def tol(dtype):
    return dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-5)


def bind_random(part, dtype, seed=0, std=0.05, norm_std=0.1):
    """Random tensors for a part's declared parameters, bound on the GPU; returns float64 numpy copies
    of exactly what the part computes with."""
    from hk_b200.parts import Precision
    from hk_b200.weights import random_tensors
    prec = Precision(dtype, torch.device("cuda"))
    tensors = random_tensors(part.param_specs(), seed, std, norm_std, "cuda", dtype_of=lambda s: prec.working_dtype(s.kind))
    host = {k: v.double().cpu().numpy() for k, v in tensors.items()}
    part.bind(tensors, prec)
    return prec, host


def make_ctx(prec, spans, cache=None, page_tokens=8, part=None):
    """spans: [(slot, first position, count)]; extends `cache` (a PagedCache) accordingly.  With `part`, the
    host-built tables that part (or its children) names are packed and uploaded as the engine does it."""
    from hk_b200.engine.context import StepContext, bind_step, pack_step, table_parts
    slot, pos, q_starts, q_lens, starts, slots = [], [], [], [], [], []
    for s, p0, c in spans:
        q_starts.append(len(slot))
        slot += [s] * c
        pos += list(range(p0, p0 + c))
        q_lens.append(c)
        starts.append(p0)
        slots.append(s)
        if cache is not None:
            assert int(cache.books.length[s]) == p0
            cache.books.extend(s, c)
    if cache is not None:
        cache.sync_tables()
    dev = prec.device
    n = len(slot)
    ctx = StepContext(prec, n, None, None, None, slots, q_starts, q_lens, starts)
    meta = np.stack([np.zeros(n, dtype=np.int32), np.asarray(pos, dtype=np.int32), np.asarray(slot, dtype=np.int32)])
    packed = pack_step(meta, ctx, table_parts(part) if part is not None else [])
    bind_step(ctx, packed, torch.from_numpy(packed.host).to(dev))
    return ctx


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_rms_norm_part(dtype):
    from hk_b200.parts import RMSNorm
    part = RMSNorm(72, 3e-6, "n.weight")
    prec, w = bind_random(part, dtype)
    assert part.weight.dtype == torch.float32
    x = torch.randn(11, 72, device="cuda") * 2
    out = torch.empty(11, 72, dtype=dtype, device="cuda")
    part.forward(x, out)
    np.testing.assert_allclose(out.double().cpu().numpy(), P.rms_norm(x.double().cpu().numpy(), w["n.weight"], 3e-6), **tol(dtype))
    # a checkpoint that stores weight - 1: the offset is a parameter of the part
    shifted = RMSNorm(72, 3e-6, "n.weight", weight_offset=1.0)
    prec, w = bind_random(shifted, dtype)
    shifted.forward(x, out)
    np.testing.assert_allclose(out.double().cpu().numpy(), P.rms_norm(x.double().cpu().numpy(), w["n.weight"] + 1.0, 3e-6), **tol(dtype))


def test_rotary_tables_match_the_plain_angles():
    from hk_b200.parts import Precision, RotaryEmbedding
    part = RotaryEmbedding(1e6, 24, 300)
    part.bind({}, Precision(torch.float32, torch.device("cuda")))
    cos, sin, rot = part.tables()
    assert rot == 24 and cos.shape == (300, 12) and cos.dtype == torch.float32
    c, s = P.rope_angles(np.arange(300), P.rope_inv_freq(1e6, 24))
    assert np.array_equal(cos.cpu().numpy(), c.astype(np.float32)) and np.array_equal(sin.cpu().numpy(), s.astype(np.float32))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_swiglu_feed_forward_part(dtype):
    from hk_b200.parts import SwiGLUFeedForward
    part = SwiGLUFeedForward(72, 200, "mlp.")
    prec, w = bind_random(part, dtype)
    xb = (torch.randn(9, 72, device="cuda")).to(dtype)
    res0 = torch.randn(9, 72, device="cuda")
    res = res0.clone()
    part.forward(xb, res, make_ctx(prec, [(0, 0, 9)]))
    x = xb.double().cpu().numpy()
    h = P.swiglu(P.linear(x, w["mlp.gate_proj.weight"]), P.linear(x, w["mlp.up_proj.weight"]))
    want = res0.double().cpu().numpy() + P.linear(h, w["mlp.down_proj.weight"])
    np.testing.assert_allclose(res.double().cpu().numpy(), want, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("window,qk_norm,rope,bias,pairing,scaling", [
    (None, True, True, False, "half", None), (7, True, True, False, "half", None), (None, False, False, False, "half", None),
    (None, True, True, True, "adjacent", None), (5, False, True, True, "half", dict(kind="yarn", factor=4.0, orig_ctx=16)),
    (None, True, True, False, "adjacent", dict(kind="llama3", factor=8.0, orig_ctx=32)),
    (None, False, True, True, "half", dict(kind="linear", factor=2.0))])
def test_attention_part_whole_then_cut(dtype, window, qk_norm, rope, bias, pairing, scaling):
    """The attention mixer alone: a whole sequence in one step equals the plain functions, and the
    same sequence cut into a portion and single tokens gives the same rows.  Its parameters one by one: a
    window, the per-head norm, the rotation with either pairing of dims and every kind of frequency scaling,
    biases on the four projections."""
    from hk_b200.cache.device import PagedCache
    from hk_b200.parts import GQAAttention, RopeScaling, RotaryEmbedding
    d, H, G, hd, T = 40, 6, 2, 16, 29
    pos_part = RotaryEmbedding(5000.0, 8, 64, pairing=pairing, scaling=RopeScaling(**scaling) if scaling else None) if rope else None
    part = GQAAttention(d, H, G, hd, "a.", qk_norm_eps=1e-5 if qk_norm else None, position=pos_part, window=window,
                        qkv_bias=bias, o_bias=bias)
    prec, w = bind_random(part, dtype, std=0.2)
    xb = torch.randn(T, d, device="cuda").to(dtype)
    x = xb.double().cpu().numpy()
    q, k, v = (P.linear(x, w[f"a.{n}_proj.weight"]) for n in "qkv")
    if bias:
        q, k, v = (t + w[f"a.{n}_proj.bias"][None, :] for t, n in ((q, "q"), (k, "k"), (v, "v")))
    if qk_norm:
        q, k = P.head_norm(q, w["a.q_norm.weight"], hd, 1e-5), P.head_norm(k, w["a.k_norm.weight"], hd, 1e-5)
    if rope:
        kind = scaling["kind"] if scaling else "none"
        sc = {k_: v_ for k_, v_ in (scaling or {}).items() if k_ != "kind"}
        cos, sin = P.rope_angles(np.arange(T), P.rope_inv_freq_scaled(5000.0, 8, kind, **sc))
        m = P.rope_mscale(kind, sc.get("factor", 1.0))
        rotate = P.rope_rotate_half if pairing == "half" else P.rope_rotate_adjacent
        q, k = rotate(q, hd, cos * m, sin * m), rotate(k, hd, cos * m, sin * m)
    want = P.linear(P.causal_gqa_attention(q, k, v, H, G, hd, window=window), w["a.o_proj.weight"])
    if bias:
        want = want + w["a.o_proj.bias"][None, :]

    def run(cuts):
        cache = PagedCache([[part.cache_spec()]], prec, 4, 16, 2, 64)
        slot = cache.open()
        other = cache.open()        # a second request shares the steps, so rows interleave
        res = torch.zeros(T, d, device="cuda")
        p = 0
        for c in cuts:
            r = torch.zeros(c + 1, d, device="cuda")
            ctx = make_ctx(prec, [(other, int(cache.books.length[other]), 1), (slot, p, c)], cache, part=part)
            if dtype == torch.bfloat16:
                assert part.step_tables_key() in ctx.tables        # the flash kernels' work items came through the hook
            part.forward(torch.cat([xb[:1], xb[p:p + c]]), r, ctx, cache.layers[0][0])
            res[p:p + c] = r[1:]
            p += c
        return res.double().cpu().numpy()

    whole = run([T])
    np.testing.assert_allclose(whole, want, **tol(dtype))
    cut = run([13, 2, 1, 1, 7, 5])
    np.testing.assert_allclose(cut, want, **tol(dtype))
    if dtype == torch.float32:
        np.testing.assert_allclose(cut, whole, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_embedding_and_output_head_parts(dtype):
    from hk_b200.parts import OutputHead, RMSNorm, TokenEmbedding
    emb = TokenEmbedding(333, 72, "emb.weight")
    prec, w = bind_random(emb, dtype)
    ids = torch.tensor([5, 332, 0, 17], dtype=torch.int32, device="cuda")
    x = torch.empty(4, 72, device="cuda")
    emb.forward(ids, x)
    assert np.array_equal(x.double().cpu().numpy(), w["emb.weight"][[5, 332, 0, 17]])
    for tied in (False, True):
        head = OutputHead(72, 333, RMSNorm(72, 1e-6, "norm.weight"), "head.weight", tied_to="emb.weight" if tied else None)
        specs = head.param_specs()
        assert specs["head.weight"].optional == tied
        from hk_b200.weights import random_tensors
        t = random_tensors(specs, 4, 0.05, 0.1, "cuda", dtype_of=lambda s: prec.working_dtype(s.kind))
        if tied:
            assert "head.weight" not in t
            t["emb.weight"] = emb.table
        head.bind(t, prec)
        res = torch.randn(6, 72, device="cuda")
        rows = torch.tensor([4, 1], dtype=torch.int32, device="cuda")
        logits = head.forward(res, rows, 2, make_ctx(prec, [(0, 0, 6)]))
        assert logits.dtype == torch.float32 and logits.shape == (2, 333)
        wh = (t["emb.weight"] if tied else t["head.weight"]).double().cpu().numpy()
        xb = P.rms_norm(res.double().cpu().numpy()[[4, 1]], t["norm.weight"].double().cpu().numpy(), 1e-6)
        np.testing.assert_allclose(logits.double().cpu().numpy(), P.linear(xb, wh), **tol(dtype))


# ---------------------------------------------------------------------------------------------
# A toy architecture defined here: a mixer whose memory is a state of fixed size (a decaying sum
# of its inputs), beside an attention layer that is run twice and a layer that reads an earlier
# layer's cache.  Nothing in the package knows about it.

@dataclass
class ToyConfig:
    architecture: str = "ToyStateForCausalLM"
    hidden_size: int = 24
    vocab_size: int = 50
    decay: float = 0.75
    initializer_range: float = 0.2
    max_position_embeddings: int = 64

    @classmethod
    def from_dict(cls, raw):
        return cls(**{k: v for k, v in raw.items() if k in cls.__dataclass_fields__})

    def to_dict(self):
        return dict(architectures=[self.architecture], hidden_size=self.hidden_size, vocab_size=self.vocab_size,
                    decay=self.decay, initializer_range=self.initializer_range)


def build_toy(cfg, max_positions):
    from hk_b200.models import LayerCall, ModelSpec
    from hk_b200.parts import (GQAAttention, MATRIX, OutputHead, ParamSpec, Part, PreNormBlock, RMSNorm, StateSpec,
                               StepTables, SwiGLUFeedForward, TokenEmbedding)

    class DecayingSumMixer(Part):
        """state <- decay * state + xb_t ; residual_t += W state   (state: one vector per request).

        Written so that a decode step through it can be captured: the rows of a request are found through a
        host-built table (`step_tables`: for every row the first row of its request; for every request its last
        row and its slot) and everything else is arithmetic on device tensors.  The scan over a request's rows is
        a product with the matrix M[t, s] = decay^(t - s) for first(t) <= s <= t."""
        graph_safe = True
        KEY = ("toy_decaying_sum_rows",)

        def __init__(self, d, decay, name):
            self.d, self.decay, self.name, self.w = d, decay, name, None

        def own_param_specs(self):
            return {self.name: ParamSpec((self.d, self.d), MATRIX)}

        def own_bind(self, tensors, precision):
            self.w = tensors[self.name]
            self.decay_dev = torch.tensor(self.decay, dtype=torch.float64, device=precision.device)   # not inside a capture

        def cache_spec(self):
            return StateSpec((self.d,), torch.float32)

        def step_tables_key(self):
            return self.KEY

        def step_tables(self, ctx):
            first = np.zeros(ctx.n_tokens, dtype=np.int32)
            for qs, ql in zip(ctx.q_starts, ctx.q_lens):
                first[qs:qs + ql] = qs
            last = np.asarray([qs + ql - 1 for qs, ql in zip(ctx.q_starts, ctx.q_lens)], dtype=np.int32)
            return StepTables({"first": first, "last": last, "slots": np.asarray(ctx.slots, dtype=np.int32)})

        def forward(self, xb, residual, ctx, cache, write_cache=True):
            tabs, _ = ctx.tables[self.KEY]
            n = xb.shape[0]
            t = torch.arange(n, device=xb.device)
            first = tabs["first"].long()
            diff = t[:, None] - t[None, :]
            inside = (diff >= 0) & (t[None, :] >= first[:, None])
            m = torch.where(inside, torch.pow(self.decay_dev, diff.clamp(min=0)), torch.zeros((), dtype=torch.float64, device=xb.device))
            before = cache.state.index_select(0, ctx.slot_of_token.long()).double()          # the request's state, per row
            carry = torch.pow(self.decay_dev, (t - first + 1))[:, None] * before
            states = (m @ xb.double() + carry).float()
            residual += states @ self.w.float().T
            cache.state.index_copy_(0, tabs["slots"].long(), states.index_select(0, tabs["last"].long()))

    d = cfg.hidden_size
    blocks = [
        PreNormBlock(RMSNorm(d, 1e-6, "l0.n1"), DecayingSumMixer(d, cfg.decay, "l0.mix"), RMSNorm(d, 1e-6, "l0.n2"),
                     SwiGLUFeedForward(d, 40, "l0.mlp.")),
        PreNormBlock(RMSNorm(d, 1e-6, "l1.n1"), GQAAttention(d, 2, 1, 16, "l1.attn."), RMSNorm(d, 1e-6, "l1.n2"),
                     SwiGLUFeedForward(d, 40, "l1.mlp.")),
    ]
    # layer 1 runs twice with a cache for each run, then once more reading the first run's cache
    schedule = [LayerCall(0), LayerCall(1), LayerCall(1), LayerCall(1, cache_of=1)]
    return ModelSpec(cfg, TokenEmbedding(cfg.vocab_size, d, "emb"), blocks,
                     OutputHead(d, cfg.vocab_size, RMSNorm(d, 1e-6, "norm"), "head"), schedule)


def toy_plain(cfg, w, ids):
    """The toy model on whole sequences in float64, from the definitions above."""
    d = cfg.hidden_size
    x = w["emb"][ids]
    T = len(ids)

    def ffn(x, p):
        xb = P.rms_norm(x, w[p + "n2"], 1e-6)
        return x + P.linear(P.swiglu(P.linear(xb, w[p + "mlp.gate_proj.weight"]), P.linear(xb, w[p + "mlp.up_proj.weight"])),
                            w[p + "mlp.down_proj.weight"])

    xb = P.rms_norm(x, w["l0.n1"], 1e-6)
    st = np.zeros(d)
    add = np.zeros_like(x)
    for t in range(T):
        st = cfg.decay * st + xb[t]
        add[t] = w["l0.mix"] @ st
    x = ffn(x + add, "l0.")
    first_kv = None
    for call in range(3):
        xb = P.rms_norm(x, w["l1.n1"], 1e-6)
        q = P.linear(xb, w["l1.attn.q_proj.weight"])
        k, v = P.linear(xb, w["l1.attn.k_proj.weight"]), P.linear(xb, w["l1.attn.v_proj.weight"])
        if call == 0:
            first_kv = (k, v)
        if call == 2:
            k, v = first_kv
        x = x + P.linear(P.causal_gqa_attention(q, k, v, 2, 1, 16), w["l1.attn.o_proj.weight"])
        x = ffn(x, "l1.")
    return P.linear(P.rms_norm(x, w["norm"], 1e-6), w["head"])


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_toy_mixer_with_state_is_registered_built_and_stepped(dtype):
    from hk_b200.config import register_architecture
    from hk_b200.engine import Engine, StepEntry
    register_architecture("ToyStateForCausalLM", ToyConfig, build_toy)
    cfg = ToyConfig()
    eng = Engine(config=cfg, random_seed=3, dtype=dtype, max_tokens=128, page_tokens=4, max_requests=3, max_context=64)
    kinds = [[lc.kind for lc in caches] for caches in eng.cache.layers]
    assert kinds == [["state"], ["pages"], ["pages"], []]
    w = {}
    blk0, blk1 = eng.model.layers
    w.update({"emb": eng.model.embedding.table, "head": eng.model.head.weight, "norm": eng.model.head.norm.weight,
              "l0.n1": blk0.mixer_norm.weight, "l0.n2": blk0.ffn_norm.weight, "l0.mix": blk0.mixer.w,
              "l1.n1": blk1.mixer_norm.weight, "l1.n2": blk1.ffn_norm.weight})
    for p, blk in (("l0.", blk0), ("l1.", blk1)):
        F = blk.feed_forward.F
        w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"] = blk.feed_forward.w_gate_up[:F], blk.feed_forward.w_gate_up[F:]
        w[p + "mlp.down_proj.weight"] = blk.feed_forward.w_down
    a = blk1.mixer
    w["l1.attn.q_proj.weight"], w["l1.attn.k_proj.weight"], w["l1.attn.v_proj.weight"] = \
        a.w_qkv[:32], a.w_qkv[32:48], a.w_qkv[48:]
    w["l1.attn.o_proj.weight"] = a.w_o
    w = {k: v.double().cpu().numpy() for k, v in w.items()}
    rng = np.random.default_rng(0)
    seqs = {"x": rng.integers(0, 50, 21).tolist(), "y": rng.integers(0, 50, 30).tolist()}
    want = {k: toy_plain(cfg, w, np.array(v)) for k, v in seqs.items()}

    def run(plan):
        got = {k: [] for k in seqs}
        fed = {k: 0 for k in seqs}
        for k in seqs:
            eng.open_request(k)
        for step in plan:
            entries = [StepEntry(k, seqs[k][fed[k]:fed[k] + n], list(range(n))) for k, n in step]
            out = eng.step(entries).double().cpu().numpy()
            r = 0
            for k, n in step:
                got[k].append(out[r:r + n])
                r += n
                fed[k] += n
        for k in seqs:
            eng.close_request(k)
        return {k: np.concatenate(v) for k, v in got.items()}

    whole = run([[("x", 21)], [("y", 30)]])
    cut = run([[("x", 5), ("y", 2)], [("y", 11)], [("x", 1), ("y", 1)], [("x", 15), ("y", 16)]])
    # single tokens of both requests, step after step: the first such step captures a graph (and runs once, eagerly),
    # the later ones replay it; the mixer's state must advance exactly once per step in both
    assert eng.decode_graphs and not eng._pad_graphs
    decoded = run([[("x", 12), ("y", 21)]] + [[("x", 1), ("y", 1)]] * 9)
    assert eng._graphs[2].graph is not None
    eager = Engine(config=cfg, random_seed=3, dtype=dtype, max_tokens=128, page_tokens=4, max_requests=3, max_context=64,
                   decode_graphs=False)
    eng_graph, eng = eng, eager
    decoded_eagerly = run([[("x", 12), ("y", 21)]] + [[("x", 1), ("y", 1)]] * 9)
    eng = eng_graph
    # the whole-model criterion of the replay tests: max |difference| relative to the largest |logit|
    scale = max(np.abs(v).max() for v in want.values())
    tol_max = 2e-5 if dtype == torch.float32 else 2e-2
    for k in seqs:
        assert np.abs(whole[k] - want[k]).max() <= tol_max * scale
        assert np.abs(cut[k] - want[k]).max() <= tol_max * scale
        assert np.abs(decoded[k] - want[k]).max() <= tol_max * scale
        assert np.array_equal(decoded[k], decoded_eagerly[k])          # a captured step computes what an eager one does
    # the state slot was cleared when the requests were opened again: the second run equals the first
    assert eng.free_pages() == [eng.cache.num_pages]


# ---------------------------------------------------------------------------------------------
# A second toy architecture defined here: a feed-forward with routing (each token goes to two of
# four experts, router logits and weights in 32-bit) and a position encoding of its own (angles
# that grow with the logarithm of the position, on part of the head).  Nothing in the package
# knows about either; they are registered as parts and built through the architecture registry.

@dataclass
class RoutedConfig:
    architecture: str = "ToyRoutedForCausalLM"
    hidden_size: int = 40
    vocab_size: int = 61
    experts: int = 4
    expert_width: int = 24
    initializer_range: float = 0.2
    max_position_embeddings: int = 96

    @classmethod
    def from_dict(cls, raw):
        return cls(**{k: v for k, v in raw.items() if k in cls.__dataclass_fields__})

    def to_dict(self):
        return dict(architectures=[self.architecture], hidden_size=self.hidden_size, vocab_size=self.vocab_size,
                    experts=self.experts, expert_width=self.expert_width, initializer_range=self.initializer_range)


def log_angles(max_positions, rotary_dim):
    """angle[p, i] = log(1 + p) * (i + 1), in float64."""
    p = np.arange(max_positions, dtype=np.float64)[:, None]
    return np.log1p(p) * (np.arange(rotary_dim // 2, dtype=np.float64)[None, :] + 1.0)


def build_routed(cfg, max_positions):
    from hk_b200.csrc import ops
    from hk_b200.models import LayerCall, ModelSpec
    from hk_b200.parts import (GQAAttention, MATRIX, VECTOR, OutputHead, ParamSpec, Part, PreNormBlock, RMSNorm,
                               SwiGLUFeedForward, TokenEmbedding, register_part)

    class LogPosition(Part):
        """A position encoding with the rotary interface (tables of cos and sin by position) and other angles."""
        graph_safe = True

        def __init__(self, rotary_dim, max_positions):
            self.rotary_dim, self.max_positions, self.cos, self.sin = rotary_dim, max_positions, None, None

        def own_bind(self, tensors, precision):
            a = torch.from_numpy(log_angles(self.max_positions, self.rotary_dim))
            self.cos = torch.cos(a).float().contiguous().to(precision.device)
            self.sin = torch.sin(a).float().contiguous().to(precision.device)

        def tables(self):
            return self.cos, self.sin, self.rotary_dim

    class TopTwoRoutedFeedForward(Part):
        """residual += sum over the token's two best experts e of p_e * down_e(silu(gate_e xb) * up_e xb), where
        p = softmax of the two router logits; router logits in 32-bit from a 32-bit router matrix."""
        graph_safe = True           # routing by weights on the device: no row list ever comes to the host

        def __init__(self, d, experts, width, prefix):
            self.d, self.E, self.prefix = d, experts, prefix
            self.router = None
            self.expert = [SwiGLUFeedForward(d, width, f"{prefix}expert{e}.") for e in range(experts)]

        def children(self):
            return self.expert

        def own_param_specs(self):
            return {self.prefix + "router": ParamSpec((self.E, self.d), VECTOR)}      # kept in float32

        def own_bind(self, tensors, precision):
            self.router = tensors[self.prefix + "router"]

        def forward(self, xb, residual, ctx):
            n = xb.shape[0]
            logits = torch.empty((n, self.E), dtype=torch.float32, device=xb.device)
            ops.gemm(xb.float().contiguous(), self.router, logits)                     # 32-bit product
            top = torch.topk(logits, 2, dim=1)
            p = torch.softmax(top.values, dim=1)
            weight = torch.zeros_like(logits).scatter_(1, top.indices, p)              # [n, E]; zero where not chosen
            for e in range(self.E):
                part = torch.zeros((n, self.d), dtype=torch.float32, device=xb.device)
                self.expert[e].forward(xb, part, ctx)
                residual += part * weight[:, e:e + 1]

    register_part("position", "toy_log", LogPosition)
    register_part("feed_forward", "toy_top2", TopTwoRoutedFeedForward)
    d = cfg.hidden_size
    pos = LogPosition(8, max_positions)          # rotates 8 of the 16 dims of a head
    blocks = [
        PreNormBlock(RMSNorm(d, 1e-6, "l0.n1"), GQAAttention(d, 4, 2, 16, "l0.attn.", qk_norm_eps=1e-6, position=pos),
                     RMSNorm(d, 1e-6, "l0.n2"), TopTwoRoutedFeedForward(d, cfg.experts, cfg.expert_width, "l0.moe.")),
        PreNormBlock(RMSNorm(d, 1e-6, "l1.n1"), GQAAttention(d, 4, 2, 16, "l1.attn.", position=pos),
                     RMSNorm(d, 1e-6, "l1.n2"), SwiGLUFeedForward(d, 56, "l1.mlp.")),
    ]
    return ModelSpec(cfg, TokenEmbedding(cfg.vocab_size, d, "emb"), blocks,
                     OutputHead(d, cfg.vocab_size, RMSNorm(d, 1e-6, "norm"), "head"), [LayerCall(0), LayerCall(1)])


def routed_plain(cfg, w, ids):
    """The routed toy model on whole sequences in float64; also returns the smallest gap between a token's
    second and third router logit (a test is only meaningful where the routing is not a coin toss)."""
    T = len(ids)
    ang = log_angles(cfg.max_position_embeddings, 8)[:T]
    cos, sin = np.cos(ang), np.sin(ang)

    def rotate(x, heads):                                    # rotate-half on the first 8 dims of each head
        x = x.reshape(T, heads, 16).copy()
        a, b = x[:, :, :4].copy(), x[:, :, 4:8].copy()
        x[:, :, :4] = a * cos[:, None, :] - b * sin[:, None, :]
        x[:, :, 4:8] = a * sin[:, None, :] + b * cos[:, None, :]
        return x.reshape(T, heads * 16)

    def swiglu_ffn(xb, p):
        return P.linear(P.swiglu(P.linear(xb, w[p + "gate_proj.weight"]), P.linear(xb, w[p + "up_proj.weight"])), w[p + "down_proj.weight"])

    x = w["emb"][ids]
    gap = np.inf
    for l in (0, 1):
        p = f"l{l}.attn."
        xb = P.rms_norm(x, w[f"l{l}.n1"], 1e-6)
        q, k, v = (P.linear(xb, w[p + n + "_proj.weight"]) for n in "qkv")
        if l == 0:
            q = P.head_norm(q, w[p + "q_norm.weight"], 16, 1e-6)
            k = P.head_norm(k, w[p + "k_norm.weight"], 16, 1e-6)
        x = x + P.linear(P.causal_gqa_attention(rotate(q, 4), rotate(k, 2), v, 4, 2, 16), w[p + "o_proj.weight"])
        xb = P.rms_norm(x, w[f"l{l}.n2"], 1e-6)
        if l == 1:
            x = x + swiglu_ffn(xb, "l1.mlp.")
            continue
        logits = xb @ w["l0.moe.router"].T
        order = np.argsort(-logits, axis=1)
        srt = np.take_along_axis(logits, order, axis=1)
        gap = min(gap, float((srt[:, 1] - srt[:, 2]).min()))
        add = np.zeros_like(x)
        for t in range(T):
            e0, e1 = order[t, 0], order[t, 1]
            z = np.exp(srt[t, :2] - srt[t, 0])
            z /= z.sum()
            for e, pe in ((e0, z[0]), (e1, z[1])):
                add[t] += pe * swiglu_ffn(xb[t:t + 1], f"l0.moe.expert{e}.")[0]
        x = x + add
    return P.linear(P.rms_norm(x, w["norm"], 1e-6), w["head"]), gap


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_toy_routed_feed_forward_and_another_position_encoding(dtype):
    from hk_b200.config import register_architecture
    from hk_b200.engine import Engine, StepEntry
    from hk_b200.parts import part_class
    register_architecture("ToyRoutedForCausalLM", RoutedConfig, build_routed)
    cfg = RoutedConfig()
    eng = Engine(config=cfg, random_seed=24, dtype=dtype, max_tokens=192, page_tokens=8, max_requests=2, max_context=96)
    assert part_class("feed_forward", "toy_top2").__name__ == "TopTwoRoutedFeedForward"
    assert eng.decode_graphs and eng._pad_graphs  # every part is graph-safe and none keeps a state
    # the weights the engine computes with, by the names the parts declared
    blk0, blk1 = eng.model.layers
    w = {"emb": eng.model.embedding.table, "head": eng.model.head.weight, "norm": eng.model.head.norm.weight,
         "l0.moe.router": blk0.feed_forward.router}
    for l, blk in ((0, blk0), (1, blk1)):
        a = blk.mixer
        w[f"l{l}.n1"], w[f"l{l}.n2"] = blk.mixer_norm.weight, blk.ffn_norm.weight
        w[f"l{l}.attn.q_proj.weight"], w[f"l{l}.attn.k_proj.weight"], w[f"l{l}.attn.v_proj.weight"] = \
            a.w_qkv[:64], a.w_qkv[64:96], a.w_qkv[96:]
        w[f"l{l}.attn.o_proj.weight"] = a.w_o
    w["l0.attn.q_norm.weight"], w["l0.attn.k_norm.weight"] = blk0.mixer.q_norm, blk0.mixer.k_norm
    ffns = [(f"l0.moe.expert{e}.", blk0.feed_forward.expert[e]) for e in range(cfg.experts)] + [("l1.mlp.", blk1.feed_forward)]
    for p, f in ffns:
        w[p + "gate_proj.weight"], w[p + "up_proj.weight"], w[p + "down_proj.weight"] = f.w_gate_up[:f.F], f.w_gate_up[f.F:], f.w_down
    w = {k: v.double().cpu().numpy() for k, v in w.items()}
    rng = np.random.default_rng(1)
    seqs = {"x": rng.integers(0, cfg.vocab_size, 37).tolist(), "y": rng.integers(0, cfg.vocab_size, 26).tolist()}
    want, gaps = {}, []
    for k, v in seqs.items():
        want[k], g = routed_plain(cfg, w, np.array(v))
        gaps.append(g)
    # in bfloat16 the router sees inputs rounded to 8 bits: the gap has to be well above that noise
    assert min(gaps) > (2e-3 if dtype == torch.float32 else 2e-2), \
        "choose another seed: a token's second and third expert are too close to call"

    def run(plan):
        got, fed = {k: [] for k in seqs}, {k: 0 for k in seqs}
        for k in seqs:
            eng.open_request(k)
        for step in plan:
            entries = [StepEntry(k, seqs[k][fed[k]:fed[k] + n], list(range(n))) for k, n in step]
            out = eng.step(entries).double().cpu().numpy()
            r = 0
            for k, n in step:
                got[k].append(out[r:r + n])
                r += n
                fed[k] += n
        for k in seqs:
            eng.close_request(k)
        return {k: np.concatenate(v) for k, v in got.items()}

    whole = run([[("x", 37)], [("y", 26)]])
    cut = run([[("x", 9), ("y", 2)], [("y", 7)], [("x", 1), ("y", 1)], [("x", 2)], [("x", 25), ("y", 16)]])
    decoded = run([[("x", 30), ("y", 19)]] + [[("x", 1), ("y", 1)]] * 7)       # the tail replays a captured graph
    assert eng._graphs[2].graph is not None
    scale = max(np.abs(v).max() for v in want.values())
    tol_max = 2e-5 if dtype == torch.float32 else 2e-2
    for k in seqs:
        assert np.abs(whole[k] - want[k]).max() <= tol_max * scale
        assert np.abs(cut[k] - want[k]).max() <= tol_max * scale
        assert np.abs(decoded[k] - want[k]).max() <= tol_max * scale


# ---------------------------------------------------------------------------------------------
# A third toy architecture: a block with TWO mixers (each with a cache of its own; one keeps keys
# and values of different widths) followed by a block with NO mixer.  The model asks its blocks,
# not their mixers, which caches they keep.

@dataclass
class TwoMixerConfig:
    architecture: str = "ToyTwoMixerForCausalLM"
    hidden_size: int = 24
    vocab_size: int = 37
    key_width: int = 8
    value_width: int = 40
    initializer_range: float = 0.3
    max_position_embeddings: int = 64

    @classmethod
    def from_dict(cls, raw):
        return cls(**{k: v for k, v in raw.items() if k in cls.__dataclass_fields__})

    def to_dict(self):
        return dict(architectures=[self.architecture], hidden_size=self.hidden_size, vocab_size=self.vocab_size,
                    key_width=self.key_width, value_width=self.value_width, initializer_range=self.initializer_range)


def build_two_mixer(cfg, max_positions):
    from hk_b200.models import ModelSpec
    from hk_b200.parts import (GQAAttention, KVCacheSpec, MATRIX, OutputHead, ParamSpec, Part, RMSNorm, SwiGLUFeedForward,
                               TokenEmbedding)

    class NarrowKeyWideValueMixer(Part):
        """One head; keys of width kw and values of width vw in pages of their own widths:
        residual_t += Wo sum_{s <= t} softmax_s(q_t . k_s / sqrt(kw)) v_s."""

        def __init__(self, d, kw, vw, prefix):
            self.d, self.kw, self.vw, self.prefix = d, kw, vw, prefix

        def own_param_specs(self):
            p = self.prefix
            return {p + "q": ParamSpec((self.kw, self.d), MATRIX), p + "k": ParamSpec((self.kw, self.d), MATRIX),
                    p + "v": ParamSpec((self.vw, self.d), MATRIX), p + "o": ParamSpec((self.d, self.vw), MATRIX)}

        def own_bind(self, tensors, precision):
            self.w = {n: tensors[self.prefix + n] for n in "qkvo"}

        def cache_spec(self):
            return KVCacheSpec(1, self.kw, None, v_head_dim=self.vw)

        def forward(self, xb, residual, ctx, cache, write_cache=True):
            x = xb.float()
            q, k, v = (x @ self.w[n].float().T for n in "qkv")
            pt = cache.page_tokens
            pos, slot = ctx.positions.long(), ctx.slot_of_token.long()
            page = cache.block_table[slot, pos // pt].long()
            assert cache.k_pages.shape[1:] == (1, pt, self.kw) and cache.v_pages.shape[1:] == (1, pt, self.vw)
            if write_cache:
                cache.k_pages[page, 0, pos % pt] = k.to(cache.k_pages.dtype)
                cache.v_pages[page, 0, pos % pt] = v.to(cache.v_pages.dtype)
            for s, qs, ql, p0 in zip(ctx.slots, ctx.q_starts, ctx.q_lens, ctx.start_positions):
                js = torch.arange(p0 + ql, device=xb.device)
                pages = cache.block_table[s, js // pt].long()
                keys, vals = cache.k_pages[pages, 0, js % pt].float(), cache.v_pages[pages, 0, js % pt].float()
                sc = q[qs:qs + ql] @ keys.T / math.sqrt(self.kw)
                sc = sc.masked_fill(js[None, :] > (p0 + torch.arange(ql, device=xb.device))[:, None], float("-inf"))
                residual[qs:qs + ql] += (torch.softmax(sc, dim=1) @ vals) @ self.w["o"].float().T

    class TwoMixerBlock(Part):
        def __init__(self, norm, first, second):
            self.norm, self.first, self.second = norm, first, second

        def children(self):
            return (self.norm, self.first, self.second)

        def cache_specs(self):
            return [self.first.cache_spec(), self.second.cache_spec()]

        def forward(self, residual, ctx, caches, write_cache=True):
            xb = torch.empty(residual.shape, dtype=ctx.precision.compute, device=residual.device)
            self.norm.forward(residual, xb)
            add = torch.zeros_like(residual)
            self.first.forward(xb, add, ctx, caches[0], write_cache)
            self.second.forward(xb, add, ctx, caches[1], write_cache)
            residual += add

    class FeedForwardOnlyBlock(Part):
        def __init__(self, norm, ffn):
            self.norm, self.ffn = norm, ffn

        def children(self):
            return (self.norm, self.ffn)

        def cache_specs(self):
            return []

        def forward(self, residual, ctx, caches, write_cache=True):
            assert list(caches) == []
            xb = torch.empty(residual.shape, dtype=ctx.precision.compute, device=residual.device)
            self.norm.forward(residual, xb)
            self.ffn.forward(xb, residual, ctx)

    d = cfg.hidden_size
    blocks = [TwoMixerBlock(RMSNorm(d, 1e-6, "b0.n"), NarrowKeyWideValueMixer(d, cfg.key_width, cfg.value_width, "b0.m."),
                            GQAAttention(d, 2, 1, 16, "b0.attn.")),
              FeedForwardOnlyBlock(RMSNorm(d, 1e-6, "b1.n"), SwiGLUFeedForward(d, 40, "b1.mlp."))]
    return ModelSpec(cfg, TokenEmbedding(cfg.vocab_size, d, "emb"), blocks, OutputHead(d, cfg.vocab_size, RMSNorm(d, 1e-6, "norm"), "head"))


def two_mixer_plain(cfg, w, ids):
    x = w["emb"][ids]
    T = len(ids)
    xb = P.rms_norm(x, w["b0.n"], 1e-6)
    q, k, v = (xb @ w["b0.m." + n].T for n in "qkv")
    sc = q @ k.T / math.sqrt(cfg.key_width)
    sc[np.triu_indices(T, 1)] = -np.inf
    pr = np.exp(sc - sc.max(1, keepdims=True))
    pr /= pr.sum(1, keepdims=True)
    add = (pr @ v) @ w["b0.m.o"].T
    qa, ka, va = (P.linear(xb, w[f"b0.attn.{n}_proj.weight"]) for n in "qkv")
    add = add + P.linear(P.causal_gqa_attention(qa, ka, va, 2, 1, 16), w["b0.attn.o_proj.weight"])
    x = x + add
    xb = P.rms_norm(x, w["b1.n"], 1e-6)
    x = x + P.linear(P.swiglu(P.linear(xb, w["b1.mlp.gate_proj.weight"]), P.linear(xb, w["b1.mlp.up_proj.weight"])),
                     w["b1.mlp.down_proj.weight"])
    return P.linear(P.rms_norm(x, w["norm"], 1e-6), w["head"])


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_toy_block_with_two_mixers_and_a_block_with_none(dtype):
    from hk_b200.config import register_architecture
    from hk_b200.engine import Engine, StepEntry
    register_architecture("ToyTwoMixerForCausalLM", TwoMixerConfig, build_two_mixer)
    cfg = TwoMixerConfig()
    eng = Engine(config=cfg, random_seed=11, dtype=dtype, max_tokens=96, page_tokens=4, max_requests=2, max_context=48)
    # entry 0 keeps two page caches in two groups (other widths), entry 1 keeps none
    assert [[lc.kind for lc in caches] for caches in eng.cache.layers] == [["pages", "pages"], []]
    first, second = eng.cache.layers[0]
    assert first.k_pages.shape[-1] == 8 and first.v_pages.shape[-1] == 40 and first.group != second.group
    b0, b1 = eng.model.layers
    w = {"emb": eng.model.embedding.table, "head": eng.model.head.weight, "norm": eng.model.head.norm.weight,
         "b0.n": b0.norm.weight, "b1.n": b1.norm.weight, "b0.attn.o_proj.weight": b0.second.w_o,
         "b0.attn.q_proj.weight": b0.second.w_qkv[:32], "b0.attn.k_proj.weight": b0.second.w_qkv[32:48],
         "b0.attn.v_proj.weight": b0.second.w_qkv[48:], "b1.mlp.gate_proj.weight": b1.ffn.w_gate_up[:40],
         "b1.mlp.up_proj.weight": b1.ffn.w_gate_up[40:], "b1.mlp.down_proj.weight": b1.ffn.w_down}
    w.update({"b0.m." + n: b0.first.w[n] for n in "qkvo"})
    w = {k: v.double().cpu().numpy() for k, v in w.items()}
    rng = np.random.default_rng(2)
    seqs = {"x": rng.integers(0, cfg.vocab_size, 23).tolist(), "y": rng.integers(0, cfg.vocab_size, 17).tolist()}
    want = {k: two_mixer_plain(cfg, w, np.array(v)) for k, v in seqs.items()}
    scale = max(np.abs(v).max() for v in want.values())
    for plan in ([[("x", 23)], [("y", 17)]], [[("x", 6), ("y", 2)], [("y", 9)], [("x", 1), ("y", 1)], [("x", 16), ("y", 5)]]):
        got, fed = {k: [] for k in seqs}, {k: 0 for k in seqs}
        for k in seqs:
            eng.open_request(k)
        for step in plan:
            out = eng.step([StepEntry(k, seqs[k][fed[k]:fed[k] + n], list(range(n))) for k, n in step]).double().cpu().numpy()
            r = 0
            for k, n in step:
                got[k].append(out[r:r + n])
                r += n
                fed[k] += n
        for k in seqs:
            eng.close_request(k)
            assert np.abs(np.concatenate(got[k]) - want[k]).max() <= (2e-5 if dtype == torch.float32 else 2e-2) * scale
    assert eng.free_pages() == [eng.cache.num_pages] * 2
