"""Each CUDA kernel alone against its plain reference (tests/ref_ops.py), at sizes other than
the engine tests': odd widths, head sizes in steps of 16, any number of heads and groups.
Tolerances: float32 kernels within accumulated float32 rounding of the float64 reference;
bfloat16 storage within half a unit in the last place of the result plus the same; matrix
products scaled by sum |a||b| (the reference's own rule, tests/test_cuda.zig:374-378)."""
import math

import numpy as np
import pytest
import torch

import ref_ops

pytestmark = pytest.mark.gpu

DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16]
IDS = ["f32", "bf16"]


def ops():
    from hk_b200.csrc import ops as o
    return o


def close(got, want, dtype, atol=1e-5, rtol=1e-5):
    got = got.double().cpu()
    want = want.double().cpu()
    if dtype == torch.bfloat16:
        rtol, atol = max(rtol, 2 ** -8), max(atol, 1e-5)
    bad = (got - want).abs() > atol + rtol * want.abs()
    assert not bad.any(), f"{int(bad.sum())} of {bad.numel()} differ; worst {(got - want).abs().max():.3g} at {tuple(np.unravel_index(int((got - want).abs().argmax()), got.shape))}"


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("n,d,vocab", [(1, 8, 3), (37, 72, 333), (5, 4100, 17)])
def test_embedding(dtype, n, d, vocab):
    g = torch.Generator().manual_seed(n + d)
    table = torch.randn(vocab, d, generator=g).to(dtype)
    ids = torch.randint(0, vocab, (n,), generator=g, dtype=torch.int32)
    out = torch.empty(n, d, dtype=torch.float32, device=DEV)
    ops().embedding(table.to(DEV), ids.to(DEV), out)
    assert torch.equal(out.cpu(), ref_ops.embedding(table, ids))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("n,d,eps", [(1, 16, 1e-6), (19, 72, 1e-5), (3, 4104, 3e-6), (130, 96, 0.0)])
def test_rms_norm(dtype, n, d, eps):
    g = torch.Generator().manual_seed(d)
    x = torch.randn(n, d, generator=g) * 3 + 0.5
    w = 1 + 0.1 * torch.randn(d, generator=g)
    out = torch.empty(n, d, dtype=dtype, device=DEV)
    ops().rms_norm(x.to(DEV), w.to(DEV), eps, out)
    close(out, ref_ops.rms_norm(x, w, eps), dtype)
    rows = torch.tensor([n - 1, 0, n // 2], dtype=torch.int32)
    out = torch.empty(3, d, dtype=dtype, device=DEV)
    ops().rms_norm(x.to(DEV), w.to(DEV), eps, out, rows.to(DEV))
    close(out, ref_ops.rms_norm(x, w, eps, rows), dtype)


def test_rms_norm_reference_fact():
    # src/engine/ops.zig:227-234
    out = torch.empty(1, 4, dtype=torch.float32, device=DEV)
    ops().rms_norm(torch.tensor([[2.0, -2, 2, -2]], device=DEV), torch.ones(4, device=DEV), 0.0, out)
    assert torch.allclose(out.cpu(), torch.tensor([[1.0, -1, 1, -1]]), atol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("n,f", [(1, 1), (7, 200), (33, 1111)])
def test_swiglu(dtype, n, f):
    gu = torch.randn(n, 2 * f, generator=torch.Generator().manual_seed(f)) * 4
    out = torch.empty(n, f, dtype=dtype, device=DEV)
    ops().swiglu(gu.to(DEV), out)
    close(out, ref_ops.swiglu(gu), dtype)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("m,n,k", [(1, 7, 5), (13, 300, 256), (65, 129, 1000), (2, 1000, 72), (128, 64, 64)])
@pytest.mark.parametrize("accumulate", [False, True])
def test_gemm_generic(dtype, m, n, k, accumulate):
    g = torch.Generator().manual_seed(m * n + k)
    a = torch.randn(m, k, generator=g).to(dtype)
    w = torch.randn(n, k, generator=g).to(dtype)
    out0 = torch.randn(m, n, generator=g)
    out = out0.clone().to(DEV)
    with ops().force(gemm="generic"):
        ops().gemm(a.to(DEV), w.to(DEV), out, accumulate=accumulate)
    want = ref_ops.gemm(a, w, out0 if accumulate else None)
    bound = a.double().abs() @ w.double().abs().T          # sum |a||b|
    err = (out.double().cpu() - want).abs()
    assert (err <= 1e-6 * bound + 1e-6 * want.abs() + 1e-7).all(), f"worst {err.max():.3g}"


def make_paged(rng, n_slots, lens, G, hd, pt, dtype, extra_pages=3):
    """Random cache contents in scattered pages; returns (k_pages, v_pages, block_table, k, v) with
    k, v the dense float64 [slot][len, G, hd] contents (already rounded to `dtype`)."""
    max_pages = max(-(-l // pt) for l in lens) + 1
    total = sum(-(-l // pt) for l in lens) + extra_pages
    perm = rng.permutation(total)
    bt = np.full((n_slots, max_pages), -1, dtype=np.int32)
    k_pages = torch.zeros(total, G, pt, hd, dtype=dtype)
    v_pages = torch.zeros(total, G, pt, hd, dtype=dtype)
    dense_k, dense_v = [], []
    nxt = 0
    for s, l in enumerate(lens):
        k = torch.from_numpy(rng.standard_normal((l, G, hd))).to(dtype)
        v = torch.from_numpy(rng.standard_normal((l, G, hd))).to(dtype)
        dense_k.append(k.double())
        dense_v.append(v.double())
        for i in range(-(-l // pt)):
            page = int(perm[nxt])
            nxt += 1
            bt[s, i] = page
            seg = slice(i * pt, min(l, (i + 1) * pt))
            k_pages[page, :, :seg.stop - seg.start] = k[seg].transpose(0, 1)
            v_pages[page, :, :seg.stop - seg.start] = v[seg].transpose(0, 1)
    return k_pages, v_pages, torch.from_numpy(bt), dense_k, dense_v


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("H,G,hd,pt,rot,norm", [
    (4, 2, 16, 4, 16, True), (5, 1, 48, 16, 24, True), (6, 3, 80, 8, 80, False), (8, 8, 128, 16, 128, True),
    (3, 1, 256, 32, 64, True), (2, 2, 32, 1, 0, False), (3, 1, 40, 8, 24, True), (2, 1, 24, 4, 24, True),
    (4, 2, 160, 16, 160, True)])
def test_qk_norm_rope_kv_write(dtype, H, G, hd, pt, rot, norm):
    rng = np.random.default_rng(H * hd + pt)
    lens = [9, 30, 17]
    k_pages, v_pages, bt, _, _ = make_paged(rng, 3, lens, G, hd, pt, dtype)
    k_pages.zero_()
    v_pages.zero_()
    # tokens: a portion of slot 1 (positions 12..29), one token of slot 0 (position 8), three of slot 2
    slot = torch.tensor([1] * 18 + [0] + [2] * 3, dtype=torch.int32)
    pos = torch.tensor(list(range(12, 30)) + [8] + [14, 15, 16], dtype=torch.int32)
    n = slot.numel()
    qkv = torch.from_numpy(rng.standard_normal((n, (H + 2 * G) * hd))).float() * 2
    qw = (1 + 0.2 * torch.from_numpy(rng.standard_normal(hd))).float() if norm else None
    kw = (1 + 0.2 * torch.from_numpy(rng.standard_normal(hd))).float() if norm else None
    eps = 1e-5
    half = max(rot // 2, 1)
    ang = torch.arange(64, dtype=torch.float64)[:, None] * torch.from_numpy(rng.uniform(0.001, 1.0, half))[None, :]
    cos, sin = torch.cos(ang).float(), torch.sin(ang).float()
    q_out = torch.empty(n, H * hd, dtype=dtype, device=DEV)
    kp, vp = k_pages.to(DEV), v_pages.to(DEV)
    d = lambda t: None if t is None else t.to(DEV)
    ops().qk_norm_rope_kv_write(qkv.to(DEV), q_out, d(qw), d(kw), eps, d(cos) if rot else None, d(sin) if rot else None,
                                rot, pos.to(DEV), slot.to(DEV), bt.to(DEV), kp, vp, H, G, hd, pt)
    q, k, v = ref_ops.qk_norm_rope(qkv, qw, kw, eps, cos, sin, rot, pos, H, G, hd)
    close(q_out, q.reshape(n, H * hd), dtype)
    rk, rv = torch.zeros_like(k_pages, dtype=torch.float64), torch.zeros_like(v_pages, dtype=torch.float64)
    ref_ops.write_pages(k, v, rk, rv, bt, slot, pos, pt)
    close(kp, rk, dtype)        # untouched places must still be zero
    close(vp, rv, dtype)
    # a layer that reads another layer's cache writes nothing
    kp2, vp2 = torch.zeros_like(kp), torch.zeros_like(vp)
    q2 = torch.empty_like(q_out)
    ops().qk_norm_rope_kv_write(qkv.to(DEV), q2, d(qw), d(kw), eps, d(cos) if rot else None, d(sin) if rot else None,
                                rot, pos.to(DEV), slot.to(DEV), bt.to(DEV), kp2, vp2, H, G, hd, pt, write_kv=False)
    assert torch.equal(q2, q_out) and not kp2.any() and not vp2.any()


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("H,G,hd,pt,rot,norm,ntok", [(32, 8, 128, 16, 128, True, 700), (7, 1, 64, 8, 32, True, 1843), (9, 3, 48, 16, 48, False, 1097)])
def test_qk_norm_rope_kv_write_many_tokens(dtype, H, G, hd, pt, rot, norm, ntok):
    # a prompt's worth of (token, head) items: item counts that are no multiple of a block, tokens of two requests at
    # places that straddle pages
    rng = np.random.default_rng(H * hd + pt + ntok)
    n0 = ntok // 3
    lens = [n0 + 5, ntok - n0 + 11]
    k_pages, v_pages, bt, _, _ = make_paged(rng, 2, lens, G, hd, pt, dtype)
    k_pages.zero_()
    v_pages.zero_()
    slot = torch.tensor([0] * n0 + [1] * (ntok - n0), dtype=torch.int32)
    pos = torch.tensor(list(range(5, 5 + n0)) + list(range(11, 11 + ntok - n0)), dtype=torch.int32)
    qkv = torch.from_numpy(rng.standard_normal((ntok, (H + 2 * G) * hd))).float() * 2
    qw = (1 + 0.2 * torch.from_numpy(rng.standard_normal(hd))).float() if norm else None
    kw = (1 + 0.2 * torch.from_numpy(rng.standard_normal(hd))).float() if norm else None
    ang = torch.arange(max(lens) + 1, dtype=torch.float64)[:, None] * torch.from_numpy(rng.uniform(0.001, 1.0, rot // 2))[None, :]
    cos, sin = torch.cos(ang).float(), torch.sin(ang).float()
    q_out = torch.empty(ntok, H * hd, dtype=dtype, device=DEV)
    kp, vp = k_pages.to(DEV), v_pages.to(DEV)
    d = lambda t: None if t is None else t.to(DEV)
    ops().qk_norm_rope_kv_write(qkv.to(DEV), q_out, d(qw), d(kw), 1e-6, d(cos), d(sin), rot, pos.to(DEV), slot.to(DEV), bt.to(DEV),
                                kp, vp, H, G, hd, pt)
    q, k, v = ref_ops.qk_norm_rope(qkv, qw, kw, 1e-6, cos, sin, rot, pos, H, G, hd)
    close(q_out, q.reshape(ntok, H * hd), dtype)
    rk, rv = torch.zeros_like(k_pages, dtype=torch.float64), torch.zeros_like(v_pages, dtype=torch.float64)
    ref_ops.write_pages(k, v, rk, rv, bt, slot, pos, pt)
    close(kp, rk, dtype)
    close(vp, rv, dtype)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("H,G,hd,pt,rot", [(4, 2, 16, 4, 16), (5, 1, 48, 16, 24), (8, 8, 128, 16, 128), (3, 1, 40, 8, 24), (2, 1, 24, 4, 22),
                                            (4, 2, 160, 16, 160), (6, 2, 64, 16, 32)])
@pytest.mark.parametrize("pairing,with_bias", [("adjacent", False), ("adjacent", True), ("half", True)])
def test_qk_norm_rope_kv_write_with_bias_and_adjacent_pairs(dtype, H, G, hd, pt, rot, pairing, with_bias):
    # both kernels (a lane with four consecutive dims; a warp over shared memory for the other sizes), a bias on
    # the projection, and the rotation of dims (2i, 2i + 1) instead of (i, i + half)
    rng = np.random.default_rng(H * hd + pt + rot)
    lens = [9, 30, 17]
    k_pages, v_pages, bt, _, _ = make_paged(rng, 3, lens, G, hd, pt, dtype)
    k_pages.zero_()
    v_pages.zero_()
    slot = torch.tensor([1] * 18 + [0] + [2] * 3, dtype=torch.int32)
    pos = torch.tensor(list(range(12, 30)) + [8] + [14, 15, 16], dtype=torch.int32)
    n = slot.numel()
    qkv = torch.from_numpy(rng.standard_normal((n, (H + 2 * G) * hd))).float() * 2
    bias = torch.from_numpy(rng.standard_normal((H + 2 * G) * hd)).float() if with_bias else None
    qw = (1 + 0.2 * torch.from_numpy(rng.standard_normal(hd))).float()
    kw = (1 + 0.2 * torch.from_numpy(rng.standard_normal(hd))).float()
    ang = torch.arange(64, dtype=torch.float64)[:, None] * torch.from_numpy(rng.uniform(0.001, 1.0, rot // 2))[None, :]
    cos, sin = torch.cos(ang).float(), torch.sin(ang).float()
    q_out = torch.empty(n, H * hd, dtype=dtype, device=DEV)
    kp, vp = k_pages.to(DEV), v_pages.to(DEV)
    ops().qk_norm_rope_kv_write(qkv.to(DEV), q_out, qw.to(DEV), kw.to(DEV), 1e-5, cos.to(DEV), sin.to(DEV), rot, pos.to(DEV),
                                slot.to(DEV), bt.to(DEV), kp, vp, H, G, hd, pt, bias=None if bias is None else bias.to(DEV),
                                pairing=pairing)
    q, k, v = ref_ops.qk_norm_rope(qkv, qw, kw, 1e-5, cos, sin, rot, pos, H, G, hd, bias=bias, pairing=pairing)
    close(q_out, q.reshape(n, H * hd), dtype)
    rk, rv = torch.zeros_like(k_pages, dtype=torch.float64), torch.zeros_like(v_pages, dtype=torch.float64)
    ref_ops.write_pages(k, v, rk, rv, bt, slot, pos, pt)
    close(kp, rk, dtype)
    close(vp, rv, dtype)


def test_adjacent_rotation_reference_fact():
    # src/engine/ops.zig:236-252, the `.norm` style: 90 degrees on pairs (x0,x1),(x2,x3): [1,0,0,1] -> [0,1,-1,0]
    qkv = torch.tensor([[1.0, 0, 0, 1] + [0.0] * 8], device=DEV)
    q_out = torch.empty(1, 4, dtype=torch.float32, device=DEV)
    z = torch.zeros(1, dtype=torch.int32, device=DEV)
    kp = torch.zeros(1, 1, 1, 4, device=DEV)
    ops().qk_norm_rope_kv_write(qkv, q_out, None, None, 0.0, torch.zeros(1, 2, device=DEV), torch.ones(1, 2, device=DEV),
                                4, z, z, torch.zeros(1, 1, dtype=torch.int32, device=DEV), kp, kp.clone(), 1, 1, 4, 1, pairing="adjacent")
    assert torch.allclose(q_out.cpu(), torch.tensor([[0.0, 1, -1, 0]]), atol=1e-6)


@pytest.mark.parametrize("n,N", [(1, 7), (33, 4096), (5, 1001)])
def test_add_bias(n, N):
    out0 = torch.randn(n, N, device=DEV)
    bias = torch.randn(N, device=DEV)
    out = out0.clone()
    ops().add_bias(out, bias)
    assert torch.equal(out, out0 + bias[None, :])


def test_rotation_reference_fact():
    # src/engine/ops.zig:236-252: 90 degrees in the half-split pairing: [1,0,0,1] -> [0,-1,1,0]
    qkv = torch.tensor([[1.0, 0, 0, 1] + [0.0] * 8], device=DEV)
    q_out = torch.empty(1, 4, dtype=torch.float32, device=DEV)
    z = torch.zeros(1, dtype=torch.int32, device=DEV)
    kp = torch.zeros(1, 1, 1, 4, device=DEV)
    ops().qk_norm_rope_kv_write(qkv, q_out, None, None, 0.0, torch.zeros(1, 2, device=DEV), torch.ones(1, 2, device=DEV),
                                4, z, z, torch.zeros(1, 1, dtype=torch.int32, device=DEV), kp, kp.clone(), 1, 1, 4, 1)
    assert torch.allclose(q_out.cpu(), torch.tensor([[0.0, -1, 1, 0]]), atol=1e-6)


ATT_SHAPES = [(4, 2, 16, 4), (5, 1, 48, 16), (6, 2, 80, 8), (8, 2, 128, 16), (3, 3, 256, 16), (7, 7, 32, 32), (8, 1, 64, 16),
              (2, 1, 112, 16), (3, 1, 40, 8), (4, 2, 160, 16), (2, 2, 24, 4)]


def attention_case(kernel, dtype, H, G, hd, pt, window, lens, q_spans, spike=None, sm_count=148, fixed_splits=0, rows=0, mass=False):
    """q_spans: per slot (first position, count) of the query rows; the cache holds lens[s] keys.  With `mass` the
    softmax-weighted mean of |v| is kept in `attention_case.mass` (see `close_probabilities_in_bfloat16`)."""
    rng = np.random.default_rng(H * 1000 + hd + pt + window)
    k_pages, v_pages, bt, dk, dv = make_paged(rng, len(lens), lens, G, hd, pt, dtype)
    slot, pos = [], []
    for s, (p0, c) in enumerate(q_spans):
        slot += [s] * c
        pos += list(range(p0, p0 + c))
    n = len(slot)
    q = torch.from_numpy(rng.standard_normal((n, H * hd))).to(dtype)
    if spike is not None:
        # make one far key dominate one query row: the output must be that key's value
        row, s, j, g = spike
        kk = dk[s][j, g].clone()
        k_page = int(bt[s, j // pt])
        big = (kk / kk.norm() * 30).to(dtype)
        k_pages[k_page, g, j % pt] = big
        dk[s][j, g] = big.double()
        group = H // G
        for h in range(g * group, (g + 1) * group):
            q[row, h * hd:(h + 1) * hd] = (big.double() * (math.sqrt(hd) * 2)).to(dtype) / 30 * 3
    slot_t, pos_t = torch.tensor(slot, dtype=torch.int32), torch.tensor(pos, dtype=torch.int32)
    scale = 1.0 / math.sqrt(hd)
    out = torch.empty(n, H * hd, dtype=dtype, device=DEV)
    plan = None
    if kernel != "generic":
        from hk_b200.csrc import attention_fast
        q_starts = [0]
        for _, c in q_spans[:-1]:
            q_starts.append(q_starts[-1] + c)
        plan = attention_fast.build_plan(list(range(len(lens))), q_starts, [c for _, c in q_spans], [p0 for p0, _ in q_spans],
                                         n, window, H, G, sm_count, lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV),
                                         fixed_splits=fixed_splits,
                                         prefill_rows=rows or (128 if kernel == "flash" and attention_fast.tc_prefill_supported(hd, H // G) else 64))
    with ops().force(attention=kernel):
        ops().paged_attention(q.to(DEV), k_pages.to(DEV), v_pages.to(DEV), bt.to(DEV), pos_t.to(DEV), slot_t.to(DEV), out,
                              H, G, hd, pt, window, scale, plan=plan)
    want = ref_ops.paged_attention(q, k_pages, v_pages, bt, pos_t, slot_t, H, G, hd, pt, window, scale)
    if mass:
        attention_case.mass = ref_ops.paged_attention(q, k_pages, v_pages.abs(), bt, pos_t, slot_t, H, G, hd, pt, window, scale)
    return out, want, (q, dk, dv, slot, pos)


def close_probabilities_in_bfloat16(got, want, mass):
    """The bound that follows from the kernel's arithmetic: probabilities are rounded to bfloat16 (unit roundoff 2^-8)
    before they multiply v, while their sum is kept in 32-bit, so an output is off by at most 2^-8 of the weighted mean
    of |v| (`mass`), plus the rounding of the output itself; twice that is allowed."""
    got, want, mass = got.double().cpu(), want.double().cpu(), mass.double().cpu()
    bad = (got - want).abs() > 2 ** -7 * (mass + want.abs()) + 1e-5
    assert not bad.any(), f"{int(bad.sum())} of {bad.numel()} differ; worst {(got - want).abs().max():.3g}"


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("H,G,hd,pt", ATT_SHAPES)
@pytest.mark.parametrize("window", [0, 13])
def test_attention_generic_mixed_batch(dtype, H, G, hd, pt, window):
    # slot 0: a decode token at position 299 of 300; slot 1: a portion 37..69 of 70; slot 2: the first 5 tokens
    out, want, _ = attention_case("generic", dtype, H, G, hd, pt, window, [300, 70, 5], [(299, 1), (37, 33), (0, 5)])
    close(out, want, dtype, atol=2e-5, rtol=1e-4)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("j", [0, 15, 16, 17, 255, 256, 481])
def test_attention_generic_finds_a_far_key(dtype, j):
    # 500 keys; key j (a page's first, last, or middle place) is made to dominate the decode query
    H, G, hd, pt = 4, 2, 64, 16
    out, want, (q, dk, dv, slot, pos) = attention_case("generic", dtype, H, G, hd, pt, 0, [500], [(499, 1)], spike=(0, 0, j, 1))
    close(out, want, dtype, atol=2e-5, rtol=1e-4)
    got = out.double().cpu().reshape(1, H, hd)
    assert torch.allclose(got[0, 2], dv[0][j, 1], atol=0.05) and torch.allclose(got[0, 3], dv[0][j, 1], atol=0.05)
    assert not torch.allclose(got[0, 0], dv[0][j, 1], atol=0.05)     # the other group did not see the spike


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_attention_generic_window_edge(dtype):
    # window 20 at position 99 reads keys 80..99: a dominant key at 80 is seen, one at 79 is not
    H, G, hd, pt = 2, 1, 32, 8
    out, want, (_, _, dv, _, _) = attention_case("generic", dtype, H, G, hd, pt, 20, [100], [(99, 1)], spike=(0, 0, 80, 0))
    close(out, want, dtype, atol=2e-5, rtol=1e-4)
    assert torch.allclose(out.double().cpu().reshape(H, hd)[0], dv[0][80, 0], atol=0.05)
    out, want, (_, _, dv, _, _) = attention_case("generic", dtype, H, G, hd, pt, 20, [100], [(99, 1)], spike=(0, 0, 79, 0))
    close(out, want, dtype, atol=2e-5, rtol=1e-4)
    assert not torch.allclose(out.double().cpu().reshape(H, hd)[0], dv[0][79, 0], atol=0.2)


def test_kernels_refuse_what_they_cannot_do():
    o = ops()
    with pytest.raises(o.KernelError):
        o.gemm(torch.zeros(2, 3, device=DEV), torch.zeros(4, 5, device=DEV), torch.zeros(2, 4, device=DEV))
    with pytest.raises(o.KernelError):
        o.rms_norm(torch.zeros(2, 8, device=DEV), torch.ones(4, device=DEV), 1e-6, torch.zeros(2, 8, device=DEV))
    with pytest.raises(o.KernelError):
        o.embedding(torch.zeros(4, 8), torch.zeros(2, dtype=torch.int32, device=DEV), torch.zeros(2, 8, device=DEV))
    with pytest.raises(o.KernelError):
        o.swiglu(torch.zeros(2, 7, device=DEV), torch.zeros(2, 3, device=DEV))
    with pytest.raises(o.KernelError):       # head size above 256
        z = torch.zeros(1, dtype=torch.int32, device=DEV)
        o.paged_attention(torch.zeros(1, 272, device=DEV), torch.zeros(1, 1, 4, 272, device=DEV), torch.zeros(1, 1, 4, 272, device=DEV),
                          torch.zeros(1, 1, dtype=torch.int32, device=DEV), z, z, torch.zeros(1, 272, device=DEV), 1, 1, 272, 4, 0, 1.0)


# ---- the tensor-core matrix products (bfloat16) ---------------------------------------------------


def gemm_case(kernel, m, n, k, accumulate, seed=0):
    g = torch.Generator().manual_seed(seed + m * 7 + n * 3 + k)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = torch.randn(n, k, generator=g).to(torch.bfloat16)
    out0 = torch.randn(m, n, generator=g)
    out = out0.clone().to(DEV)
    with ops().force(gemm=kernel):
        ops().gemm(a.to(DEV), w.to(DEV), out, accumulate=accumulate)
    from hk_b200.csrc import gemm_fast
    gemm_fast.check_status(torch.device(DEV))
    want = ref_ops.gemm(a, w, out0 if accumulate else None)
    bound = a.double().abs() @ w.double().abs().T
    err = (out.double().cpu() - want).abs()
    ok = err <= 2e-6 * bound + 1e-6 * want.abs() + 1e-6
    assert ok.all(), f"{int((~ok).sum())} of {ok.numel()} wrong; worst {err.max():.3g} at {tuple(np.unravel_index(int(err.argmax()), err.shape))}"


@pytest.mark.parametrize("m,n,k", [
    (128, 256, 64), (128, 128, 64), (256, 512, 128), (130, 300, 72), (65, 1000, 4096), (2048, 6144, 512), (300, 151936 // 8, 256),
    (128, 256, 8), (1000, 136, 1024), (129, 257, 200)])
@pytest.mark.parametrize("accumulate", [False, True])
def test_gemm_tcgen05(m, n, k, accumulate):
    gemm_case("tc", m, n, k, accumulate)


@pytest.mark.parametrize("m,n,k", [(64, 4096, 12288), (17, 4096, 4096), (33, 6144, 4096), (64, 1000, 1040), (128, 384, 8192)])
@pytest.mark.parametrize("accumulate", [False, True])
def test_gemm_tcgen05_with_k_slices(m, n, k, accumulate):
    # fewer output tiles than SMs: K is cut into slices whose partial sums are added in order
    from hk_b200.csrc import gemm_fast
    assert gemm_fast.tc_config(m, n, k, 148)[1] > 1
    gemm_case("tc", m, n, k, accumulate)


def test_gemm_tcgen05_many_tiles_per_cta():
    # more tiles than SMs x 2: every CTA walks several tiles through both accumulator buffers
    gemm_case("tc", 2048, 24576, 256, False)
    gemm_case("tc", 4096, 4096, 4096, True)


@pytest.mark.parametrize("m", [1, 2, 7, 8, 9, 16, 17, 32, 33, 64])
@pytest.mark.parametrize("n,k", [(16, 64), (300, 72), (1000, 4096), (4096, 12288), (6144, 512), (40, 8), (18992, 128)])
def test_gemm_small_m(m, n, k):
    gemm_case("smallm", m, n, k, False)
    gemm_case("smallm", m, n, k, True, seed=1)


@pytest.mark.parametrize("rw", [8, 4, 2, 1])
@pytest.mark.parametrize("m", [1, 3, 8, 9, 16, 17, 32])
@pytest.mark.parametrize("n,k", [(16, 64), (300, 192), (1000, 4096), (4096, 12288), (6144, 512), (40, 64), (18992, 128), (2400, 320)])
def test_gemm_stream(rw, m, n, k):
    # the persistent streaming kernel: tiles of 128, 64, 32 or 16 weight rows; ragged N and K; CTAs that share tiles
    from hk_b200.csrc import gemm_fast
    if rw == 1 and m > 16:
        pytest.skip("no such variant")
    gemm_fast._stream_rw = rw
    try:
        gemm_case("stream", m, n, k, False)
        gemm_case("stream", m, n, k, True, seed=1)
    finally:
        gemm_fast._stream_rw = 0


@pytest.mark.parametrize("ctas", [1, 3, 7, 50, 148])
@pytest.mark.parametrize("m,n,k", [(8, 1000, 4096), (5, 200, 1088), (16, 4096, 640), (3, 9536, 256)])
def test_gemm_stream_hand_over_between_ctas_is_exact_and_repeatable(ctas, m, n, k):
    # fewer CTAs move the places where one CTA's share of a tile ends and the next one's begins; the partial sums
    # are added in K order whoever arrives last, so two runs agree to the bit, and the counters are left at zero
    from hk_b200.csrc import gemm_fast
    gemm_fast._stream_ctas = ctas
    try:
        gemm_case("stream", m, n, k, False)
        gemm_case("stream", m, n, k, True, seed=3)
        g = torch.Generator().manual_seed(11)
        a = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
        w = torch.randn(n, k, generator=g).to(torch.bfloat16).to(DEV)
        outs = [torch.empty(m, n, device=DEV) for _ in range(3)]
        with ops().force(gemm="stream"):
            for o in outs:
                ops().gemm(a, w, o)
        assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
        assert int(gemm_fast._stream_scratch[0][1].abs().sum()) == 0
    finally:
        gemm_fast._stream_ctas = 0
    gemm_fast.check_status(torch.device(DEV))


@pytest.mark.parametrize("rw", [8, 4, 2, 1])
@pytest.mark.parametrize("m,f,k", [(1, 128, 64), (8, 384, 192), (7, 1536, 4096), (20, 256, 1024), (32, 12288, 256)])
def test_gemm_stream_swiglu_epilogue(rw, m, f, k):
    from hk_b200.csrc import gemm_fast
    if rw == 1 and m > 16:
        pytest.skip("no such variant")
    g = torch.Generator().manual_seed(m + f + k)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16)
    gate = (torch.randn(f, k, generator=g) / math.sqrt(k)).to(torch.bfloat16)
    up = (torch.randn(f, k, generator=g) / math.sqrt(k)).to(torch.bfloat16)
    out = torch.empty(m, f, dtype=torch.bfloat16, device=DEV)
    gemm_fast._stream_rw = rw
    try:
        with ops().force(gemm="stream"):
            ops().gemm_swiglu(a.to(DEV), torch.cat([gate, up]).to(DEV), out)
    finally:
        gemm_fast._stream_rw = 0
    gemm_fast.check_status(torch.device(DEV))
    want = ref_ops.swiglu(torch.cat([ref_ops.gemm(a, gate), ref_ops.gemm(a, up)], dim=1))
    close(out, want, torch.bfloat16, atol=2e-3)


def test_fast_gemms_refuse_unaligned_shapes_and_the_generic_kernel_takes_them():
    a = torch.randn(4, 70).to(torch.bfloat16).to(DEV)      # K % 8 != 0
    w = torch.randn(9, 70).to(torch.bfloat16).to(DEV)
    out = torch.empty(4, 9, device=DEV)
    for kernel in ("tc", "smallm", "stream"):
        with pytest.raises(ops().KernelError):
            with ops().force(gemm=kernel):
                ops().gemm(a, w, out)
    ops().gemm(a, w, out)                                  # free choice: falls to the generic kernel
    close(out, ref_ops.gemm(a.cpu(), w.cpu()), torch.float32, atol=1e-4, rtol=1e-4)
    with pytest.raises(ops().KernelError):
        with ops().force(gemm="smallm"):
            ops().gemm(torch.zeros(65, 64, dtype=torch.bfloat16, device=DEV), torch.zeros(8, 64, dtype=torch.bfloat16, device=DEV),
                       torch.zeros(65, 8, device=DEV))
    with pytest.raises(ops().KernelError):
        with ops().force(gemm="stream"):
            ops().gemm(torch.zeros(33, 64, dtype=torch.bfloat16, device=DEV), torch.zeros(8, 64, dtype=torch.bfloat16, device=DEV),
                       torch.zeros(33, 8, device=DEV))


@pytest.mark.parametrize("m,f,k", [(128, 128, 64), (300, 384, 200), (2048, 1536, 512), (7, 256, 128), (64, 128, 64), (65, 128, 64),
                                   (40, 1024, 4096), (64, 12288, 512), (33, 1000, 256), (200, 328, 64), (19, 77, 128), (500, 2056, 72)])
def test_gemm_swiglu_in_the_epilogue(m, f, k):
    # w = [F gate rows | F up rows]; widths that are no multiple of a tile, of 128 or of 8
    from hk_b200.csrc import gemm_fast
    g = torch.Generator().manual_seed(m + f + k)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16)
    gate = (torch.randn(f, k, generator=g) / math.sqrt(k)).to(torch.bfloat16)
    up = (torch.randn(f, k, generator=g) / math.sqrt(k)).to(torch.bfloat16)
    w = torch.cat([gate, up]).to(DEV)
    out = torch.empty(m, f, dtype=torch.bfloat16, device=DEV)
    ops().gemm_swiglu(a.to(DEV), w, out)
    gemm_fast.check_status(torch.device(DEV))
    want = ref_ops.swiglu(torch.cat([ref_ops.gemm(a, gate), ref_ops.gemm(a, up)], dim=1))
    close(out, want, torch.bfloat16, atol=2e-3)
    with ops().force(gemm="generic"):          # the unfused route
        out2 = torch.empty_like(out)
        ops().gemm_swiglu(a.to(DEV), w, out2)
    close(out2, want, torch.bfloat16, atol=2e-3)


@pytest.mark.parametrize("bn", [32, 64, 96, 160, 192, 224, 256])
@pytest.mark.parametrize("m,f,k,splits", [(70, 672, 256, 1), (130, 1000, 72, 1), (64, 1344, 1024, 2), (9, 4032, 512, 3)])
def test_gemm_swiglu_tcgen05_every_tile_width(bn, m, f, k, splits):
    # the tile width is a run-time value: half a tile's rows are gates, half their ups; K slices where tiles fit F
    from hk_b200.csrc import gemm_fast
    if splits > 1 and f % (bn // 2):
        pytest.skip("K slices need tiles that fit the width")
    g = torch.Generator().manual_seed(bn + m + f + k)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16)
    gate = (torch.randn(f, k, generator=g) / math.sqrt(k)).to(torch.bfloat16)
    up = (torch.randn(f, k, generator=g) / math.sqrt(k)).to(torch.bfloat16)
    out = torch.empty(m, f, dtype=torch.bfloat16, device=DEV)
    gemm_fast._tc_bn, gemm_fast._tc_splits = bn, splits
    try:
        with ops().force(gemm="tc"):
            ops().gemm_swiglu(a.to(DEV), torch.cat([gate, up]).to(DEV), out)
    finally:
        gemm_fast._tc_bn = gemm_fast._tc_splits = 0
    gemm_fast.check_status(torch.device(DEV))
    want = ref_ops.swiglu(torch.cat([ref_ops.gemm(a, gate), ref_ops.gemm(a, up)], dim=1))
    close(out, want, torch.bfloat16, atol=2e-3)


@pytest.mark.parametrize("bn", [16, 48, 80, 112, 144, 176, 208, 240])
@pytest.mark.parametrize("m,n,k,splits", [(64, 1000, 256, 1), (300, 777, 72, 1), (33, 4096, 2048, 4), (128, 250, 520, 2)])
@pytest.mark.parametrize("accumulate", [False, True])
def test_gemm_tcgen05_every_tile_width(bn, m, n, k, splits, accumulate):
    from hk_b200.csrc import gemm_fast
    gemm_fast._tc_bn, gemm_fast._tc_splits = bn, splits
    try:
        gemm_case("tc", m, n, k, accumulate, seed=bn)
    finally:
        gemm_fast._tc_bn = gemm_fast._tc_splits = 0


# ---- the flash attention kernel (bfloat16) -----------------------------------------------------

FLASH_SHAPES = [(4, 2, 16, 4), (5, 1, 48, 16), (6, 2, 80, 8), (8, 2, 128, 16), (7, 7, 32, 32), (8, 1, 64, 16), (2, 1, 112, 16),
                (32, 8, 128, 16), (12, 4, 96, 64), (40, 2, 64, 16)]


@pytest.mark.parametrize("kernel", ["flash", "flash_cp"])
@pytest.mark.parametrize("H,G,hd,pt", FLASH_SHAPES)
@pytest.mark.parametrize("window", [0, 13, 100])
def test_attention_flash_mixed_batch(kernel, H, G, hd, pt, window):
    # a decode token deep in a long request, a portion that starts off-tile, a fresh request, a two-token portion.
    # 'flash' takes the tcgen05 kernel for head sizes 64 and 128, 'flash_cp' always the mma.sync one.
    out, want, _ = attention_case(kernel, torch.bfloat16, H, G, hd, pt, window, [300, 170, 5, 131],
                                  [(299, 1), (37, 133), (0, 5), (129, 2)])
    close(out, want, torch.bfloat16, atol=3e-3, rtol=2 ** -7)
    from hk_b200.csrc import gemm_fast
    gemm_fast.check_status(torch.device(DEV))


@pytest.mark.parametrize("H,G,hd,pt,window", [(32, 8, 128, 16, 0), (8, 2, 64, 16, 0), (6, 2, 128, 32, 200), (5, 1, 64, 16, 0),
                                              (16, 1, 128, 16, 0), (3, 3, 128, 8, 0)])
def test_attention_tcgen05_prefill_long_prompt(H, G, hd, pt, window):
    # several 128-key tiles per CTA and several CTAs per request: a 700-token prompt whole, and a portion that starts
    # at position 391 of another request
    out, want, _ = attention_case("flash", torch.bfloat16, H, G, hd, pt, window, [700, 650], [(0, 700), (391, 259)])
    close(out, want, torch.bfloat16, atol=3e-3, rtol=2 ** -7)
    from hk_b200.csrc import gemm_fast
    gemm_fast.check_status(torch.device(DEV))


@pytest.mark.parametrize("H,G,hd,pt,window", [(32, 8, 128, 16, 0), (8, 2, 64, 16, 0), (6, 2, 128, 32, 200), (5, 1, 64, 16, 0), (16, 1, 128, 8, 0),
                                              (3, 3, 128, 64, 0), (4, 1, 64, 128, 150), (8, 2, 128, 256, 0), (12, 4, 64, 16, 131)])
def test_attention_tcgen05_two_query_tiles(H, G, hd, pt, window):
    # items of 256 rows (two query tiles per CTA, K and V by TMA, P written over S): a 700-token prompt whole, a portion
    # that starts at position 391 of another request, a portion of 40 tokens (rows in the first tile only for some
    # groupings) and a single token at position 299
    out, want, _ = attention_case("flash", torch.bfloat16, H, G, hd, pt, window, [700, 650, 77, 300],
                                  [(0, 700), (391, 259), (37, 40), (299, 1)], rows=256, mass=True)
    close_probabilities_in_bfloat16(out, want, attention_case.mass)
    from hk_b200.csrc import gemm_fast
    gemm_fast.check_status(torch.device(DEV))


@pytest.mark.parametrize("j", [0, 15, 127, 128, 129, 255, 256, 383, 384, 600, 699])
def test_attention_tcgen05_two_query_tiles_find_a_far_key(j):
    # row 699 of a 700-token prompt (the last row of some CTA's second tile) with one dominant key at a tile's or a
    # page's edge; and the first row of a second tile (row 32 * 5 + 128 / 4 ...) likewise
    H, G, hd, pt = 8, 2, 128, 16
    for row in (699, 32 * 21):
        if j > row:
            continue
        out, want, (q, dk, dv, slot, pos) = attention_case("flash", torch.bfloat16, H, G, hd, pt, 0, [700], [(0, 700)],
                                                           spike=(row, 0, j, 1), rows=256, mass=True)
        close_probabilities_in_bfloat16(out, want, attention_case.mass)
        got = out.double().cpu().reshape(700, H, hd)
        assert torch.allclose(got[row, 4], dv[0][j, 1], atol=0.05) and not torch.allclose(got[row, 0], dv[0][j, 1], atol=0.05)


@pytest.mark.parametrize("kernel", ["flash", "flash_cp"])
@pytest.mark.parametrize("H,G,hd,pt", [(8, 2, 128, 16), (5, 1, 48, 16), (4, 4, 64, 8), (32, 8, 128, 16), (6, 2, 64, 32), (4, 1, 128, 64),
                                       (16, 1, 64, 128)])
@pytest.mark.parametrize("sm_count,fixed_splits", [(148, 0), (4000, 0), (148, 5), (148, 1)])
@pytest.mark.parametrize("window", [0, 77])
def test_attention_flash_decode_with_split_keys(kernel, H, G, hd, pt, sm_count, fixed_splits, window):
    # decode only: 16 rows per CTA, warps split the keys of a tile; few requests and long contexts are also
    # split along the keys among CTAs and merged.  'flash' takes the TMA-fed variant where it applies
    # (head size 64/128, pages of 16+ tokens), 'flash_cp' always the cp.async one.
    out, want, _ = attention_case(kernel, torch.bfloat16, H, G, hd, pt, window, [700, 64, 1, 129, 333],
                                  [(699, 1), (63, 1), (0, 1), (128, 1), (332, 1)], sm_count=sm_count, fixed_splits=fixed_splits)
    close(out, want, torch.bfloat16, atol=3e-3, rtol=2 ** -7)
    from hk_b200.csrc import gemm_fast
    gemm_fast.check_status(torch.device(DEV))


@pytest.mark.parametrize("j", [0, 15, 16, 63, 64, 65, 255, 256, 481])
@pytest.mark.parametrize("fixed_splits", [0, 3])
def test_attention_flash_finds_a_far_key(j, fixed_splits):
    H, G, hd, pt = 4, 2, 64, 16
    out, want, (q, dk, dv, slot, pos) = attention_case("flash", torch.bfloat16, H, G, hd, pt, 0, [500], [(499, 1)],
                                                       spike=(0, 0, j, 1), fixed_splits=fixed_splits)
    close(out, want, torch.bfloat16, atol=3e-3, rtol=2 ** -7)
    got = out.double().cpu().reshape(1, H, hd)
    assert torch.allclose(got[0, 2], dv[0][j, 1], atol=0.05) and not torch.allclose(got[0, 0], dv[0][j, 1], atol=0.05)


@pytest.mark.parametrize("kernel", ["flash", "flash_cp"])
@pytest.mark.parametrize("window,pos,fixed_splits,sm_count", [(128, 190, 2, 148), (100, 133, 2, 148), (1000, 1500, 16, 148),
                                                             (128, 133, 0, 4000), (300, 1337, 4, 148), (64, 200, 3, 148)])
def test_attention_decode_split_keys_reach_the_newest_key_of_a_window(kernel, window, pos, fixed_splits, sm_count):
    # A window whose first key is no multiple of 64: the splits start at the tile boundary below it, and the last
    # split must still reach the token's own key.  That key (and then the window's first) is made to dominate.
    H, G, hd, pt = 4, 2, 64, 16
    for j in (pos, pos - window + 1):
        out, want, (_, _, dv, _, _) = attention_case(kernel, torch.bfloat16, H, G, hd, pt, window, [pos + 1], [(pos, 1)],
                                                     spike=(0, 0, j, 1), sm_count=sm_count, fixed_splits=fixed_splits)
        close(out, want, torch.bfloat16, atol=3e-3, rtol=2 ** -7)
        assert torch.allclose(out.double().cpu().reshape(H, hd)[2], dv[0][j, 1], atol=0.05)
    out, want, (_, _, dv, _, _) = attention_case(kernel, torch.bfloat16, H, G, hd, pt, window, [pos + 1], [(pos, 1)],
                                                 spike=(0, 0, pos - window, 1), sm_count=sm_count, fixed_splits=fixed_splits)
    close(out, want, torch.bfloat16, atol=3e-3, rtol=2 ** -7)       # the key just outside the window is not seen
    assert not torch.allclose(out.double().cpu().reshape(H, hd)[2], dv[0][pos - window, 1], atol=0.2)


def test_attention_flash_window_edge_in_a_portion():
    # rows at positions 90..99 with window 20: row 99 reads 80..99.  A dominant key at 80 is seen by row 99
    # (the last row of the portion) and one at 79 is not, although rows 90..98 of the same tile do see 79.
    H, G, hd, pt = 2, 1, 32, 8
    out, want, (_, _, dv, _, _) = attention_case("flash", torch.bfloat16, H, G, hd, pt, 20, [100], [(90, 10)], spike=(9, 0, 80, 0))
    close(out, want, torch.bfloat16, atol=3e-3, rtol=2 ** -7)
    assert torch.allclose(out.double().cpu().reshape(10, H, hd)[9, 0], dv[0][80, 0], atol=0.05)
    out, want, (_, _, dv, _, _) = attention_case("flash", torch.bfloat16, H, G, hd, pt, 20, [100], [(90, 10)], spike=(9, 0, 79, 0))
    close(out, want, torch.bfloat16, atol=3e-3, rtol=2 ** -7)
    assert not torch.allclose(out.double().cpu().reshape(10, H, hd)[9, 0], dv[0][79, 0], atol=0.2)


def test_attention_flash_refuses_large_heads_and_generic_takes_them():
    out, want, _ = attention_case(None, torch.bfloat16, 3, 3, 256, 16, 0, [40], [(0, 40)])
    close(out, want, torch.bfloat16, atol=3e-3, rtol=2 ** -7)
