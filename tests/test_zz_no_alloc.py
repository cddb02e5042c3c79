"""The decode attention entry point that allocates nothing (hk_b200/csrc/attention_noalloc.h).

Some users of this library run where device allocations are not theirs to make: a host program
that gave the library a fixed memory budget, a real-time loop that cannot afford an allocation's
latency or its synchronisation, a plugin that is only ever handed device pointers.  For them
`hk_attention_decode_noalloc` keeps the partial results of split key ranges in an array inside
the library image instead of caller-allocated scratch.  This test calls it through its exported
C symbol, twice in a row and once more with the first inputs (the shared array then holds another
call's leftovers), and compares with the ordinary entry point on the same inputs and with the plain
per-kernel reference (`ref_ops.paged_attention`), so that a fault shared by both entry points shows too.
It also checks that a request beyond the array's stated size is refused, and that the driver's count of
free device memory is the same before and after the calls (torch's allocator cannot see a cudaMalloc made
inside a C entry point; the driver's figure can).

The file sorts last on purpose: a run that stops at the first failure has then run everything else.
"""
import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"
ERR_SCRATCH_TOO_SMALL = 100002
SCRATCH_BYTES = 4 << 20


def make_case(seed, H, G, hd, pt, lens, splits, window):
    """Decode tokens (the last position of each request) over random paged caches."""
    from test_kernels_gpu import make_paged
    from hk_b200.csrc import attention_fast
    rng = np.random.default_rng(seed)
    k_pages, v_pages, bt, _, _ = make_paged(rng, len(lens), lens, G, hd, pt, torch.bfloat16)
    n = len(lens)
    q = torch.from_numpy(rng.standard_normal((n, H * hd))).to(torch.bfloat16)
    pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32)
    slot = torch.arange(n, dtype=torch.int32)
    plan = attention_fast.build_plan(list(range(n)), list(range(n)), [1] * n, [l - 1 for l in lens], n, window, H, G, 148,
                                     lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV), fixed_splits=splits)
    assert plan.nw == 1 and plan.n_parts == n * splits
    import ref_ops
    want = ref_ops.paged_attention(q, k_pages, v_pages, bt, pos, slot, H, G, hd, pt, window, 1.0 / math.sqrt(hd))
    return dict(q=q.to(DEV), k=k_pages.to(DEV), v=v_pages.to(DEV), bt=bt.to(DEV), pos=pos.to(DEV), slot=slot.to(DEV),
                plan=plan, H=H, G=G, hd=hd, pt=pt, window=window, n=n, plain=want.reshape(n, H * hd))


def close_to(got, want):
    diff = (got.double().cpu() - want.double().cpu()).abs()
    assert (diff <= 3e-3 + 2 ** -7 * want.double().cpu().abs()).all(), f"worst {diff.max():.3g}"


def ordinary(case):
    from hk_b200.csrc import ops
    out = torch.empty_like(case["q"])
    with ops.force(attention="flash_cp"):      # the same kernels as the entry point under test
        ops.paged_attention(case["q"], case["k"], case["v"], case["bt"], case["pos"], case["slot"], out, case["H"], case["G"],
                            case["hd"], case["pt"], case["window"], 1.0 / math.sqrt(case["hd"]), plan=case["plan"])
    return out


def no_alloc(lib, case, out, n_parts=None):
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    plan = case["plan"]
    return lib.hk_attention_decode_noalloc(
        p(case["q"]), p(case["k"]), p(case["v"]), p(case["bt"]), int(case["bt"].shape[1]), p(plan.items), plan.n_items,
        plan.n_parts if n_parts is None else n_parts, p(plan.first), p(plan.count), p(plan.row0), p(out), case["n"], case["H"],
        case["G"], case["hd"], case["pt"], case["window"], ctypes.c_float(math.log2(math.e) / math.sqrt(case["hd"])),
        plan.max_keys // case["pt"] + 2, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_no_alloc_entry_point_matches_the_ordinary_one_on_calls_in_a_row():
    from hk_b200.csrc import build
    lib = build.load("attention_flash")
    a = make_case(1, 8, 2, 128, 16, [700, 64, 129, 333], 5, 0)
    # b: windows of 40 and 100 keys whose first key is no multiple of the 64-key tile (257 - 40, 190 - 100)
    b = make_case(2, 6, 3, 64, 8, [90, 257, 31], 3, 40)
    c = make_case(4, 4, 2, 64, 16, [191, 134], 2, 100)
    want_a, want_b, want_c = ordinary(a), ordinary(b), ordinary(c)
    outs = [torch.empty_like(a["q"]), torch.empty_like(b["q"]), torch.empty_like(a["q"]), torch.empty_like(c["q"])]
    warm = torch.empty_like(a["q"])
    assert no_alloc(lib, a, warm) == 0          # the first call on a device resolves the array's address
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    codes = [no_alloc(lib, a, outs[0]), no_alloc(lib, b, outs[1]), no_alloc(lib, a, outs[2]), no_alloc(lib, c, outs[3])]
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert codes == [0, 0, 0, 0]
    assert free_after == free_before, "the entry point took device memory from the driver"
    for got, want, case in ((outs[0], want_a, a), (outs[1], want_b, b), (outs[2], want_a, a), (outs[3], want_c, c)):
        close_to(got, want)
        close_to(got, case["plain"])
    assert torch.equal(outs[0], outs[2]) and torch.equal(outs[0], warm)


def test_no_alloc_entry_point_refuses_what_its_array_cannot_hold():
    from hk_b200.csrc import build
    lib = build.load("attention_flash")
    a = make_case(3, 8, 2, 128, 16, [200, 300], 2, 0)
    out = torch.full_like(a["q"], 7.0)
    per_part = a["G"] * 16 * (a["hd"] + 2) * 4
    too_many = SCRATCH_BYTES // per_part + 1
    assert no_alloc(lib, a, out, n_parts=too_many) == ERR_SCRATCH_TOO_SMALL
    torch.cuda.synchronize()
    assert (out == 7.0).all(), "a refused call must launch nothing"
    assert no_alloc(lib, a, out) == 0
    torch.cuda.synchronize()
    assert torch.equal(out, ordinary(a))
    close_to(out, a["plain"])
