"""The allocation-free down projection against the regular one.

`b200moe_down_noalloc` serves hosts that cannot call cudaMalloc where they run
the layer (an allocator callback, a runtime that owns the device heap, a decode
loop that bans allocator calls): it keeps the k-split partial sums in an array
built into the library.  Same inputs, same kernel: its result must equal the
regular entry point's partial sums added in split order.  Two calls in a row
check that nothing left in the shared array by one call leaks into the next.
This file sorts last so that a run stopping at the first failure has already
run every other test."""
import ctypes

import pytest
import torch

from shark_platform_b200 import synthetic as syn

pytestmark = pytest.mark.gpu

TOL = 1e-6  # relative L2; both sides add the same fp32 partials in the same order


def _rel(a, b):
    return float(torch.linalg.norm((a - b).double()) / torch.linalg.norm(b.double()).clamp_min(1e-30))


def _down_both_ways(seed, tokens, hidden=256, ffn=1024, experts=8, top_k=2):
    from shark_platform_b200 import _cabi as C, moe, types as T

    gen = torch.Generator().manual_seed(seed)
    planes = syn.q8_0_planes(gen, experts, hidden, ffn)
    lay = T.BlockScaledLayout([experts, hidden, ffn], planes["d"].cuda(), planes["qs"].cuda())
    w = moe.prepare_weight(T.PlanarQuantizedTensor(shape=[experts, hidden, ffn], layout=lay))
    ex = torch.stack([torch.randperm(experts, generator=gen)[:top_k] for _ in range(tokens)])
    plan = moe.route_plan(ex.cuda(), experts)
    pairs = tokens * top_k
    a = (torch.randn(pairs, ffn, generator=gen) * 0.5).to(torch.float16).cuda()
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: ctypes.c_void_p(t.data_ptr())

    ks = C.lib.b200moe_down_ksplit(ctypes.byref(w.desc), pairs, tokens, C.REGIME_STREAM)
    part = torch.zeros(ks, pairs, hidden, dtype=torch.float32, device="cuda")
    C.check(C.lib.b200moe_down(p(a), p(plan.seg_offsets), pairs, tokens, ctypes.byref(w.desc),
                               C.REGIME_STREAM, ks, p(part), st), "down")
    want = part[0].clone()
    for c in range(1, ks):
        want += part[c]

    got = torch.full((pairs, hidden), float("nan"), dtype=torch.float32, device="cuda")
    C.check(C.lib.b200moe_down_noalloc(p(a), p(plan.seg_offsets), pairs, tokens,
                                       ctypes.byref(w.desc), p(got), st), "down_noalloc")
    torch.cuda.synchronize()
    assert ks > 1, "the case must exercise the k-split scratch"
    return got.cpu(), want.cpu()


def test_no_alloc_down_matches_regular_entry_point_twice():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    # two calls in a row on different data and sizes share the built-in array
    got1, want1 = _down_both_ways(seed=21, tokens=24)
    got2, want2 = _down_both_ways(seed=22, tokens=9)
    assert torch.isfinite(got1).all() and torch.isfinite(got2).all()
    assert _rel(got1, want1) < TOL
    assert _rel(got2, want2) < TOL


def test_no_alloc_down_rejects_oversized_calls():
    from shark_platform_b200 import _cabi as C

    desc = C.WeightDesc(C.LAYOUT_Q8_0, 8, 4096, 14336, 16, 16, None)
    dummy = ctypes.c_void_p(256)
    rc = C.lib.b200moe_down_noalloc(dummy, dummy, 4096, 4096, ctypes.byref(desc), dummy, None)
    assert rc == -1
    assert "exceeds the built-in scratch" in C.last_error()
