"""Peer-to-peer dispatch / return index arithmetic with several emulated ranks on
ONE GPU: every "rank" gets its own buffers on the same device and the kernels of
all ranks run one after another (no kernel waits for another: the barrier kernel
is not used here, its segment offsets are recomputed with torch)."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world,E,k,tokens", [(2, 8, 2, 37), (4, 8, 2, 50), (8, 8, 2, 16), (2, 4, 1, 9)])
def test_dispatch_and_return_round_trip(world, E, k, tokens):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from shark_platform_b200 import _cabi as C, moe

    d, el = 64, E // world
    gen = torch.Generator().manual_seed(world * 100 + tokens)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    cap, ret_rows = tokens * world * min(k, el), tokens * k
    counts_all = [torch.zeros(world, E, dtype=torch.int32, device="cuda") for _ in range(world)]
    flags = [torch.zeros(world, dtype=torch.int32, device="cuda") for _ in range(world)]
    recv = [torch.zeros(cap, d, dtype=torch.float16, device="cuda") for _ in range(world)]
    ret = [torch.zeros(ret_rows, d, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    eps = []
    for r in range(world):
        ep = C.EpDesc()
        ep.world, ep.rank, ep.experts_local = world, r, el
        for i in range(world):
            ep.counts_all[i], ep.flags[i] = counts_all[i].data_ptr(), flags[i].data_ptr()
            ep.recv_x[i], ep.ret_y[i] = recv[i].data_ptr(), ret[i].data_ptr()
        eps.append(ep)
    xs, exs, plans = [], [], []
    for r in range(world):
        # small integers (exact in fp16 and bf16): column 1 holds the rank, the others the token
        x = (torch.arange(tokens).view(-1, 1) + torch.zeros(tokens, d))
        x[:, 1] = r
        x = x.to(torch.float16).cuda()
        ex = torch.stack([torch.randperm(E, generator=gen)[:k] for _ in range(tokens)]).to(torch.int32).cuda()
        plan = moe.route_plan(ex, E)
        C.check(C.lib.b200moe_ep_publish_counts(ctypes.byref(eps[r]), p(plan.counts), st))
        xs.append(x); exs.append(ex); plans.append(plan)
    torch.cuda.synchronize()
    full = torch.stack([pl.counts.cpu() for pl in plans])  # [src, E]
    for r in range(world):
        assert torch.equal(counts_all[r].cpu(), full)
    for r in range(world):
        C.check(C.lib.b200moe_ep_dispatch(ctypes.byref(eps[r]), p(xs[r]), p(exs[r]), p(plans[r].perm),
                                          p(plans[r].seg_offsets), tokens * k, k, d, 0, cap, st))
    torch.cuda.synchronize()
    assert moe.device_status() == 0
    seg2s = []
    for q in range(world):
        # expected receive buffer: experts ascending, then source ranks ascending, then the
        # source's own stable order (ascending pair id)
        want = []
        seg2 = [0]
        for e in range(el):
            g = q * el + e
            for src in range(world):
                pairs = torch.nonzero(exs[src].reshape(-1).cpu() == g).reshape(-1)
                want += [(float(int(pp) // k), float(src)) for pp in pairs]
            seg2.append(len(want))
        got = [tuple(v) for v in recv[q][:len(want), 0:2].float().cpu().tolist()]
        assert got == want, (q, got[:8], want[:8])
        seg2s.append(torch.tensor(seg2, dtype=torch.int32, device="cuda"))
    # "expert computation": result row = 2 * input row, as fp32 in two k-split halves
    for q in range(world):
        dpart = torch.stack([recv[q].float() * 1.5, recv[q].float() * 0.5])
        C.check(C.lib.b200moe_ep_return(ctypes.byref(eps[q]), p(dpart), 2, cap, p(seg2s[q]), d, ret_rows, st))
        torch.cuda.synchronize()
    assert moe.device_status() == 0
    for r in range(world):
        # ret_y is in rank r's expert-sorted order: position i holds pair perm[i]
        perm = plans[r].perm.cpu().long()
        want = 2.0 * (perm // k).float()
        assert torch.equal(ret[r][:tokens * k, 0].float().cpu(), want)
        assert torch.equal(ret[r][:tokens * k, -1].float().cpu(), want)
        assert torch.equal(ret[r][:tokens * k, 1].float().cpu(), torch.full_like(want, 2.0 * r))


def test_barrier_gives_up_when_a_peer_never_arrives():
    """A lost rank: a world-2 descriptor whose second rank never signals.  The
    barrier's bounded spin runs out (limit shortened to ~50 us for the test), the
    kernel returns, the status word reports the timeout once, and the library
    keeps working afterwards.  Nothing faults or hangs: the wait simply ends."""
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from shark_platform_b200 import _cabi as C, moe, synthetic as syn

    assert moe.device_status() == 0
    world, el = 2, 4
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    counts_all = [torch.zeros(world, world * el, dtype=torch.int32, device="cuda") for _ in range(world)]
    flags = [torch.zeros(world, dtype=torch.int32, device="cuda") for _ in range(world)]
    rows = [torch.zeros(8, 64, dtype=torch.float16, device="cuda") for _ in range(world)]
    ep = C.EpDesc()
    ep.world, ep.rank, ep.experts_local = world, 0, el
    for i in range(world):
        ep.counts_all[i], ep.flags[i] = counts_all[i].data_ptr(), flags[i].data_ptr()
        ep.recv_x[i], ep.ret_y[i] = rows[i].data_ptr(), rows[i].data_ptr()
    seg2 = torch.full((el + 1,), -1, dtype=torch.int32, device="cuda")
    C.check(C.lib.b200moe_set_wait_limit(100_000))
    try:
        C.check(C.lib.b200moe_ep_barrier(ctypes.byref(ep), 1, ctypes.c_void_p(seg2.data_ptr()), st))
        torch.cuda.synchronize()  # the kernel came back
    finally:
        C.check(C.lib.b200moe_set_wait_limit(0))
    assert flags[1].cpu().tolist() == [1, 0]   # rank 0 signalled its peer
    assert flags[0].cpu().tolist() == [1, 0]   # and itself; the peer's flag never came
    word = ctypes.c_int32(0)
    rc = C.lib.b200moe_device_status(st, ctypes.byref(word))
    assert rc == -4 and word.value & 1, (rc, word.value)       # B200MOE_ERR_DEVICE, wait timed out
    assert "timed out" in C.last_error()
    with pytest.raises(C.B200MoeError):
        C.check(rc, "device_status")
    assert moe.device_status() == 0                             # cleared by the read
    # the library is still usable: an ordinary layer call, checked for a clean status
    case = syn.make_case(syn.CASES["small_q8"])
    blk = syn.case_block(case)
    y = blk(syn.case_input(case))
    assert torch.isfinite(y.float()).all()
    assert moe.device_status() == 0


@pytest.mark.parametrize("name,tokens", [("small_q8", 40), ("small_grok", 130), ("small_q4k", 300)])
def test_single_call_expert_parallel_layer_with_one_rank(name, tokens):
    """`b200moe_ep_layer_forward` with a world of one: the whole sequence
    (publish, three barriers, dispatch, grouped products, return, combine) runs on
    one GPU with nobody to wait for, and must reproduce the ordinary layer up to
    the bf16 rounding of the returned rows.  Called three times in a row with
    advancing epochs, the way a stack of layers shares one exchange."""
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from oracle import moe_oracle as orc
    from helpers import oracle_params
    from shark_platform_b200 import _cabi as C, moe, synthetic as syn

    case = syn.make_case(syn.CASES[name], tokens=tokens)
    s = case.spec
    blk = syn.case_block(case)
    layer = blk.layer
    h = syn.case_input(case).reshape(tokens, s.hidden).contiguous()
    want = blk.layer.forward(h)
    ref, _ = orc.moe_block(case.h, oracle_params(case), form="per_expert")
    E, k, d = s.experts, s.top_k, s.hidden
    cap, ret_rows = tokens * k, tokens * k
    counts_all = torch.zeros(1, E, dtype=torch.int32, device="cuda")
    flags = torch.zeros(1, dtype=torch.int32, device="cuda")
    recv = torch.zeros(cap, d, dtype=torch.float16, device="cuda")
    ret = torch.zeros(ret_rows, d, dtype=torch.bfloat16, device="cuda")
    ep = C.EpDesc()
    ep.world, ep.rank, ep.experts_local = 1, 0, E
    ep.counts_all[0], ep.flags[0] = counts_all.data_ptr(), flags.data_ptr()
    ep.recv_x[0], ep.ret_y[0] = recv.data_ptr(), ret.data_ptr()
    desc = ctypes.byref(layer.desc)
    ks = C.lib.b200moe_down_ksplit(ctypes.byref(layer.down.desc), tokens * k, tokens, C.REGIME_AUTO)
    nbytes = C.lib.b200moe_ep_workspace_bytes(desc, tokens, cap, ks)
    assert nbytes > 0
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    dt = C.DT_BF16 if h.dtype == torch.bfloat16 else C.DT_F32
    epoch = 0
    for _ in range(3):
        y = torch.zeros_like(h)
        C.check(C.lib.b200moe_ep_layer_forward(desc, ctypes.byref(ep), p(h), p(y), dt, tokens, C.REGIME_AUTO,
                                               cap, ret_rows, tokens, ks, epoch, p(ws), nbytes, st),
                "ep_layer_forward")
        epoch += 3
        torch.cuda.synchronize()
        assert moe.device_status() == 0
        assert orc.rel_l2(y.float().cpu(), want.float().cpu()) < 1e-2
        assert orc.rel_l2(y.float().cpu().view(1, tokens, d), ref) < 2e-2
    assert int(flags[0]) == epoch
    # too small a workspace or return buffer is refused before anything is launched
    rc = C.lib.b200moe_ep_layer_forward(desc, ctypes.byref(ep), p(h), p(y), dt, tokens, C.REGIME_AUTO,
                                        cap, ret_rows, tokens, ks, epoch, p(ws), nbytes - 1, st)
    assert rc == -3
    rc = C.lib.b200moe_ep_layer_forward(desc, ctypes.byref(ep), p(h), p(y), dt, tokens, C.REGIME_AUTO,
                                        cap, ret_rows - 1, tokens, ks, epoch, p(ws), nbytes, st)
    assert rc == -1 and "return buffer" in C.last_error()
