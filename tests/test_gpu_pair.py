"""CTA-pair tensor kernel (tcgen05, cta_group::2) against the single-CTA tensor
kernel.  Both accumulate every output element over k in the same order, so the
two expert products are compared bit for bit at an equal k split; the whole
layer is compared within rounding (the down projection's k split differs
between the regimes) and against the oracle."""
import ctypes

import pytest
import torch

from oracle import moe_oracle as orc
from shark_platform_b200 import synthetic as syn
from helpers import b200_block, device_input, oracle_params

pytestmark = pytest.mark.gpu


# hidden a multiple of 512 so that the down projection also runs on CTA pairs
PAIR_CASES = {
    "pair_q8": syn.CaseSpec("pair_q8", 300, 512, 1024, kind=syn.Q8_0, norm_weight="perturbed", seed=31),
    "pair_q4k": syn.CaseSpec("pair_q4k", 257, 512, 1024, kind=syn.Q4_K, norm_weight="perturbed", seed=32),
    "pair_grok": syn.CaseSpec("pair_grok", 777, 512, 768, kind=syn.Q8_0, activation="gelu", out_norm=True,
                              router_bias="zipf", norm_weight="perturbed", seed=33),
}
RUNS = [("pair_q8", 64), ("pair_q8", 300), ("pair_q4k", 257), ("pair_grok", 777), ("small_q8", 300)]


@pytest.mark.parametrize("name,tokens", RUNS)
def test_pair_products_equal_the_single_cta_products_bit_for_bit(name, tokens):
    from shark_platform_b200 import _cabi as C, moe

    spec = PAIR_CASES.get(name) or syn.CASES[name]
    case = syn.make_case(spec, tokens=tokens)
    layer = b200_block(case).layer
    gen = torch.Generator().manual_seed(tokens)
    experts = torch.stack([torch.randperm(spec.experts, generator=gen)[:spec.top_k] for _ in range(tokens)])
    plan = moe.route_plan(experts.cuda(), spec.experts)
    pairs = tokens * spec.top_k
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    xs = torch.randn(pairs, spec.hidden, generator=gen).to(torch.float16).cuda()
    act = C.ACT_SILU if spec.activation == "silu" else C.ACT_GELU
    outs = {}
    for regime in (C.REGIME_TENSOR, C.REGIME_TENSOR_PAIR):
        a = torch.zeros(pairs, spec.ffn, dtype=torch.float16, device="cuda")
        C.check(C.lib.b200moe_gate_up(p(xs), p(plan.seg_offsets), pairs, tokens, ctypes.byref(layer.gate.desc),
                                      ctypes.byref(layer.up.desc), act, regime, 0, p(a), st), "gate_up")
        d = torch.zeros(1, pairs, spec.hidden, dtype=torch.float32, device="cuda")
        C.check(C.lib.b200moe_down(p(a), p(plan.seg_offsets), pairs, tokens, ctypes.byref(layer.down.desc),
                                   regime, 1, p(d), st), "down")
        torch.cuda.synchronize()
        assert moe.device_status() == 0
        outs[regime] = (a, d)
    a1, d1 = outs[C.REGIME_TENSOR]
    a2, d2 = outs[C.REGIME_TENSOR_PAIR]
    diff_a = int((a1 != a2).sum())
    diff_d = int((d1 != d2).sum())
    print(f"{name} T={tokens}: gate/up elements that differ {diff_a}/{a1.numel()}, down {diff_d}/{d1.numel()}")
    assert diff_a == 0
    assert diff_d == 0


@pytest.mark.parametrize("name,tokens", RUNS)
def test_pair_regime_layer_matches_tensor_regime_and_oracle(name, tokens):
    from shark_platform_b200 import moe

    spec = PAIR_CASES.get(name) or syn.CASES[name]
    case = syn.make_case(spec, tokens=tokens)
    h = device_input(case)
    want = b200_block(case, regime="tensor")(h)
    blk = b200_block(case, regime="tensor_pair")
    got = blk(h)
    got2 = blk(h)
    torch.cuda.synchronize()
    assert moe.device_status() == 0
    assert torch.equal(got, got2), "two runs differ: a race"
    assert orc.rel_l2(got.float().cpu(), want.float().cpu()) < 5e-3  # both rounded to bf16
    ref, _ = orc.moe_block(case.h, oracle_params(case), form="per_expert")
    assert orc.rel_l2(got.float().cpu(), ref) < 2e-2
