"""CTA-pair tensor kernel against the single-CTA tensor kernel (bit-equal:
both accumulate every output element over k in the same order)."""
import pytest
import torch

from shark_platform_b200 import synthetic as syn
from helpers import b200_block, device_input

pytestmark = pytest.mark.gpu


# hidden a multiple of 512 so that the down projection also runs on CTA pairs
PAIR_CASES = {
    "pair_q8": syn.CaseSpec("pair_q8", 300, 512, 1024, kind=syn.Q8_0, norm_weight="perturbed", seed=31),
    "pair_q4k": syn.CaseSpec("pair_q4k", 257, 512, 1024, kind=syn.Q4_K, norm_weight="perturbed", seed=32),
    "pair_grok": syn.CaseSpec("pair_grok", 777, 512, 768, kind=syn.Q8_0, activation="gelu", out_norm=True,
                              router_bias="zipf", norm_weight="perturbed", seed=33),
}


@pytest.mark.parametrize("name,tokens", [("pair_q8", 64), ("pair_q8", 300), ("pair_q4k", 257),
                                         ("pair_grok", 777), ("small_q8", 300)])
def test_pair_regime_equals_tensor_regime(name, tokens):
    from shark_platform_b200 import moe

    spec = PAIR_CASES.get(name) or syn.CASES[name]
    case = syn.make_case(spec, tokens=tokens)
    h = device_input(case)
    want = b200_block(case, regime="tensor")(h)
    got = b200_block(case, regime="tensor_pair")(h)
    torch.cuda.synchronize()
    assert moe.device_status() == 0
    assert torch.equal(got, want)
