"""CTA-pair tensor kernel against the single-CTA tensor kernel (bit-equal:
both accumulate every output element over k in the same order)."""
import pytest
import torch

from shark_platform_b200 import synthetic as syn
from helpers import b200_block, device_input

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,tokens", [("small_q8", 64), ("small_q8", 300), ("small_q4k", 257),
                                         ("small_grok", 777)])
def test_pair_regime_equals_tensor_regime(name, tokens):
    from shark_platform_b200 import moe

    case = syn.make_case(syn.CASES[name], tokens=tokens)
    h = device_input(case)
    want = b200_block(case, regime="tensor")(h)
    got = b200_block(case, regime="tensor_pair")(h)
    torch.cuda.synchronize()
    assert moe.device_status() == 0
    assert torch.equal(got, want)
