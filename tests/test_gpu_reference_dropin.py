"""The real drop-in: sharktank's OWN `MoeBlock` / `PreGatherFFNMOE` (the
unmodified reference, imported from $SHARKTANK_SRC or baseline/_ref) over
sharktank's own `PlanarQuantizedTensor`s on CUDA, after `plugin.register()`.

The reference cannot evaluate these layers itself: `weights[experts,:,:]` on a
Q8_0 / Q4_K tensor has no implementation there (ops/default_impls.py:204-218
covers Q4_1 only).  With the plugin registered, its forward runs unchanged and
the three expert einsums land in this library.  Values are checked against the
oracle, dispatch against the reference registry's own bookkeeping
(ops/_registry.py:36-55)."""
import pytest
import torch
import torch.nn.functional as F

from oracle import moe_oracle as orc
from shark_platform_b200 import synthetic as syn
from helpers import import_sharktank, oracle_params, reference_path

pytestmark = [
    pytest.mark.gpu,
    pytest.mark.skipif(reference_path() is None,
                       reason="sharktank not available ($SHARKTANK_SRC or baseline/_ref)"),
]

REL_L2_TOL = 2e-2


def _reference_theta(case, dev="cuda"):
    from sharktank.types import DefaultPrimitiveTensor, PlanarQuantizedTensor, Theta
    from sharktank.types.layouts import BlockScaledLayout, SuperBlockOffsetScaled_4_6_Layout

    s = case.spec
    e, f, d = s.experts, s.ffn, s.hidden

    def weight(planes, shape):
        p = {k: v.to(dev) for k, v in planes.items()}
        if s.kind == syn.Q8_0:
            lay = BlockScaledLayout(shape, p["d"], p["qs"])
        else:
            lay = SuperBlockOffsetScaled_4_6_Layout(shape, **p)
        return PlanarQuantizedTensor(shape=shape, layout=lay)

    tree = {
        "ffn_gate_inp": {"weight": DefaultPrimitiveTensor(data=case.router_w.to(dev))},
        "ffn_norm": {"weight": DefaultPrimitiveTensor(data=case.norm_w.to(dev))},
        "ffn_gate_exps": {"weight": weight(case.gate, [e, f, d])},
        "ffn_up_exps": {"weight": weight(case.up, [e, f, d])},
        "ffn_down_exps": {"weight": weight(case.down, [e, d, f])},
    }
    if case.router_b is not None:
        tree["ffn_gate_inp"]["bias"] = DefaultPrimitiveTensor(data=case.router_b.to(dev))
    if case.out_norm_w is not None:
        tree["layer_output_norm"] = {"weight": DefaultPrimitiveTensor(data=case.out_norm_w.to(dev))}
    return Theta(tree)


@pytest.mark.parametrize("name", ["small_q8", "small_q4k", "small_grok"])
def test_reference_moeblock_runs_on_quantized_experts_through_the_plugin(name):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    import_sharktank()
    from sharktank.layers.mixture_of_experts_block import MoeBlock
    from sharktank.ops import _registry as st_registry

    from shark_platform_b200 import moe, plugin

    plugin.register()
    case = syn.make_case(syn.CASES[name])
    s = case.spec
    act = F.silu if s.activation == "silu" else F.gelu
    block = MoeBlock(_reference_theta(case), s.experts, s.top_k, s.eps, moe_activation=act)
    p = oracle_params(case)

    # the reference's own forward, twice with different activations: the second
    # call routes differently through a fresh top-k tensor of the same shape
    gen = torch.Generator().manual_seed(99)
    for h in (case.h, torch.randn(case.h.shape, generator=gen)):
        want, mid = orc.moe_block(h, p, form="pregather")
        assert orc.topk_margin(mid["prob"], s.top_k) > 1e-6
        y = block(h.cuda())
        assert moe.device_status() == 0
        assert orc.rel_l2(y.cpu(), want) < REL_L2_TOL
        assert orc.rel_l2(y.cpu() - h, want - h) < REL_L2_TOL  # the MoE term alone

    # dispatch, as the reference's registry records it
    xn = orc.rms_norm(case.h, p.norm_w, p.eps).view(-1, s.hidden)
    gate, idx, _ = orc.router(xn, p.router_w, p.router_b, p.top_k)
    st_registry._test_enable_last_op_dispatch(True)
    try:
        gathered = block.experts.ffn_gate[idx.cuda(), :, :]
        assert st_registry._test_get_last_op_dispatch() is moe.get_index_quantized
        assert isinstance(gathered, moe.GatheredExperts)
        out = block.experts.pre_matmul_gather(xn.cuda(), block.experts.ffn_up, idx.cuda())
        assert st_registry._test_get_last_op_dispatch() is moe.einsum_2args_gathered
    finally:
        st_registry._test_enable_last_op_dispatch(False)
    want_up = torch.einsum("mk,menk->men", xn, p.w_up[idx].float())
    assert orc.rel_l2(out.cpu(), want_up) < 5e-3

    # PreGatherFFNMOE.forward on its own
    got = block.experts(xn.cuda(), idx.cuda(), gate.cuda())
    want = orc.experts_pregather(xn, idx, gate, p.w_gate, p.w_up, p.w_down, act)
    assert orc.rel_l2(got.cpu(), want) < REL_L2_TOL
    assert moe.device_status() == 0


def test_reference_pregather_on_expert_sharded_split_tensor():
    """sharktank's own `SplitPrimitiveTensor(ts=[PlanarQuantizedTensor...],
    shard_dim=0)` (types/tensors.py:957-1096) as expert weights of its own
    PreGatherFFNMOE.  The reference can neither index nor multiply it; after
    `plugin.register()` each shard serves the pairs routed to its experts."""
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    import_sharktank()
    from sharktank.layers.ffn_moe_block import PreGatherFFNMOE
    from sharktank.types import PlanarQuantizedTensor, SplitPrimitiveTensor, Theta

    from shark_platform_b200 import moe, plugin

    plugin.register()
    case = syn.make_case(syn.CASES["small_q8"])
    s = case.spec
    whole = _reference_theta(case)

    def shard(key):
        full = whole.tensor(key, "weight")
        lay = full.unpack()
        parts = []
        for e0, e1 in ((0, 3), (3, 8)):
            shape = [e1 - e0] + [int(v) for v in full.shape[1:]]
            planes = {k: v[e0:e1].contiguous() for k, v in lay.planes.items()}
            parts.append(PlanarQuantizedTensor(shape=shape, layout=type(lay)(shape, **planes)))
        return SplitPrimitiveTensor(ts=parts, shard_dim=0)

    theta = Theta({k: {"weight": shard(k)} for k in ("ffn_gate_exps", "ffn_up_exps", "ffn_down_exps")})
    experts_layer = PreGatherFFNMOE(theta, activation=F.silu)
    p = oracle_params(case)
    xn = orc.rms_norm(case.h, p.norm_w, p.eps).view(-1, s.hidden)
    gate, idx, _ = orc.router(xn, p.router_w, p.router_b, p.top_k)
    got = experts_layer(xn.cuda(), idx.cuda(), gate.cuda())
    want = orc.experts_pregather(xn, idx, gate, p.w_gate, p.w_up, p.w_down, F.silu)
    assert orc.rel_l2(got.cpu(), want) < REL_L2_TOL
    assert moe.device_status() == 0
