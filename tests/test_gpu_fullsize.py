"""Parity at the benchmark's own shapes: the Mixtral-8x7B layer with Q8_0 and
Q4_K experts and the Grok-1 layer, at the token counts the benchmark times.

The layer is drawn on the device (seeded; the routing inputs come from the CPU
generator), the CUDA path runs through the C ABI, and the oracle evaluates
norm + router for every token and the expert FFN for a seeded token sample,
one dequantised expert at a time.  Checked per run: the oracle's top-k margin
(> 1e-5, so that index equality is well defined), expert indices of ALL tokens,
the permutation, output relative L2 on the sample, the device status word and
run-twice bit-equality.
"""
import dataclasses

import pytest
import torch

from oracle import moe_oracle as orc
from shark_platform_b200 import synthetic as syn
from helpers import ExpertWeightStream, sampled_oracle

pytestmark = pytest.mark.gpu

REL_L2_TOL = 2e-2
MARGIN = 1e-5
SAMPLE = 512

# seeds chosen so that the oracle's top-k margin over all tokens exceeds MARGIN
FULL = {
    "mixtral_q8": (syn.CaseSpec("mixtral_q8_full", 4096, 4096, 14336, kind=syn.Q8_0, seed=102),
                   [1, 32, 128, 4096]),
    "mixtral_q4k": (syn.CaseSpec("mixtral_q4k_full", 2048, 4096, 14336, kind=syn.Q4_K, seed=202),
                    [32, 2048]),
    "grok_q8": (syn.CaseSpec("grok_q8_full", 8192, 6144, 32768, kind=syn.Q8_0, activation="gelu",
                             out_norm=True, seed=3), [8192]),
}
RUNS = [(name, t) for name, (_, ts) in FULL.items() for t in ts]
_results = {}


def _evaluate(name):
    """All runs of one layer; the layer and its dequantised experts are dropped
    before the next layer is drawn."""
    from shark_platform_b200 import moe as M

    spec, runs = FULL[name]
    case = syn.make_case_on_device(spec, "cuda")
    blk = syn.case_block(case, "auto", "cuda")
    stream = ExpertWeightStream(case, keep=len(runs) > 1)
    out = {}
    for tokens in runs:
        h = syn.case_input(dataclasses.replace(case, h=case.h[:, :tokens].contiguous()), "cuda")
        y, experts, gates = blk.layer.forward(h, want_routing=True)
        y2 = blk.layer.forward(h)
        status = M.device_status()
        plan = M.route_plan(experts, spec.experts)
        if tokens <= SAMPLE:
            sel = torch.arange(tokens)
        else:
            gen = torch.Generator().manual_seed(tokens)
            first = experts[:, 0].cpu()
            e0 = int(torch.bincount(first.to(torch.int64), minlength=spec.experts).argmax())
            whole_segment = torch.nonzero((experts.cpu() == e0).any(dim=1)).reshape(-1)
            if name == "grok_q8":  # 2.4 GFLOP per token on the host: the random sample only
                whole_segment = whole_segment[:0]
            sel = torch.unique(torch.cat([torch.randperm(tokens, generator=gen)[:SAMPLE], whole_segment]))
        want, mid = sampled_oracle(case, tokens, sel, stream)
        counts, seg, perm, inv = orc.route_plan(mid["experts"], spec.experts)
        out[tokens] = dict(
            margin=orc.topk_margin(mid["prob"], spec.top_k),
            experts_equal=torch.equal(experts.cpu().to(torch.int64), mid["experts"]),
            gate_err=float((gates.cpu() - mid["gate"]).abs().max()),
            plan_equal=(plan.seg_offsets.cpu().tolist() == seg.tolist()
                        and plan.perm.cpu().tolist() == perm.tolist()
                        and plan.inv.cpu().tolist() == inv.tolist()),
            rel_l2=orc.rel_l2(y.reshape(tokens, -1)[sel.cuda()].float().cpu(), want),
            sampled=int(sel.numel()), status=status, twice_equal=torch.equal(y, y2),
            finite=bool(torch.isfinite(y.float()).all()),
        )
    del blk, case, stream
    torch.cuda.empty_cache()
    return out


@pytest.mark.parametrize("name,tokens", RUNS)
def test_full_size_layer_matches_oracle(name, tokens):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    if name not in _results:
        _results.clear()  # one layer's results at a time
        _results[name] = _evaluate(name)
    r = _results[name][tokens]
    print(f"{name} T={tokens}: {r}")
    assert r["margin"] > MARGIN, "seed has a near-tie in the oracle's top-k; pick another"
    assert r["experts_equal"], "expert indices differ from the oracle"
    assert r["plan_equal"], "permutation differs from the stable sort"
    assert r["gate_err"] < 2e-6
    assert r["status"] == 0
    assert r["finite"]
    assert r["twice_equal"], "two runs differ: a race"
    assert r["rel_l2"] < REL_L2_TOL
