"""Shared helpers for the test-suite: fixture loading and oracle parameter setup."""
import hashlib
import os

import numpy as np
import torch

from oracle import moe_oracle as orc
from shark_platform_b200 import synthetic as syn

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def reference_path():
    """Directory that holds the `sharktank` package, or None: $SHARKTANK_SRC (a
    source checkout) first, then the offline install `baseline/_ref` of this
    repository (`pip install --no-deps --target baseline/_ref <checkout>/sharktank`)."""
    for cand in (os.environ.get("SHARKTANK_SRC", ""), os.path.join(ROOT, "baseline", "_ref")):
        if cand and os.path.isdir(os.path.join(cand, "sharktank")):
            return cand
    return None


def import_sharktank():
    """Imports the unmodified reference with the iree stand-in (test scaffolding:
    iree-turbine only supplies tracing traits and export machinery on this path)."""
    import sys

    path = reference_path()
    assert path is not None, "sharktank is not available"
    for p in (GOLDEN, path):
        if p not in sys.path:
            sys.path.insert(0, p)
    import iree_stub

    iree_stub.install()
    import sharktank

    return sharktank


def load_golden(name):
    return np.load(os.path.join(GOLDEN, name))


def np_planes(planes):
    return {k: v.numpy() for k, v in planes.items()}


def dense_weight(kind, planes):
    """The dense tensor the reference's eager kernels see for a weight."""
    if kind == syn.DENSE:
        return planes["w"]
    if planes["qs"].numel() > (1 << 26):
        # full-size layers: the multi-threaded restatement (bit-equal to the numpy
        # one, tests/test_oracle.py), seconds instead of a minute
        return orc.dequant_torch(kind, planes)
    return torch.from_numpy(orc.dequant(kind, np_planes(planes)))


def oracle_params(case):
    s = case.spec
    return orc.MoeParams(
        norm_w=case.norm_w,
        router_w=case.router_w,
        router_b=case.router_b,
        out_norm_w=case.out_norm_w,
        w_gate=dense_weight(s.kind, case.gate),
        w_up=dense_weight(s.kind, case.up),
        w_down=dense_weight(s.kind, case.down),
        top_k=s.top_k,
        eps=s.eps,
        activation=s.activation,
    )


def case_digest(case) -> str:
    m = hashlib.sha256()
    tensors = [case.h, case.norm_w, case.router_w]
    if case.router_b is not None:
        tensors.append(case.router_b)
    if case.out_norm_w is not None:
        tensors.append(case.out_norm_w)
    for planes in (case.gate, case.up, case.down):
        tensors += [planes[k] for k in sorted(planes)]
    for t in tensors:
        m.update(t.contiguous().numpy().tobytes())
    return m.hexdigest()


# ---------------------------------------------------------------- GPU side
def mirror_theta(case, device="cuda"):
    return syn.case_theta(case, device)


def b200_block(case, regime="auto", device="cuda"):
    return syn.case_block(case, regime, device)


def device_input(case, device="cuda"):
    return syn.case_input(case, device)


# ------------------------------------------- full-size layers (GPU + oracle)
class ExpertWeightStream:
    """Dense fp16 weights of one expert at a time for `orc.moe_block_sampled`:
    the expert's planes are copied from the device and dequantised with the
    oracle's torch restatement.  `keep=True` holds the dequantised experts for
    reuse by a later evaluation of the same layer (about 2.8 GB for a Mixtral
    layer); otherwise only one expert is resident."""

    def __init__(self, case, keep=False):
        self.case, self.keep, self.cache = case, keep, {}

    def __call__(self, e):
        if e in self.cache:
            return self.cache[e]
        kind = self.case.spec.kind
        out = tuple(
            orc.dequant_torch(kind, {k: v[e].cpu() for k, v in planes.items()})
            for planes in (self.case.gate, self.case.up, self.case.down))
        if self.keep:
            self.cache[e] = out
        return out


def sampled_oracle(case, tokens, token_index, stream):
    """Oracle rows for `token_index` of the layer applied to the first `tokens`
    tokens of the case, plus the intermediates (indices, probabilities) of all
    of them."""
    s = case.spec
    cpu = lambda t: None if t is None else t.cpu()
    p = orc.MoeParams(norm_w=cpu(case.norm_w), router_w=cpu(case.router_w), router_b=cpu(case.router_b),
                      out_norm_w=cpu(case.out_norm_w), w_gate=None, w_up=None, w_down=None,
                      top_k=s.top_k, eps=s.eps, activation=s.activation)
    h = case.h[:, :tokens].cpu()
    return orc.moe_block_sampled(h, p, stream, token_index)
