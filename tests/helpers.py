"""Shared helpers for the test-suite: fixture loading and oracle parameter setup."""
import hashlib
import os

import numpy as np
import torch

from oracle import moe_oracle as orc
from shark_platform_b200 import synthetic as syn

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_golden(name):
    return np.load(os.path.join(GOLDEN, name))


def np_planes(planes):
    return {k: v.numpy() for k, v in planes.items()}


def dense_weight(kind, planes):
    """The dense tensor the reference's eager kernels see for a weight."""
    if kind == syn.DENSE:
        return planes["w"]
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
