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
    """The case as a Theta of this package's mirror types on `device`."""
    from shark_platform_b200 import types as T

    s = case.spec
    e, f, d = s.experts, s.ffn, s.hidden

    def weight(planes, shape):
        if s.kind == syn.DENSE:
            return T.DefaultPrimitiveTensor(data=planes["w"].to(device))
        p = {k: v.to(device) for k, v in planes.items()}
        if s.kind == syn.Q8_0:
            lay = T.BlockScaledLayout(shape, p["d"], p["qs"])
        else:
            lay = T.SuperBlockOffsetScaled_4_6_Layout(shape, **p)
        return T.PlanarQuantizedTensor(shape=shape, layout=lay)

    tree = {
        "ffn_gate_inp": {"weight": T.DefaultPrimitiveTensor(data=case.router_w.to(device))},
        "ffn_norm": {"weight": T.DefaultPrimitiveTensor(data=case.norm_w.to(device))},
        "ffn_gate_exps": {"weight": weight(case.gate, [e, f, d])},
        "ffn_up_exps": {"weight": weight(case.up, [e, f, d])},
        "ffn_down_exps": {"weight": weight(case.down, [e, d, f])},
    }
    if case.router_b is not None:
        tree["ffn_gate_inp"]["bias"] = T.DefaultPrimitiveTensor(data=case.router_b.to(device))
    if case.out_norm_w is not None:
        tree["layer_output_norm"] = {"weight": T.DefaultPrimitiveTensor(data=case.out_norm_w.to(device))}
    return T.Theta(tree)


def b200_block(case, regime="auto", device="cuda"):
    import torch.nn.functional as F
    from shark_platform_b200.moe import B200MoeBlock

    s = case.spec
    act = F.silu if s.activation == "silu" else F.gelu
    return B200MoeBlock(mirror_theta(case, device), s.experts, s.top_k, s.eps, act, regime=regime)


def device_input(case, device="cuda"):
    h = case.h.to(device)
    return h.to(torch.bfloat16) if case.spec.act_dtype == "bf16" else h
