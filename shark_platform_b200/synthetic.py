"""Seeded synthetic MoE layers in the reference's tensor formats.

Real Mixtral / Grok checkpoints cannot be fetched, so benchmarks and tests use
random layers with the shapes of the public model configs and the value
distributions the benchmark definition gives.  One CPU generator per case,
draws in a fixed order: activations, router weight, [router bias], then the
gate, up and down expert planes.  Plane names and shapes are those of
sharktank's BlockScaledLayout (types/layouts.py:194-299) and
SuperBlockOffsetScaled_4_6_Layout (types/layouts.py:360-530).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

Q8_0 = "Q8_0"
Q4_K = "Q4_K"
Q4_1 = "Q4_1"
DENSE = "DENSE"


@dataclass
class CaseSpec:
    name: str
    tokens: int
    hidden: int
    ffn: int
    experts: int = 8
    top_k: int = 2
    kind: str = Q8_0
    activation: str = "silu"
    act_dtype: str = "bf16"  # "bf16": activations rounded to bf16; "f32": kept
    out_norm: bool = False
    router_bias: Optional[str] = None  # None | "zipf" | "normal"
    norm_weight: str = "ones"  # "ones" | "perturbed"
    seed: int = 0
    eps: float = 1e-5


# The five benchmark configurations plus reduced shapes used by fixtures.
CASES = {
    "toy": CaseSpec("toy", 64, 512, 1024, kind=DENSE, act_dtype="f32", seed=0),
    "mixtral_q8": CaseSpec("mixtral_q8", 32, 4096, 14336, kind=Q8_0, seed=1),
    "mixtral_q4k": CaseSpec("mixtral_q4k", 32, 4096, 14336, kind=Q4_K, seed=2),
    "grok_q8": CaseSpec(
        "grok_q8", 8192, 6144, 32768, kind=Q8_0, activation="gelu", out_norm=True, seed=3
    ),
    "small_q8": CaseSpec(
        "small_q8", 40, 256, 512, kind=Q8_0, norm_weight="perturbed", seed=11
    ),
    "small_q4k": CaseSpec(
        "small_q4k", 33, 256, 512, kind=Q4_K, norm_weight="perturbed", seed=12
    ),
    "small_grok": CaseSpec(
        "small_grok", 17, 256, 768, kind=Q8_0, activation="gelu", out_norm=True,
        router_bias="zipf", norm_weight="perturbed", seed=13,
    ),
    "small_top4": CaseSpec(
        "small_top4", 29, 256, 512, kind=Q8_0, top_k=4, router_bias="normal",
        norm_weight="perturbed", seed=14,
    ),
    "small_q41": CaseSpec(
        "small_q41", 37, 256, 512, kind=Q4_1, norm_weight="perturbed", seed=16
    ),
    "small_dense": CaseSpec(
        "small_dense", 21, 256, 512, kind=DENSE, act_dtype="f32",
        norm_weight="perturbed", seed=15,
    ),
}


def zipf_bias(gen: torch.Generator, experts: int, s: float = 1.2) -> torch.Tensor:
    """Per-expert router bias from a Zipf(s) ranking: a random permutation gives
    expert e a rank r_e in 1..E and the bias is -s*ln(r_e) (prior odds r^-s)."""
    rank = torch.randperm(experts, generator=gen) + 1
    return (-s * torch.log(rank.to(torch.float32))).contiguous()


def q8_0_planes(gen, experts: int, n: int, k: int) -> dict:
    """int8 quants uniform in [-127,127], fp16 scales |N(0,1)|*0.002."""
    qs = torch.randint(-127, 128, (experts, n, k // 32, 32), generator=gen, dtype=torch.int8)
    d = (torch.randn(experts, n, k // 32, 1, generator=gen).abs() * 0.002).to(torch.float16)
    return {"d": d, "qs": qs}


def q4_k_planes(gen, experts: int, n: int, k: int) -> dict:
    """Uniform 4-bit quants, uniform 6-bit sub-scales and sub-mins in the
    planar hi/low planes; d = |N(0,1)|*2.5e-4 and dmin = |N(0,1)|*2e-3 keep the
    weights zero-mean and comparable in size to the Q8_0 case."""
    sup = k // 256
    qs = torch.randint(0, 256, (experts, n, sup, 8, 16), generator=gen, dtype=torch.uint8)

    def six_bit():
        v = torch.randint(0, 64, (experts, n, sup, 8), generator=gen, dtype=torch.uint8)
        lo, hi = v & 0xF, v >> 4
        low = lo[..., 0::2] | (lo[..., 1::2] << 4)
        high = hi[..., 0::4] | (hi[..., 1::4] << 2) | (hi[..., 2::4] << 4) | (hi[..., 3::4] << 6)
        return high.contiguous(), low.contiguous()

    sc_hi, sc_lo = six_bit()
    mn_hi, mn_lo = six_bit()
    d = (torch.randn(experts, n, sup, 1, generator=gen).abs() * 2.5e-4).to(torch.float16)
    dmin = (torch.randn(experts, n, sup, 1, generator=gen).abs() * 2.0e-3).to(torch.float16)
    return {
        "d": d, "dmin": dmin,
        "sb_scales_high": sc_hi, "sb_scales_low": sc_lo,
        "sb_mins_high": mn_hi, "sb_mins_low": mn_lo,
        "qs": qs,
    }


def q4_1_planes(gen, experts: int, n: int, k: int) -> dict:
    """GGUF Q4_1 as sharktank holds it (BlockScaledI4Layout, types/layouts.py:
    303-347): blocks of 32 unsigned 4-bit quants packed two per byte, fp16 scale
    d = |N(0,1)|*0.02 and fp16 offset m = -7.5*d*(1 + 0.1*N(0,1)) (roughly zero-mean
    weights of the size of the other layouts')."""
    qs = torch.randint(0, 256, (experts, n, k // 32, 16), generator=gen, dtype=torch.uint8)
    d32 = torch.randn(experts, n, k // 32, 1, generator=gen).abs() * 0.02
    m32 = -7.5 * d32 * (1.0 + 0.1 * torch.randn(experts, n, k // 32, 1, generator=gen))
    return {"d": d32.to(torch.float16), "m": m32.to(torch.float16), "qs": qs}


def dense_planes(gen, experts: int, n: int, k: int) -> dict:
    return {"w": torch.randn(experts, n, k, generator=gen) * 0.02}


_PLANE_MAKERS = {Q8_0: q8_0_planes, Q4_K: q4_k_planes, Q4_1: q4_1_planes, DENSE: dense_planes}


@dataclass
class Case:
    spec: CaseSpec
    h: torch.Tensor  # [1, T, d] fp32 holding values representable in act_dtype
    norm_w: torch.Tensor
    router_w: torch.Tensor
    router_b: Optional[torch.Tensor]
    out_norm_w: Optional[torch.Tensor]
    gate: dict
    up: dict
    down: dict


def make_case(spec: CaseSpec, tokens: Optional[int] = None, seed: Optional[int] = None) -> Case:
    T = spec.tokens if tokens is None else tokens
    d, f, e = spec.hidden, spec.ffn, spec.experts
    gen = torch.Generator(device="cpu").manual_seed(spec.seed if seed is None else seed)
    h = torch.randn(1, T, d, generator=gen)
    if spec.act_dtype == "bf16":
        h = h.to(torch.bfloat16).to(torch.float32)
    router_w = torch.randn(e, d, generator=gen) * 0.02
    router_b = None
    if spec.router_bias == "zipf":
        router_b = zipf_bias(gen, e)
    elif spec.router_bias == "normal":
        router_b = torch.randn(e, generator=gen) * 0.5
    if spec.norm_weight == "perturbed":
        norm_w = 1.0 + 0.1 * torch.randn(d, generator=gen)
    else:
        norm_w = torch.ones(d)
    out_norm_w = None
    if spec.out_norm:
        if spec.norm_weight == "perturbed":
            out_norm_w = 1.0 + 0.1 * torch.randn(d, generator=gen)
        else:
            out_norm_w = torch.ones(d)
    mk = _PLANE_MAKERS[spec.kind]
    gate = mk(gen, e, f, d)
    up = mk(gen, e, f, d)
    down = mk(gen, e, d, f)
    return Case(spec, h, norm_w, router_w, router_b, out_norm_w, gate, up, down)


def weight_bytes(kind: str, n: int, k: int) -> int:
    """Bytes one [n, k] expert matrix occupies in its quantized planes."""
    if kind == Q8_0:
        return n * k // 32 * 34
    if kind == Q4_K:
        return n * k // 256 * 144
    if kind == Q4_1:
        return n * k // 32 * 20
    return n * k * 2  # dense weights are held as fp16 on the device


def layer_flops(tokens: int, top_k: int, hidden: int, ffn: int) -> int:
    """Expert-GEMM flops of one layer call: three [ffn x hidden] products per
    (token, slot), 2 flops per multiply-add."""
    return tokens * top_k * 3 * 2 * ffn * hidden


def case_theta(case: Case, device="cuda"):
    """The case as a Theta of this package's tensor types on `device`, with the
    theta keys MoeBlock reads (layers/mixture_of_experts_block.py:31-62)."""
    from . import types as T

    s = case.spec
    e, f, d = s.experts, s.ffn, s.hidden

    def weight(planes, shape):
        if s.kind == DENSE:
            return T.DefaultPrimitiveTensor(data=planes["w"].to(device))
        p = {k: v.to(device) for k, v in planes.items()}
        if s.kind == Q8_0:
            lay = T.BlockScaledLayout(shape, p["d"], p["qs"])
        elif s.kind == Q4_1:
            lay = T.BlockScaledI4Layout(shape, p["d"], p["qs"], m=p["m"])
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


def case_block(case: Case, regime: str = "auto", device="cuda"):
    """B200MoeBlock for the case (weights uploaded to `device`)."""
    import torch.nn.functional as F

    from .moe import B200MoeBlock

    s = case.spec
    act = F.silu if s.activation == "silu" else F.gelu
    return B200MoeBlock(case_theta(case, device), s.experts, s.top_k, s.eps, act, regime=regime)


def case_input(case: Case, device="cuda") -> torch.Tensor:
    h = case.h.to(device)
    return h.to(torch.bfloat16) if case.spec.act_dtype == "bf16" else h


def make_case_on_device(spec: CaseSpec, device="cuda", seed: Optional[int] = None) -> Case:
    """Same distributions as `make_case` for layers too large to draw on the
    host (tens of gigabytes for the 32-layer stack, a minute per Mixtral layer):
    the expert planes come from the device generator, the small tensors
    (activations, router, bias) from the seeded CPU generator, so the routing of
    a seed is reproducible on any machine.  The expert values differ from the
    CPU-seeded case of the same seed."""
    T, d, f, e = spec.tokens, spec.hidden, spec.ffn, spec.experts
    sd = spec.seed if seed is None else seed
    cpu_gen = torch.Generator(device="cpu").manual_seed(sd)
    h = torch.randn(1, T, d, generator=cpu_gen)
    if spec.act_dtype == "bf16":
        h = h.to(torch.bfloat16).to(torch.float32)
    router_w = torch.randn(e, d, generator=cpu_gen) * 0.02
    router_b = None
    if spec.router_bias == "zipf":
        router_b = zipf_bias(cpu_gen, e)
    elif spec.router_bias == "normal":
        router_b = torch.randn(e, generator=cpu_gen) * 0.5
    h, router_w = h.to(device), router_w.to(device)
    router_b = None if router_b is None else router_b.to(device)
    norm_w = torch.ones(d, device=device)
    out_norm_w = torch.ones(d, device=device) if spec.out_norm else None
    gen = torch.Generator(device=device).manual_seed(sd)
    rn = lambda *shape: torch.randn(*shape, generator=gen, device=device)

    def q8(n, k):
        qs = torch.randint(-127, 128, (e, n, k // 32, 32), generator=gen, device=device, dtype=torch.int8)
        dd = (rn(e, n, k // 32, 1).abs() * 0.002).to(torch.float16)
        return {"d": dd, "qs": qs}

    def q4k(n, k):
        sup = k // 256
        u8 = lambda hi, *shape: torch.randint(0, hi, shape, generator=gen, device=device, dtype=torch.uint8)

        def six_bit():
            v = u8(64, e, n, sup, 8)
            lo, hi = v & 0xF, v >> 4
            low = lo[..., 0::2] | (lo[..., 1::2] << 4)
            high = hi[..., 0::4] | (hi[..., 1::4] << 2) | (hi[..., 2::4] << 4) | (hi[..., 3::4] << 6)
            return high.contiguous(), low.contiguous()

        sc_hi, sc_lo = six_bit()
        mn_hi, mn_lo = six_bit()
        return {
            "d": (rn(e, n, sup, 1).abs() * 2.5e-4).to(torch.float16),
            "dmin": (rn(e, n, sup, 1).abs() * 2.0e-3).to(torch.float16),
            "sb_scales_high": sc_hi, "sb_scales_low": sc_lo,
            "sb_mins_high": mn_hi, "sb_mins_low": mn_lo,
            "qs": u8(256, e, n, sup, 8, 16),
        }

    if spec.kind == Q8_0:
        planes = q8
    elif spec.kind == Q4_K:
        planes = q4k
    else:
        raise NotImplementedError("device-side generation covers the quantized layouts")
    return Case(spec, h, norm_w, router_w, router_b, out_norm_w, planes(f, d), planes(f, d), planes(d, f))


# ------------------------------------------------------------ attention block
@dataclass
class AttnCase:
    """Seeded inputs of one paged attention block call sequence (a batched
    prefill, then one decode step), shapes as in the reference's
    PagedLlamaAttentionBlock (layers/paged_llama_attention_block.py:26-85)."""

    hidden: int
    head_count: int
    head_count_kv: int
    head_dim: int
    stride: int
    blocks: int
    block_index: int
    softcap: Optional[float]
    h: torch.Tensor            # [bs, sl, d] prefill activations
    h_decode: torch.Tensor     # [bs, 1, d]
    seq_lens: torch.Tensor     # [bs]
    page_ids: torch.Tensor     # [bs, pages per sequence] (room for the decode step)
    pages: int
    norm_w: torch.Tensor
    wq: torch.Tensor
    wk: torch.Tensor
    wv: torch.Tensor
    wo: torch.Tensor
    eps: float = 1e-5
    rope_base: float = 10000.0


def make_attn_case(seed: int = 0, bs: int = 2, sl: int = 32, hidden: int = 256, head_count: int = 4,
                   head_count_kv: int = 2, head_dim: int = 64, stride: int = 16, blocks: int = 2,
                   block_index: int = 1, softcap: Optional[float] = None, seq_lens=None) -> AttnCase:
    assert hidden == head_count * head_dim and sl % stride == 0
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s, sc=1.0: torch.randn(*s, generator=g) * sc
    h, h_decode = rn(bs, sl, hidden), rn(bs, 1, hidden)
    if seq_lens is None:
        seq_lens = torch.tensor([sl - (7 * b) % sl for b in range(bs)])
    per_seq = sl // stride + 1
    pages = bs * per_seq + 3
    page_ids = torch.randperm(pages, generator=g)[: bs * per_seq].view(bs, per_seq)
    kv = head_count_kv * head_dim
    return AttnCase(hidden, head_count, head_count_kv, head_dim, stride, blocks, block_index, softcap,
                    h, h_decode, seq_lens, page_ids, pages,
                    1.0 + 0.1 * rn(hidden), rn(hidden, hidden, sc=0.06), rn(kv, hidden, sc=0.06),
                    rn(kv, hidden, sc=0.06), rn(hidden, hidden, sc=0.06))
