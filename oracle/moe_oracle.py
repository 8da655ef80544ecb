"""CPU oracle for the mixture-of-experts FFN hot path.  TEST INFRASTRUCTURE ONLY.

This file restates, on the CPU, the algorithm of sharktank's torch-eager MoE
layer and of the GGUF block formats it consumes.  It is the checker for the
CUDA path: only the test-suite, the smoke entry and the CPU-baseline leg of the
benchmark may import it.  The product package never does.

Parity status: PINNED.  Every function below is checked (a) against fixtures
under tests/golden/ that were produced by importing the reference itself
(tests/golden/make_golden.py), (b) against the reference's own known-answer
vectors for the bit-unpack helpers, and (c) for the block formats against the
independent `gguf.quants.dequantize` implementation.

torch's CPU operators are used for softmax / top-k / matmul because the
reference's arithmetic *is* those operators; numpy is used for the byte-level
format work.  Each function cites the reference file:line it follows (paths
relative to the sharktank project root).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Optional

import numpy as np
import torch
import torch.nn.functional as F

Q8_0 = "Q8_0"
Q4_K = "Q4_K"
Q4_1 = "Q4_1"
DENSE = "DENSE"

# --------------------------------------------------------------------------
# Bit-field helpers (sharktank/types/layout_utils.py:20-113)
# --------------------------------------------------------------------------


def _u8(a) -> np.ndarray:
    a = np.asarray(a)
    if a.dtype == np.int8:
        a = a.view(np.uint8)
    assert a.dtype == np.uint8, a.dtype
    return a


def deinterleave_i4(block) -> np.ndarray:
    """layout_utils.py:20-44 (`linearize_interleaved_i4_block`).

    Input byte i holds element i in its low nibble and element i+n in its high
    nibble (n = bytes per block).  Output is the linear packing: byte j holds
    element 2j (low nibble) and 2j+1 (high nibble)."""
    b = _u8(block)
    lo, hi = b & 0xF, b >> 4
    first = lo[..., 0::2] | (lo[..., 1::2] << 4)
    second = hi[..., 0::2] | (hi[..., 1::2] << 4)
    return np.concatenate([first, second], axis=-1)


def interleave_i4(block) -> np.ndarray:
    """layout_utils.py:47-64 (`interleave_linear_i4_block`), inverse of the above."""
    b = _u8(block)
    n = b.shape[-1] // 2
    a, c = b[..., :n], b[..., n:]
    out = np.empty(b.shape, dtype=np.uint8)
    out[..., 0::2] = (a & 0xF) | ((c & 0xF) << 4)
    out[..., 1::2] = (a >> 4) | ((c >> 4) << 4)
    return out


def unpack_i4(packed, signed: bool = False) -> np.ndarray:
    """layout_utils.py:67-86 (`promote_linear_i4_block_to_i8`): two values per
    byte, low nibble first."""
    b = _u8(packed)
    out = np.empty(b.shape[:-1] + (b.shape[-1] * 2,), dtype=np.uint8)
    out[..., 0::2] = b & 0xF
    out[..., 1::2] = b >> 4
    if signed:
        out = ((out.astype(np.int16) ^ 8) - 8).astype(np.int8)
    return out


def unpack_i2(packed) -> np.ndarray:
    """layout_utils.py:89-101 (`promote_linear_i2_block_to_i8`): four 2-bit
    fields per byte, least-significant field first."""
    b = _u8(packed)
    out = np.empty(b.shape[:-1] + (b.shape[-1] * 4,), dtype=np.uint8)
    for f in range(4):
        out[..., f::4] = (b >> (2 * f)) & 3
    return out


def unpack_i6(high2, low4) -> np.ndarray:
    """layout_utils.py:104-113 (`promote_linear_i6_block_to_i8`): value =
    low nibble | (2-bit high field << 4)."""
    lo = unpack_i4(low4)
    hi = unpack_i2(high2)
    assert lo.shape == hi.shape, (lo.shape, hi.shape)
    return lo | (hi << 4)


# --------------------------------------------------------------------------
# Packed GGUF blocks -> planar planes (sharktank/types/gguf_interop/layouts.py)
# --------------------------------------------------------------------------


def q8_0_unpack(raw, shape) -> dict:
    """gguf_interop/layouts.py:51-60.  34-byte blocks: fp16 scale then 32 int8.
    Returns contiguous planes d [..., K/32, 1] fp16 and qs [..., K/32, 32] int8."""
    raw = _u8(raw).reshape(-1, 34)
    lead = tuple(shape[:-1])
    nblk = shape[-1] // 32
    d = raw[:, 0:2].copy().view(np.float16).reshape(lead + (nblk, 1))
    qs = raw[:, 2:].copy().view(np.int8).reshape(lead + (nblk, 32))
    return {"d": d, "qs": qs}


def q4_k_scale_min_fields(s12) -> tuple[np.ndarray, np.ndarray]:
    """The eight 6-bit sub-scales and sub-mins of one Q4_K super-block from its
    12 packed bytes (ggml's get_scale_min_k4, restated; this is what
    gguf_interop/layouts.py:163-217 re-packs into hi/low planes)."""
    s = _u8(s12).astype(np.uint8)
    sc = np.empty(s.shape[:-1] + (8,), dtype=np.uint8)
    mn = np.empty_like(sc)
    for b in range(4):
        sc[..., b] = s[..., b] & 63
        mn[..., b] = s[..., b + 4] & 63
        sc[..., b + 4] = (s[..., b + 8] & 0xF) | ((s[..., b] >> 6) << 4)
        mn[..., b + 4] = (s[..., b + 8] >> 4) | ((s[..., b + 4] >> 6) << 4)
    return sc, mn


def pack_i6_planes(v6) -> tuple[np.ndarray, np.ndarray]:
    """Eight 6-bit values -> (high [.., 2], low [.., 4]) planes in the planar
    convention of SuperBlockOffsetScaled_4_6_Layout (types/layouts.py:447-470):
    low byte j = low nibbles of fields 2j (bits 0-3) and 2j+1 (bits 4-7); high
    byte j = top two bits of fields 4j..4j+3 at bit positions 0, 2, 4, 6."""
    v = np.asarray(v6, dtype=np.uint8)
    lo4 = v & 0xF
    hi2 = v >> 4
    low = lo4[..., 0::2] | (lo4[..., 1::2] << 4)
    high = (
        hi2[..., 0::4]
        | (hi2[..., 1::4] << 2)
        | (hi2[..., 2::4] << 4)
        | (hi2[..., 3::4] << 6)
    )
    return high.astype(np.uint8), low.astype(np.uint8)


def q4_k_unpack(raw, shape) -> dict:
    """gguf_interop/layouts.py:112-153.  144-byte super-blocks of 256 weights:
    fp16 d, fp16 dmin, 12 bytes of 6-bit scales/mins, 128 bytes of nibbles.
    In the file, byte i of 32-byte group g holds quant i of sub-block 2g (low
    nibble) and quant i of sub-block 2g+1 (high nibble); the planar `qs`
    [.., SUP, 8, 16] holds sub-block b linearly (byte i = quants 2i, 2i+1)."""
    raw = _u8(raw).reshape(-1, 144)
    lead = tuple(shape[:-1])
    sup = shape[-1] // 256
    d = raw[:, 0:2].copy().view(np.float16).reshape(lead + (sup, 1))
    dmin = raw[:, 2:4].copy().view(np.float16).reshape(lead + (sup, 1))
    sc, mn = q4_k_scale_min_fields(raw[:, 4:16])
    sc_hi, sc_lo = pack_i6_planes(sc)
    mn_hi, mn_lo = pack_i6_planes(mn)
    groups = raw[:, 16:].reshape(-1, 4, 32)
    qs = deinterleave_i4(groups).reshape(-1, 8, 16)
    return {
        "d": d,
        "dmin": dmin,
        "sb_scales_high": sc_hi.reshape(lead + (sup, 2)),
        "sb_scales_low": sc_lo.reshape(lead + (sup, 4)),
        "sb_mins_high": mn_hi.reshape(lead + (sup, 2)),
        "sb_mins_low": mn_lo.reshape(lead + (sup, 4)),
        "qs": qs.reshape(lead + (sup, 8, 16)),
    }


# --------------------------------------------------------------------------
# Dequantisation (sharktank/types/layouts.py)
# --------------------------------------------------------------------------


def q8_0_dequant(planes: dict, dtype=np.float16) -> np.ndarray:
    """BlockScaledLayout.dequant, types/layouts.py:274-290:
    `d.to(dtype) * qs.to(dtype)`; the default dtype is d's (fp16), so the
    default result is the fp16 rounding of the exact product."""
    d = np.asarray(planes["d"])
    qs = np.asarray(planes["qs"])
    prod = d.astype(np.float32) * qs.astype(np.float32)  # exact: 11 x 8 bits
    out = prod.astype(dtype)
    return out.reshape(out.shape[:-2] + (out.shape[-2] * out.shape[-1],))


def q4_1_dequant(planes: dict) -> np.ndarray:
    """BlockScaledI4Layout (types/layouts.py:303-347, unsigned, with offsets `m`:
    GGUF Q4_1): `qs` holds two 4-bit values per byte, low nibble first
    (layout_utils.py:67-86), and dequant is BlockScaledLayout's
    `d * qs + m` evaluated in fp16 (types/layouts.py:277-290): one rounding after
    the product, one after the sum."""
    d = np.asarray(planes["d"]).astype(np.float32)
    m = np.asarray(planes["m"]).astype(np.float32)
    q = unpack_i4(planes["qs"]).astype(np.float32)  # [..., K/32, 32]
    h = lambda a: a.astype(np.float16).astype(np.float32)
    w = h(h(d * q) + m).astype(np.float16)
    return w.reshape(w.shape[:-2] + (w.shape[-2] * w.shape[-1],))


def q4_k_fields(planes: dict) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
    sc = unpack_i6(planes["sb_scales_high"], planes["sb_scales_low"])
    mn = unpack_i6(planes["sb_mins_high"], planes["sb_mins_low"])
    q = unpack_i4(planes["qs"])
    return sc, mn, q


def q4_k_dequant(planes: dict) -> np.ndarray:
    """SuperBlockOffsetScaled_4_6_Layout.dequant, types/layouts.py:505-517.
    The reference evaluates `(d*sc)*q - dmin*m` entirely in fp16 (its dtype
    argument is ignored), i.e. with one rounding after each of the four
    operations.  Each step below is computed exactly in fp32 and rounded once,
    which is what IEEE fp16 arithmetic does."""
    sc, mn, q = q4_k_fields(planes)
    d = np.asarray(planes["d"]).astype(np.float32)
    dmin = np.asarray(planes["dmin"]).astype(np.float32)
    h = lambda a: a.astype(np.float16).astype(np.float32)
    t1 = h(d * sc.astype(np.float32))[..., None]  # [.., SUP, 8, 1]
    t2 = h(dmin * mn.astype(np.float32))[..., None]
    w = h(h(t1 * q.astype(np.float32)) - t2).astype(np.float16)
    return w.reshape(w.shape[:-3] + (w.shape[-3] * 256,))


def q4_k_dequant_f32(planes: dict) -> np.ndarray:
    """The same formula in fp32 without intermediate rounding; equals ggml's
    own Q4_K dequantisation (used for the independent `gguf.quants` pin)."""
    sc, mn, q = q4_k_fields(planes)
    d = np.asarray(planes["d"]).astype(np.float32)
    dmin = np.asarray(planes["dmin"]).astype(np.float32)
    w = (d * sc)[..., None] * q.astype(np.float32) - (dmin * mn)[..., None]
    return w.reshape(w.shape[:-3] + (w.shape[-3] * 256,))


def dequant(kind: str, planes: dict) -> np.ndarray:
    """What `unbox_tensor` hands to the eager kernels for a quantized weight
    (types/tensors.py:1276-1284): `layout.dequant()` with no dtype, fp16."""
    if kind == Q8_0:
        return q8_0_dequant(planes)
    if kind == Q4_K:
        return q4_k_dequant(planes)
    if kind == Q4_1:
        return q4_1_dequant(planes)
    raise ValueError(kind)


# The same two dequantisations with torch's multi-threaded CPU operators, for
# full-size layers (hundreds of millions of weights per matrix, where the numpy
# versions above take minutes).  tests/test_oracle.py checks them bit for bit
# against the numpy versions, which are the ones pinned to the reference.


def q8_0_dequant_torch(planes: dict) -> torch.Tensor:
    """BlockScaledLayout.dequant (types/layouts.py:274-290) on torch tensors:
    fp16(d * q), the product formed exactly in fp32 and rounded once."""
    d, qs = planes["d"], planes["qs"]
    out = (d.to(torch.float32) * qs.to(torch.float32)).to(torch.float16)
    return out.reshape(*out.shape[:-2], out.shape[-2] * out.shape[-1])


def _unpack_i4_torch(b: torch.Tensor) -> torch.Tensor:
    b = b.view(torch.uint8)
    return torch.stack([b & 0xF, b >> 4], dim=-1).reshape(*b.shape[:-1], b.shape[-1] * 2)


def _unpack_i6_torch(high2: torch.Tensor, low4: torch.Tensor) -> torch.Tensor:
    lo = _unpack_i4_torch(low4)
    h = high2.view(torch.uint8)
    hi = torch.stack([(h >> (2 * f)) & 3 for f in range(4)], dim=-1).reshape(*h.shape[:-1], h.shape[-1] * 4)
    return lo | (hi << 4)


def q4_k_dequant_torch(planes: dict) -> torch.Tensor:
    """SuperBlockOffsetScaled_4_6_Layout.dequant (types/layouts.py:505-517) on
    torch tensors, one fp16 rounding after each of the four operations."""
    sc = _unpack_i6_torch(planes["sb_scales_high"], planes["sb_scales_low"]).to(torch.float32)
    mn = _unpack_i6_torch(planes["sb_mins_high"], planes["sb_mins_low"]).to(torch.float32)
    q = _unpack_i4_torch(planes["qs"]).to(torch.float32)  # [.., SUP, 8, 32]
    h = lambda a: a.to(torch.float16).to(torch.float32)
    t1 = h(planes["d"].to(torch.float32) * sc).unsqueeze(-1)
    t2 = h(planes["dmin"].to(torch.float32) * mn).unsqueeze(-1)
    w = (h(t1 * q) - t2).to(torch.float16)
    return w.reshape(*w.shape[:-3], w.shape[-3] * 256)


def dequant_torch(kind: str, planes: dict) -> torch.Tensor:
    if kind == Q8_0:
        return q8_0_dequant_torch(planes)
    if kind == Q4_K:
        return q4_k_dequant_torch(planes)
    raise ValueError(kind)


# --------------------------------------------------------------------------
# Layer stages (sharktank/layers/mixture_of_experts_block.py,
# layers/ffn_moe_block.py, ops/default_impls.py)
# --------------------------------------------------------------------------


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNormLayer.forward (layers/norm.py:34-41) over rms_norm_default
    (ops/default_impls.py:402-408): fp32 compute, weight applied after a cast
    to the weight dtype, result cast back to the input dtype."""
    xf = x.to(torch.float32)
    var = xf.pow(2).mean(-1, keepdim=True)
    out = xf * torch.rsqrt(var + eps)
    out = weight * out.to(weight.dtype)
    return out.to(x.dtype)


def router(
    xn: torch.Tensor,
    w_router: torch.Tensor,
    bias: Optional[torch.Tensor],
    top_k: int,
):
    """mixture_of_experts_block.py:72-83 with linear_default
    (ops/default_impls.py:328-341): logits in the activation dtype, fp32
    softmax, descending top-k, renormalised gates cast to the activation dtype.
    Returns (gates [T,k], experts [T,k] int64, probabilities [T,E])."""
    w = w_router.to(xn.dtype)
    logits = torch.matmul(xn, w.mT)
    if bias is not None:
        logits = logits + bias
    p = F.softmax(logits, dim=1, dtype=torch.float)
    gate, idx = torch.topk(p, top_k, dim=-1)
    gate = gate / gate.sum(dim=-1, keepdim=True)
    return gate.to(xn.dtype), idx, p


def topk_margin(p: torch.Tensor, top_k: int) -> float:
    """Smallest gap between consecutive sorted probabilities among the first
    k+1 of any token.  torch.topk leaves tie order unspecified, so bit-exact
    index parity is only defined for inputs whose margin is > 0."""
    s = torch.sort(p, dim=-1, descending=True).values[:, : top_k + 1]
    return float((s[:, :-1] - s[:, 1:]).min())


def route_plan(experts: torch.Tensor, expert_count: int):
    """Definition of the token permutation (the reference has no such step; it
    gathers weights per token instead, layers/ffn_moe_block.py:39).  Pairs
    (token, slot) are numbered p = token*k + slot; `perm` lists them by
    ascending expert id, ties by ascending p; `seg_offsets` is the exclusive
    prefix sum of the per-expert counts; `inv[p]` is p's position in `perm`."""
    flat = experts.reshape(-1).to(torch.int64)
    perm = torch.sort(flat, stable=True).indices
    counts = torch.bincount(flat, minlength=expert_count)
    seg = torch.zeros(expert_count + 1, dtype=torch.int64)
    seg[1:] = torch.cumsum(counts, 0)
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(perm.numel())
    return counts, seg, perm, inv


def experts_pregather(
    xn: torch.Tensor,
    experts: torch.Tensor,
    gate: torch.Tensor,
    w_gate: torch.Tensor,
    w_up: torch.Tensor,
    w_down: torch.Tensor,
    activation: Callable,
    chunk: int = 16,
) -> torch.Tensor:
    """PreGatherFFNMOE.forward (layers/ffn_moe_block.py:60-74) with its three
    einsum lowerings mk_menk_men / mek_menk_men / me_men_men
    (ops/default_impls.py:72-105): the expert matrices of every (token, slot)
    are gathered into a dense [T,k,N,K] copy and multiplied as batched GEMVs.
    Weights are cast to the activation dtype (default_impls.py:351).  Tokens are
    processed in chunks because the gather is 470 MB per token at Mixtral size;
    chunking does not change any value (rows are independent)."""
    T, k = experts.shape
    outs = []
    for t0 in range(0, T, chunk):
        x = xn[t0 : t0 + chunk]
        ex = experts[t0 : t0 + chunk]
        g = gate[t0 : t0 + chunk]
        m = x.shape[0]

        def mk_menk(inp, w):
            wg = w[ex].to(inp.dtype)  # [m,k,N,K]
            r = torch.matmul(inp.unsqueeze(1), wg.view(m, k * wg.shape[2], -1).mT)
            return r.view(m, k, wg.shape[2])

        a = activation(mk_menk(x, w_gate)) * mk_menk(x, w_up)
        wd = w_down[ex].to(a.dtype)  # [m,k,d,F]
        dn = torch.matmul(
            a.reshape(m * k, 1, -1), wd.view(m * k, wd.shape[2], wd.shape[3]).mT
        ).view(m, k, -1)
        scaled = torch.matmul(
            g.reshape(m * k, 1, 1), dn.reshape(m * k, -1, 1).mT
        ).view(m, k, -1)
        outs.append(torch.sum(scaled, dim=1))
    return torch.cat(outs, 0)


def experts_per_expert(
    xn, experts, gate, w_gate, w_up, w_down, activation
) -> torch.Tensor:
    """The per-expert dense formulation (FFNMOE, layers/ffn_moe_block.py:120-127)
    applied to each expert's tokens.  Mathematically the same layer; used where
    the gather form is too slow (large token counts) after being validated
    against `experts_pregather` on small shapes.  Summation over slots is done
    in slot order like the reference's torch.sum(dim=1)."""
    T, k = experts.shape
    parts = torch.zeros(T, k, w_down.shape[1], dtype=xn.dtype)
    for e in range(w_gate.shape[0]):
        tok, slot = torch.nonzero(experts == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        x = xn[tok]
        a = activation(x @ w_gate[e].to(x.dtype).mT) * (x @ w_up[e].to(x.dtype).mT)
        parts[tok, slot] = (a @ w_down[e].to(x.dtype).mT) * gate[tok, slot].unsqueeze(1)
    return parts.sum(dim=1)


@dataclass
class MoeParams:
    """Everything MoeBlock reads from its theta (mixture_of_experts_block.py:
    31-62): `ffn_norm.weight`, `ffn_gate_inp.weight` (+ optional `.bias`),
    optional `layer_output_norm.weight`, and `ffn_{gate,up,down}_exps.weight`
    as dense tensors (already dequantised for quantized layouts)."""

    norm_w: torch.Tensor
    router_w: torch.Tensor
    w_gate: torch.Tensor
    w_up: torch.Tensor
    w_down: torch.Tensor
    router_b: Optional[torch.Tensor] = None
    out_norm_w: Optional[torch.Tensor] = None
    top_k: int = 2
    eps: float = 1e-5
    activation: str = "silu"


ACTIVATIONS = {"silu": F.silu, "gelu": F.gelu}


def moe_block(h: torch.Tensor, p: MoeParams, form: str = "pregather", chunk: int = 16):
    """MoeBlock.forward (mixture_of_experts_block.py:64-90).  `h` is
    [bs, sl, d]; returns (output [bs,sl,d], dict of intermediates)."""
    bs, sl, d = h.shape
    xn = rms_norm(h, p.norm_w, p.eps).view(-1, d)
    gate, idx, prob = router(xn, p.router_w, p.router_b, p.top_k)
    act = ACTIVATIONS[p.activation]
    if form == "pregather":
        y = experts_pregather(xn, idx, gate, p.w_gate, p.w_up, p.w_down, act, chunk)
    else:
        y = experts_per_expert(xn, idx, gate, p.w_gate, p.w_up, p.w_down, act)
    y = y.reshape(bs, sl, d)
    if p.out_norm_w is not None:
        y = rms_norm(y, p.out_norm_w, p.eps)
    return h + y, {"xn": xn, "gate": gate, "experts": idx, "prob": prob}


def moe_block_sampled(h: torch.Tensor, p: MoeParams, expert_weights: Callable, token_index: torch.Tensor):
    """MoeBlock.forward (mixture_of_experts_block.py:64-90) for layers too large
    to hold dequantised: norm and router for EVERY token, the expert FFN (the
    per-expert form, `experts_per_expert`) only for the tokens in `token_index`,
    with the dense weights of one expert at a time fetched through
    `expert_weights(e) -> (w_gate[N,K], w_up[N,K], w_down[d,F])`.  `p.w_*` are
    ignored.  Returns (output rows [len(token_index), d], intermediates of all
    tokens).  Tokens are independent, so the sampled rows equal the same rows
    of the full evaluation."""
    bs, sl, d = h.shape
    xn = rms_norm(h, p.norm_w, p.eps).view(-1, d)
    gate, idx, prob = router(xn, p.router_w, p.router_b, p.top_k)
    act = ACTIVATIONS[p.activation]
    tok_sel = token_index.to(torch.int64)
    xs, ex_s, g_s = xn[tok_sel], idx[tok_sel], gate[tok_sel]
    parts = torch.zeros(tok_sel.numel(), p.top_k, d, dtype=xn.dtype)
    n_experts = p.router_w.shape[0]
    for e in range(n_experts):
        tok, slot = torch.nonzero(ex_s == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        wg, wu, wd = expert_weights(e)
        x = xs[tok]
        a = act(x @ wg.to(x.dtype).mT) * (x @ wu.to(x.dtype).mT)
        parts[tok, slot] = (a @ wd.to(x.dtype).mT) * g_s[tok, slot].unsqueeze(1)
        del wg, wu, wd
    y = parts.sum(dim=1)
    if p.out_norm_w is not None:
        y = rms_norm(y, p.out_norm_w, p.eps)
    out = h.view(-1, d)[tok_sel] + y
    return out, {"xn": xn, "gate": gate, "experts": idx, "prob": prob}


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    a = a.double().flatten()
    b = b.double().flatten()
    return float(torch.linalg.norm(a - b) / torch.linalg.norm(b).clamp_min(1e-30))
