"""CPU oracle for the attention block that precedes every MoE layer.  TEST
INFRASTRUCTURE ONLY: the product package never imports it.

Restates sharktank's `PagedLlamaAttentionBlock.forward`
(layers/paged_llama_attention_block.py:86-303, the "decomposed" kernel), the
paged KV cache it reads and writes (layers/kv_cache.py:222-526) and the rotary
embedding (layers/rotary_embedding.py:115-240 with the linalg template
kernels/templates/rotary_embedding.mlir).

Parity status: PINNED for norm, projections, cache write / write_timestep / read,
GQA expansion, softcap, mask, softmax and output projection — fixtures under
tests/golden/attn_*.npz come from running sharktank's own block
(tests/golden/make_golden.py).  UNPINNED for the rotary kernel alone: the
reference implements it as an IREE custom kernel that cannot run without
iree-turbine, so the fixtures were produced with the eager restatement of the
kernel template in tests/golden/iree_stub.py, which this file restates again.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch


def rotary_angles(positions: torch.Tensor, dim: int, base: float) -> torch.Tensor:
    """`RotaryEmbeddingLayer._compute_rotary_embed_table`
    (layers/rotary_embedding.py:222-228): angle[t, j] = t * base^-(2*(j//2)/dim),
    the same angle for both elements of a pair.  [T] -> [T, dim] fp32."""
    freqs = 1.0 / (base ** ((torch.arange(0, dim) // 2).float() / dim * 2.0))
    return torch.outer(positions, freqs).float()


def apply_rotary(x: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """The rotary kernel (kernels/templates/rotary_embedding.mlir:30-60): x
    [bs, sl, heads, dim], table [bs, sl, dim]; pairs (2i, 2i+1) are rotated, every
    output element with the angle stored at its own index."""
    t = table.unsqueeze(2)
    cos, sin = torch.cos(t), torch.sin(t)
    real, imag = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = real * cos[..., 0::2] - imag * sin[..., 0::2]
    out[..., 1::2] = imag * cos[..., 1::2] + real * sin[..., 1::2]
    return out


@dataclass
class CacheGeometry:
    """`PagedKVCache` (layers/kv_cache.py:246-277): a page holds, for every
    transformer block, a K and a V partition of `stride` positions x kv_heads x
    head_dim; the slab is [page_count, blocks * 2 * stride * kv_heads * head_dim]."""

    blocks: int
    stride: int
    kv_heads: int
    head_dim: int

    @property
    def sub_page_dims(self):
        return [self.blocks, 2, self.stride, self.kv_heads, self.head_dim]

    @property
    def flat(self):
        return math.prod(self.sub_page_dims)

    def allocate(self, pages: int, dtype=torch.float32) -> torch.Tensor:
        return torch.zeros(pages, self.flat, dtype=dtype)


def cache_write(slab, geo: CacheGeometry, parts, block_index: int, page_ids: torch.Tensor):
    """`PagedKVCache.write` (layers/kv_cache.py:485-526): whole pages of K and V
    ([bs, sl, kv_heads, hd], sl a multiple of the stride) to the listed pages."""
    table = slab.unflatten(1, geo.sub_page_dims).flatten(0, 2)  # [page*block*2, stride, heads, hd]
    bs, nblk = page_ids.shape
    base = page_ids * (geo.blocks * 2) + block_index * 2
    for index, part in enumerate(parts):
        view = part.unflatten(1, (nblk, geo.stride)).flatten(0, 1)
        table.index_copy_(0, (base + index).flatten(0, 1), view.to(table.dtype))


def cache_write_timestep(slab, geo: CacheGeometry, parts, block_index: int, positions: torch.Tensor,
                         page_ids: torch.Tensor):
    """`PagedKVCache.write_timestep` (layers/kv_cache.py:428-483): one position
    per sequence ([bs, 1, kv_heads, hd]) at `positions` [bs]."""
    table = slab.unflatten(1, geo.sub_page_dims)
    page = torch.gather(page_ids, 1, (positions // geo.stride).unsqueeze(1)).squeeze(1)
    off = positions % geo.stride
    for index, part in enumerate(parts):
        for b in range(positions.shape[0]):
            table[page[b], block_index, index, off[b]] = part[b, 0].to(table.dtype)


def cache_read(slab, geo: CacheGeometry, block_index: int, page_ids: torch.Tensor):
    """`PagedKVCache.read` (layers/kv_cache.py:351-426): K and V of every listed
    page, linearised to [bs, nblk * stride, kv_heads, hd]."""
    table = slab.unflatten(1, geo.sub_page_dims).flatten(0, 2)
    bs, nblk = page_ids.shape
    base = page_ids * (geo.blocks * 2) + block_index * 2
    out = []
    for index in range(2):
        sel = torch.index_select(table, 0, (base + index).flatten(0, 1))
        out.append(sel.unflatten(0, (bs, nblk)).flatten(1, 2))
    return out


@dataclass
class AttnParams:
    """What the block reads from its theta (paged_llama_attention_block.py:57-85):
    `attn_norm.weight`, `attn_{q,k,v,output}.weight` (dense here), optional
    `attn_output_norm.weight`."""

    norm_w: torch.Tensor
    wq: torch.Tensor
    wk: torch.Tensor
    wv: torch.Tensor
    wo: torch.Tensor
    head_count: int
    head_count_kv: int
    head_dim: int
    eps: float = 1e-5
    rope_base: float = 10000.0
    block_index: int = 0
    softcap: Optional[float] = None
    attention_scale: Optional[float] = None
    out_norm_w: Optional[torch.Tensor] = None


def _rms_norm(x, w, eps):
    xf = x.to(torch.float32)
    out = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (w * out.to(w.dtype)).to(x.dtype)


def attention_block(h: torch.Tensor, p: AttnParams, slab: torch.Tensor, geo: CacheGeometry,
                    seq_block_ids: torch.Tensor, attention_mask: Optional[torch.Tensor],
                    start_positions: Optional[torch.Tensor] = None):
    """`PagedLlamaAttentionBlock.forward` with the decomposed attention kernel.
    Prefill when `start_positions` is None (start_index 0, the K/V just computed
    are attended and written to the cache), else one decode step at ragged start
    positions (the new row is written, then all listed pages are read back)."""
    bs, sl, d = h.shape
    H, Hkv, hd = p.head_count, p.head_count_kv, p.head_dim
    x = _rms_norm(h, p.norm_w, p.eps)
    xq = (x @ p.wq.to(x.dtype).mT).view(bs, sl, H, hd)
    xk = (x @ p.wk.to(x.dtype).mT).view(bs, sl, Hkv, hd)
    xv = (x @ p.wv.to(x.dtype).mT).view(bs, sl, Hkv, hd)
    if start_positions is None:
        pos = torch.arange(sl).unsqueeze(0).expand(bs, sl)
    else:
        pos = torch.arange(sl).unsqueeze(0) + start_positions.unsqueeze(1)
    table = rotary_angles(pos.flatten(), hd, p.rope_base).view(bs, sl, hd)
    xq = apply_rotary(xq.to(table.dtype), table).to(x.dtype)
    xk = apply_rotary(xk.to(table.dtype), table).to(x.dtype)
    if start_positions is None:
        cache_write(slab, geo, [xk, xv], p.block_index, seq_block_ids)
    else:
        assert sl == 1
        cache_write_timestep(slab, geo, [xk, xv], p.block_index, start_positions, seq_block_ids)
        xk, xv = (t.to(x.dtype) for t in cache_read(slab, geo, p.block_index, seq_block_ids))
    rep = H // Hkv
    if rep > 1:
        xk = xk.unsqueeze(-2).expand(*xk.shape[:3], rep, hd).flatten(2, 3)
        xv = xv.unsqueeze(-2).expand(*xv.shape[:3], rep, hd).flatten(2, 3)
    q, keys, values = xq.transpose(1, 2), xk.transpose(1, 2), xv.transpose(1, 2)
    w = torch.matmul(q, keys.transpose(2, 3))
    w = w / math.sqrt(hd) if p.attention_scale is None else w * p.attention_scale
    if p.softcap is not None:
        w = p.softcap * torch.tanh(w / p.softcap)
    if attention_mask is not None:
        w = w + attention_mask
    w = torch.softmax(w.to(torch.float32), dim=-1).to(q.dtype)
    out = torch.matmul(w, values).transpose(1, 2).flatten(2, 3)
    out = out @ p.wo.to(out.dtype).mT
    if p.out_norm_w is not None:
        out = _rms_norm(out, p.out_norm_w, p.eps)
    return h + out
