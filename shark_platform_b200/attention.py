"""The attention block that precedes every MoE layer, on the GPU.

`B200PagedAttentionBlock` has the constructor and `forward` of sharktank's
`PagedLlamaAttentionBlock` (layers/paged_llama_attention_block.py:26-303) and
works on the same objects: the model's theta (`attn_norm`, `attn_q`, `attn_k`,
`attn_v`, `attn_output`, optional `attn_output_norm`), a `PagedKVCache`
(layers/kv_cache.py:222-526; sharktank's own or the mirror below), the list
`cache_state` holding the page slab, and a rotary embedding layer.

What runs where:
  * RMS norm, rotary embedding fused with the KV page write, and the decode
    attention over the pages: this library's kernels (`b200moe_rms_norm`,
    `b200moe_attn_rope_kv_write`, `b200moe_attn_decode`).  Decode never
    materialises the linear K/V temporaries the reference reads the cache into
    (`xk_temp` / `xv_temp` are accepted and ignored).
  * the four projections: one dense product each (q, k and v fused into one) —
    a library GEMM for dense weights, this library's quantized linear for Q8_0 /
    Q4_K / Q4_1 weights;
  * the prefill attention core over the freshly computed K/V: torch's fused
    scaled-dot-product attention, which the reference also offers as
    `attention_kernel="torch"` (:215-224); with a softcap (Grok) the decomposed
    torch operators, since the fused kernel has no cap.

There is no CPU path: CPU tensors are rejected.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch
import torch.nn.functional as F

from . import _cabi as C
from . import moe as _moe

_DT = {torch.float32: C.DT_F32, torch.float16: C.DT_F16, torch.bfloat16: C.DT_BF16}


def _p(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


class PagedKVCache:
    """Mirror of sharktank's PagedKVCache (layers/kv_cache.py:222-340) for use
    without sharktank: geometry plus `allocate`.  Reads and writes happen inside
    the attention block's kernels."""

    def __init__(self, *, transformer_block_count: int, attn_head_count: int, attn_head_dim: int,
                 cache_partition_count: int = 2, block_seq_stride: int = 16,
                 dtype: torch.dtype = torch.float32, device=None, shard_count: int = 1):
        if cache_partition_count != 2 or shard_count != 1:
            raise C.B200MoeError("the cache holds K and V on one device")
        self.transformer_block_count = transformer_block_count
        self.attn_head_count = attn_head_count
        self.attn_head_dim = attn_head_dim
        self.cache_partition_count = cache_partition_count
        self.block_seq_stride = block_seq_stride
        self.shard_count = shard_count
        self.dtype, self.device = dtype, device
        self.sub_page_dims = [transformer_block_count, 2, block_seq_stride, attn_head_count, attn_head_dim]
        self.page_slab_flat_dim = math.prod(self.sub_page_dims)

    def allocate(self, page_count: int) -> list[torch.Tensor]:
        return [torch.zeros(page_count, self.page_slab_flat_dim, dtype=self.dtype, device=self.device)]


class RotaryEmbeddingLayer:
    """What the block needs of sharktank's RotaryEmbeddingLayer
    (layers/rotary_embedding.py:20-40): the dimension count and the frequency base."""

    def __init__(self, *, rope_dimension_count: int, max_seqlen: int, rope_freq_base: Optional[float] = None,
                 device=None, use_hf: bool = False):
        self.rope_dimension_count = rope_dimension_count
        self.max_seqlen = max_seqlen
        self.rope_freq_base = rope_freq_base if rope_freq_base is not None else 10000.0
        self.device, self.use_hf = device, use_hf


def _is_quantized(t) -> bool:
    return _moe._layout_name(t) in _moe._SUPPORTED


class B200PagedAttentionBlock(torch.nn.Module):
    """Drop-in for PagedLlamaAttentionBlock (same constructor keywords, same
    `forward` keywords)."""

    def __init__(self, theta, *, block_index: int, cache, head_count: int, head_dim: int, head_count_kv: int,
                 rms_epsilon: float, attention_kernel: str = "decomposed", attention_scale: Optional[float] = None,
                 softcap: Optional[float] = None, fake_quant: Optional[bool] = True):
        super().__init__()
        self.theta = theta
        self.block_index, self.cache = block_index, cache
        self.head_count, self.head_dim, self.head_count_kv = head_count, head_dim, head_count_kv
        self.rms_epsilon = rms_epsilon
        self.attention_kernel, self.attention_scale, self.softcap = attention_kernel, attention_scale, softcap
        if "kv_cache" in getattr(theta, "keys", ()):
            raise C.B200MoeError("a quantized KV cache (kv_cache.quantizer) is not supported")
        if head_count % head_count_kv != 0 or head_count // head_count_kv > 8:
            raise C.B200MoeError("head_count must be 1..8 times head_count_kv")
        if head_dim not in (64, 128):
            raise C.B200MoeError(f"head_dim {head_dim}: 64 and 128 are built")
        if cache.attn_head_count != head_count_kv or cache.attn_head_dim != head_dim:
            raise C.B200MoeError("the cache's heads / head_dim differ from the block's")
        w = lambda name: theta(name).tensor("weight")
        self._norm_w = _moe._unbox(w("attn_norm")).to(torch.float32).contiguous()
        _moe._require_cuda(self._norm_w, "attn_norm.weight")
        self._out_norm_w = None
        if theta.optional_tensor("attn_output_norm") is not None:
            self._out_norm_w = _moe._unbox(w("attn_output_norm")).to(torch.float32).contiguous()
        wq, wk, wv, self._wo = w("attn_q"), w("attn_k"), w("attn_v"), w("attn_output")
        self._bias = {n: theta(n).optional_tensor("bias") if "bias" in theta(n).keys else None
                      for n in ("attn_q", "attn_k", "attn_v", "attn_output")}
        if any(_is_quantized(t) for t in (wq, wk, wv)):
            self._wqkv, self._wq, self._wk, self._wv = None, wq, wk, wv
        else:  # one fused projection
            self._wqkv = torch.cat([_moe._unbox(t) for t in (wq, wk, wv)], dim=0).contiguous()
        self._freqs = None
        self._scratch = None
        self._desc = C.KvCacheDesc(cache.transformer_block_count, cache.block_seq_stride, head_count_kv, head_dim, 0)

    # ---------------------------------------------------------------- pieces
    def _linear(self, x, weight, bias):
        if _is_quantized(weight):
            y = _moe.linear_quantized(x, weight, bias)
            if y is NotImplemented:
                raise C.B200MoeError("quantized projection weight has an unsupported shape")
            return y
        wt = _moe._unbox(weight) if not isinstance(weight, torch.Tensor) else weight
        return F.linear(x, wt.to(x.dtype), None if bias is None else _moe._unbox(bias).to(x.dtype))

    def _norm(self, x, weight):
        y = torch.empty_like(x)
        rows = x.numel() // x.shape[-1]
        with torch.cuda.device(x.device):
            C.check(C.lib.b200moe_rms_norm(_p(x), _DT[x.dtype], _p(weight), rows, x.shape[-1],
                                           float(self.rms_epsilon), _p(y), _DT[y.dtype], _moe._stream()), "rms_norm")
        return y

    def _freq_table(self, embedding, device):
        if self._freqs is None or self._freqs.device != device:
            if getattr(embedding, "use_hf", False):
                raise C.B200MoeError("the HuggingFace rotary ordering (use_hf) is not supported")
            dim = embedding.rope_dimension_count
            if dim != self.head_dim:
                raise C.B200MoeError("rope_dimension_count must equal head_dim")
            base = embedding.rope_freq_base
            # layers/rotary_embedding.py:222-228, one entry per pair
            freqs = 1.0 / (base ** ((torch.arange(0, dim) // 2).float() / dim * 2.0))
            self._freqs = freqs[0::2].contiguous().to(device)
        return self._freqs

    # --------------------------------------------------------------- forward
    def forward(self, h: torch.Tensor, *, embedding, seq_block_ids: torch.Tensor,
                start_index: Optional[int] = None, start_positions: Optional[torch.Tensor] = None,
                attention_mask: Optional[torch.Tensor] = None, embedding_batch_mask: Optional[torch.Tensor] = None,
                cache_state: list = None, xk_temp: Optional[torch.Tensor] = None,
                xv_temp: Optional[torch.Tensor] = None) -> torch.Tensor:
        _moe._require_cuda(h, "h")
        if h.dtype not in _DT:
            raise C.B200MoeError(f"activations must be fp32, fp16 or bf16, got {h.dtype}")
        if (start_index is not None) == (start_positions is not None):
            raise C.B200MoeError("exactly one of start_index (prefill) and start_positions (decode) is given")
        slab = cache_state[0]
        if slab.dtype not in _DT or not slab.is_contiguous():
            raise C.B200MoeError("the page slab must be a contiguous fp32, fp16 or bf16 tensor")
        dev = h.device
        bs, sl, d = h.shape
        H, Hkv, hd = self.head_count, self.head_count_kv, self.head_dim
        stride = self.cache.block_seq_stride
        decode = start_positions is not None
        if decode and sl != 1:
            raise C.B200MoeError("a decode step brings one token per sequence")
        x = self._norm(h.contiguous(), self._norm_w)
        if self._wqkv is not None:
            qkv = F.linear(x, self._wqkv.to(x.dtype))
            q, k, v = torch.split(qkv, [H * hd, Hkv * hd, Hkv * hd], dim=-1)
            q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        else:
            q = self._linear(x, self._wq, self._bias["attn_q"]).contiguous()
            k = self._linear(x, self._wk, self._bias["attn_k"]).contiguous()
            v = self._linear(x, self._wv, self._bias["attn_v"]).contiguous()
        if self._wqkv is not None and any(self._bias[n] is not None for n in ("attn_q", "attn_k", "attn_v")):
            raise C.B200MoeError("projection biases are supported with unfused (quantized) weights only")
        tokens = bs * sl
        if decode:
            positions = start_positions.to(torch.int32).contiguous()
        else:
            positions = (torch.arange(sl, device=dev, dtype=torch.int32) + int(start_index)).repeat(bs)
        page_ids = seq_block_ids.to(torch.int32).contiguous()
        self._desc.page_count = slab.shape[0]
        k_out = v_out = None
        if not decode:
            k_out, v_out = torch.empty_like(k), torch.empty_like(v)
        with torch.cuda.device(dev):
            C.check(C.lib.b200moe_attn_rope_kv_write(
                _p(q), _p(k), _p(v), _p(k_out), _p(v_out), _DT[q.dtype], _p(slab), _DT[slab.dtype],
                ctypes.byref(self._desc), self.block_index, _p(positions), _p(page_ids),
                _p(self._freq_table(embedding, dev)), tokens, sl, page_ids.shape[1], H, _moe._stream()),
                "attn_rope_kv_write")
        scale = self.attention_scale if self.attention_scale is not None else 1.0 / math.sqrt(hd)
        if decode:
            # positions to attend: everything up to and including the new row (what the
            # reference's decode mask leaves unmasked)
            seq_lens = (positions + 1).contiguous()
            max_len = page_ids.shape[1] * stride
            out = torch.empty(bs, H * hd, dtype=h.dtype, device=dev)
            nbytes = C.lib.b200moe_attn_decode_scratch_bytes(ctypes.byref(self._desc), bs, H, max_len)
            if self._scratch is None or self._scratch.numel() < nbytes or self._scratch.device != dev:
                self._scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
            with torch.cuda.device(dev):
                C.check(C.lib.b200moe_attn_decode(
                    _p(q), _DT[q.dtype], _p(slab), _DT[slab.dtype], ctypes.byref(self._desc), self.block_index,
                    _p(page_ids), _p(seq_lens), bs, page_ids.shape[1], H, max_len, float(scale),
                    float(self.softcap) if self.softcap is not None else 0.0, _p(out), _DT[out.dtype],
                    _p(self._scratch), self._scratch.numel(), _moe._stream()), "attn_decode")
            attn = out.view(bs, 1, H * hd)
        else:
            qh = q.view(bs, sl, H, hd).transpose(1, 2)
            kh = k_out.view(bs, sl, Hkv, hd).transpose(1, 2)
            vh = v_out.view(bs, sl, Hkv, hd).transpose(1, 2)
            mask = None if attention_mask is None else attention_mask.to(q.dtype)
            if self.softcap is None:
                attn = F.scaled_dot_product_attention(qh, kh, vh, attn_mask=mask, is_causal=mask is None,
                                                      scale=scale, enable_gqa=H != Hkv)
            else:
                rep = H // Hkv
                kh, vh = kh.repeat_interleave(rep, dim=1), vh.repeat_interleave(rep, dim=1)
                w = torch.matmul(qh, kh.transpose(2, 3)) * scale
                w = self.softcap * torch.tanh(w / self.softcap)
                if mask is not None:
                    w = w + mask
                else:
                    w = w + torch.full((sl, sl), float("-inf"), device=dev, dtype=w.dtype).triu(1)
                attn = torch.matmul(torch.softmax(w.float(), dim=-1).to(qh.dtype), vh)
            attn = attn.transpose(1, 2).reshape(bs, sl, H * hd)
        y = self._linear(attn, self._wo, self._bias["attn_output"])
        if self._out_norm_w is not None:
            y = self._norm(y.contiguous(), self._out_norm_w)
        return h + y


def patch_attention_blocks(model) -> int:
    """Replaces every PagedLlamaAttentionBlock-shaped child of `model` (anything
    with `.theta`, `.cache`, `.head_count_kv` and `.block_index`) by a
    B200PagedAttentionBlock built from the same theta and cache.  Returns the
    number of blocks replaced."""
    replaced = 0
    for parent in list(model.modules()):
        for name, child in list(parent.named_children()):
            if isinstance(child, B200PagedAttentionBlock):
                continue
            if not all(hasattr(child, a) for a in ("theta", "cache", "head_count_kv", "block_index", "attn_norm")):
                continue
            new = B200PagedAttentionBlock(
                child.theta, block_index=child.block_index, cache=child.cache, head_count=child.head_count,
                head_dim=child.head_dim, head_count_kv=child.head_count_kv, rms_epsilon=child.attn_norm.epsilon,
                attention_kernel=getattr(child, "attention_kernel", "decomposed"),
                attention_scale=getattr(child, "attention_scale", None), softcap=getattr(child, "softcap", None))
            setattr(parent, name, new)
            replaced += 1
    return replaced
