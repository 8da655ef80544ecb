"""The attention oracle against fixtures produced by sharktank's own
PagedLlamaAttentionBlock / PagedKVCache (tests/golden/make_golden.py)."""
import numpy as np
import pytest
import torch

from oracle import attention_oracle as ao
from shark_platform_b200 import synthetic as syn
from helpers import load_golden

CASES = {"attn_plain": (70, None), "attn_softcap": (71, 30.0)}


def attn_params(c):
    return ao.AttnParams(c.norm_w, c.wq, c.wk, c.wv, c.wo, c.head_count, c.head_count_kv, c.head_dim,
                         eps=c.eps, rope_base=c.rope_base, block_index=c.block_index, softcap=c.softcap)


def masks(c):
    """The masks the reference's driver builds (layers/causal_llm.py:82-140)."""
    bs, sl, _ = c.h.shape
    neg = torch.finfo(torch.float32).min
    causal = torch.triu(torch.ones(sl, sl, dtype=torch.bool), diagonal=1)[None, None]
    pad = (torch.arange(sl)[None, :] >= c.seq_lens[:, None])[:, None, None, :]
    kv_len = c.page_ids.shape[1] * c.stride
    dmask = torch.where(torch.arange(kv_len)[None, :] >= (c.seq_lens + 1)[:, None], neg, 0.0)[:, None, None, :]
    return torch.where(causal | pad, neg, 0.0), dmask


@pytest.mark.parametrize("name", sorted(CASES))
def test_attention_oracle_reproduces_the_reference_block(name):
    seed, softcap = CASES[name]
    g = load_golden(f"{name}.npz")
    c = syn.make_attn_case(seed=seed, softcap=softcap)
    geo = ao.CacheGeometry(c.blocks, c.stride, c.head_count_kv, c.head_dim)
    slab = geo.allocate(c.pages)
    mask, dmask = masks(c)
    sl = c.h.shape[1]
    y = ao.attention_block(c.h, attn_params(c), slab, geo, c.page_ids[:, : sl // c.stride], mask)
    assert np.array_equal(slab.numpy(), g["slab_prefill"])
    assert np.abs(y.numpy() - g["y"]).max() < 1e-5
    yd = ao.attention_block(c.h_decode, attn_params(c), slab, geo, c.page_ids, dmask, start_positions=c.seq_lens)
    assert np.array_equal(slab.numpy(), g["slab_decode"])
    assert np.abs(yd.numpy() - g["y_decode"]).max() < 1e-5


def test_cache_read_is_the_inverse_of_write():
    geo = ao.CacheGeometry(3, 4, 2, 8)
    slab = geo.allocate(7)
    gen = torch.Generator().manual_seed(1)
    k, v = torch.randn(2, 8, 2, 8, generator=gen), torch.randn(2, 8, 2, 8, generator=gen)
    ids = torch.tensor([[5, 1], [0, 6]])
    ao.cache_write(slab, geo, [k, v], 2, ids)
    rk, rv = ao.cache_read(slab, geo, 2, ids)
    assert torch.equal(rk, k) and torch.equal(rv, v)
    assert float(slab.unflatten(1, geo.sub_page_dims)[:, :2].abs().sum()) == 0.0  # other blocks untouched
