"""The paged attention block on the GPU against fixtures made by sharktank's
own PagedLlamaAttentionBlock and against the attention oracle."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import attention_oracle as ao
from shark_platform_b200 import synthetic as syn
from helpers import load_golden
from test_attention_oracle import CASES, attn_params, masks

pytestmark = pytest.mark.gpu


def _block(c, dev="cuda", cache_dtype=torch.float32, act_dtype=torch.float32):
    from shark_platform_b200 import attention as A, types as T

    P = lambda t: T.DefaultPrimitiveTensor(data=t.to(dev))
    theta = T.Theta({"attn_norm": {"weight": P(c.norm_w)}, "attn_q": {"weight": P(c.wq)},
                     "attn_k": {"weight": P(c.wk)}, "attn_v": {"weight": P(c.wv)},
                     "attn_output": {"weight": P(c.wo)}})
    cache = A.PagedKVCache(transformer_block_count=c.blocks, attn_head_count=c.head_count_kv,
                           attn_head_dim=c.head_dim, block_seq_stride=c.stride, dtype=cache_dtype, device=dev)
    blk = A.B200PagedAttentionBlock(theta, block_index=c.block_index, cache=cache, head_count=c.head_count,
                                    head_dim=c.head_dim, head_count_kv=c.head_count_kv, rms_epsilon=c.eps,
                                    softcap=c.softcap)
    rope = A.RotaryEmbeddingLayer(rope_dimension_count=c.head_dim, max_seqlen=4096, rope_freq_base=c.rope_base)
    return blk, cache, rope


@pytest.mark.parametrize("name", sorted(CASES))
def test_attention_block_matches_the_reference_fixture(name):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from shark_platform_b200 import moe

    seed, softcap = CASES[name]
    g = load_golden(f"{name}.npz")
    c = syn.make_attn_case(seed=seed, softcap=softcap)
    blk, cache, rope = _block(c)
    state = cache.allocate(c.pages)
    mask, dmask = masks(c)
    sl = c.h.shape[1]
    y = blk(c.h.cuda(), embedding=rope, start_index=0, attention_mask=mask.cuda(), cache_state=state,
            seq_block_ids=c.page_ids[:, : sl // c.stride].cuda())
    assert moe.device_status() == 0
    assert np.abs(state[0].cpu().numpy() - g["slab_prefill"]).max() < 2e-5  # K/V pages, rotated keys included
    # rows of padded positions attend nothing meaningful in either implementation: compare the valid ones
    for b, n in enumerate(c.seq_lens.tolist()):
        assert np.abs(y[b, :n].cpu().numpy() - g["y"][b, :n]).max() < 2e-4
    yd = blk(c.h_decode.cuda(), embedding=rope, start_positions=c.seq_lens.cuda(), embedding_batch_mask=None,
             attention_mask=dmask.cuda(), cache_state=state, seq_block_ids=c.page_ids.cuda())
    assert moe.device_status() == 0
    assert np.abs(state[0].cpu().numpy() - g["slab_decode"]).max() < 2e-5
    assert np.abs(yd.cpu().numpy() - g["y_decode"]).max() < 2e-4


@pytest.mark.parametrize("cache_dtype,act_dtype,tol", [(torch.float32, torch.float32, 2e-4),
                                                      (torch.float16, torch.float16, 2e-2),
                                                      (torch.bfloat16, torch.bfloat16, 6e-2)])
@pytest.mark.parametrize("hd,heads,kv_heads,seq", [(128, 8, 2, 1000), (64, 4, 4, 300), (128, 8, 1, 2049)])
def test_decode_attention_over_long_ragged_sequences(hd, heads, kv_heads, seq, cache_dtype, act_dtype, tol):
    """The decode kernel alone (b200moe_attn_decode): sequences long enough for
    several position splits, ragged lengths, scattered pages, GQA groups of 1, 4
    and 8, against softmax(q K^T / sqrt(hd)) V over the same (rounded) cache."""
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from shark_platform_b200 import _cabi as C, moe

    bs, stride, blocks, blk_i = 3, 16, 2, 1
    gen = torch.Generator().manual_seed(seq + hd)
    geo = ao.CacheGeometry(blocks, stride, kv_heads, hd)
    per = (seq + stride - 1) // stride + 1
    pages = bs * per + 5
    slab = (torch.randn(pages, geo.flat, generator=gen) * 0.5).to(cache_dtype)
    page_ids = torch.randperm(pages, generator=gen)[: bs * per].view(bs, per)
    seq_lens = torch.tensor([seq, max(1, seq // 3), seq - 17])
    q = torch.randn(bs, heads, hd, generator=gen).to(act_dtype)
    # expected, from the rounded cache contents
    k, v = ao.cache_read(slab.float(), geo, blk_i, page_ids)
    rep = heads // kv_heads
    want = torch.zeros(bs, heads, hd)
    for b in range(bs):
        n = int(seq_lens[b])
        kk = k[b, :n].repeat_interleave(rep, dim=1)  # [n, heads, hd]
        vv = v[b, :n].repeat_interleave(rep, dim=1)
        w = torch.einsum("hd,nhd->hn", q[b].float(), kk) / hd ** 0.5
        want[b] = torch.einsum("hn,nhd->hd", torch.softmax(w, dim=-1), vv)
    desc = C.KvCacheDesc(blocks, stride, kv_heads, hd, pages)
    dt = {torch.float32: C.DT_F32, torch.float16: C.DT_F16, torch.bfloat16: C.DT_BF16}
    max_len = per * stride
    nbytes = C.lib.b200moe_attn_decode_scratch_bytes(ctypes.byref(desc), bs, heads, max_len)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    out = torch.empty(bs, heads, hd, dtype=act_dtype, device="cuda")
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    slab_d, q_d = slab.cuda(), q.cuda()
    ids_d, lens_d = page_ids.to(torch.int32).cuda(), seq_lens.to(torch.int32).cuda()
    for _ in range(2):
        C.check(C.lib.b200moe_attn_decode(p(q_d), dt[act_dtype], p(slab_d), dt[cache_dtype], ctypes.byref(desc), blk_i,
                                          p(ids_d), p(lens_d), bs, per, heads, max_len, 1.0 / hd ** 0.5, 0.0,
                                          p(out), dt[act_dtype], p(scratch), nbytes, st), "attn_decode")
    torch.cuda.synchronize()
    assert moe.device_status() == 0
    err = float((out.float().cpu() - want).abs().max() / want.abs().max())
    assert err < tol, err


def test_a_missing_page_is_reported_not_followed():
    """A page id outside the slab: the write is skipped and the status word says so."""
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from shark_platform_b200 import _cabi as C, moe

    c = syn.make_attn_case(seed=5)
    blk, cache, rope = _block(c)
    state = cache.allocate(c.pages)
    ids = c.page_ids[:, :2].clone()
    ids[0, 1] = c.pages + 7
    mask, _ = masks(c)
    blk(c.h.cuda(), embedding=rope, start_index=0, attention_mask=mask.cuda(), cache_state=state,
        seq_block_ids=ids.cuda())
    with pytest.raises(C.B200MoeError, match="status word"):
        moe.device_status()
    assert moe.device_status() == 0
