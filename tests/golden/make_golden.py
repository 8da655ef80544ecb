"""Generate the golden fixtures in this directory by running the reference itself.

Usage (needs a sharktank source checkout; iree-turbine is replaced by
iree_stub.py, which only has to make the torch-eager path importable):

    python tests/golden/make_golden.py --sharktank /path/to/reference/sharktank

Writes:
  formats.npz      packed Q8_0 / Q4_K blocks, the planes the reference's
                   `unpack()` produces and its `dequant()` values; outputs of
                   the bit-unpack helpers on random bytes
  moe_bf16act.npz  sharktank's MoeBlock on bf16 activations (its bf16 router path)
  attn_*.npz       sharktank's PagedLlamaAttentionBlock: prefill and decode outputs and
                   the KV page slab after each
  moe_<case>.npz   outputs of sharktank's MoeBlock for the small seeded cases
                   of shark_platform_b200.synthetic (quantized weights go
                   through `layout.dequant()` -> DefaultPrimitiveTensor, the
                   only way the reference can evaluate them)
The inputs are regenerated from the seed by the tests; each fixture carries a
SHA-256 of the inputs so that a drifting generator is detected, not ignored.
"""
import argparse
import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, HERE)
sys.path.insert(0, ROOT)


def digest(case) -> str:
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sharktank", default=os.environ.get("SHARKTANK_SRC", ""),
                    help="path of a sharktank source checkout (the directory that contains the sharktank package)")
    args = ap.parse_args()
    if not args.sharktank:
        ap.error("--sharktank (or SHARKTANK_SRC) is required")
    sys.path.insert(0, args.sharktank)
    import iree_stub

    iree_stub.install()
    import torch.nn.functional as F
    from sharktank.layers.mixture_of_experts_block import MoeBlock
    from sharktank.types import DefaultPrimitiveTensor, PlanarQuantizedTensor, Theta
    from sharktank.types.gguf_interop.layouts import Q4_K as RefQ4K, Q8_0 as RefQ8
    from sharktank.types.layouts import (
        BlockScaledI4Layout,
        BlockScaledLayout,
        SuperBlockOffsetScaled_4_6_Layout,
    )
    from sharktank.types import layout_utils as lu

    from shark_platform_b200 import synthetic as syn

    # ---------------- formats ----------------
    rng = np.random.default_rng(1234)
    out = {}
    n, k = 6, 512
    raw8 = rng.integers(0, 256, size=(n * k // 32, 34), dtype=np.uint8)
    sc = (np.abs(rng.standard_normal(n * k // 32)) * 0.01).astype(np.float16)
    raw8[:, 0:2] = sc.view(np.uint8).reshape(-1, 2)
    lay = RefQ8(raw=torch.from_numpy(raw8.reshape(-1)), shape=[n, k]).unpack()
    out["q8_raw"] = raw8
    out["q8_d"] = lay.d.contiguous().numpy()
    out["q8_qs"] = lay.qs.contiguous().numpy()
    out["q8_dequant_f16"] = lay.dequant().numpy()
    out["q8_dequant_f32"] = lay.dequant(torch.float32).numpy()

    raw4 = rng.integers(0, 256, size=(n * k // 256, 144), dtype=np.uint8)
    dd = (np.abs(rng.standard_normal((n * k // 256, 2))) * [3e-4, 2e-3]).astype(np.float16)
    raw4[:, 0:4] = dd.view(np.uint8).reshape(-1, 4)
    lay4 = RefQ4K(raw=torch.from_numpy(raw4.reshape(-1)), shape=[n, k]).unpack()
    out["q4k_raw"] = raw4
    for name, t in lay4.planes.items():
        out["q4k_" + name] = t.contiguous().numpy()
    out["q4k_sb_scales"] = lay4.sb_scales.numpy()
    out["q4k_sb_mins"] = lay4.sb_mins.numpy()
    out["q4k_qs_i8"] = lay4.qs.numpy()
    out["q4k_dequant_f16"] = lay4.dequant().numpy()

    # Q4_1 as sharktank holds it: BlockScaledI4Layout with offsets
    gq = torch.Generator().manual_seed(77)
    p41 = syn.q4_1_planes(gq, 1, n, k)
    lay41 = BlockScaledI4Layout([n, k], p41["d"][0], p41["qs"][0], m=p41["m"][0])
    out["q41_d"] = p41["d"][0].numpy()
    out["q41_m"] = p41["m"][0].numpy()
    out["q41_qs"] = p41["qs"][0].numpy()
    out["q41_dequant_f16"] = lay41.dequant().numpy()

    b = rng.integers(0, 256, size=(5, 16), dtype=np.uint8)
    tb = torch.from_numpy(b)
    out["bits_in"] = b
    out["bits_linearize_i4"] = lu.linearize_interleaved_i4_block(tb).numpy()
    out["bits_interleave_i4"] = lu.interleave_linear_i4_block(tb).numpy()
    out["bits_i4_unsigned"] = lu.promote_linear_i4_block_to_i8(tb).numpy()
    out["bits_i4_signed"] = lu.promote_linear_i4_block_to_i8(tb, signed=True).numpy()
    out["bits_i2"] = lu.promote_linear_i2_block_to_i8(tb).numpy()
    out["bits_i6"] = lu.promote_linear_i6_block_to_i8(tb[:, :4], tb[:, 8:16]).numpy()
    np.savez_compressed(os.path.join(HERE, "formats.npz"), **out)
    print("formats.npz written")

    # ---------------- MoE layer ----------------
    def ref_weight(kind, planes, shape):
        if kind == syn.Q8_0:
            lay = BlockScaledLayout(shape, planes["d"], planes["qs"])
        elif kind == syn.Q4_K:
            lay = SuperBlockOffsetScaled_4_6_Layout(shape, **planes)
        elif kind == syn.Q4_1:
            lay = BlockScaledI4Layout(shape, planes["d"], planes["qs"], m=planes["m"])
        else:
            return DefaultPrimitiveTensor(data=planes["w"])
        qt = PlanarQuantizedTensor(shape=shape, layout=lay)
        return DefaultPrimitiveTensor(data=qt.unpack().dequant())

    for name in ["toy", "small_q8", "small_q4k", "small_q41", "small_grok", "small_top4", "small_dense"]:
        spec = syn.CASES[name]
        case = syn.make_case(spec)
        e, f, d = spec.experts, spec.ffn, spec.hidden
        tree = {
            "ffn_gate_inp": {"weight": DefaultPrimitiveTensor(data=case.router_w)},
            "ffn_norm": {"weight": DefaultPrimitiveTensor(data=case.norm_w)},
            "ffn_gate_exps": {"weight": ref_weight(spec.kind, case.gate, [e, f, d])},
            "ffn_up_exps": {"weight": ref_weight(spec.kind, case.up, [e, f, d])},
            "ffn_down_exps": {"weight": ref_weight(spec.kind, case.down, [e, d, f])},
        }
        if case.router_b is not None:
            tree["ffn_gate_inp"]["bias"] = DefaultPrimitiveTensor(data=case.router_b)
        if case.out_norm_w is not None:
            tree["layer_output_norm"] = {"weight": DefaultPrimitiveTensor(data=case.out_norm_w)}
        act = F.silu if spec.activation == "silu" else F.gelu
        block = MoeBlock(Theta(tree), e, spec.top_k, spec.eps, moe_activation=act)

        captured = {}
        orig = block.experts.forward

        def spy(h, experts, expert_gate):
            captured["xn"] = h.clone()
            captured["experts"] = experts.clone()
            captured["gate"] = expert_gate.clone()
            return orig(h, experts, expert_gate)

        block.experts.forward = spy
        y = block(case.h)
        np.savez_compressed(
            os.path.join(HERE, f"moe_{name}.npz"),
            y=y.numpy(),
            experts=captured["experts"].numpy(),
            gate=captured["gate"].numpy(),
            xn=captured["xn"].numpy(),
            digest=np.array(digest(case)),
        )
        print(f"moe_{name}.npz written  |y|={float(y.abs().mean()):.4f}")

    # ---------------- bf16 activations through the reference ----------------
    # With bf16 `h` the reference rounds the normalised row to bf16
    # (layers/norm.py:39-41), computes the router logits in bf16 (the weight is
    # cast to the input dtype, ops/default_impls.py:332-333) and casts the expert
    # weights to bf16 as well (:351).  The CUDA path keeps norm, logits and gates
    # in fp32; this fixture measures how far the two routings are apart.
    spec = syn.CaseSpec("bf16act", 512, 256, 512, kind=syn.Q8_0, norm_weight="perturbed", seed=21)
    case = syn.make_case(spec)
    e, f, d = spec.experts, spec.ffn, spec.hidden
    tree = {
        "ffn_gate_inp": {"weight": DefaultPrimitiveTensor(data=case.router_w)},
        "ffn_norm": {"weight": DefaultPrimitiveTensor(data=case.norm_w)},
        "ffn_gate_exps": {"weight": ref_weight(spec.kind, case.gate, [e, f, d])},
        "ffn_up_exps": {"weight": ref_weight(spec.kind, case.up, [e, f, d])},
        "ffn_down_exps": {"weight": ref_weight(spec.kind, case.down, [e, d, f])},
    }
    block = MoeBlock(Theta(tree), e, spec.top_k, spec.eps, moe_activation=F.silu)
    captured = {}
    orig = block.experts.forward

    def spy16(h, experts, expert_gate):
        captured["experts"] = experts.clone()
        captured["gate"] = expert_gate.clone()
        return orig(h, experts, expert_gate)

    block.experts.forward = spy16
    y16 = block(case.h.to(torch.bfloat16))
    assert y16.dtype == torch.bfloat16
    np.savez_compressed(
        os.path.join(HERE, "moe_bf16act.npz"),
        y=y16.float().numpy(),
        experts=captured["experts"].numpy(),
        gate=captured["gate"].float().numpy(),
        digest=np.array(digest(case)),
    )
    print("moe_bf16act.npz written")

    # ---------------- paged attention block ----------------
    # sharktank's own PagedLlamaAttentionBlock + PagedKVCache + RotaryEmbeddingLayer:
    # a batched prefill, then one decode step on the cache it filled.  The rotary
    # kernel is the eager stand-in of iree_stub.py (the IREE kernel cannot run).
    from sharktank.layers import PagedKVCache, PagedLlamaAttentionBlock, RotaryEmbeddingLayer

    for name, softcap in (("attn_plain", None), ("attn_softcap", 30.0)):
        c = syn.make_attn_case(seed=70 if softcap is None else 71, softcap=softcap)
        bs, sl, _ = c.h.shape
        cache = PagedKVCache(transformer_block_count=c.blocks, attn_head_count=c.head_count_kv,
                             attn_head_dim=c.head_dim, block_seq_stride=c.stride, dtype=torch.float32)
        theta = Theta({
            "attn_norm": {"weight": DefaultPrimitiveTensor(data=c.norm_w)},
            "attn_q": {"weight": DefaultPrimitiveTensor(data=c.wq)},
            "attn_k": {"weight": DefaultPrimitiveTensor(data=c.wk)},
            "attn_v": {"weight": DefaultPrimitiveTensor(data=c.wv)},
            "attn_output": {"weight": DefaultPrimitiveTensor(data=c.wo)},
        })
        block = PagedLlamaAttentionBlock(theta, block_index=c.block_index, cache=cache,
                                         head_count=c.head_count, head_dim=c.head_dim,
                                         head_count_kv=c.head_count_kv, rms_epsilon=c.eps, softcap=softcap)
        rope = RotaryEmbeddingLayer(rope_dimension_count=c.head_dim, max_seqlen=256, rope_freq_base=c.rope_base)
        state = cache.allocate(c.pages)
        state[0].zero_()
        neg = torch.finfo(torch.float32).min
        causal = torch.triu(torch.ones(sl, sl, dtype=torch.bool), diagonal=1)[None, None]
        pad = (torch.arange(sl)[None, :] >= c.seq_lens[:, None])[:, None, None, :]
        mask = torch.where(causal | pad, neg, 0.0)
        y = block(c.h, embedding=rope, start_index=0, attention_mask=mask, cache_state=state,
                  seq_block_ids=c.page_ids[:, : sl // c.stride])
        slab_prefill = state[0].clone()
        kv_len = c.page_ids.shape[1] * c.stride
        dmask = torch.where(torch.arange(kv_len)[None, :] >= (c.seq_lens + 1)[:, None], neg, 0.0)[:, None, None, :]
        xk_temp = torch.zeros(bs, 256, c.head_count_kv, c.head_dim)
        xv_temp = torch.zeros(bs, 256, c.head_count_kv, c.head_dim)
        yd = block(c.h_decode, embedding=rope, start_positions=c.seq_lens,
                   embedding_batch_mask=rope.compute_batch_mask(c.seq_lens, batch_seq_len=1),
                   attention_mask=dmask, cache_state=state, seq_block_ids=c.page_ids,
                   xk_temp=xk_temp, xv_temp=xv_temp)
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), y=y.numpy(), slab_prefill=slab_prefill.numpy(),
                            y_decode=yd.numpy(), slab_decode=state[0].numpy())
        print(f"{name}.npz written  |y|={float(y.abs().mean()):.4f} |yd|={float(yd.abs().mean()):.4f}")


if __name__ == "__main__":
    main()
