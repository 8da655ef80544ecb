"""Model level: sharktank's own `PagedMixtralModelV1` (models/mixtral/mixtral.py:
30-240) — token embedding, paged-KV attention blocks, MoE blocks, output head —
with every `moe_block` swapped for the B200 block by `plugin.patch_moe_blocks`,
driven the way `examples/paged_llm_v1.py:120-225` drives it: one batched prefill,
then a decode step on the paged cache.

Reference side: the unmodified model on the CPU with the expert weights
dequantised (`layout.dequant()`), which is the only way the reference can
evaluate quantized experts.  B200 side: the same theta on the GPU with the
experts left quantized (Q8_0 / Q4_K planar tensors); attention, embedding and
head stay the reference's torch-eager code, now on CUDA tensors.  The IREE
rotary kernel is replaced by the eager stand-in of tests/golden/iree_stub.py on
both sides."""
import pytest
import torch

from shark_platform_b200 import synthetic as syn
from helpers import dense_weight, import_sharktank, reference_path

pytestmark = [
    pytest.mark.gpu,
    pytest.mark.skipif(reference_path() is None,
                       reason="sharktank not available ($SHARKTANK_SRC or baseline/_ref)"),
]

BLOCKS, HIDDEN, FFN, VOCAB, STRIDE = 2, 256, 512, 128, 16


def _build(dev, kind, quantized):
    from sharktank.layers.configs.llm_configs import LlamaHParams, LlamaModelConfig
    from sharktank.models.mixtral.mixtral import PagedMixtralModelV1
    from sharktank.types import DefaultPrimitiveTensor, PlanarQuantizedTensor, Theta
    from sharktank.types.layouts import BlockScaledLayout, SuperBlockOffsetScaled_4_6_Layout

    hp = LlamaHParams(model_arch="llama", context_length=128, embedding_length=HIDDEN, block_count=BLOCKS,
                      feed_forward_length=FFN, attention_head_count=4, attn_head_dim=64,
                      attention_layer_norm_rms_epsilon=1e-5, attention_head_count_kv=2,
                      rope_dimension_count=64, rope_freq_base=10000.0, expert_count=8, expert_used_count=2)
    cfg = LlamaModelConfig(hp=hp, block_seq_stride=STRIDE, device=torch.device(dev),
                           activation_dtype=torch.float32, attention_dtype=torch.float32)
    g = torch.Generator().manual_seed(3)
    rn = lambda *s, sc=0.05: (torch.randn(*s, generator=g) * sc).to(dev)
    P = lambda t: DefaultPrimitiveTensor(data=t)
    tree = {"token_embd": {"weight": P(rn(VOCAB, HIDDEN, sc=1.0))},
            "output_norm": {"weight": P(1 + rn(HIDDEN, sc=0.1))},
            "output": {"weight": P(rn(VOCAB, HIDDEN))}, "blk": {}}
    for n in range(BLOCKS):
        case = syn.make_case(syn.CaseSpec(f"blk{n}", 1, HIDDEN, FFN, kind=kind, seed=40 + n))
        # keep the residual stream at unit scale, like a trained model's blocks
        for name in ("d", "dmin"):
            if name in case.down:
                case.down[name] = (case.down[name].float() * 0.05).half()

        def w(planes, shape):
            if not quantized:
                return P(dense_weight(kind, planes).float().to(dev))
            p = {k: v.to(dev) for k, v in planes.items()}
            lay = (BlockScaledLayout(shape, p["d"], p["qs"]) if kind == syn.Q8_0
                   else SuperBlockOffsetScaled_4_6_Layout(shape, **p))
            return PlanarQuantizedTensor(shape=shape, layout=lay)

        tree["blk"][str(n)] = {
            "attn_norm": {"weight": P(1 + rn(HIDDEN, sc=0.1))},
            "attn_q": {"weight": P(rn(256, HIDDEN))}, "attn_k": {"weight": P(rn(128, HIDDEN))},
            "attn_v": {"weight": P(rn(128, HIDDEN))}, "attn_output": {"weight": P(rn(HIDDEN, 256))},
            "ffn_norm": {"weight": P(1 + rn(HIDDEN, sc=0.1))},
            "ffn_gate_inp": {"weight": P(case.router_w.to(dev))},
            "ffn_gate_exps": {"weight": w(case.gate, [8, FFN, HIDDEN])},
            "ffn_up_exps": {"weight": w(case.up, [8, FFN, HIDDEN])},
            "ffn_down_exps": {"weight": w(case.down, [8, HIDDEN, FFN])},
        }
    return PagedMixtralModelV1(Theta(tree), cfg)


def _prefill_and_decode(model, dev):
    bs, sl = 2, 32
    g = torch.Generator().manual_seed(9)
    tokens = torch.randint(0, VOCAB, (bs, sl), generator=g).to(dev)
    seq_lens = torch.tensor([32, 20]).to(dev)
    cache_state = model.cache.allocate(page_count=16)
    for t in cache_state:
        t.zero_()  # freshly allocated pages are uninitialised memory
    seq_block_ids = torch.tensor([[0, 1, 2], [3, 4, 5]]).to(dev)
    mask = model.attention_mask(model.input_mask(seq_lens, sl))
    logits = model.prefill(tokens, attention_mask=mask, seq_block_ids=seq_block_ids[:, :2],
                           cache_state=cache_state)
    nxt = torch.randint(0, VOCAB, (bs, 1), generator=g).to(dev)
    start = seq_lens.clone()
    dmask = model.decode_attention_mask(model.input_mask(start + 1, seq_block_ids.shape[1] * STRIDE))
    dlogits = model.decode(nxt, attention_mask=dmask, start_positions=start, seq_block_ids=seq_block_ids,
                           cache_state=cache_state)
    return logits.float().cpu(), dlogits.float().cpu(), seq_lens.cpu()


@pytest.mark.parametrize("kind", [syn.Q8_0, syn.Q4_K])
def test_mixtral_model_with_every_moe_block_swapped(kind):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    import_sharktank()
    from oracle import moe_oracle as orc
    from shark_platform_b200 import moe, plugin

    # the reference builds its rotary table from a CPU `arange` whatever the
    # device of the positions (layers/rotary_embedding.py:222-228), which stops its
    # own model on CUDA; the same formula with the range on the positions' device
    from sharktank.layers.rotary_embedding import RotaryEmbeddingLayer

    def table_on_the_positions_device(self, t):
        dim = self.rope_dimension_count
        freqs = 1.0 / (self.rope_freq_base ** ((torch.arange(0, dim, device=t.device) // 2).float() / dim * 2.0))
        return torch.outer(t, freqs).float()

    RotaryEmbeddingLayer._compute_rotary_embed_table = table_on_the_positions_device
    reference = _build("cpu", kind, quantized=False)
    want_p, want_d, seq_lens = _prefill_and_decode(reference, "cpu")

    model = _build("cuda:0", kind, quantized=True)
    assert plugin.patch_moe_blocks(model) == BLOCKS
    assert all(isinstance(b, moe.B200MoeBlock) for b in model.moe_blocks)
    got_p, got_d, _ = _prefill_and_decode(model, "cuda:0")
    assert moe.device_status() == 0
    # positions past a sequence's length are padding: compare the valid ones
    for b, n in enumerate(seq_lens.tolist()):
        assert orc.rel_l2(got_p[b, :n], want_p[b, :n]) < 2e-2
    assert orc.rel_l2(got_d, want_d) < 2e-2
    # the greedy tokens the driver would pick (causal_llm.py extract_tokens_from_logits)
    for b, n in enumerate(seq_lens.tolist()):
        assert int(got_p[b, n - 1].argmax()) == int(want_p[b, n - 1].argmax())
    assert torch.equal(got_d.argmax(-1), want_d.argmax(-1))

    # the attention blocks as well: rotary + paged-KV write and the paged decode
    # attention from this library, projections and prefill core from torch
    from shark_platform_b200 import attention

    assert attention.patch_attention_blocks(model) == BLOCKS
    assert all(isinstance(b, attention.B200PagedAttentionBlock) for b in model.attn_blocks)
    got_p2, got_d2, _ = _prefill_and_decode(model, "cuda:0")
    assert moe.device_status() == 0
    for b, n in enumerate(seq_lens.tolist()):
        assert orc.rel_l2(got_p2[b, :n], want_p[b, :n]) < 2e-2
    assert orc.rel_l2(got_d2, want_d) < 2e-2
    assert torch.equal(got_d2.argmax(-1), want_d.argmax(-1))
