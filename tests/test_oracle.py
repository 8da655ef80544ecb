"""The CPU oracle against the reference: golden fixtures made by running
sharktank itself, the reference's known-answer vectors for the bit helpers
(sharktank/tests/types/layout_utils_test.py:14-94) and `gguf.quants`."""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as orc
from shark_platform_b200 import synthetic as syn
from helpers import case_digest, load_golden, oracle_params

MOE_CASES = ["toy", "small_q8", "small_q4k", "small_q41", "small_grok", "small_top4", "small_dense"]


# ---- known-answer vectors from the reference's own tests -------------------
def test_kat_linearize_and_interleave_i4():
    src = np.array([[0x80, 0x91, 0xA2, 0xB3, 0xC4, 0xD5, 0xE6, 0xF7]], dtype=np.uint8)
    lin = orc.deinterleave_i4(src)
    assert lin.tolist() == [[0x10, 0x32, 0x54, 0x76, 0x98, 0xBA, 0xDC, 0xFE]]
    assert orc.interleave_i4(lin).tolist() == src.tolist()


def test_kat_promote_i4():
    lin = np.array([[0x10, 0x32, 0x54, 0x76, 0x98, 0xBA, 0xDC, 0xFE]], dtype=np.uint8)
    assert orc.unpack_i4(lin).tolist() == [list(range(16))]
    assert orc.unpack_i4(lin, signed=True).tolist() == [
        [0, 1, 2, 3, 4, 5, 6, 7, -8, -7, -6, -5, -4, -3, -2, -1]
    ]


def test_kat_promote_i2():
    data = np.array([[0xC1, 0xB2, 0xA3, 0x94, 0x85]], dtype=np.uint8)
    want = [[1, 0, 0, 3, 2, 0, 3, 2, 3, 0, 2, 2, 0, 1, 1, 2, 1, 1, 0, 2]]
    assert orc.unpack_i2(data).tolist() == want


def test_kat_promote_i6():
    high = np.array([[0xDC, 0xCD]], dtype=np.uint8)
    low = np.array([[0xCB, 0x32, 0x11, 0x76]], dtype=np.uint8)
    assert orc.unpack_i6(high, low).tolist() == [
        [0xB, 0x3C, 0x12, 0x33, 0x11, 0x31, 0x6, 0x37]
    ]


# ---- fixtures produced by the reference -----------------------------------
def test_bit_helpers_match_reference_outputs():
    g = load_golden("formats.npz")
    b = g["bits_in"]
    assert np.array_equal(orc.deinterleave_i4(b), g["bits_linearize_i4"])
    assert np.array_equal(orc.interleave_i4(b), g["bits_interleave_i4"])
    assert np.array_equal(orc.unpack_i4(b), g["bits_i4_unsigned"])
    assert np.array_equal(orc.unpack_i4(b, signed=True), g["bits_i4_signed"])
    assert np.array_equal(orc.unpack_i2(b), g["bits_i2"])
    assert np.array_equal(orc.unpack_i6(b[:, :4], b[:, 8:16]), g["bits_i6"])


def test_q8_0_unpack_and_dequant_match_reference():
    g = load_golden("formats.npz")
    shape = [6, 512]
    planes = orc.q8_0_unpack(g["q8_raw"], shape)
    assert np.array_equal(planes["d"].view(np.uint16), g["q8_d"].view(np.uint16))
    assert np.array_equal(planes["qs"], g["q8_qs"])
    f16 = orc.q8_0_dequant(planes)
    assert f16.dtype == np.float16
    assert np.array_equal(f16.view(np.uint16), g["q8_dequant_f16"].view(np.uint16))
    f32 = orc.q8_0_dequant(planes, np.float32)
    assert np.array_equal(f32.view(np.uint32), g["q8_dequant_f32"].view(np.uint32))


def test_q4_k_unpack_and_dequant_match_reference():
    g = load_golden("formats.npz")
    shape = [6, 512]
    planes = orc.q4_k_unpack(g["q4k_raw"], shape)
    for name in ("sb_scales_high", "sb_scales_low", "sb_mins_high", "sb_mins_low", "qs"):
        assert np.array_equal(planes[name], g["q4k_" + name]), name
    for name in ("d", "dmin"):
        assert np.array_equal(planes[name].view(np.uint16), g["q4k_" + name].view(np.uint16))
    sc, mn, q = orc.q4_k_fields(planes)
    assert np.array_equal(sc, g["q4k_sb_scales"])
    assert np.array_equal(mn, g["q4k_sb_mins"])
    assert np.array_equal(q, g["q4k_qs_i8"])
    w = orc.q4_k_dequant(planes)
    assert np.array_equal(w.view(np.uint16), g["q4k_dequant_f16"].view(np.uint16))


def test_formats_match_gguf_package():
    """Independent pin: ggml's own dequantisation as shipped in `gguf`."""
    quants = pytest.importorskip("gguf.quants")
    import gguf

    g = load_golden("formats.npz")
    want8 = quants.dequantize(g["q8_raw"].reshape(6, -1), gguf.GGMLQuantizationType.Q8_0)
    got8 = orc.q8_0_dequant(orc.q8_0_unpack(g["q8_raw"], [6, 512]), np.float32)
    assert np.array_equal(got8, want8)
    want4 = quants.dequantize(g["q4k_raw"].reshape(6, -1), gguf.GGMLQuantizationType.Q4_K)
    got4 = orc.q4_k_dequant_f32(orc.q4_k_unpack(g["q4k_raw"], [6, 512]))
    assert np.array_equal(got4, want4)


@pytest.mark.parametrize("name", MOE_CASES)
def test_moe_block_matches_reference(name):
    g = load_golden(f"moe_{name}.npz")
    case = syn.make_case(syn.CASES[name])
    assert case_digest(case) == str(g["digest"]), "synthetic generator drifted"
    p = oracle_params(case)
    y, mid = orc.moe_block(case.h, p, form="pregather")
    assert np.array_equal(mid["experts"].numpy(), g["experts"])
    assert np.array_equal(mid["gate"].numpy(), g["gate"])
    assert np.array_equal(mid["xn"].numpy(), g["xn"])
    assert np.array_equal(y.numpy(), g["y"])  # same operators, same order: bit-equal
    # the per-expert formulation is the same layer up to fp32 summation order
    y2, _ = orc.moe_block(case.h, p, form="per_expert")
    assert orc.rel_l2(y2, y) < 1e-5
    assert orc.topk_margin(mid["prob"], case.spec.top_k) > 1e-6


def test_route_plan_definition():
    ex = torch.tensor([[3, 1], [1, 0], [3, 2], [1, 3]])
    counts, seg, perm, inv = orc.route_plan(ex, 5)
    assert counts.tolist() == [1, 3, 1, 3, 0]
    assert seg.tolist() == [0, 1, 4, 5, 8, 8]
    assert perm.tolist() == [3, 1, 2, 6, 5, 0, 4, 7]
    assert inv[perm].tolist() == list(range(8))


# ---- the multi-threaded torch restatements used for full-size layers --------
@pytest.mark.parametrize("kind", [syn.Q8_0, syn.Q4_K])
def test_torch_dequant_equals_the_pinned_numpy_dequant(kind):
    gen = torch.Generator().manual_seed(21)
    mk = syn.q8_0_planes if kind == syn.Q8_0 else syn.q4_k_planes
    planes = mk(gen, 3, 24, 1024)
    want = orc.dequant(kind, {k: v.numpy() for k, v in planes.items()})
    got = orc.dequant_torch(kind, planes).numpy()
    assert got.shape == want.shape
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    g = load_golden("formats.npz")  # and on the reference-made fixture planes
    if kind == syn.Q8_0:
        t = orc.q8_0_dequant_torch({"d": torch.from_numpy(g["q8_d"]), "qs": torch.from_numpy(g["q8_qs"])})
        assert np.array_equal(t.numpy().view(np.uint16), g["q8_dequant_f16"].view(np.uint16))
    else:
        names = ("d", "dmin", "sb_scales_high", "sb_scales_low", "sb_mins_high", "sb_mins_low", "qs")
        t = orc.q4_k_dequant_torch({n: torch.from_numpy(np.ascontiguousarray(g["q4k_" + n])) for n in names})
        assert np.array_equal(t.numpy().view(np.uint16), g["q4k_dequant_f16"].view(np.uint16))


@pytest.mark.parametrize("name", ["small_q8", "small_grok", "small_top4"])
def test_sampled_streamed_evaluation_equals_the_full_one(name):
    case = syn.make_case(syn.CASES[name])
    p = oracle_params(case)
    want, mid = orc.moe_block(case.h, p, form="pregather")
    sel = torch.tensor([0, 3, 4, case.spec.tokens - 1])
    got, mid2 = orc.moe_block_sampled(case.h, p, lambda e: (p.w_gate[e], p.w_up[e], p.w_down[e]), sel)
    assert torch.equal(mid2["experts"], mid["experts"])
    assert orc.rel_l2(got, want.view(-1, case.spec.hidden)[sel]) < 1e-6


def test_oracle_follows_the_reference_on_bf16_activations():
    """With bf16 `h` the reference rounds the normalised row, the router logits
    and the expert weights to bf16 (layers/norm.py:39-41, ops/default_impls.py:
    332-333, :351).  The oracle makes the same casts: indices and outputs equal
    the fixture sharktank produced."""
    g = load_golden("moe_bf16act.npz")
    spec = syn.CaseSpec("bf16act", 512, 256, 512, kind=syn.Q8_0, norm_weight="perturbed", seed=21)
    case = syn.make_case(spec)
    assert case_digest(case) == str(g["digest"])
    y, mid = orc.moe_block(case.h.to(torch.bfloat16), oracle_params(case), form="pregather")
    assert np.array_equal(mid["experts"].numpy(), g["experts"])
    assert y.dtype == torch.bfloat16
    assert orc.rel_l2(y.float(), torch.from_numpy(g["y"])) < 1e-6


def test_q4_1_dequant_matches_reference():
    """BlockScaledI4Layout with offsets (GGUF Q4_1), the one quantized MoE layout
    the reference itself can index (ops/default_impls.py:204-218)."""
    g = load_golden("formats.npz")
    got = orc.q4_1_dequant({"d": g["q41_d"], "m": g["q41_m"], "qs": g["q41_qs"]})
    assert np.array_equal(got.view(np.uint16), g["q41_dequant_f16"].view(np.uint16))
