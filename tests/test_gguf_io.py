"""GGUF loader: file structure on the CPU, GPU unpack against the oracle.

Mirrors what the reference's loader promises
(sharktank/types/gguf_interop/base.py:141-163): reversed shapes, packed Q8_0 /
Q4_K tensor classes, dense tensors as DefaultPrimitiveTensor, key/value fields
as Python values.
"""
import os

import numpy as np
import pytest
import torch

from oracle import moe_oracle as orc
from shark_platform_b200 import gguf_io
from shark_platform_b200 import types as T

gguf = pytest.importorskip("gguf")

E, F, D = 8, 256, 256  # experts, ffn, hidden of the file's single MoE layer


def _raw_q8(rng, *lead, k):
    nb = int(np.prod(lead)) * k // 32
    raw = rng.integers(0, 256, size=(nb, 34), dtype=np.uint8)
    d = (np.abs(rng.standard_normal(nb)) * 0.002).astype(np.float16)
    raw[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    return raw.reshape(*lead, k // 32 * 34)


def _raw_q4k(rng, *lead, k):
    nb = int(np.prod(lead)) * k // 256
    raw = rng.integers(0, 256, size=(nb, 144), dtype=np.uint8)
    dd = (np.abs(rng.standard_normal((nb, 2))) * [2.5e-4, 2e-3]).astype(np.float16)
    raw[:, 0:4] = dd.view(np.uint8).reshape(-1, 4)
    return raw.reshape(*lead, k // 256 * 144)


def write_file(path, kind, seed=21):
    """One MoE layer (blk.0) with packed expert weights of `kind`."""
    from gguf import GGMLQuantizationType as QT
    from gguf import GGUFWriter

    rng = np.random.default_rng(seed)
    mk, qt = (_raw_q8, QT.Q8_0) if kind == "Q8_0" else (_raw_q4k, QT.Q4_K)
    raws = {
        "blk.0.ffn_gate_exps.weight": (mk(rng, E, F, k=D), [E, F, D]),
        "blk.0.ffn_up_exps.weight": (mk(rng, E, F, k=D), [E, F, D]),
        "blk.0.ffn_down_exps.weight": (mk(rng, E, D, k=F), [E, D, F]),
    }
    dense = {
        "blk.0.ffn_gate_inp.weight": (rng.standard_normal((E, D)) * 0.02).astype(np.float32),
        "blk.0.ffn_norm.weight": (1.0 + 0.1 * rng.standard_normal(D)).astype(np.float32),
        "token_embd.weight": rng.standard_normal((16, D)).astype(np.float16),
    }
    w = GGUFWriter(path, "llama")
    w.add_uint32("llama.expert_count", E)
    w.add_uint32("llama.expert_used_count", 2)
    w.add_float32("llama.attention.layer_norm_rms_epsilon", 1e-5)
    w.add_string("general.name", "tiny-moe")
    w.add_array("tokenizer.ggml.tokens", ["a", "b", "c"])
    w.add_array("some.ints", [3, 1, 4])
    for name, (raw, _) in raws.items():
        w.add_tensor(name, raw, raw_dtype=qt)
    for name, arr in dense.items():
        w.add_tensor(name, arr)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    return raws, dense


@pytest.mark.parametrize("kind", ["Q8_0", "Q4_K"])
def test_load_file_structure_on_cpu(tmp_path, kind):
    path = os.path.join(tmp_path, "m.gguf")
    raws, dense = write_file(path, kind)
    ds = gguf_io.load_file(path, device="cpu")
    p = ds.properties
    assert p["schema"] == "GGUF"
    assert p["general.architecture"] == "llama" and p["general.name"] == "tiny-moe"
    assert p["llama.expert_count"] == E and isinstance(p["llama.expert_count"], int)
    assert abs(p["llama.attention.layer_norm_rms_epsilon"] - 1e-5) < 1e-12
    assert p["tokenizer.ggml.tokens"] == ["a", "b", "c"] and p["some.ints"] == [3, 1, 4]

    flat = ds.root_theta.flatten()
    assert set(flat) == set(raws) | set(dense)
    blk = ds.root_theta("blk", 0)
    cls = gguf_io.Q8_0 if kind == "Q8_0" else gguf_io.Q4_K
    lay = T.BlockScaledLayout if kind == "Q8_0" else T.SuperBlockOffsetScaled_4_6_Layout
    for name, (raw, shape) in raws.items():
        t = flat[name]
        assert isinstance(t, cls) and isinstance(t, T.QuantizedTensor)
        assert t.name == name and t.shape == shape and t.layout_type is lay
        assert np.array_equal(t.raw.numpy(), raw.reshape(-1))
    assert blk.tensor("ffn_gate_exps", "weight") is flat["blk.0.ffn_gate_exps.weight"]
    for name, arr in dense.items():
        t = flat[name]
        assert isinstance(t, T.DefaultPrimitiveTensor) and t.shape == list(arr.shape)
        assert np.array_equal(t.as_torch().numpy(), arr)


def test_packed_tensors_reject_inconsistent_sizes():
    raw = np.zeros(34 * 4, dtype=np.uint8)
    with pytest.raises(ValueError):
        gguf_io.Q8_0(raw=raw, shape=[4, 48])  # 48 is not a multiple of 32
    with pytest.raises(ValueError):
        gguf_io.Q8_0(raw=raw, shape=[8, 32])  # 8 blocks expected, 4 given
    with pytest.raises(ValueError):
        gguf_io.Q4_K(raw=np.zeros(144, dtype=np.uint8), shape=[2, 256])
    with pytest.raises(ValueError):
        gguf_io.wrap_tensor("x", [32, 2], "Q6_K", np.zeros(10, dtype=np.uint8), device="cpu")


def test_wrap_tensor_bf16_and_reversed_shape():
    vals = torch.randn(3, 8).to(torch.bfloat16)
    data = vals.view(torch.int16).numpy().view(np.uint8).reshape(-1)
    t = gguf_io.wrap_tensor("w", [8, 3], "BF16", data, device="cpu")
    assert t.shape == [3, 8] and t.as_torch().dtype == torch.bfloat16
    assert torch.equal(t.as_torch(), vals)


# ------------------------------------------------------------------ GPU
@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["Q8_0", "Q4_K"])
def test_unpack_on_gpu_matches_oracle_planes(tmp_path, kind):
    path = os.path.join(tmp_path, "m.gguf")
    raws, _ = write_file(path, kind)
    ds = gguf_io.load_file(path)
    unpack = orc.q8_0_unpack if kind == "Q8_0" else orc.q4_k_unpack
    for name, (raw, shape) in raws.items():
        lay = ds.root_theta.flatten()[name].unpack()
        want = unpack(raw.reshape(-1), shape)
        assert set(lay.planes) == set(want)
        for key, plane in lay.planes.items():
            got = plane.cpu().numpy()
            assert list(got.shape) == list(want[key].shape), (name, key)
            assert np.array_equal(got.view(np.uint8), np.ascontiguousarray(want[key]).view(np.uint8)), (name, key)


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["Q8_0", "Q4_K"])
def test_moe_block_from_gguf_file(tmp_path, kind):
    """A layer built from the file's theta gives the oracle's result and the
    same bits as one built from host-unpacked planes."""
    import torch.nn.functional as Fn

    from shark_platform_b200 import synthetic as syn
    from shark_platform_b200.moe import B200MoeBlock

    path = os.path.join(tmp_path, "m.gguf")
    raws, dense = write_file(path, kind)
    ds = gguf_io.load_file(path)
    theta = ds.root_theta("blk", 0)
    k = ds.properties["llama.expert_used_count"]
    eps = ds.properties["llama.attention.layer_norm_rms_epsilon"]
    blk = B200MoeBlock(theta, E, k, eps, Fn.silu)

    unpack = orc.q8_0_unpack if kind == "Q8_0" else orc.q4_k_unpack
    planes = {n: unpack(raw.reshape(-1), shape) for n, (raw, shape) in raws.items()}

    def planar(name):
        raw, shape = raws[name]
        p = {key: torch.from_numpy(np.ascontiguousarray(v)).cuda() for key, v in planes[name].items()}
        lay = (T.BlockScaledLayout(shape, p["d"], p["qs"]) if kind == "Q8_0"
               else T.SuperBlockOffsetScaled_4_6_Layout(shape, **p))
        return T.PlanarQuantizedTensor(shape=shape, layout=lay)

    tree = {
        "ffn_gate_inp": {"weight": T.DefaultPrimitiveTensor(data=torch.from_numpy(dense["blk.0.ffn_gate_inp.weight"]).cuda())},
        "ffn_norm": {"weight": T.DefaultPrimitiveTensor(data=torch.from_numpy(dense["blk.0.ffn_norm.weight"]).cuda())},
        "ffn_gate_exps": {"weight": planar("blk.0.ffn_gate_exps.weight")},
        "ffn_up_exps": {"weight": planar("blk.0.ffn_up_exps.weight")},
        "ffn_down_exps": {"weight": planar("blk.0.ffn_down_exps.weight")},
    }
    blk2 = B200MoeBlock(T.Theta(tree), E, k, eps, Fn.silu)

    gen = torch.Generator().manual_seed(3)
    h = torch.randn(1, 37, D, generator=gen).to(torch.bfloat16)
    y = blk(h.cuda())
    y2 = blk2(h.cuda())
    assert torch.equal(y, y2)

    okind = syn.Q8_0 if kind == "Q8_0" else syn.Q4_K
    deq = lambda n: torch.from_numpy(orc.dequant(okind, planes[n]))
    params = orc.MoeParams(
        norm_w=torch.from_numpy(dense["blk.0.ffn_norm.weight"]),
        router_w=torch.from_numpy(dense["blk.0.ffn_gate_inp.weight"]),
        router_b=None, out_norm_w=None,
        w_gate=deq("blk.0.ffn_gate_exps.weight"), w_up=deq("blk.0.ffn_up_exps.weight"),
        w_down=deq("blk.0.ffn_down_exps.weight"),
        top_k=k, eps=eps, activation="silu",
    )
    want, mid = orc.moe_block(h.float(), params, form="per_expert")
    assert orc.topk_margin(mid["prob"], k) > 1e-5  # the routing decision is well defined
    assert orc.rel_l2(y.float().cpu(), want) <= 2e-2
