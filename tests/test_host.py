"""Host-side logic that needs no GPU: the C ABI loads and exports what the
header declares, the registry mirror follows the reference's dispatch rules,
the type mirror behaves like sharktank's containers."""
import os
import sys

import pytest
import torch

from helpers import import_sharktank, reference_path


@pytest.fixture(scope="module", autouse=True)
def built_library():
    from shark_platform_b200 import build

    build.build()


def test_cabi_exports_every_declared_symbol():
    from shark_platform_b200 import _cabi as C

    names = C.declared_symbols()
    assert len(names) >= 18
    for n in names:
        assert hasattr(C.lib, n), n
        assert n in C._PROTOS, f"{n} has no ctypes prototype"
    assert set(C._PROTOS) == set(names)
    assert b"sm_100a" in C.lib.b200moe_version()


def test_registry_salience_order_and_decline():
    from shark_platform_b200 import ops

    disp = ops.SignatureDispatcher(lambda a, b: None, (0, 1))
    calls = []

    @disp.override(torch.Tensor, torch.Tensor)
    def base(a, b):
        calls.append("base")
        return "base"

    @disp.override(torch.Tensor, torch.Tensor)
    def later(a, b):
        calls.append("later")
        return NotImplemented

    @disp.override(torch.Tensor, torch.Tensor, salience=5)
    def salient(a, b):
        calls.append("salient")
        return NotImplemented

    x = torch.zeros(1)
    assert disp(x, x) == "base"
    assert calls == ["salient", "later", "base"]  # salience first, then latest registered
    with pytest.raises(NotImplementedError):
        disp(x, 3)


def test_overrides_are_registered_in_the_mirror():
    from shark_platform_b200 import moe, ops, types as T

    lay = T.BlockScaledLayout([2, 64, 256], torch.zeros(2, 64, 8, 1, dtype=torch.float16),
                              torch.zeros(2, 64, 8, 32, dtype=torch.int8))
    q = T.PlanarQuantizedTensor(shape=[2, 64, 256], layout=lay)
    assert moe.get_index_quantized in list(ops.get_index.find_overrides((q,)))
    # CPU index tensors are declined, never computed on the host
    with pytest.raises(NotImplementedError):
        q[torch.zeros(3, 2, dtype=torch.int64), :, :]
    g = moe.GatheredExperts(q, torch.zeros(3, 2, dtype=torch.int64))
    assert g.shape == [3, 2, 64, 256]
    assert moe.einsum_2args_gathered in list(ops.einsum_2args.find_overrides((torch.zeros(1), g)))
    with pytest.raises(NotImplementedError):
        ops.einsum_2args(torch.zeros(3, 256), g, "mk,menk->men")  # CPU activations: declined


def test_theta_mirror_matches_reference_accessors():
    from shark_platform_b200 import types as T

    w = T.DefaultPrimitiveTensor(data=torch.ones(4))
    th = T.Theta({"ffn_norm": {"weight": w}, "ffn_gate_inp": {"weight": w, "bias": w}})
    assert th.tensor("ffn_norm", "weight") is w
    assert th("ffn_gate_inp").tensor("bias") is w
    assert th.optional_tensor("layer_output_norm") is None
    assert th.optional_tensor("ffn_norm") is not None
    assert "bias" in th("ffn_gate_inp").keys
    with pytest.raises(KeyError):
        th.tensor("nope", "weight")


def test_product_never_imports_the_oracle():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    pkg = os.path.join(root, "shark_platform_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.replace("# oracle", ""), f"{f} mentions the oracle"


@pytest.mark.skipif(reference_path() is None, reason="sharktank not available ($SHARKTANK_SRC or baseline/_ref)")
def test_plugin_registers_ahead_of_sharktank_overrides():
    import_sharktank()
    import sharktank.ops as st_ops
    from sharktank.types import PlanarQuantizedTensor
    from sharktank.types.layouts import BlockScaledLayout

    from shark_platform_b200 import moe, plugin

    plugin.register()
    lay = BlockScaledLayout([2, 64, 256], torch.zeros(2, 64, 8, 1, dtype=torch.float16),
                            torch.zeros(2, 64, 8, 32, dtype=torch.int8))
    q = PlanarQuantizedTensor(shape=[2, 64, 256], layout=lay)
    first = next(iter(st_ops.get_index.find_overrides((q,))))
    assert first is moe.get_index_quantized
    g = moe.GatheredExperts(q, torch.zeros(3, 2, dtype=torch.int64))
    first = next(iter(st_ops.einsum_2args.find_overrides((torch.zeros(1), g))))
    assert first is moe.einsum_2args_gathered
    # CPU tensors: our overrides decline and the reference's own error surfaces
    with pytest.raises(NotImplementedError):
        q[torch.zeros(3, 2, dtype=torch.int64), :, :]
    # dense quantized linear / matmul: consulted first, declined on the CPU, after
    # which dispatch goes on to the reference's own IREE kernel (stubbed out here)
    lay2 = BlockScaledLayout([256, 256], torch.ones(256, 8, 1, dtype=torch.float16),
                             torch.ones(256, 8, 32, dtype=torch.int8))
    q2 = PlanarQuantizedTensor(shape=[256, 256], layout=lay2)
    x = torch.ones(3, 256)
    assert next(iter(st_ops.matmul.find_overrides((x, q2)))) is moe.matmul_quantized
    assert next(iter(st_ops.linear.find_overrides((x, q2)))) is moe.linear_quantized
    with pytest.raises(RuntimeError, match="mmt_block_scaled_q8 unavailable"):
        st_ops.linear(x, q2)


def _desc(layout, experts, rows, cols):
    from shark_platform_b200 import _cabi as C

    return C.WeightDesc(layout, experts, rows, cols, 16, 16, 16)


def test_down_ksplit_heuristics_need_no_gpu():
    """Pure host arithmetic behind b200moe_down_ksplit (148 SMs assumed without a device)."""
    import ctypes

    from shark_platform_b200 import _cabi as C

    mixtral_down = _desc(C.LAYOUT_Q8_0, 8, 4096, 14336)
    ks = lambda d, pairs, seg, regime: C.lib.b200moe_down_ksplit(ctypes.byref(d), pairs, seg, regime)
    assert ks(mixtral_down, 64, 32, C.REGIME_STREAM) == 4      # decode: 1024 items = 6.9 waves
    assert ks(mixtral_down, 8192, 4096, C.REGIME_STREAM) == 1  # many rows: no partials
    assert ks(mixtral_down, 8192, 4096, C.REGIME_AUTO) == 1    # prefill, 768 tiles >= 2 waves
    one_expert = _desc(C.LAYOUT_Q8_0, 1, 4096, 14336)
    assert ks(one_expert, 1024, 4096, C.REGIME_AUTO) == 4      # one expert per rank: 96 tiles
    small_k = _desc(C.LAYOUT_Q8_0, 8, 256, 512)
    assert ks(small_k, 64, 32, C.REGIME_STREAM) == 1           # two stages only


def test_kperm_and_workspace_need_no_gpu():
    import ctypes

    from shark_platform_b200 import _cabi as C

    assert C.lib.b200moe_kperm(C.LAYOUT_Q8_0, C.REGIME_AUTO, 32) == 0
    assert C.lib.b200moe_kperm(C.LAYOUT_Q4_K, C.REGIME_AUTO, 32) == 1
    assert C.lib.b200moe_kperm(C.LAYOUT_Q4_K, C.REGIME_TENSOR, 4096) == 1
    layer = C.LayerDesc()
    layer.hidden, layer.ffn, layer.experts, layer.top_k = 4096, 14336, 8, 2
    layer.gate = _desc(C.LAYOUT_Q8_0, 8, 14336, 4096)
    layer.up = _desc(C.LAYOUT_Q8_0, 8, 14336, 4096)
    layer.down = _desc(C.LAYOUT_Q8_0, 8, 4096, 14336)
    small = C.lib.b200moe_workspace_bytes(ctypes.byref(layer), 32)
    big = C.lib.b200moe_workspace_bytes(ctypes.byref(layer), 4096)
    # xs + A + D dominate: pairs * (d*2 + F*2 + ksplit*d*4) bytes
    assert 64 * (4096 * 2 + 14336 * 2 + 4 * 4096 * 4) <= small < 16 * 2**20
    assert 8192 * (4096 * 2 + 14336 * 2 + 4096 * 4) <= big < 600 * 2**20
    assert C.lib.b200moe_workspace_bytes(None, 32) == 0


def test_entry_points_reject_bad_arguments_without_touching_the_gpu():
    import ctypes

    from shark_platform_b200 import _cabi as C

    dummy = ctypes.c_void_p(256)
    bad = _desc(7, 8, 256, 512)  # unknown layout
    rc = C.lib.b200moe_dequant(ctypes.byref(bad), C.DT_F16, dummy, None)
    assert rc == -1 and "unknown layout" in C.last_error()
    rc = C.lib.b200moe_gate_up(dummy, dummy, 8, 8, None, None, 0, 0, 0, dummy, None)
    assert rc == -1 and "NULL" in C.last_error()
    ep = C.EpDesc()
    ep.world, ep.rank, ep.experts_local = 40, 0, 1
    rc = C.lib.b200moe_ep_barrier(ctypes.byref(ep), 1, None, None)
    assert rc == -1 and "out of range" in C.last_error()
    with pytest.raises(C.B200MoeError):
        C.check(rc, "ep_barrier")


def test_patch_moe_blocks_leaves_other_modules_alone():
    from shark_platform_b200 import plugin

    model = torch.nn.Sequential(torch.nn.Linear(4, 4), torch.nn.ReLU())
    assert plugin.patch_moe_blocks(model) == 0
    assert isinstance(model[0], torch.nn.Linear)


def test_debug_flags_parse_like_the_reference_switch():
    """B200MOE_DEBUG uses the `[+|-]name[=value]` list syntax of sharktank's
    TURBINE_LLM_DEBUG (utils/debugging.py:28-83)."""
    from shark_platform_b200 import debugging as dbg

    f = dbg.DebugFlags.parse("tensor_trace, +nvtx,-nan_checks,dump_path=/tmp/b200moe_dump")
    assert f.tensor_trace and f.nvtx and not f.nan_checks and str(f.dump_path) == "/tmp/b200moe_dump" and f.any
    assert not dbg.DebugFlags.parse("").any
    with pytest.raises(ValueError):
        dbg.DebugFlags.parse("no_such_flag")
