"""Host side of the MoE FFN path: weight preparation, the staged calls into the
C ABI, the fused `B200MoeBlock`, and the op-level overrides.

Two ways in, mirroring how the reference layer is written:

* `B200MoeBlock(theta, expert_count, expert_used_count, rms_epsilon,
  moe_activation)` has the constructor and `forward(h)` of sharktank's
  `MoeBlock` (layers/mixture_of_experts_block.py:23-90) and runs the whole layer
  as one library call.
* `get_index` / `einsum_2args` overrides make sharktank's own
  `PreGatherFFNMOE.forward` (layers/ffn_moe_block.py:60-74) work on quantized
  expert tensors: `weights[experts, :, :]` returns a lazy `GatheredExperts`
  handle instead of a dense copy, and the three MoE einsums run as grouped
  products over the permuted tokens.

Everything computes on the GPU through libb200moe; tensors on the CPU are
declined (`NotImplemented`) or rejected, never evaluated.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Any, Optional

import torch
import torch.nn.functional as F

from . import _cabi as C
from . import debugging as _debug
from . import ops as _ops

_DT = {torch.float32: C.DT_F32, torch.float16: C.DT_F16, torch.bfloat16: C.DT_BF16}
REGIMES = {"auto": C.REGIME_AUTO, "stream": C.REGIME_STREAM, "tensor": C.REGIME_TENSOR,
           "tensor_pair": C.REGIME_TENSOR_PAIR}


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _require_cuda(t: torch.Tensor, what: str):
    if not t.is_cuda:
        raise C.B200MoeError(f"{what} must be a CUDA tensor (there is no CPU path)")


def device_status() -> int:
    """Reads and clears the device status word; raises if a kernel reported an
    error (bounded wait timed out, bounds check failed)."""
    st = ctypes.c_int32(0)
    C.check(C.lib.b200moe_device_status(_stream(), ctypes.byref(st)), "device_status")
    return st.value


# ---------------------------------------------------------------- weights
@dataclass
class PreparedWeight:
    """Device buffers of one stacked expert tensor plus its C descriptor."""

    desc: C.WeightDesc
    layout: int
    experts: int
    rows: int
    cols: int
    keep: tuple  # tensors the descriptor points into

    @property
    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.keep)


def _layout_name(t) -> Optional[str]:
    lt = getattr(t, "layout_type", None)
    return getattr(lt, "__name__", None)


def _unbox(t) -> torch.Tensor:
    if isinstance(t, torch.Tensor):
        return t
    if hasattr(t, "as_torch"):
        return t.as_torch()
    raise TypeError(f"expected a tensor, got {type(t).__name__}")


def prepare_weight(t: Any, tile_scales: bool = True) -> PreparedWeight:
    """Turns `ffn_*_exps.weight` (a PlanarQuantizedTensor with a Q8_0 /
    Q4_K planar layout — sharktank's or this package's — or a dense tensor) into
    the descriptor the kernels take.  Q8_0 planes are used in place; Q4_K gets
    one derived array (per-sub-block scale/min pairs).  The result is cached on
    the tensor object."""
    cached = getattr(t, "_b200moe_prepared", None)
    if cached is not None:
        return cached
    name = _layout_name(t)
    if name is None:
        w = _unbox(t)
        _require_cuda(w, "expert weight")
        assert w.dim() == 3, "expert weights are [experts, rows, cols]"
        w16 = w.to(torch.float16).contiguous()
        e, n, k = w16.shape
        desc = C.WeightDesc(C.LAYOUT_F16, e, n, k, w16.data_ptr(), None, None)
        prep = PreparedWeight(desc, C.LAYOUT_F16, e, n, k, (w16,))
    else:
        e, n, k = (int(v) for v in t.shape)
        planes = t.unpack().planes
        for p in planes.values():
            _require_cuda(p, "expert weight plane")
        if name == "BlockScaledLayout":
            if "m" in planes:
                raise C.B200MoeError("BlockScaledLayout with offsets is not supported")
            qs = planes["qs"].contiguous().view(torch.int8)
            d = planes["d"].contiguous()
            assert d.dtype == torch.float16 and qs.numel() == e * n * k and d.numel() == e * n * k // 32
            sub = None
            if k % 256 == 0 and tile_scales:
                sub = torch.empty_like(d)
                with torch.cuda.device(qs.device):
                    C.check(C.lib.b200moe_q8_prepare(_ptr(d), e * n, k, _ptr(sub), _stream()),
                            "q8_prepare")
            desc = C.WeightDesc(C.LAYOUT_Q8_0, e, n, k, qs.data_ptr(), d.data_ptr(),
                                None if sub is None else sub.data_ptr())
            prep = PreparedWeight(desc, C.LAYOUT_Q8_0, e, n, k, (qs, d) + ((sub,) if sub is not None else ()))
        elif name == "SuperBlockOffsetScaled_4_6_Layout":
            qs = planes["qs"].contiguous().view(torch.uint8)
            assert qs.numel() == e * n * k // 2
            blocks = e * n * k // 256
            sub = torch.empty(blocks * 8, 2, dtype=torch.float16, device=qs.device)
            args = [planes[nm].contiguous() for nm in
                    ("d", "dmin", "sb_scales_high", "sb_scales_low", "sb_mins_high", "sb_mins_low")]
            with torch.cuda.device(qs.device):
                C.check(C.lib.b200moe_q4k_prepare(*[_ptr(a) for a in args], blocks, _ptr(sub),
                                                  _stream()), "q4k_prepare")
            desc = C.WeightDesc(C.LAYOUT_Q4_K, e, n, k, qs.data_ptr(), None, sub.data_ptr())
            prep = PreparedWeight(desc, C.LAYOUT_Q4_K, e, n, k, (qs, sub))
        elif name == "BlockScaledI4Layout":
            # GGUF Q4_1: w = fp16(fp16(d*q) + m) per block of 32, two quants per byte,
            # low nibble first — the nibble order of the Q4_K planar plane and the
            # same two roundings as its fp16(fp16(ds*q) - dm), so it runs on the Q4_K
            # kernels with the per-block pairs (d, -m)
            lay = t.unpack()
            if getattr(lay, "signed", False):
                raise C.B200MoeError("signed BlockScaledI4Layout is not supported")
            if k % 256 != 0:
                raise C.B200MoeError(f"BlockScaledI4Layout: cols ({k}) must be a multiple of 256")
            qs = planes["qs"].contiguous().view(torch.uint8)
            d = planes["d"].contiguous().to(torch.float16).reshape(-1)
            assert qs.numel() == e * n * k // 2 and d.numel() == e * n * k // 32
            m = planes.get("m")
            neg_m = torch.zeros_like(d) if m is None else -m.contiguous().to(torch.float16).reshape(-1)
            sub = torch.stack([d, neg_m], dim=1).contiguous()
            desc = C.WeightDesc(C.LAYOUT_Q4_K, e, n, k, qs.data_ptr(), None, sub.data_ptr())
            prep = PreparedWeight(desc, C.LAYOUT_Q4_K, e, n, k, (qs, sub))
        else:
            raise C.B200MoeError(f"unsupported quantized layout {name}")
    try:
        t._b200moe_prepared = prep
    except AttributeError:
        pass
    return prep


def dequant_layout(layout, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """`layout.dequant(dtype)` on the GPU, bit-exact with the reference
    (types/layouts.py:274-290 and :505-517)."""

    class _Holder:
        pass

    h = _Holder()
    h.layout_type = type(layout)
    h.shape = list(layout.shape)
    h.unpack = lambda: layout
    shape = list(layout.shape)
    if len(shape) == 2:
        h.shape = [1] + shape
    elif len(shape) != 3:
        lead = 1
        for v in shape[:-2]:
            lead *= int(v)
        h.shape = [lead] + shape[-2:]
    if type(layout).__name__ == "BlockScaledI4Layout" and dtype not in (None, torch.float16):
        raise C.B200MoeError("BlockScaledI4Layout dequantises to fp16 only")
    prep = prepare_weight(h)
    is_q4k = prep.layout == C.LAYOUT_Q4_K
    out_dtype = torch.float16 if (dtype is None or is_q4k) else dtype
    if out_dtype not in (torch.float16, torch.float32):
        raise C.B200MoeError(f"dequant to {out_dtype} is not supported")
    dev = prep.keep[0].device
    out = torch.empty(shape, dtype=out_dtype, device=dev)
    with torch.cuda.device(dev):
        C.check(C.lib.b200moe_dequant(ctypes.byref(prep.desc), _DT[out_dtype], _ptr(out), _stream()),
                "dequant")
    return out


# ------------------------------------------------------------ staged calls
@dataclass
class RoutePlan:
    counts: torch.Tensor       # int32 [E_local]
    seg_offsets: torch.Tensor  # int32 [E_local + 1]
    perm: torch.Tensor         # int32 [pairs]: sorted position -> pair
    inv: torch.Tensor          # int32 [pairs]: pair -> sorted position (or -1)
    pairs: int
    top_k: int


def route_plan(experts: torch.Tensor, expert_count: int, expert_begin: int = 0) -> RoutePlan:
    """Stable grouping of (token, slot) pairs by expert id on the GPU."""
    _require_cuda(experts, "experts")
    ex = experts.to(torch.int32).contiguous()
    pairs = ex.numel()
    top_k = ex.shape[-1] if ex.dim() > 1 else 1
    dev = ex.device
    counts = torch.empty(expert_count, dtype=torch.int32, device=dev)
    seg = torch.empty(expert_count + 1, dtype=torch.int32, device=dev)
    # zero-filled: with an expert range that drops pairs, positions past the last
    # kept pair are not written and must still be valid row numbers
    perm = torch.zeros(max(pairs, 1), dtype=torch.int32, device=dev)
    inv = torch.empty(max(pairs, 1), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        C.check(C.lib.b200moe_route_plan(_ptr(ex), pairs, expert_begin, expert_count, _ptr(counts),
                                         _ptr(seg), _ptr(perm), _ptr(inv), _stream()), "route_plan")
    return RoutePlan(counts, seg, perm[:pairs], inv[:pairs], pairs, top_k)


def grouped_matmul(xs: torch.Tensor, plan_seg: torch.Tensor, w: PreparedWeight, max_segment: int,
                   regime: int = C.REGIME_AUTO) -> torch.Tensor:
    """out[p,:] = W[e(p)] @ xs[p,:] for rows p sorted by expert (fp16 in, fp32 out)."""
    pairs = xs.shape[0]
    dev = xs.device
    ks = C.lib.b200moe_down_ksplit(ctypes.byref(w.desc), pairs, max_segment, regime)
    part = torch.empty(ks, max(pairs, 1), w.rows, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        C.check(C.lib.b200moe_down(_ptr(xs), _ptr(plan_seg), pairs, max_segment,
                                   ctypes.byref(w.desc), regime, ks, _ptr(part), _stream()), "down")
    out = part[0] if ks == 1 else part.sum(dim=0)
    return out[:pairs]


# -------------------------------------------------------------- the layer
class PreparedLayer:
    """All device-side state of one MoE layer: descriptor, weights, workspace."""

    def __init__(self, theta, expert_count: int, expert_used_count: int, rms_epsilon: float,
                 activation: str):
        self.gate = prepare_weight(theta.tensor("ffn_gate_exps", "weight"))
        self.up = prepare_weight(theta.tensor("ffn_up_exps", "weight"))
        self.down = prepare_weight(theta.tensor("ffn_down_exps", "weight"))
        dev = self.gate.keep[0].device
        self.device = dev

        def f32(t):
            return None if t is None else _unbox(t).to(device=dev, dtype=torch.float32).contiguous()

        self.norm_w = f32(theta.tensor("ffn_norm", "weight"))
        router = theta("ffn_gate_inp")
        self.router_w = f32(router.tensor("weight"))
        self.router_b = f32(router.optional_tensor("bias")) if "bias" in router.keys else None
        self.out_norm_w = None
        if theta.optional_tensor("layer_output_norm") is not None:
            self.out_norm_w = f32(theta("layer_output_norm").tensor("weight"))
        self.expert_count = expert_count
        self.top_k = expert_used_count
        self.hidden = self.gate.cols
        self.ffn = self.gate.rows
        self.desc = C.LayerDesc(
            self.hidden, self.ffn, expert_count, expert_used_count,
            C.ACT_SILU if activation == "silu" else C.ACT_GELU, float(rms_epsilon),
            self.norm_w.data_ptr(), self.router_w.data_ptr(),
            None if self.router_b is None else self.router_b.data_ptr(),
            None if self.out_norm_w is None else self.out_norm_w.data_ptr(),
            self.gate.desc, self.up.desc, self.down.desc, 0,
        )
        self._workspace: Optional[torch.Tensor] = None
        self._workspace_tokens = 0

    def workspace(self, tokens: int) -> torch.Tensor:
        if self._workspace is None or tokens > self._workspace_tokens:
            nbytes = C.lib.b200moe_workspace_bytes(ctypes.byref(self.desc), tokens)
            self._workspace = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
            self._workspace_tokens = tokens
        return self._workspace

    def forward(self, h: torch.Tensor, regime: int = C.REGIME_AUTO, want_routing: bool = False):
        _require_cuda(h, "h")
        if h.dtype not in (torch.float32, torch.bfloat16):
            raise C.B200MoeError(f"activations must be fp32 or bf16, got {h.dtype}")
        shape = h.shape
        x = h.reshape(-1, shape[-1]).contiguous()
        tokens = x.shape[0]
        y = torch.empty_like(x)
        experts = gates = None
        if want_routing:
            experts = torch.empty(tokens, self.top_k, dtype=torch.int32, device=x.device)
            gates = torch.empty(tokens, self.top_k, dtype=torch.float32, device=x.device)
        ws = self.workspace(tokens)
        with torch.cuda.device(self.device):
            C.check(C.lib.b200moe_layer_forward(
                ctypes.byref(self.desc), _ptr(x), _ptr(y), _DT[x.dtype], tokens, regime, _ptr(ws),
                ws.numel(), _ptr(experts), _ptr(gates), _stream()), "layer_forward")
        y = y.reshape(shape)
        return (y, experts, gates) if want_routing else y


class HostPipeline:
    """Batches that live in (pinned) host memory, streamed through one layer
    with `depth` steps in flight: a step's input copy, its kernels and its
    output copy run on three streams, so consecutive steps overlap
    (`b200moe_pipeline_*`).  `submit(h_host, y_host)` returns at once; `y_host`
    is complete after `drain()` or once `depth` further steps were submitted."""

    def __init__(self, layer: PreparedLayer, max_tokens: int, dtype: torch.dtype, depth: int = 2,
                 regime: int = C.REGIME_AUTO):
        if dtype not in (torch.float32, torch.bfloat16):
            raise C.B200MoeError(f"activations must be fp32 or bf16, got {dtype}")
        self.layer, self.dtype, self.max_tokens = layer, dtype, max_tokens
        nbytes = C.lib.b200moe_pipeline_bytes(ctypes.byref(layer.desc), _DT[dtype], max_tokens, depth)
        if nbytes == 0:
            raise C.B200MoeError("pipeline: bad size or depth (1..8)")
        self._mem = torch.empty(nbytes, dtype=torch.uint8, device=layer.device)
        self._handle = ctypes.c_void_p()
        with torch.cuda.device(layer.device):
            C.check(C.lib.b200moe_pipeline_create(ctypes.byref(layer.desc), _DT[dtype], max_tokens, regime,
                                                  depth, _ptr(self._mem), nbytes,
                                                  ctypes.byref(self._handle)), "pipeline_create")
        self._keep = []

    def submit(self, h_host: torch.Tensor, y_host: torch.Tensor):
        if h_host.is_cuda or y_host.is_cuda:
            raise C.B200MoeError("pipeline buffers live in host memory")
        if h_host.dtype != self.dtype or y_host.dtype != self.dtype or not (
                h_host.is_contiguous() and y_host.is_contiguous()):
            raise C.B200MoeError("pipeline buffers must be contiguous and of the pipeline's dtype")
        tokens = h_host.numel() // self.layer.hidden
        if y_host.numel() != h_host.numel():
            raise C.B200MoeError("pipeline: input and output sizes differ")
        with torch.cuda.device(self.layer.device):
            C.check(C.lib.b200moe_pipeline_submit(self._handle, _ptr(h_host), _ptr(y_host), tokens,
                                                  _stream()), "pipeline_submit")

    def drain(self):
        C.check(C.lib.b200moe_pipeline_drain(self._handle), "pipeline_drain")

    def close(self):
        if self._handle:
            C.check(C.lib.b200moe_pipeline_destroy(self._handle), "pipeline_destroy")
            self._handle = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_LAYERS: dict[int, PreparedLayer] = {}


@torch.library.custom_op("b200moe::layer_forward", mutates_args=())
def _layer_forward_op(h: torch.Tensor, handle: int, regime: int) -> torch.Tensor:
    return _LAYERS[handle].forward(h, regime)


@_layer_forward_op.register_fake
def _(h, handle, regime):
    return torch.empty_like(h)


def _activation_name(fn) -> str:
    if fn in (F.silu, torch.nn.functional.silu) or getattr(fn, "__name__", "") == "silu":
        return "silu"
    if fn in (F.gelu, torch.nn.functional.gelu) or getattr(fn, "__name__", "") == "gelu":
        return "gelu"
    raise C.B200MoeError(f"unsupported MoE activation {fn!r} (silu and gelu are implemented)")


class B200MoeBlock(torch.nn.Module):
    """Drop-in for sharktank's MoeBlock: same constructor, same theta keys
    (`ffn_gate_inp`, `ffn_norm`, optional `layer_output_norm`,
    `ffn_{gate,up,down}_exps.weight`), same `forward(h[bs, sl, d])`."""

    def __init__(self, theta, expert_count: int, expert_used_count: int, rms_epsilon: float,
                 moe_activation=F.silu, *, regime: str = "auto"):
        super().__init__()
        self.theta = theta
        self.expert_count = expert_count
        self.expert_used_count = expert_used_count
        self.layer = PreparedLayer(theta, expert_count, expert_used_count, rms_epsilon,
                                   _activation_name(moe_activation))
        self.regime = REGIMES[regime]
        self._handle = id(self.layer)
        _LAYERS[self._handle] = self.layer

    def __del__(self):
        if _LAYERS is not None:
            _LAYERS.pop(getattr(self, "_handle", None), None)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        if not _debug.flags.any:
            return torch.ops.b200moe.layer_forward(h, self._handle, self.regime)
        if _debug.flags.nvtx:
            torch.cuda.nvtx.range_push(f"b200moe.layer[{h.numel() // h.shape[-1]} tokens]")
        y, experts, gates = self.layer.forward(h, self.regime, want_routing=True)
        if _debug.flags.nvtx:
            torch.cuda.nvtx.range_pop()
        _debug.after_layer("moe", y, experts, gates)
        return y


class B200MoeStack(torch.nn.Module):
    """Several MoE layers applied back to back (the MoE halves of consecutive
    transformer blocks, without the attention in between): the output of layer i
    is the input of layer i+1."""

    def __init__(self, blocks):
        super().__init__()
        self.blocks = torch.nn.ModuleList(blocks)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        for blk in self.blocks:
            h = blk(h)
        return h


# ------------------------------------------------------ op-level overrides
class GatheredExperts:
    """What `ffn_*_exps.weight[experts, :, :]` returns for a quantized tensor: a
    handle on (weights, experts) with the logical shape [T, k, N, K] of the dense
    gather the reference would have materialised (layers/ffn_moe_block.py:39).
    For one shard of an expert-sharded tensor, `expert_begin` is the global id of
    the shard's first expert; pairs routed elsewhere contribute zero rows."""

    def __init__(self, base, experts: torch.Tensor, expert_begin: int = 0):
        self.base = base
        self.experts = experts
        self.expert_begin = expert_begin
        t, k = experts.shape
        self.shape = [t, k, int(base.shape[1]), int(base.shape[2])]

    def plan(self, device) -> RoutePlan:
        return _cached_plan(self.experts, int(self.base.shape[0]), self.expert_begin, device)


def _cached_plan(experts: torch.Tensor, expert_count: int, expert_begin: int = 0,
                 device=None) -> RoutePlan:
    """One route plan per `experts` tensor OBJECT (and expert range), kept on the
    tensor itself.

    PreGatherFFNMOE.forward indexes all three expert tensors with the same
    `experts` object (layers/ffn_moe_block.py:60-74), so the plan built for the
    gate product is found again for up and down.  The plan dies with the tensor.
    Nothing is keyed on the address: the next layer's (or decode step's)
    `torch.topk` result has the same shape, version 0 and, from the caching
    allocator, very often the same address as the one just freed."""
    device = experts.device if device is None else torch.device(device)
    plans = getattr(experts, "_b200moe_plans", None)
    if plans is None or plans.get("version") != experts._version:
        plans = {"version": experts._version}
        experts._b200moe_plans = plans
    key = (expert_begin, expert_count, str(device))
    if key not in plans:
        plans[key] = route_plan(experts.to(device), expert_count, expert_begin)
    return plans[key]


class ShardedGatheredExperts:
    """`weights[experts, :, :]` on an expert-sharded `SplitPrimitiveTensor`
    (shard_dim 0, shards = quantized tensors; types/tensors.py:957-1096): one
    GatheredExperts per shard, each knowing its first global expert id."""

    def __init__(self, base, experts: torch.Tensor):
        self.base = base
        self.experts = experts
        self.parts = []
        begin = 0
        for shard in base.shards:
            self.parts.append(GatheredExperts(shard, experts, begin))
            begin += int(shard.shape[0])
        t, k = experts.shape
        self.shape = [t, k, int(base.shape[1]), int(base.shape[2])]


_SUPPORTED = ("BlockScaledLayout", "SuperBlockOffsetScaled_4_6_Layout", "BlockScaledI4Layout")


def get_index_quantized(tensor, key):
    """`get_index` override: `weights[experts, :, :]` on a Q8_0 / Q4_K planar
    tensor -> lazy GatheredExperts.  Anything else is declined."""
    if _layout_name(tensor) not in _SUPPORTED:
        return NotImplemented
    if not (isinstance(key, tuple) and len(key) == 3 and isinstance(key[0], torch.Tensor)):
        return NotImplemented
    idx = key[0]
    if idx.dtype not in (torch.int64, torch.int32) or idx.dim() != 2 or not idx.is_cuda:
        return NotImplemented
    if key[1] != slice(None) or key[2] != slice(None):
        return NotImplemented
    return GatheredExperts(tensor, idx)


def _gathered_product(x: torch.Tensor, g: GatheredExperts, einsum_str: str):
    """[T, k, N] fp32 on the weights' device: rows of pairs whose expert lies in
    g's expert range, zeros elsewhere.  None for an einsum string that is not one
    of the two MoE products."""
    w = prepare_weight(g.base)
    dev = w.keep[0].device
    plan = g.plan(dev)
    t, k = g.experts.shape
    x = x.to(dev)
    kperm = C.lib.b200moe_kperm(w.layout, C.REGIME_AUTO, t)
    if einsum_str == "mk,menk->men":
        rows = x.to(torch.float16).contiguous()
        xs = torch.empty(plan.pairs, w.cols, dtype=torch.float16, device=dev)
        with torch.cuda.device(dev):
            C.check(C.lib.b200moe_permute_rows(_ptr(rows), _ptr(plan.perm), _ptr(plan.seg_offsets),
                                               w.experts, plan.pairs, k, w.cols, kperm, _ptr(xs),
                                               _stream()), "permute_rows")
    elif einsum_str == "mek,menk->men":
        rows = x.reshape(t * k, -1).to(torch.float16)
        xs = rows.index_select(0, plan.perm.to(torch.int64)).contiguous()
        if kperm:
            xs = xs.view(plan.pairs, -1, 2, 4).transpose(2, 3).reshape(plan.pairs, -1).contiguous()
    else:
        return None
    out = grouped_matmul(xs, plan.seg_offsets, w, t)
    inv = plan.inv.to(torch.int64)
    res = out.index_select(0, inv.clamp_min(0))
    if g.expert_begin != 0 or w.experts != _total_experts(g):
        res = res * (inv >= 0).unsqueeze(1)  # rows past the kept pairs were never computed
    return res.view(t, k, w.rows)


def _total_experts(g: GatheredExperts) -> int:
    return getattr(g, "total_experts", int(g.base.shape[0]))


def einsum_2args_gathered(input0, input1, einsum_str):
    """`einsum_2args` override for the MoE strings with a GatheredExperts rhs
    (ops/default_impls.py:72-94): "mk,menk->men" and "mek,menk->men"."""
    if not isinstance(input1, GatheredExperts):
        return NotImplemented
    x = _unbox(input0)
    if not x.is_cuda:
        return NotImplemented
    res = _gathered_product(x, input1, einsum_str)
    if res is None:
        return NotImplemented
    return res.to(device=x.device, dtype=x.dtype)


def get_index_split(tensor, key):
    """`get_index` override for an expert-sharded `SplitPrimitiveTensor` whose
    shards are Q8_0 / Q4_K planar tensors (the reference has no sharded
    get_index at all, ops/sharded_impls.py)."""
    shards = getattr(tensor, "shards", None)
    if not shards or getattr(tensor, "shard_dim", None) != 0:
        return NotImplemented
    if any(_layout_name(sh) not in _SUPPORTED for sh in shards):
        return NotImplemented
    if not (isinstance(key, tuple) and len(key) == 3 and isinstance(key[0], torch.Tensor)):
        return NotImplemented
    idx = key[0]
    if idx.dtype not in (torch.int64, torch.int32) or idx.dim() != 2 or not idx.is_cuda:
        return NotImplemented
    if key[1] != slice(None) or key[2] != slice(None):
        return NotImplemented
    return ShardedGatheredExperts(tensor, idx)


def einsum_2args_sharded_gathered(input0, input1, einsum_str):
    """The two MoE products against an expert-sharded weight: every shard
    multiplies, on its own device, the pairs routed to its experts; the disjoint
    partial results are added on the device of the activations.  `input0` is a
    plain tensor (result: a plain tensor on its device) or a `ReplicatedTensor`
    (shard i feeds weight shard i; result: replicated again).  One process
    holding all shards, as in the reference's sharding model
    (types/tensors.py:743-955); with one process per GPU use
    `parallel.build_block` instead, which exchanges tokens rather than results."""
    if not isinstance(input1, ShardedGatheredExperts):
        return NotImplemented
    rep = getattr(input0, "shards", None)
    if rep is not None and getattr(input0, "shard_dim", None) is not None:
        return NotImplemented  # split activations are not a replicated operand
    xs = [_unbox(sh) for sh in rep] if rep is not None else None
    x0 = xs[0] if xs is not None else _unbox(input0)
    if not x0.is_cuda:
        return NotImplemented
    total = None
    n_parts = len(input1.parts)
    for i, part in enumerate(input1.parts):
        part.total_experts = int(input1.base.shape[0])
        xi = xs[i] if xs is not None and len(xs) == n_parts else x0
        res = _gathered_product(xi, part, einsum_str)
        if res is None:
            return NotImplemented
        res = res.to(x0.device)
        total = res if total is None else total + res
    total = total.to(x0.dtype)
    if rep is None:
        return total
    return type(input0)(ts=[total.to(x.device) for x in xs])


def einsum_2args_gate_scale(input0, input1, einsum_str):
    """"me,men->men" on CUDA tensors: the gate scaling (ops/default_impls.py:97-105)."""
    if einsum_str != "me,men->men":
        return NotImplemented
    a, b = _unbox(input0), _unbox(input1)
    return a.unsqueeze(-1) * b


def matmul_quantized(lhs, rhs, *, transpose_rhs: bool = False):
    """`matmul(x, W, transpose_rhs=True)` with a Q8_0 / Q4_K planar weight
    [N, K]: the dense quantized linear of the same models (attention
    projections, output head), run as the grouped product with one expert.
    Replaces the IREE kernel routing of ops/custom_impls.py:66-128 and the
    dequantise-then-matmul default (ops/default_impls.py:345-359)."""
    if not transpose_rhs or _layout_name(rhs) not in _SUPPORTED:
        return NotImplemented
    x = _unbox(lhs)
    if not x.is_cuda or len(rhs.shape) != 2:
        return NotImplemented
    n, k = (int(v) for v in rhs.shape)
    if k % 256 != 0 or n % 256 != 0 or x.shape[-1] != k:
        return NotImplemented

    class _AsExperts:  # the same planes seen as a stack of one expert
        pass

    holder = getattr(rhs, "_b200moe_as_experts", None)
    if holder is None:
        holder = _AsExperts()
        holder.layout_type = rhs.layout_type
        holder.shape = [1, n, k]
        holder.unpack = rhs.unpack
        try:
            rhs._b200moe_as_experts = holder
        except AttributeError:
            pass
    w = prepare_weight(holder)
    rows = x.reshape(-1, k).to(torch.float16).contiguous()
    m = rows.shape[0]
    if C.lib.b200moe_kperm(w.layout, C.REGIME_AUTO, m):
        rows = rows.view(m, -1, 2, 4).transpose(2, 3).reshape(m, -1).contiguous()
    seg = torch.tensor([0, m], dtype=torch.int32, device=x.device)
    out = grouped_matmul(rows, seg, w, max(m, 1))
    return out.view(*x.shape[:-1], n).to(x.dtype)


def linear_quantized(input, weight, bias=None, *, accum_dtype=None):
    """`linear(x, W, bias)` for the same weights (ops/qlinear_impls.py:158-172)."""
    y = matmul_quantized(input, weight, transpose_rhs=True)
    if y is NotImplemented:
        return NotImplemented
    if bias is not None:
        y = y + _unbox(bias).to(y.dtype)
    return y


def register_overrides(ops_module=_ops, quantized_type=None, tensor_type=torch.Tensor, salience=10,
                       split_type=None, replicated_type=None):
    """Registers the overrides with an ops registry: this package's mirror by
    default, sharktank's own when called from `plugin.register`."""
    from . import types as _types

    qt = quantized_type or _types.QuantizedTensor
    split = split_type or _types.SplitPrimitiveTensor
    repl = replicated_type or _types.ReplicatedTensor
    ops_module.get_index.override(qt, salience=salience)(get_index_quantized)
    ops_module.get_index.override(split, salience=salience)(get_index_split)
    ops_module.einsum_2args.override(tensor_type, GatheredExperts, salience=salience)(
        einsum_2args_gathered)
    ops_module.einsum_2args.override(tensor_type, ShardedGatheredExperts, salience=salience)(
        einsum_2args_sharded_gathered)
    ops_module.einsum_2args.override(repl, ShardedGatheredExperts, salience=salience)(
        einsum_2args_sharded_gathered)
    ops_module.matmul.override(tensor_type, qt, salience=salience)(matmul_quantized)
    if ops_module is _ops:
        ops_module.linear.override(tensor_type, qt, salience=salience)(linear_quantized)
        ops_module.einsum_2args.override(torch.Tensor, torch.Tensor)(einsum_2args_gate_scale)
    else:
        # sharktank dispatches linear on (input, weight) and (input, weight, bias)
        ops_module.linear.override(tensor_type, qt, salience=salience)(linear_quantized)
        ops_module.linear.override(tensor_type, qt, tensor_type, salience=salience)(linear_quantized)


register_overrides()
