"""Expert-parallel MoE layer: one process per GPU, experts partitioned over ranks.

Rank r owns the contiguous experts [r*E/W, (r+1)*E/W) (the shard an
expert-sharded `SplitPrimitiveTensor(ts=[...], shard_dim=0)` of
`ffn_*_exps.weight` gives it), the router and norm weights are replicated, and
every rank brings its own slice of the tokens.  Per layer call:

  1. route the local tokens (replicated router), sort the (token, slot) pairs by
     global expert id — which also sorts them by destination rank;
  2. all-to-all the per-expert counts, then the fp16 activation rows (dispatch);
  3. group the received rows by local expert, run the grouped gate/up and down
     products, put the results back in arrival order;
  4. all-to-all the fp32 result rows back (combine), scale by the gates, sum the
     slots, output norm, residual.

The reference has no expert parallelism (its sharded tensors are lists held by
one process and it has no sharded einsum/get_index); this is new behaviour with
the layer semantics of MoeBlock.forward.  The exchange logic is written
against a small compute backend so that it runs under `gloo` on CPUs in tests
with a stand-in backend; the product backend is the CUDA library.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class Exchange:
    """Split sizes of one dispatch/combine pair, all in rows."""

    send_splits: list[int]       # rows this rank sends to each rank
    recv_splits: list[int]       # rows this rank receives from each rank
    recv_counts: torch.Tensor    # int32 [world, E_local] on the device: rows per (source, expert)
    max_segment: int             # most rows any local expert receives


def plan_exchange(counts_local: torch.Tensor, world: int, group) -> Exchange:
    """counts_local: int32 [E] rows this rank routes to each *global* expert.
    One small all-to-all tells every rank how many rows arrive per (source
    rank, local expert).  Synchronises with the host once (NCCL needs
    host-side split sizes)."""
    E = counts_local.numel()
    el = E // world
    send_counts = counts_local.reshape(world, el).contiguous()
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    both = torch.stack([send_counts, recv_counts]).cpu()
    send_splits = both[0].sum(dim=1).tolist()
    recv_splits = both[1].sum(dim=1).tolist()
    max_segment = int(both[1].sum(dim=0).max()) if el > 0 else 0
    return Exchange(send_splits, recv_splits, recv_counts, max_segment)


def exchange_rows(rows: torch.Tensor, send_splits, recv_splits, group) -> torch.Tensor:
    out = rows.new_empty((sum(recv_splits),) + tuple(rows.shape[1:]))
    dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=list(recv_splits),
                           input_split_sizes=list(send_splits), group=group)
    return out


class ExpertParallelMoeBlock(torch.nn.Module):
    """MoeBlock.forward with the experts of this rank only.

    backend methods (CUDA implementation: `CudaBackend` below):
      route(h)                         -> xn [T,d], experts int32 [T,k], gates f32 [T,k]
      plan(experts, n_experts, begin)  -> counts, seg_offsets, perm, inv
      regroup(recv_counts, n)          -> seg_offsets, perm, inv of the arrived rows by local expert
      gather(rows, perm, top_k, n)     -> rows[perm // top_k] for the first n positions
      expert_ffn(xs, seg, max_segment) -> [rows, d] in the wire dtype of the return trip
      combine(rows, inv, gates, h)     -> y
    """

    def __init__(self, backend, expert_count: int, top_k: int, group=None):
        super().__init__()
        self.backend = backend
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        assert expert_count % self.world == 0, "experts must divide evenly over the ranks"
        self.expert_count = expert_count
        self.experts_local = expert_count // self.world
        self.top_k = top_k
        self.launches_per_step = 10

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        b = self.backend
        shape = h.shape
        x = h.reshape(-1, shape[-1])
        xn, experts, gates = b.route(x)
        counts, seg, perm, inv = b.plan(experts.reshape(-1), self.expert_count, 0)
        pairs = experts.numel()
        send_rows = b.gather(xn, perm, self.top_k, pairs)
        ex = plan_exchange(counts, self.world, self.group)
        recv_rows = exchange_rows(send_rows, ex.send_splits, ex.recv_splits, self.group)
        n_recv = recv_rows.shape[0]
        seg2, perm2, inv2 = b.regroup(ex.recv_counts, n_recv)
        xs = b.gather(recv_rows, perm2, 1, n_recv)
        d_sorted = b.expert_ffn(xs, seg2, max(ex.max_segment, 1))
        d_arrival = b.gather(d_sorted, inv2, 1, n_recv)
        d_back = exchange_rows(d_arrival, ex.recv_splits, ex.send_splits, self.group)
        y = b.combine(d_back, inv, gates, x)
        return y.reshape(shape)


class CudaBackend:
    """The compute stages on this rank's GPU through the C ABI."""

    def __init__(self, layer, regime: int = 0):
        from . import _cabi as C

        self.C = C
        self.layer = layer  # moe.PreparedLayer built on the local expert shard
        self.regime = regime
        self.dev = layer.device
        self.profile = False
        self.timings = []  # (gate_up_ms_event_pair, down_event_pair, rows) while profiling

    def _st(self):
        return ctypes.c_void_p(torch.cuda.current_stream(self.dev).cuda_stream)

    @staticmethod
    def _p(t: Optional[torch.Tensor]):
        return None if t is None else ctypes.c_void_p(t.data_ptr())

    def route(self, h):
        C, L = self.C, self.layer
        h = h.contiguous()
        tokens = h.shape[0]
        xn = torch.empty(tokens, L.hidden, dtype=torch.float16, device=self.dev)
        experts = torch.empty(tokens, L.top_k, dtype=torch.int32, device=self.dev)
        gates = torch.empty(tokens, L.top_k, dtype=torch.float32, device=self.dev)
        dt = C.DT_F32 if h.dtype == torch.float32 else C.DT_BF16
        C.check(C.lib.b200moe_router(self._p(h), dt, tokens, ctypes.byref(L.desc), self._p(xn),
                                     self._p(experts), self._p(gates), self._st()), "router")
        return xn, experts, gates

    def plan(self, experts, n_experts, begin):
        from . import moe

        p = moe.route_plan(experts, n_experts, begin)
        return p.counts, p.seg_offsets, p.perm, p.inv

    def gather(self, rows, perm, top_k, n):
        """out[i] = rows[perm[i] // top_k] for i < n (rows of fp16 or fp32)."""
        C = self.C
        rows = rows.contiguous()
        out = torch.empty((n,) + tuple(rows.shape[1:]), dtype=rows.dtype, device=self.dev)
        if n == 0:
            return out
        C.check(C.lib.b200moe_gather_rows(self._p(rows), self._p(perm), n, top_k,
                                          rows.shape[1] * rows.element_size(), self._p(out),
                                          self._st()), "gather_rows")
        return out

    def regroup(self, recv_counts, n):
        C = self.C
        world, el = recv_counts.shape
        seg = torch.empty(el + 1, dtype=torch.int32, device=self.dev)
        perm = torch.empty(max(n, 1), dtype=torch.int32, device=self.dev)
        inv = torch.empty(max(n, 1), dtype=torch.int32, device=self.dev)
        C.check(C.lib.b200moe_exchange_plan(self._p(recv_counts), world, el, self._p(seg),
                                            self._p(perm), self._p(inv), self._st()), "exchange_plan")
        return seg, perm[:n], inv[:n]

    def expert_ffn(self, xs, seg, max_segment):
        C, L = self.C, self.layer
        n = xs.shape[0]
        a = torch.empty(max(n, 1), L.ffn, dtype=torch.float16, device=self.dev)
        if L.gate.layout == C.LAYOUT_Q4_K:
            # the Q4_K kernels read interleaved columns
            xs = xs.view(n, -1, 2, 4).transpose(2, 3).reshape(n, -1).contiguous()
        kp = C.lib.b200moe_kperm(L.down.layout, self.regime, max_segment)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)] if self.profile else None
        if ev:
            ev[0].record()
        C.check(C.lib.b200moe_gate_up(self._p(xs), self._p(seg), n, max_segment,
                                      ctypes.byref(L.gate.desc), ctypes.byref(L.up.desc),
                                      L.desc.activation, self.regime, kp, self._p(a), self._st()),
                "gate_up")
        ks = C.lib.b200moe_down_ksplit(ctypes.byref(L.down.desc), n, max_segment, self.regime)
        part = torch.empty(ks, max(n, 1), L.hidden, dtype=torch.float32, device=self.dev)
        if ev:
            ev[1].record()
        C.check(C.lib.b200moe_down(self._p(a), self._p(seg), n, max_segment,
                                   ctypes.byref(L.down.desc), self.regime, ks, self._p(part),
                                   self._st()), "down")
        if ev:
            ev[2].record()
            self.timings.append((ev, n))
        out = part[0] if ks == 1 else part.sum(dim=0)
        # result rows travel back as bf16: half the NVLink bytes, and the layer
        # output is rounded to the activation dtype anyway
        return out[:n].to(torch.bfloat16)

    def combine(self, rows, inv, gates, h):
        C, L = self.C, self.layer
        h = h.contiguous()
        tokens = h.shape[0]
        y = torch.empty_like(h)
        dt = C.DT_F32 if h.dtype == torch.float32 else C.DT_BF16
        rows = rows.contiguous()
        ddt = C.DT_BF16 if rows.dtype == torch.bfloat16 else C.DT_F32
        C.check(C.lib.b200moe_combine(self._p(rows), ddt, 1, rows.shape[0], self._p(inv), self._p(gates),
                                      self._p(h), dt, tokens, ctypes.byref(L.desc), 1, self._p(y),
                                      dt, self._st()), "combine")
        return y


class P2PExchange:
    """The symmetric buffers of the peer-to-peer token exchange and its barrier
    epoch counter.  One exchange serves any number of layers of the same hidden
    size on this rank (a stack of MoE layers): the buffers are reused layer after
    layer, the epochs keep counting.  `max_tokens` bounds the tokens of the whole
    job per call (it sizes the receive buffer for the worst routing: every token
    on this rank's experts); `max_local_tokens` bounds this rank's own tokens."""

    def __init__(self, hidden: int, expert_count: int, top_k: int, max_tokens: int, max_local_tokens: int,
                 group=None, device=None):
        import torch.distributed._symmetric_memory as symm_mem

        from . import _cabi as C

        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        assert expert_count % self.world == 0 and self.world <= 16
        self.expert_count, self.top_k, self.hidden = expert_count, top_k, hidden
        self.el = expert_count // self.world
        self.dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        d = hidden
        self.cap_rows = max_tokens * min(top_k, self.el)
        self.ret_rows = max_local_tokens * top_k
        self.max_segment = max_tokens

        def up(n):
            return (n + 1023) // 1024 * 1024

        off_counts = 0
        off_flags = up(self.world * expert_count * 4)
        off_recv = off_flags + 1024
        off_ret = off_recv + up(self.cap_rows * d * 2)
        total = off_ret + up(self.ret_rows * d * 2)
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=self.dev)
        self.buf.zero_()
        self.hdl = symm_mem.rendezvous(self.buf, group=self.group)
        torch.cuda.synchronize(self.dev)
        dist.barrier(group=self.group)  # every rank's flags are zero before anyone signals
        ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        ep = C.EpDesc()
        ep.world, ep.rank, ep.experts_local = self.world, self.rank, self.el
        for i, base in enumerate(ptrs):
            ep.counts_all[i] = base + off_counts
            ep.flags[i] = base + off_flags
            ep.recv_x[i] = base + off_recv
            ep.ret_y[i] = base + off_ret
        self.ep = ep
        self.epoch = 0
        self._workspace = None

    def workspace(self, nbytes: int) -> torch.Tensor:
        if self._workspace is None or self._workspace.numel() < nbytes:
            self._workspace = torch.empty(nbytes, dtype=torch.uint8, device=self.dev)
        return self._workspace


class P2PExpertParallelMoeBlock(torch.nn.Module):
    """The same layer with dispatch and combine as direct peer-to-peer stores into
    symmetric buffers: no host synchronisation and no library collective per
    call, and the whole sequence is one C call (`b200moe_ep_layer_forward`).
    Layers of a stack share one `P2PExchange` (and its workspace)."""

    def __init__(self, layer, expert_count: int, top_k: int, max_tokens: int = 0, max_local_tokens: int = 0,
                 group=None, regime: int = 0, exchange: Optional[P2PExchange] = None):
        super().__init__()
        from . import _cabi as C

        self.C = C
        self.layer = layer
        self.regime = regime
        self.x = exchange if exchange is not None else P2PExchange(
            layer.hidden, expert_count, top_k, max_tokens, max_local_tokens, group, layer.device)
        assert self.x.hidden == layer.hidden and self.x.expert_count == expert_count
        self.group, self.world, self.rank = self.x.group, self.x.world, self.x.rank
        self.expert_count, self.top_k = expert_count, top_k
        self.dev = layer.device
        # the layer descriptor of this rank's shard: local experts, global numbering
        self.desc = C.LayerDesc.from_buffer_copy(layer.desc)
        self.desc.experts = expert_count
        self.desc.expert_begin = self.rank * self.x.el
        # load balance is steered by the rows expected under uniform routing, the
        # buffers are sized for the worst case
        expected = max(1, self.x.max_segment * top_k // self.world)
        self.ks = C.lib.b200moe_down_ksplit(ctypes.byref(layer.down.desc), expected, self.x.max_segment, regime)
        self.backend = CudaBackend(layer, regime)  # carries the profile switch for benchmarks
        self.launches_per_step = 11

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        C, x = self.C, self.x
        shape = h.shape
        xin = h.reshape(-1, shape[-1]).contiguous()
        tokens = xin.shape[0]
        if xin.dtype not in (torch.float32, torch.bfloat16):
            raise C.B200MoeError(f"activations must be fp32 or bf16, got {xin.dtype}")
        dt = C.DT_F32 if xin.dtype == torch.float32 else C.DT_BF16
        y = torch.empty_like(xin)
        nbytes = C.lib.b200moe_ep_workspace_bytes(ctypes.byref(self.desc), tokens, x.cap_rows, self.ks)
        ws = x.workspace(nbytes)
        p = CudaBackend._p
        with torch.cuda.device(self.dev):
            C.check(C.lib.b200moe_ep_layer_forward(
                ctypes.byref(self.desc), ctypes.byref(x.ep), p(xin), p(y), dt, tokens, self.regime,
                x.cap_rows, x.ret_rows, x.max_segment, self.ks, x.epoch, p(ws), ws.numel(),
                ctypes.c_void_p(torch.cuda.current_stream(self.dev).cuda_stream)), "ep_layer_forward")
        x.epoch += 3
        return y.reshape(shape)


class ExpertParallelStack(torch.nn.Module):
    """Several expert-parallel MoE layers applied back to back on this rank's
    tokens (the MoE halves of consecutive transformer blocks): the output of
    layer i is the input of layer i+1.  Peer-to-peer layers share one
    `P2PExchange` — one set of symmetric buffers and one epoch counter for the
    whole stack."""

    def __init__(self, blocks):
        super().__init__()
        self.blocks = torch.nn.ModuleList(blocks)
        xs = {id(b.x) for b in blocks if isinstance(b, P2PExpertParallelMoeBlock)}
        assert len(xs) <= 1, "peer-to-peer layers of a stack must share their exchange"

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        for blk in self.blocks:
            h = blk(h)
        return h


def shard_theta(theta, rank: int):
    """This rank's view of a (possibly sharded) theta: `SplitPrimitiveTensor` /
    `ReplicatedTensor` entries are replaced by their shard for `rank`."""
    from . import types as T

    def pick(node):
        if isinstance(node, dict):
            return {k: pick(v) for k, v in node.items()}
        shards = getattr(node, "shards", None)
        if shards is not None:
            return shards[rank] if len(shards) > 1 else shards[0]
        return node

    return T.Theta(pick(theta.tree))


def build_block(theta_local, expert_count: int, top_k: int, rms_epsilon: float, activation: str,
                group=None, regime: str = "auto", transport: str = "nccl", max_tokens: int = 0,
                max_local_tokens: int = 0, exchange: Optional[P2PExchange] = None):
    """theta_local holds this rank's expert shard ([E/W, ...] tensors) and the
    replicated router / norm weights, all on this rank's GPU.  transport "nccl":
    all-to-all collectives; "p2p": direct stores into symmetric buffers (needs
    max_tokens / max_local_tokens to size them, or an existing `exchange`)."""
    from . import moe

    layer = moe.PreparedLayer(theta_local, expert_count, top_k, rms_epsilon, activation)
    if transport == "p2p":
        return P2PExpertParallelMoeBlock(layer, expert_count, top_k, max_tokens, max_local_tokens,
                                         group, moe.REGIMES[regime], exchange)
    return ExpertParallelMoeBlock(CudaBackend(layer, moe.REGIMES[regime]), expert_count, top_k, group)


def build_from_case(case, group=None, regime: str = "auto", transport: str = "nccl",
                    max_local_tokens: int = 0, exchange: Optional[P2PExchange] = None):
    """Benchmark/test helper: slice a synthetic case's expert planes for this rank."""
    from . import types as T
    from .synthetic import DENSE, Q8_0

    group = group if group is not None else dist.group.WORLD
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    s = case.spec
    el = s.experts // world
    e0, e1 = rank * el, (rank + 1) * el
    dev = torch.device("cuda", torch.cuda.current_device())

    def weight(planes, n, k):
        shape = [el, n, k]
        if s.kind == DENSE:
            return T.DefaultPrimitiveTensor(data=planes["w"][e0:e1].to(dev))
        p = {name: v[e0:e1].contiguous().to(dev) for name, v in planes.items()}
        if s.kind == Q8_0:
            lay = T.BlockScaledLayout(shape, p["d"], p["qs"])
        elif s.kind == "Q4_1":
            lay = T.BlockScaledI4Layout(shape, p["d"], p["qs"], m=p["m"])
        else:
            lay = T.SuperBlockOffsetScaled_4_6_Layout(shape, **p)
        return T.PlanarQuantizedTensor(shape=shape, layout=lay)

    tree = {
        "ffn_gate_inp": {"weight": T.DefaultPrimitiveTensor(data=case.router_w.to(dev))},
        "ffn_norm": {"weight": T.DefaultPrimitiveTensor(data=case.norm_w.to(dev))},
        "ffn_gate_exps": {"weight": weight(case.gate, s.ffn, s.hidden)},
        "ffn_up_exps": {"weight": weight(case.up, s.ffn, s.hidden)},
        "ffn_down_exps": {"weight": weight(case.down, s.hidden, s.ffn)},
    }
    if case.router_b is not None:
        tree["ffn_gate_inp"]["bias"] = T.DefaultPrimitiveTensor(data=case.router_b.to(dev))
    if case.out_norm_w is not None:
        tree["layer_output_norm"] = {"weight": T.DefaultPrimitiveTensor(data=case.out_norm_w.to(dev))}
    tokens = case.h.shape[1]
    return build_block(T.Theta(tree), s.experts, s.top_k, s.eps, s.activation, group, regime,
                       transport, tokens, max_local_tokens or -(-tokens // world), exchange)


def build_stack_from_cases(cases, group=None, regime: str = "auto", max_local_tokens: int = 0):
    """Benchmark/test helper: a stack of peer-to-peer expert-parallel layers, one
    per synthetic case (same shape), sharing one exchange."""
    group = group if group is not None else dist.group.WORLD
    world = dist.get_world_size(group)
    s = cases[0].spec
    tokens = cases[0].h.shape[1]
    dev = torch.device("cuda", torch.cuda.current_device())
    x = P2PExchange(s.hidden, s.experts, s.top_k, tokens, max_local_tokens or -(-tokens // world), group, dev)
    return ExpertParallelStack([build_from_case(c, group, regime, "p2p", max_local_tokens, x) for c in cases])
