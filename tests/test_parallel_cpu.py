"""Expert-parallel dispatch/combine protocol under gloo, world size 2, on CPUs.
The exchange logic is the product's (shark_platform_b200.parallel); the compute
stages are stood in by the oracle so that the test needs no GPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import moe_oracle as orc
from shark_platform_b200 import synthetic as syn
from helpers import dense_weight, oracle_params


class OracleBackend:
    """CPU stand-in for parallel.CudaBackend with the same method contract."""

    def __init__(self, case, e0, e1):
        s = case.spec
        self.p = oracle_params(case)
        self.e0, self.e1 = e0, e1
        self.act = orc.ACTIVATIONS[s.activation]

    def route(self, h):
        xn = orc.rms_norm(h, self.p.norm_w, self.p.eps)
        gate, idx, _ = orc.router(xn, self.p.router_w, self.p.router_b, self.p.top_k)
        return xn, idx.to(torch.int32), gate

    def plan(self, experts, n_experts, begin):
        flat = experts.reshape(-1).to(torch.int64) - begin
        counts, seg, perm, inv = orc.route_plan(flat, n_experts)
        return counts.to(torch.int32), seg.to(torch.int32), perm.to(torch.int32), inv.to(torch.int32)

    def regroup(self, recv_counts, n):
        world, el = recv_counts.shape
        ids = torch.arange(el).repeat(world)
        arrival_expert = torch.repeat_interleave(ids, recv_counts.reshape(-1).to(torch.int64))
        assert arrival_expert.numel() == n
        _, seg, perm, inv = orc.route_plan(arrival_expert, el)
        return seg.to(torch.int32), perm.to(torch.int32), inv.to(torch.int32)

    def gather(self, rows, perm, top_k, n):
        return rows[(perm[:n].to(torch.int64) // top_k)]

    def expert_ffn(self, xs, seg, max_segment):
        out = torch.zeros(xs.shape[0], self.p.w_down.shape[1])
        assert max_segment >= int((seg[1:] - seg[:-1]).max())
        for le in range(self.e1 - self.e0):
            a, b = int(seg[le]), int(seg[le + 1])
            if a == b:
                continue
            e = self.e0 + le
            x = xs[a:b]
            hid = self.act(x @ self.p.w_gate[e].float().mT) * (x @ self.p.w_up[e].float().mT)
            out[a:b] = hid @ self.p.w_down[e].float().mT
        return out

    def combine(self, rows, inv, gates, h):
        t, k = gates.shape
        y = (rows[inv.to(torch.int64)].view(t, k, -1) * gates.unsqueeze(-1)).sum(dim=1)
        if self.p.out_norm_w is not None:
            y = orc.rms_norm(y, self.p.out_norm_w, self.p.eps)
        return h + y


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, name, tokens, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from shark_platform_b200.parallel import ExpertParallelMoeBlock

        torch.set_num_threads(2)
        case = syn.make_case(syn.CASES[name], tokens=tokens)
        s = case.spec
        el = s.experts // world
        block = ExpertParallelMoeBlock(OracleBackend(case, rank * el, (rank + 1) * el), s.experts, s.top_k)
        full = case.h.reshape(tokens, s.hidden)
        # uneven token split: rank 0 takes a third, the last rank the rest
        bounds = [0] + [tokens * (i + 1) // (world + 1) for i in range(world - 1)] + [tokens]
        y = block(full[bounds[rank]:bounds[rank + 1]].contiguous())
        want, _ = orc.moe_block(case.h, oracle_params(case), form="per_expert")
        want = want.reshape(tokens, s.hidden)[bounds[rank]:bounds[rank + 1]]
        out[rank] = orc.rel_l2(y, want)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("name,tokens", [("small_q8", 40), ("small_grok", 17), ("small_top4", 29)])
def test_expert_parallel_world2_matches_single_process(name, tokens):
    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), name, tokens, out), nprocs=world, join=True)
        assert len(out) == world
        for r in range(world):
            assert out[r] < 1e-5, (r, out[r])


def test_plan_exchange_single_rank_is_identity():
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(_free_port())
    dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        from shark_platform_b200.parallel import plan_exchange

        counts = torch.tensor([3, 0, 2, 5], dtype=torch.int32)
        ex = plan_exchange(counts, 1, dist.group.WORLD)
        assert ex.send_splits == [10] and ex.recv_splits == [10]
        assert ex.recv_counts.tolist() == [[3, 0, 2, 5]]
        assert ex.max_segment == 5
    finally:
        dist.destroy_process_group()
