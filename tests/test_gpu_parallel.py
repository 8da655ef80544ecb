"""Expert parallelism on real GPUs: two processes, two GPUs, NCCL all-to-all.
Skipped on a single-GPU machine (the CPU suite covers the protocol under gloo)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import moe_oracle as orc
from shark_platform_b200 import synthetic as syn
from helpers import oracle_params

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, name, tokens, regime, out, transport="nccl"):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from shark_platform_b200 import moe, parallel

        spec = syn.CASES[name]
        case = syn.make_case(spec, tokens=tokens)
        block = parallel.build_from_case(case, regime=regime, transport=transport,
                                         max_local_tokens=tokens)
        per = tokens // world
        full = case.h.reshape(tokens, spec.hidden)
        lo, hi = rank * per, (tokens if rank == world - 1 else (rank + 1) * per)
        h = full[lo:hi].cuda()
        if spec.act_dtype == "bf16":
            h = h.to(torch.bfloat16)
        y = block(h).float().cpu()
        y2 = block(h).float().cpu()  # second call: buffers and barrier epochs are reused
        torch.cuda.synchronize()
        assert torch.equal(y, y2)
        assert moe.device_status() == 0
        want, _ = orc.moe_block(case.h, oracle_params(case), form="per_expert")
        out[rank] = orc.rel_l2(y, want.reshape(tokens, spec.hidden)[lo:hi])
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("name,tokens,regime", [("small_q8", 40, "auto"), ("small_q4k", 33, "auto"),
                                                ("small_grok", 300, "tensor")])
def test_expert_parallel_two_gpus(name, tokens, regime):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), name, tokens, regime, out), nprocs=world, join=True)
        for r in range(world):
            assert out[r] < 2e-2, (r, out[r])


@pytest.mark.parametrize("name,tokens,regime", [("small_q8", 40, "auto"), ("small_q4k", 33, "auto"),
                                                ("small_grok", 300, "tensor")])
def test_expert_parallel_two_gpus_peer_to_peer(name, tokens, regime):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), name, tokens, regime, out, "p2p"),
                 nprocs=world, join=True)
        for r in range(world):
            assert out[r] < 2e-2, (r, out[r])


def _stack_worker(rank, world, port, tokens, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from shark_platform_b200 import moe, parallel

        cases, params = [], []
        for i in range(3):
            spec = syn.CaseSpec(f"stack{i}", tokens, 256, 512, kind=syn.Q8_0, router_bias="zipf",
                                seed=500 + i, act_dtype="f32")
            case = syn.make_case(spec)
            case.down["d"] = (case.down["d"].float() * 0.05).half()  # keep the residual stream at unit scale
            cases.append(case)
            params.append(oracle_params(case))
        stack = parallel.build_stack_from_cases(cases, max_local_tokens=tokens)
        per = tokens // world
        lo, hi = rank * per, (tokens if rank == world - 1 else (rank + 1) * per)
        h0 = cases[0].h.reshape(tokens, 256)
        y = stack(h0[lo:hi].cuda()).cpu()
        y2 = stack(h0[lo:hi].cuda()).cpu()
        torch.cuda.synchronize()
        assert torch.equal(y, y2)
        assert moe.device_status() == 0
        want = cases[0].h
        for p in params:
            want, _ = orc.moe_block(want, p, form="per_expert")
        out[rank] = orc.rel_l2(y, want.reshape(tokens, 256)[lo:hi])
    finally:
        dist.destroy_process_group()


def test_stack_of_expert_parallel_layers_shares_one_exchange():
    """Three layers with Zipf-skewed routing back to back on two GPUs: one set of
    symmetric buffers, one epoch counter (BASELINE config 5 in miniature)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_stack_worker, args=(world, _free_port(), 64, out), nprocs=world, join=True)
        for r in range(world):
            assert out[r] < 2e-2, (r, out[r])
