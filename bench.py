"""Benchmark of the MoE FFN layer: Mixtral-8x7B-shaped, Q8_0 expert weights.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One "step" is one MoE-layer forward over one batch of synthetic tokens.  Prints
ONE JSON line (rank 0).  Workloads (all hidden 4096, ffn 14336, 8 experts,
top-2, SiLU, Q8_0 weights, bf16 activations, seeded synthetic values):
  prefill4096  4096 tokens (default; tensor-core bound)
  decode32     32 tokens   (HBM bound: the weights are streamed once per call)
  decode1 / decode128
  q4k_decode32 / q4k_prefill2048   the same layer with Q4_K expert weights
  grok_prefill8192                 Grok-1 shape (hidden 6144, ffn 32768, GELU, output norm)
  stack32_decode64                 32 Mixtral layers back to back, 64 tokens, Zipf(1.2)
                                   router bias per layer (weights drawn on the device)

With N > 1 (torchrun, one process per GPU) the experts are partitioned over the
ranks, each rank routes tokens/N tokens and the token rows move by NCCL
all-to-all; the total token count stays fixed ("strong" scaling).

`--impl reference` times the CPU restatement of the reference's torch-eager
layer (oracle/moe_oracle.py, the gather + batched-GEMV form sharktank runs) on
the host cores, on a bounded token sample per step.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

WORKLOADS = {
    "prefill4096": ("mixtral_q8", 4096),
    "decode32": ("mixtral_q8", 32),
    "decode1": ("mixtral_q8", 1),
    "decode128": ("mixtral_q8", 128),
    "q4k_decode32": ("mixtral_q4k", 32),
    "q4k_prefill2048": ("mixtral_q4k", 2048),
    "grok_prefill8192": ("grok_q8", 8192),
    "stack32_decode64": ("mixtral_q8", 64),
}
STAGES = ["router", "route_plan", "permute", "gate_up", "down", "combine"]


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while running."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc = index, None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "100", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def cpu_reference_setup(case, sample_tokens):
    """Host-side dequantised weights and the token sample for the CPU arm."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from helpers import oracle_params

    t0 = time.time()
    params = oracle_params(case)
    h = case.h[:, :sample_tokens].contiguous()
    return params, h, time.time() - t0


def time_cpu(params, h, steps, warmup, chunk=4):
    from oracle import moe_oracle as orc

    for _ in range(warmup):
        orc.moe_block(h, params, form="pregather", chunk=chunk)
    t0 = time.perf_counter()
    for _ in range(steps):
        orc.moe_block(h, params, form="pregather", chunk=chunk)
    dt = time.perf_counter() - t0
    return h.shape[1] * steps / dt, dt / steps


def run_reference(args, spec_name, tokens):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from shark_platform_b200 import synthetic as syn

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    sample = min(tokens, 8)
    spec = syn.CASES[spec_name]
    case = syn.make_case(spec, tokens=sample)
    params, h, _ = cpu_reference_setup(case, sample)
    steps, warmup = min(args.steps, 8), min(args.warmup, 1)
    tps, per_step = time_cpu(params, h, steps, warmup)
    sample_txt = (f"{sample} tokens per step of the {tokens}-token workload, torch-eager gather + "
                  f"batched-GEMV form on dequantised fp16->fp32 weights, {steps} steps")
    print(json.dumps({
        "impl": "reference", "metric": "moe_layer_tokens_per_s", "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": per_step * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": args.workload,
                   "layer": f"{spec_name} MoE FFN ({spec.kind} experts, {spec.activation})",
                   "tokens": tokens, "hidden": spec.hidden, "ffn": spec.ffn,
                   "experts": spec.experts, "top_k": spec.top_k},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": torch.get_num_threads(),
                         "kind": "port", "sample": sample_txt},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="prefill4096", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--regime", default="auto", choices=["auto", "stream", "tensor"])
    ap.add_argument("--ep", default="p2p", choices=["p2p", "nccl"],
                    help="token exchange between ranks: peer-to-peer stores or NCCL all-to-all")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    spec_name, tokens = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, spec_name, tokens)
        return
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    import torch.distributed as dist

    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from shark_platform_b200 import _cabi as C, moe, synthetic as syn
    b200_block, device_input = syn.case_block, syn.case_input
    spec = syn.CASES[spec_name]
    if world > 1:
        # every rank draws the same full layer on its own GPU (same seed, same
        # generator) and keeps its expert shard: seconds instead of a minute of
        # host-side generation per rank
        import dataclasses
        case = syn.make_case_on_device(dataclasses.replace(spec, tokens=tokens), dev)
    else:
        case = syn.make_case(spec, tokens=tokens)
    peaks = measured_peaks()
    flops = syn.layer_flops(tokens, spec.top_k, spec.hidden, spec.ffn)
    w_bytes_expert = 3 * syn.weight_bytes(spec.kind, spec.ffn, spec.hidden)

    layers = 1
    if args.workload == "stack32_decode64":
        assert world == 1, "the layer stack runs on one GPU in this build"
        from shark_platform_b200.moe import B200MoeStack
        import dataclasses

        layers = 32
        blocks = []
        for i in range(layers):
            sp = dataclasses.replace(spec, tokens=tokens, router_bias="zipf", seed=1000 + i)
            blocks.append(b200_block(syn.make_case_on_device(sp, dev), regime=args.regime, device=dev))
        block = blocks[0]
        stack = B200MoeStack(blocks)
        h = device_input(case, dev).reshape(tokens, spec.hidden).contiguous()
        step = lambda: stack(h)
        fused = C.lib.b200moe_front_supported(tokens, ctypes.byref(block.layer.desc))
        launches_per_step = (4 if fused else 6) * layers
    elif world == 1:
        block = b200_block(case, regime=args.regime, device=dev)
        h = device_input(case, dev).reshape(tokens, spec.hidden).contiguous()
        step = lambda: block(h)
        # router, plan and permutation are one launch for small token counts
        fused = C.lib.b200moe_front_supported(tokens, ctypes.byref(block.layer.desc))
        launches_per_step = 4 if fused else 6
    else:
        from shark_platform_b200 import parallel

        transport = args.ep
        if transport == "p2p":
            try:
                block = parallel.build_from_case(case, dist.group.WORLD, regime=args.regime,
                                                 transport="p2p")
            except Exception as exc:  # symmetric memory not available on this machine
                transport = f"nccl (p2p set-up failed: {type(exc).__name__}: {str(exc)[:120]})"
                block = parallel.build_from_case(case, dist.group.WORLD, regime=args.regime)
        else:
            block = parallel.build_from_case(case, dist.group.WORLD, regime=args.regime)
        per = tokens // world
        h = device_input(case, dev).reshape(tokens, spec.hidden)[rank * per:(rank + 1) * per].contiguous()
        step = lambda: block(h)
        launches_per_step = block.launches_per_step

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        y = step()
    barrier()
    moe.device_status()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)  # let nvidia-smi come up so that it samples the timed region
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(args.steps):
        y = step()
    ev1.record()
    barrier()
    ms_total = ev0.elapsed_time(ev1)
    if world > 1:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    value = tokens * layers / (ms_step * 1e-3)
    moe.device_status()

    # ---- same K steps again with CUDA events around every stage (the events
    # cost a few microseconds per step, so they stay out of the timed region);
    # if the timed region was too short for nvidia-smi's 100 ms period, this pass
    # is repeated until the sampler has seen the same load for half a second
    C.check(C.lib.b200moe_profile_enable(1))
    if world > 1:
        block.backend.profile = True
    t_soak = time.perf_counter()
    for _ in range(args.steps):
        y = step()
    torch.cuda.synchronize()
    stage_ms = (ctypes.c_float * 6)()
    calls = ctypes.c_int32(0)
    C.check(C.lib.b200moe_profile_read(stage_ms, ctypes.byref(calls)))
    C.check(C.lib.b200moe_profile_enable(0))
    if world > 1:
        block.backend.profile = False
    soak_steps = 0
    if world == 1:
        while ms_total < 500.0 and time.perf_counter() - t_soak < 0.6:
            y = step()
            soak_steps += 1
    elif ms_total < 500.0:
        # every rank must run the same number of collective steps
        soak_steps = max(1, min(2000, int(500.0 / max(ms_step, 1e-3))))
        for _ in range(soak_steps):
            y = step()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None:
        clocks["window"] = ("timed region + stage-event pass" +
                            (f" + {soak_steps} more steps of the same load" if soak_steps else ""))

    # ---- end to end through the C ABI with host buffers (pinned), copies timed
    e2e = None
    if world == 1 and layers > 1:
        hp = h.cpu().pin_memory()
        yp = torch.empty_like(hp).pin_memory()
        h_dev = torch.empty_like(h)
        nbytes = hp.numel() * hp.element_size()

        def e2e_step():
            h_dev.copy_(hp, non_blocking=True)
            yp.copy_(stack(h_dev), non_blocking=True)
            torch.cuda.current_stream().synchronize()

        for _ in range(3):
            e2e_step()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            e2e_step()
        dt = time.perf_counter() - t0
        e2e = {"value": tokens * layers * args.steps / dt, "unit": "tokens/s",
               "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes}
    elif world == 1:
        layer = block.layer
        hp = h.cpu().pin_memory()
        yp = torch.empty_like(hp).pin_memory()
        nbytes = hp.numel() * hp.element_size()
        dev_io = torch.empty(2 * (nbytes + 1024), dtype=torch.uint8, device=dev)
        ws = layer.workspace(tokens)
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        regime = moe.REGIMES[args.regime]

        def e2e_step():
            C.check(C.lib.b200moe_layer_forward_host(
                ctypes.byref(layer.desc), ctypes.c_void_p(hp.data_ptr()),
                ctypes.c_void_p(yp.data_ptr()), C.DT_BF16, tokens, regime,
                ctypes.c_void_p(dev_io.data_ptr()), ctypes.c_void_p(ws.data_ptr()), ws.numel(), st))
            torch.cuda.current_stream().synchronize()

        for _ in range(3):
            e2e_step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            e2e_step()
        dt = time.perf_counter() - t0
        assert torch.equal(yp.to(dev), y.reshape(yp.shape)), "host path and device path disagree"
        e2e = {"value": tokens * args.steps / dt, "unit": "tokens/s",
               "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes}
    else:
        hp = h.cpu().pin_memory()
        yp = torch.empty_like(hp).pin_memory()
        h_dev = torch.empty_like(h)
        nbytes = hp.numel() * hp.element_size()

        def e2e_step():
            h_dev.copy_(hp, non_blocking=True)
            yy = block(h_dev)
            yp.copy_(yy, non_blocking=True)
            torch.cuda.current_stream().synchronize()

        for _ in range(3):
            e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            e2e_step()
        barrier()
        dt = torch.tensor([time.perf_counter() - t0], device=dev)
        dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        e2e = {"value": tokens * args.steps / float(dt.item()), "unit": "tokens/s",
               "h2d_bytes_per_step": nbytes * world, "d2h_bytes_per_step": nbytes * world}

    # ---- roofline of the dominant kernel (gate/up), from the stage events
    n_calls = max(int(calls.value), 1)
    stage = {n: stage_ms[i] / n_calls for i, n in enumerate(STAGES)}
    if world == 1:
        experts_active = min(spec.experts, tokens * spec.top_k)
        if tokens >= 512:
            gu_flops = tokens * spec.top_k * 2 * 2 * spec.ffn * spec.hidden
            ach = gu_flops / (stage["gate_up"] * 1e-3) / 1e12
            peak = peaks["bf16_tflops"]
            roofline = {"bound": "tensor", "kernel": "gate_up", "achieved": ach, "peak": peak,
                        "unit": "TFLOP/s", "frac": ach / peak, "traffic": None,
                        "frac_of_sustained": ach / peaks["bf16_tflops_sustained"],
                        "peak_source": peaks["source"] + " (cuBLAS bf16 burst)"}
        else:
            gu_bytes = experts_active * 2 * syn.weight_bytes(spec.kind, spec.ffn, spec.hidden)
            ach = gu_bytes / (stage["gate_up"] * 1e-3) / 1e9
            peak = peaks["hbm_gbs"]
            # DRAM traffic of this kernel per launch: an ncu capture of a 374 MB case of
            # the same kernel read 1.0028 x its quantised bytes; traffic grows with them
            roofline = {"bound": "hbm", "kernel": "gate_up", "achieved": ach, "peak": peak,
                        "unit": "GB/s", "frac": ach / peak, "traffic": gu_bytes * 1.0028,
                        "peak_source": peaks["source"] + " (copy)"}
        layer_bytes = experts_active * w_bytes_expert + 2 * tokens * spec.hidden * 2 + spec.experts * spec.hidden * 4
        whole = {"tensor_frac": layers * flops / (ms_step * 1e-3) / 1e12 / peaks["bf16_tflops"],
                 "hbm_frac": layers * layer_bytes / (ms_step * 1e-3) / 1e9 / peaks["hbm_gbs"]}
    else:
        # gate/up kernel on every rank: flops of the rows each rank received over
        # the slowest rank's mean kernel time, against N x the single-GPU peak
        tm = block.backend.timings
        gu_ms = sum(ev[0].elapsed_time(ev[1]) for ev, _ in tm) / max(len(tm), 1)
        rows = sum((n if n >= 0 else tokens * spec.top_k / world) for _, n in tm) / max(len(tm), 1)
        t = torch.tensor([gu_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        r = torch.tensor([rows], device=dev)
        dist.all_reduce(r, op=dist.ReduceOp.SUM)
        gu_flops = float(r.item()) * 2 * 2 * spec.ffn * spec.hidden
        ach = gu_flops / (float(t.item()) * 1e-3) / 1e12
        peak = peaks["bf16_tflops"] * world
        roofline = {"bound": "tensor", "kernel": "gate_up", "achieved": ach, "peak": peak,
                    "unit": "TFLOP/s", "frac": ach / peak, "traffic": None,
                    "peak_source": peaks["source"] + f" (cuBLAS bf16 burst x {world} GPUs)"}
        stage = {"gate_up_max_over_ranks": float(t.item())}
        whole = {"tensor_frac": flops / (ms_step * 1e-3) / 1e12 / peak}

    # ---- L2-cold variant for the HBM-bound decode workloads: a 256 MB buffer
    # (twice the L2) is rewritten before every step; each step has its own events
    l2_cold = None
    if world == 1 and layers == 1 and tokens <= 512:
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        pairs_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                    for _ in range(args.steps)]
        for i, (a, b) in enumerate(pairs_ev):
            flush.fill_(i & 0xFF)
            a.record()
            y = step()
            b.record()
        torch.cuda.synchronize()
        cold = sorted(a.elapsed_time(b) for a, b in pairs_ev)
        cold_ms = cold[len(cold) // 2]
        l2_cold = {"ms_per_step": cold_ms, "value": tokens / (cold_ms * 1e-3), "unit": "tokens/s",
                   "flush_bytes": flush.numel(), "statistic": f"median of {args.steps} single-step timings"}
        del flush
        moe.device_status()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        torch.set_num_threads(os.cpu_count() or 1)
        sample = min(tokens, 8)
        params, hs, _ = cpu_reference_setup(case, sample)
        tps, _ = time_cpu(params, hs, steps=3, warmup=1)
        cpu = {"value": tps, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
               "sample": f"{sample} tokens x 3 steps of the same layer on the host (torch-eager "
                         f"gather + batched-GEMV form of the reference, dequantised weights)"}

    if rank == 0:
        out = {
            "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16 operands (exact Q8_0 dequant), f32 accumulate, bf16 activations in/out",
            "data": "synthetic",
            "config": {"workload": args.workload,
                       "layer": f"{spec_name} MoE FFN ({spec.kind} experts, {spec.activation})"
                                + (f", stack of {layers} layers, value = layer-tokens/s" if layers > 1 else ""),
                       "tokens": tokens, "hidden": spec.hidden, "ffn": spec.ffn,
                       "experts": spec.experts, "top_k": spec.top_k, "regime": args.regime,
                       "parallelism": "single GPU" if world == 1 else f"ep{world}, exchange: {transport}",
                       "l2": "expert weights (>= 0.8 GB per layer) exceed L2 (126 MB); no flush"},
            "e2e": e2e, "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks, "roofline": roofline, "stage_ms": stage, "whole_layer": whole,
            "cpu_baseline": cpu,
        }
        if l2_cold is not None:
            out["l2_cold"] = l2_cold
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
