"""Benchmark of the MoE FFN layer: Mixtral-8x7B-shaped, Q8_0 expert weights.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One "step" is one MoE-layer forward over one batch of synthetic tokens.  Prints
ONE JSON line (rank 0).  Workloads (hidden 4096, ffn 14336, 8 experts, top-2,
SiLU, Q8_0 weights, bf16 activations, seeded synthetic values unless noted):
  prefill4096  4096 tokens (default; tensor-core bound).  On one GPU the line
               also carries `secondary.decode32`: the 32-token decode workload
               measured on the same layer in the same run
  decode32     32 tokens   (HBM bound: the weights are streamed once per call)
  decode1 / decode128
  q4k_decode32 / q4k_prefill2048   the same layer with Q4_K expert weights
  grok_prefill8192                 Grok-1 shape (hidden 6144, ffn 32768, GELU, output norm)
  stack32_decode64                 32 Mixtral layers back to back, 64 tokens, Zipf(1.2)
                                   router bias per layer (weights drawn on the device)
  attn_decode                      the attention block's paged decode kernel alone, Mixtral
                                   shape (32 heads, 8 kv heads, head_dim 128), 32 sequences
                                   of 4096 cached positions, fp16 cache (HBM bound)
  profile_small                    the Mixtral layer with a quarter of the ffn rows (3584;
                                   374 MB of Q8_0 weights, larger than L2) for profiler
                                   captures: --tokens sets the token count, --regime the
                                   kernel family, --kind Q4_K the other layout

With N > 1 (torchrun, one process per GPU) the experts are partitioned over the
ranks, each rank routes tokens/N tokens and the token rows move between GPUs;
the total token count stays fixed ("strong" scaling).

`--impl reference` times the reference's own torch-eager layer on the host
cores: sharktank's MoeBlock itself when the package is importable (from
$SHARKTANK_SRC or baseline/_ref, through the iree stand-in of tests/golden),
else the CPU restatement in oracle/moe_oracle.py, on dequantised weights, a
bounded token sample per step.
"""
from __future__ import annotations

import argparse
import ctypes
import dataclasses
import json
import math
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
    "profile_small": ("mixtral_q8", 256),
    "attn_decode": ("mixtral_q8", 32),
}
STAGES = ["router", "route_plan", "permute", "gate_up", "down", "combine"]
SOAK_S = 0.6          # same load before the timed region, so that it runs at the settled clock
CPU_CHUNK = 4         # tokens per call of the reference layer (its gather is 470 MB fp32 per token and matrix)


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


def workload_config(args, spec_name, spec, tokens, layers, world, transport):
    """The `config` object; both arms print exactly this."""
    return {"workload": args.workload,
            "layer": f"{spec_name} MoE FFN ({spec.kind} experts, {spec.activation})"
                     + (f", stack of {layers} layers, value = layer-tokens/s" if layers > 1 else ""),
            "tokens": tokens, "hidden": spec.hidden, "ffn": spec.ffn,
            "experts": spec.experts, "top_k": spec.top_k, "regime": args.regime,
            "parallelism": "single GPU" if world == 1 else f"ep{world}, exchange: {transport}",
            "l2": "expert weights (>= 0.8 GB per layer) exceed L2 (126 MB); no flush"}


# ------------------------------------------------------------------ CPU arm
def reference_source():
    for cand in (os.environ.get("SHARKTANK_SRC", ""), os.path.join(ROOT, "baseline", "_ref")):
        if cand and os.path.isdir(os.path.join(cand, "sharktank")):
            return cand
    return None


class CpuLayer:
    """The layer on the host cores with dequantised weights: sharktank's own
    MoeBlock when it can be imported (kind "reference"), else the oracle's
    restatement of it (kind "port").  Tokens go through in chunks of CPU_CHUNK:
    the reference gathers a dense [tokens, k, N, K] copy of the expert weights."""

    def __init__(self, case):
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        from helpers import oracle_params

        import torch.nn.functional as F

        self.spec = case.spec
        params = oracle_params(case)  # dequantised the way the reference's unbox_tensor does (fp16)
        self.kind = "port"
        self.how = "oracle/moe_oracle.py restatement of sharktank's MoeBlock (gather + batched-GEMV form)"
        src = reference_source()
        if src is not None:
            try:
                for p in (os.path.join(ROOT, "tests", "golden"), src):
                    if p not in sys.path:
                        sys.path.insert(0, p)
                import iree_stub

                iree_stub.install()
                from sharktank.layers.mixture_of_experts_block import MoeBlock
                from sharktank.types import DefaultPrimitiveTensor, Theta

                tree = {
                    "ffn_gate_inp": {"weight": DefaultPrimitiveTensor(data=params.router_w)},
                    "ffn_norm": {"weight": DefaultPrimitiveTensor(data=params.norm_w)},
                    "ffn_gate_exps": {"weight": DefaultPrimitiveTensor(data=params.w_gate)},
                    "ffn_up_exps": {"weight": DefaultPrimitiveTensor(data=params.w_up)},
                    "ffn_down_exps": {"weight": DefaultPrimitiveTensor(data=params.w_down)},
                }
                if params.router_b is not None:
                    tree["ffn_gate_inp"]["bias"] = DefaultPrimitiveTensor(data=params.router_b)
                if params.out_norm_w is not None:
                    tree["layer_output_norm"] = {"weight": DefaultPrimitiveTensor(data=params.out_norm_w)}
                act = F.silu if self.spec.activation == "silu" else F.gelu
                self.block = MoeBlock(Theta(tree), self.spec.experts, self.spec.top_k, self.spec.eps,
                                      moe_activation=act)
                self.kind = "reference"
                self.how = (f"sharktank's own MoeBlock.forward (unmodified, from {os.path.relpath(src, ROOT)}; "
                            "iree-turbine replaced by the import stand-in of tests/golden)")
            except Exception as exc:  # fall back to the restatement, say why
                self.how += f" [sharktank import failed: {type(exc).__name__}: {str(exc)[:80]}]"
        if self.kind == "port":
            from oracle import moe_oracle as orc

            self.block = lambda h: orc.moe_block(h, params, form="pregather", chunk=CPU_CHUNK)[0]

    def forward(self, h):
        """h: [1, T, d] fp32."""
        with torch.no_grad():
            return torch.cat([self.block(h[:, t0:t0 + CPU_CHUNK]) for t0 in range(0, h.shape[1], CPU_CHUNK)], 1)

    def time(self, h, steps, warmup):
        for _ in range(warmup):
            self.forward(h)
        t0 = time.perf_counter()
        for _ in range(steps):
            self.forward(h)
        dt = time.perf_counter() - t0
        return h.shape[1] * steps / dt, dt / steps


def cpu_sample_tokens(tokens, steps):
    """Tokens per step of the CPU arm: at least 256 tokens over the timed steps
    (the reference is linear in tokens: it processes them in independent
    chunks), at least 16 and at most 256 per step, never more than the workload."""
    per = max(16, -(-256 // max(steps, 1)))
    per = -(-per // CPU_CHUNK) * CPU_CHUNK
    return max(1, min(tokens, per, 256))


def run_reference(args, spec_name, tokens):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from shark_platform_b200 import synthetic as syn

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    spec = syn.CASES[spec_name]
    layers = 32 if args.workload == "stack32_decode64" else 1
    steps, warmup = args.steps, args.warmup
    sample = cpu_sample_tokens(tokens, steps)
    t0 = time.time()
    case = syn.make_case(spec, tokens=sample)
    cpu = CpuLayer(case)
    setup_s = time.time() - t0
    tps, per_step = cpu.time(case.h, steps, warmup)
    sample_txt = (f"{sample} tokens per step ({CPU_CHUNK} per layer call) of the {tokens}-token workload, "
                  f"{steps} timed steps = {sample * steps} tokens after {warmup} warm-up steps; {cpu.how}; "
                  f"weights dequantised to fp16 as the reference's unbox_tensor does, fp32 activations; "
                  f"one layer" + (" of the 32 (every layer costs the same)" if layers > 1 else "")
                  + f"; set-up {setup_s:.0f} s outside the timed region")
    world = args.gpus
    print(json.dumps({
        "impl": "reference", "metric": "moe_layer_tokens_per_s", "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": per_step * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": workload_config(args, spec_name, spec, tokens, layers, world, args.ep),
        "sample_tokens": sample,
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": torch.get_num_threads(),
                         "kind": cpu.kind, "sample": sample_txt},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


# ----------------------------------------------------------- one GPU, one layer
def event_ms(fn, steps):
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(steps):
        fn()
    ev1.record()
    torch.cuda.synchronize()
    return ev0.elapsed_time(ev1)


def soak(fn, seconds=SOAK_S):
    """Runs the step for `seconds` of wall time; returns the number of steps."""
    n, t0 = 0, time.perf_counter()
    while time.perf_counter() - t0 < seconds:
        for _ in range(4):
            fn()
        torch.cuda.synchronize()
        n += 4
    return n


def stage_times(C, fn, steps):
    C.check(C.lib.b200moe_profile_enable(1))
    for _ in range(steps):
        fn()
    torch.cuda.synchronize()
    stage_ms = (ctypes.c_float * 6)()
    calls = ctypes.c_int32(0)
    C.check(C.lib.b200moe_profile_read(stage_ms, ctypes.byref(calls)))
    C.check(C.lib.b200moe_profile_enable(0))
    n = max(int(calls.value), 1)
    return {name: stage_ms[i] / n for i, name in enumerate(STAGES)}


def roofline_single(syn, spec, tokens, stage, peaks, experts_total=None):
    E = experts_total or spec.experts
    experts_active = min(E, tokens * spec.top_k)
    if tokens >= 512:
        gu_flops = tokens * spec.top_k * 2 * 2 * spec.ffn * spec.hidden
        ach = gu_flops / (stage["gate_up"] * 1e-3) / 1e12
        # the kernel is timed inside a long run at the settled clock (SOAK_S of the
        # same steps come first), so the denominator is the sustained cuBLAS figure
        peak = peaks["bf16_tflops_sustained"]
        return {"bound": "tensor", "kernel": "gate_up", "achieved": ach, "peak": peak,
                "unit": "TFLOP/s", "frac": ach / peak, "traffic": None,
                "frac_of_burst": ach / peaks["bf16_tflops"],
                "peak_source": peaks["source"] + " (cuBLAS bf16, sustained under the power cap; "
                               f"burst {peaks['bf16_tflops']})"}
    gu_bytes = experts_active * 2 * syn.weight_bytes(spec.kind, spec.ffn, spec.hidden)
    ach = gu_bytes / (stage["gate_up"] * 1e-3) / 1e9
    peak = peaks["hbm_gbs"]
    # traffic is not measured inside this run (an ncu capture of the same kernel
    # on a 374 MB case is summarised under profiles/)
    return {"bound": "hbm", "kernel": "gate_up", "achieved": ach, "peak": peak,
            "unit": "GB/s", "frac": ach / peak, "traffic": None,
            "algorithmic_bytes": gu_bytes, "peak_source": peaks["source"] + " (copy)"}


def e2e_pipeline(C, moe, layer, h, steps, regime, depth):
    """The same metric through the host-buffer entry points: every step copies
    its input from pinned host memory and its output back; `depth` steps are in
    flight (depth 1 = one step at a time)."""
    tokens = h.shape[0]
    dev = h.device
    hp = [h.cpu().pin_memory() for _ in range(max(depth, 1))]
    yp = [torch.empty_like(hp[0]).pin_memory() for _ in range(max(depth, 1))]
    nbytes = hp[0].numel() * hp[0].element_size()
    pipe = moe.HostPipeline(layer, tokens, h.dtype, depth=depth, regime=regime)
    # the same soak as the device-timed region: the pipeline runs for SOAK_S
    # seconds first, so that the timed steps see the settled clock and not the
    # boost the GPU returns to while the host sets the pipeline up
    soaked = 0
    t_end = time.perf_counter() + SOAK_S
    while time.perf_counter() < t_end or soaked < 3:
        pipe.submit(hp[soaked % depth], yp[soaked % depth])  # waits for its slot: at most `depth` in flight
        soaked += 1
    pipe.drain()
    t0 = time.perf_counter()
    for i in range(steps):
        pipe.submit(hp[i % depth], yp[i % depth])
    pipe.drain()
    dt = time.perf_counter() - t0
    y_last = yp[(steps - 1) % depth].to(dev)
    pipe.close()
    return {"value": tokens * steps / dt, "unit": "tokens/s", "h2d_bytes_per_step": nbytes,
            "d2h_bytes_per_step": nbytes, "steps_in_flight": depth,
            "soak_steps_before_timing": soaked}, y_last


def measure_layer(C, moe, syn, block, h, spec, args, peaks, sampler=None, cold=True):
    """value / stages / roofline / e2e / L2-cold of one layer on one GPU for the
    tokens in h ([T, d] on the device)."""
    tokens = h.shape[0]
    step = lambda: block(h)
    for _ in range(args.warmup):
        y = step()
    torch.cuda.synchronize()
    moe.device_status()
    if sampler is not None:
        sampler.start()
    soak_steps = soak(step)
    ms_total = event_ms(step, args.steps)
    ms_step = ms_total / args.steps
    moe.device_status()
    stage = stage_times(C, step, args.steps)
    clocks = None
    if sampler is not None:
        soak(step, 0.25)  # the sampler's period is 100 ms: a few more samples of the same load
        clocks = sampler.stop()
        clocks["window"] = (f"{SOAK_S} s of the same steps before the timed region, the timed region, the "
                            "stage-event pass and 0.25 s more of the same steps")
    y = step()
    out = {"value": tokens / (ms_step * 1e-3), "ms_per_step": ms_step, "stage_ms": stage, "clocks": clocks,
           "soak_steps_before_timing": soak_steps,
           "roofline": roofline_single(syn, spec, tokens, stage, peaks)}
    flops = syn.layer_flops(tokens, spec.top_k, spec.hidden, spec.ffn)
    experts_active = min(spec.experts, tokens * spec.top_k)
    layer_bytes = (experts_active * 3 * syn.weight_bytes(spec.kind, spec.ffn, spec.hidden)
                   + 2 * tokens * spec.hidden * 2 + spec.experts * spec.hidden * 4)
    out["whole_layer"] = {"tensor_frac": flops / (ms_step * 1e-3) / 1e12 / peaks["bf16_tflops_sustained"],
                          "tensor_frac_of_burst": flops / (ms_step * 1e-3) / 1e12 / peaks["bf16_tflops"],
                          "hbm_frac": layer_bytes / (ms_step * 1e-3) / 1e9 / peaks["hbm_gbs"]}
    regime = moe.REGIMES[args.regime]
    e2e, y_host = e2e_pipeline(C, moe, block.layer, h, args.steps, regime, depth=2)
    assert torch.equal(y_host, y.reshape(y_host.shape)), "host path and device path disagree"
    one, _ = e2e_pipeline(C, moe, block.layer, h, args.steps, regime, depth=1)
    e2e["one_step_at_a_time"] = one["value"]
    out["e2e"] = e2e
    if cold and tokens <= 512:
        # L2-cold variant for the HBM-bound decode workloads: a 256 MB buffer
        # (twice the L2) is rewritten before every step; each step has its own events
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=h.device)
        pairs_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                    for _ in range(args.steps)]
        for i, (a, b) in enumerate(pairs_ev):
            flush.fill_(i & 0xFF)
            a.record()
            step()
            b.record()
        torch.cuda.synchronize()
        t = sorted(a.elapsed_time(b) for a, b in pairs_ev)
        cold_ms = t[len(t) // 2]
        out["l2_cold"] = {"ms_per_step": cold_ms, "value": tokens / (cold_ms * 1e-3), "unit": "tokens/s",
                          "hbm_frac": layer_bytes / (cold_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                          "flush_bytes": flush.numel(),
                          "statistic": f"median of {args.steps} single-step timings"}
        del flush
        moe.device_status()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="prefill4096", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--regime", default="auto", choices=["auto", "stream", "tensor", "tensor_pair"])
    ap.add_argument("--ep", default="p2p", choices=["p2p", "nccl"],
                    help="token exchange between ranks: peer-to-peer stores or NCCL all-to-all")
    ap.add_argument("--tokens", type=int, default=0, help="profile_small only: token count")
    ap.add_argument("--kind", default="Q8_0", choices=["Q8_0", "Q4_K"], help="profile_small only")
    ap.add_argument("--token-tile", type=int, default=0, choices=[0, 64, 128, 192],
                    help="upper bound of the tensor kernel's token tile (0 = the library's default)")
    ap.add_argument("--stream-wide", type=int, default=-1, choices=[-1, 0, 1],
                    help="streaming kernel: 16 consumer warps (1), 8 (0), by layout (-1, the default)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true")
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
    peaks = measured_peaks()
    spec = syn.CASES[spec_name]
    transport = args.ep
    if args.token_tile:
        C.check(C.lib.b200moe_set_token_tile(args.token_tile))
    if args.stream_wide >= 0:
        C.check(C.lib.b200moe_set_stream_wide(args.stream_wide))

    # ------------------------------------------ decode attention over the pages
    if args.workload == "attn_decode":
        bs, seq, heads, kvh, hd, stride, blocks = 32, args.tokens or 4096, 32, 8, 128, 32, 1
        per = seq // stride + 1
        pages = bs * per
        desc = C.KvCacheDesc(blocks, stride, kvh, hd, pages)
        gen = torch.Generator(device=dev).manual_seed(7)
        slab = (torch.randn(pages, blocks * 2 * stride * kvh * hd, generator=gen, device=dev) * 0.5).half()
        q = torch.randn(bs, heads, hd, generator=gen, device=dev).half()
        ids = torch.randperm(pages, generator=gen, device=dev).to(torch.int32).view(bs, per)
        lens = torch.full((bs,), seq, dtype=torch.int32, device=dev)
        out = torch.empty_like(q)
        nbytes = C.lib.b200moe_attn_decode_scratch_bytes(ctypes.byref(desc), bs, heads, per * stride)
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        pp = lambda t: ctypes.c_void_p(t.data_ptr())
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

        def step():
            C.check(C.lib.b200moe_attn_decode(pp(q), C.DT_F16, pp(slab), C.DT_F16, ctypes.byref(desc), 0, pp(ids),
                                              pp(lens), bs, per, heads, per * stride, 1.0 / hd ** 0.5, 0.0, pp(out),
                                              C.DT_F16, pp(scratch), nbytes, st), "attn_decode")

        for _ in range(args.warmup):
            step()
        torch.cuda.synchronize()
        soak(step, 0.3)
        ms = event_ms(step, args.steps) / args.steps
        moe.device_status()
        kv_bytes = bs * seq * kvh * hd * 2 * 2
        ach = kv_bytes / (ms * 1e-3) / 1e9
        print(json.dumps({"metric": "attention_decode_tokens_per_s", "value": bs / (ms * 1e-3), "unit": "tokens/s",
                          "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
                          "higher_is_better": True, "data": "synthetic", "dtype": "f16 cache, f32 softmax",
                          "config": {"workload": "attn_decode", "sequences": bs, "cached_positions": seq,
                                     "heads": heads, "kv_heads": kvh, "head_dim": hd, "page_stride": stride},
                          "roofline": {"bound": "hbm", "kernel": "attn_decode", "achieved": ach,
                                       "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"],
                                       "traffic": None, "algorithmic_bytes": kv_bytes,
                                       "peak_source": peaks["source"] + " (copy)"}}), flush=True)
        return

    # ------------------------------------------------------------ profiler case
    if args.workload == "profile_small":
        tokens = args.tokens or tokens
        sp = dataclasses.replace(spec, tokens=tokens, ffn=3584, kind=args.kind)
        case = syn.make_case_on_device(sp, dev)
        block = syn.case_block(case, args.regime, dev)
        h = syn.case_input(case, dev).reshape(tokens, sp.hidden).contiguous()
        for _ in range(args.warmup):
            block(h)
        torch.cuda.synchronize()
        ms = event_ms(lambda: block(h), args.steps) / args.steps
        moe.device_status()
        print(json.dumps({"metric": "moe_layer_tokens_per_s", "value": tokens / (ms * 1e-3),
                          "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
                          "ms_per_step": ms, "higher_is_better": True, "data": "synthetic",
                          "config": {"workload": "profile_small", "tokens": tokens, "experts": sp.experts,
                                     "hidden": sp.hidden, "ffn": sp.ffn, "kind": sp.kind,
                                     "regime": args.regime}}), flush=True)
        return

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    layers = 1
    secondary = None
    cpu = None
    sampler = ClockSampler(local_rank)

    # ----------------------------------------------------------- one GPU, one layer
    if world == 1 and args.workload != "stack32_decode64":
        case = syn.make_case(spec, tokens=tokens)
        block = syn.case_block(case, args.regime, dev)
        h = syn.case_input(case, dev).reshape(tokens, spec.hidden).contiguous()
        fused = C.lib.b200moe_front_supported(tokens, ctypes.byref(block.layer.desc))
        launches_per_step = 4 if fused else 6
        m = measure_layer(C, moe, syn, block, h, spec, args, peaks, sampler)
        clocks = m["clocks"]
        if args.workload == "prefill4096" and not args.no_secondary:
            # the other headline target, on the same layer in the same run
            h32 = h[:32].contiguous()
            m2 = measure_layer(C, moe, syn, block, h32, spec, args, peaks, ClockSampler(local_rank))
            c2 = m2["clocks"]
            secondary = {"decode32": {
                "config": {"workload": "decode32", "tokens": 32, "note": "first 32 tokens of the same batch, same layer"},
                "value": m2["value"], "unit": "tokens/s", "ms_per_step": m2["ms_per_step"],
                "roofline": m2["roofline"], "whole_layer": m2["whole_layer"], "stage_ms": m2["stage_ms"],
                "l2_cold": m2.get("l2_cold"), "e2e": m2["e2e"], "clocks": c2,
                "gpu_launches": 4 * args.steps}}
        if not args.no_cpu_baseline:
            torch.set_num_threads(os.cpu_count() or 1)
            sample = max(1, min(tokens, 128))
            sub = dataclasses.replace(case, h=case.h[:, :sample].contiguous())
            cl = CpuLayer(sub)
            tps, _ = cl.time(sub.h, steps=1, warmup=0)
            cpu = {"value": tps, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": cl.kind,
                   "sample": f"the first {sample} tokens of the same batch, one pass ({CPU_CHUNK} tokens per "
                             f"layer call), same layer on the host: {cl.how}"}
        value, ms_step = m["value"], m["ms_per_step"]
        e2e, roofline, stage, whole = m["e2e"], m["roofline"], m["stage_ms"], m["whole_layer"]
        l2_cold = m.get("l2_cold")
    elif world == 1:
        # ------------------------------------------- 32-layer stack on one GPU
        from shark_platform_b200.moe import B200MoeStack

        layers = 32
        blocks = []
        for i in range(layers):
            sp = dataclasses.replace(spec, tokens=tokens, router_bias="zipf", seed=1000 + i)
            blocks.append(syn.case_block(syn.make_case_on_device(sp, dev), args.regime, dev))
        stack = B200MoeStack(blocks)
        case0 = syn.make_case_on_device(dataclasses.replace(spec, tokens=tokens, seed=999), dev)
        h = syn.case_input(case0, dev).reshape(tokens, spec.hidden).contiguous()
        step = lambda: stack(h)
        fused = C.lib.b200moe_front_supported(tokens, ctypes.byref(blocks[0].layer.desc))
        launches_per_step = (4 if fused else 6) * layers
        for _ in range(args.warmup):
            step()
        torch.cuda.synchronize()
        moe.device_status()
        sampler.start()
        time.sleep(0.3)
        soak(step)
        ms_step = event_ms(step, args.steps) / args.steps
        stage = stage_times(C, step, min(args.steps, 512 // layers))
        clocks = sampler.stop()
        clocks["window"] = f"{SOAK_S} s of the same steps before the timed region, the timed region, the stage-event pass"
        moe.device_status()
        value = tokens * layers / (ms_step * 1e-3)
        roofline = roofline_single(syn, spec, tokens, stage, peaks)
        layer_bytes = (spec.experts * 3 * syn.weight_bytes(spec.kind, spec.ffn, spec.hidden)
                       + 2 * tokens * spec.hidden * 2 + spec.experts * spec.hidden * 4)
        whole = {"hbm_frac": layers * layer_bytes / (ms_step * 1e-3) / 1e9 / peaks["hbm_gbs"]}
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
               "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes, "steps_in_flight": 1}
        l2_cold = None
    elif args.workload == "stack32_decode64":
        # ------------------- 32-layer stack, expert parallel (peer-to-peer)
        from shark_platform_b200 import parallel
        from shark_platform_b200.moe import B200MoeStack

        layers = 32
        per = tokens // world
        case0 = syn.make_case_on_device(dataclasses.replace(spec, tokens=tokens, seed=999), dev)
        h_all = syn.case_input(case0, dev).reshape(tokens, spec.hidden)
        h = h_all[rank * per:(rank + 1) * per].contiguous()
        # layer by layer: draw the full layer (same seed on every rank), route this
        # rank's slice of the running activations through the single-GPU layer as
        # the correctness witness, keep the expert shard, drop the rest
        x = parallel.P2PExchange(spec.hidden, spec.experts, spec.top_k, tokens, per, dist.group.WORLD, dev)
        blocks, rows = [], torch.zeros(spec.experts, device=dev)
        want, inputs, wants = h, [], []
        for i in range(layers):
            sp = dataclasses.replace(spec, tokens=tokens, router_bias="zipf", seed=1000 + i)
            c = syn.make_case_on_device(sp, dev)
            full = syn.case_block(c, args.regime, dev)
            inputs.append(want)
            want, ex_i, _ = full.layer.forward(want, want_routing=True)
            wants.append(want)
            rows += torch.bincount(ex_i.reshape(-1).to(torch.int64), minlength=spec.experts).float()
            del full
            blocks.append(parallel.build_from_case(c, dist.group.WORLD, args.regime, "p2p", per, x))
            del c
            torch.cuda.empty_cache()
        stack = parallel.ExpertParallelStack(blocks)
        step = lambda: stack(h)
        launches_per_step = blocks[0].launches_per_step * layers
        # witness per layer, every layer fed the single-GPU chain's own input (a
        # chain of 32 random layers amplifies a rounding difference into different
        # expert choices further down, so end-to-end distance is not a measure)
        worst = torch.zeros(1, device=dev)
        for blk, xin, ref_out in zip(blocks, inputs, wants):
            got = blk(xin)
            agg = torch.stack([torch.linalg.norm((got.float() - ref_out.float()).double()) ** 2,
                               torch.linalg.norm(ref_out.float().double()) ** 2])
            dist.all_reduce(agg)
            worst = torch.maximum(worst, torch.sqrt(agg[0] / agg[1]).float().reshape(1))
        ep_check = {"rel_l2_vs_single_gpu": float(worst.item()),
                    "what": "largest over the 32 layers: each expert-parallel layer against the full "
                            "single-GPU layer on the same input (the single-GPU chain's), all ranks' tokens"}
        del inputs, wants
        for _ in range(args.warmup):
            step()
        barrier()
        moe.device_status()
        if rank == 0:
            sampler.start()
        for _ in range(40):  # ~0.5 s of the same load on every rank before timing
            step()
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(args.steps):
            y = step()
        ev1.record()
        barrier()
        t = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step = float(t.item()) / args.steps
        value = tokens * layers / (ms_step * 1e-3)
        moe.device_status()
        stage = stage_times(C, step, min(args.steps, 512 // layers))
        barrier()
        clocks = sampler.stop() if rank == 0 else None
        if clocks is not None:
            clocks["window"] = "40 steps of the same load before the timed region, the timed region, the stage-event pass"
        dist.all_reduce(rows)
        per_rank = rows.view(world, -1).sum(dim=1)
        # every rank streams the weights of its own experts once per layer call
        el = spec.experts // world
        rank_bytes = el * 3 * syn.weight_bytes(spec.kind, spec.ffn, spec.hidden)
        gu = torch.tensor([stage["gate_up"]], device=dev)
        dist.all_reduce(gu, op=dist.ReduceOp.MAX)
        ach = el * 2 * syn.weight_bytes(spec.kind, spec.ffn, spec.hidden) / (float(gu.item()) * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": "gate_up", "achieved": ach, "peak": peaks["hbm_gbs"],
                    "unit": "GB/s", "frac": ach / peaks["hbm_gbs"], "traffic": None,
                    "note": "per GPU: this rank's expert weights over the slowest rank's gate/up time",
                    "peak_source": peaks["source"] + " (copy)"}
        whole = {"hbm_frac_per_gpu": layers * rank_bytes / (ms_step * 1e-3) / 1e9 / peaks["hbm_gbs"],
                 "ep_check": ep_check,
                 "rows_per_rank": {"max": float(per_rank.max()), "mean": float(per_rank.mean()),
                                   "note": "rows routed to each rank's experts, summed over the 32 layers"}}
        stage = {"rank0": stage}
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
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            e2e_step()
        barrier()
        dt = torch.tensor([time.perf_counter() - t0], device=dev)
        dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        e2e = {"value": tokens * layers * args.steps / float(dt.item()), "unit": "tokens/s",
               "h2d_bytes_per_step": nbytes * world, "d2h_bytes_per_step": nbytes * world,
               "steps_in_flight": 1}
        l2_cold = None
    else:
        # ------------------------------------------------ expert parallelism
        from shark_platform_b200 import parallel

        # every rank draws the same full layer on its own GPU (same seed) and keeps
        # its expert shard: seconds instead of a minute of host-side generation
        case = syn.make_case_on_device(dataclasses.replace(spec, tokens=tokens), dev)
        per = tokens // world
        h_all = syn.case_input(case, dev).reshape(tokens, spec.hidden)
        h = h_all[rank * per:(rank + 1) * per].contiguous()
        # correctness witness, outside the timed region: this rank's token slice
        # through the single-GPU layer, before the other ranks' experts are dropped
        full_block = syn.case_block(case, args.regime, dev)
        y_single, ex_single, _ = full_block.layer.forward(h, want_routing=True)
        y_single = y_single.clone()
        del full_block
        torch.cuda.empty_cache()
        if transport == "p2p":
            try:
                block = parallel.build_from_case(case, dist.group.WORLD, regime=args.regime, transport="p2p")
            except Exception as exc:  # symmetric memory not available on this machine
                transport = f"nccl (p2p set-up failed: {type(exc).__name__}: {str(exc)[:120]})"
                block = parallel.build_from_case(case, dist.group.WORLD, regime=args.regime)
        else:
            block = parallel.build_from_case(case, dist.group.WORLD, regime=args.regime)
        del case
        torch.cuda.empty_cache()
        step = lambda: block(h)
        launches_per_step = block.launches_per_step
        y = step()
        num = torch.linalg.norm((y.float() - y_single.float()).double()) ** 2
        den = torch.linalg.norm(y_single.float().double()) ** 2
        agg = torch.stack([num, den])
        dist.all_reduce(agg)
        ep_check = {"rel_l2_vs_single_gpu": float(torch.sqrt(agg[0] / agg[1])),
                    "what": "every rank's own token slice through the full single-GPU layer vs the "
                            "expert-parallel result, all ranks' tokens together"}
        for _ in range(args.warmup):
            step()
        barrier()
        moe.device_status()
        if rank == 0:
            sampler.start()
            time.sleep(0.3)
        # the same number of soak steps on every rank (collective steps)
        t0 = time.perf_counter()
        step()
        torch.cuda.synchronize()
        n_soak = torch.tensor([max(8, int(SOAK_S / max(time.perf_counter() - t0, 1e-4)))], device=dev)
        dist.all_reduce(n_soak, op=dist.ReduceOp.MIN)
        for _ in range(min(int(n_soak.item()), 4000)):
            step()
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(args.steps):
            y = step()
        ev1.record()
        barrier()
        t = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step = float(t.item()) / args.steps
        value = tokens / (ms_step * 1e-3)
        moe.device_status()
        if isinstance(block, parallel.P2PExpertParallelMoeBlock):
            st_ms = stage_times(C, step, args.steps)  # per-stage events inside the C call
            gu_ms, dn_ms = st_ms["gate_up"], st_ms["down"]
        else:
            block.backend.profile = True
            for _ in range(args.steps):
                step()
            torch.cuda.synchronize()
            block.backend.profile = False
            tm = block.backend.timings
            gu_ms = sum(ev[0].elapsed_time(ev[1]) for ev, _ in tm) / max(len(tm), 1)
            dn_ms = sum(ev[1].elapsed_time(ev[2]) for ev, _ in tm) / max(len(tm), 1)
            st_ms = {}
        barrier()
        clocks = sampler.stop() if rank == 0 else None
        if clocks is not None:
            clocks["window"] = f"~{SOAK_S} s of the same steps before the timed region, the timed region, the stage-event pass"
        # gate/up kernel on every rank: flops of all routed rows over the slowest
        # rank's mean kernel time, against N x the single-GPU peak
        tt = torch.tensor([gu_ms, dn_ms], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        gu_flops = float(tokens * spec.top_k) * 2 * 2 * spec.ffn * spec.hidden
        ach = gu_flops / (float(tt[0].item()) * 1e-3) / 1e12
        peak = peaks["bf16_tflops_sustained"] * world
        roofline = {"bound": "tensor", "kernel": "gate_up", "achieved": ach, "peak": peak,
                    "unit": "TFLOP/s", "frac": ach / peak, "traffic": None,
                    "frac_of_burst": ach / (peaks["bf16_tflops"] * world),
                    "peak_source": peaks["source"] + f" (cuBLAS bf16, sustained under the power cap, x {world} GPUs)"}
        stage = {"gate_up_max_over_ranks": float(tt[0].item()), "down_max_over_ranks": float(tt[1].item()),
                 "rank0": st_ms}
        flops = syn.layer_flops(tokens, spec.top_k, spec.hidden, spec.ffn)
        whole = {"tensor_frac": flops / (ms_step * 1e-3) / 1e12 / peak, "ep_check": ep_check}
        # load balance: rows each rank's experts received
        rows = torch.bincount(ex_single.reshape(-1).to(torch.int64), minlength=spec.experts).float()
        dist.all_reduce(rows)
        per_rank = rows.view(world, -1).sum(dim=1)
        whole["rows_per_rank"] = {"max": float(per_rank.max()), "mean": float(per_rank.mean())}
        hp = h.cpu().pin_memory()
        yp = torch.empty_like(hp).pin_memory()
        h_dev = torch.empty_like(h)
        nbytes = hp.numel() * hp.element_size()

        def e2e_step():
            h_dev.copy_(hp, non_blocking=True)
            yp.copy_(block(h_dev), non_blocking=True)
            torch.cuda.current_stream().synchronize()

        def timed(fn):
            barrier()
            t0 = time.perf_counter()
            fn()
            barrier()
            dt = torch.tensor([time.perf_counter() - t0], device=dev)
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
            return tokens * args.steps / float(dt.item())

        for _ in range(3):
            e2e_step()
        one_at_a_time = timed(lambda: [e2e_step() for _ in range(args.steps)])

        # Two steps in flight: the copy-in of step i+1 and the copy-out of step
        # i-1 run on their own streams beside the layer call of step i; the host
        # reads every step's result (waits for its copy-out) one step later.
        depth = 2
        comp = torch.cuda.current_stream()
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        h_devs = [torch.empty_like(h) for _ in range(depth)]
        yps = [torch.empty_like(hp).pin_memory() for _ in range(depth)]
        ev_in = [torch.cuda.Event() for _ in range(depth)]
        ev_comp = [torch.cuda.Event() for _ in range(depth)]
        ev_out = [torch.cuda.Event() for _ in range(depth)]

        def pipelined(steps):
            for i in range(steps):
                s = i % depth
                with torch.cuda.stream(s_in):
                    if i >= depth:
                        s_in.wait_event(ev_comp[s])  # the layer of step i-depth has read this buffer
                    h_devs[s].copy_(hp, non_blocking=True)
                    ev_in[s].record(s_in)
                comp.wait_event(ev_in[s])
                y = block(h_devs[s])
                ev_comp[s].record(comp)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_comp[s])
                    yps[s].copy_(y, non_blocking=True)
                    y.record_stream(s_out)
                    ev_out[s].record(s_out)
                if i >= 1:
                    ev_out[(i - 1) % depth].synchronize()
            ev_out[(steps - 1) % depth].synchronize()

        pipelined(3)
        torch.cuda.synchronize()
        piped = timed(lambda: pipelined(args.steps))
        torch.cuda.synchronize()
        e2e = {"value": piped, "unit": "tokens/s",
               "h2d_bytes_per_step": nbytes * world, "d2h_bytes_per_step": nbytes * world,
               "steps_in_flight": depth, "one_step_at_a_time": one_at_a_time,
               "pipelined_equals_serial": bool(torch.equal(yps[(args.steps - 1) % depth], yp))}
        l2_cold = None

    if rank == 0:
        sm = clocks.get("sm_mhz") if clocks else None
        out = {
            "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16 operands (exact Q8_0 dequant), f32 accumulate, bf16 activations in/out",
            "data": "synthetic",
            "config": workload_config(args, spec_name, spec, tokens, layers, world, transport),
            "e2e": e2e, "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks, "ms_x_mhz": (ms_step * sm) if sm else None,
            "roofline": roofline, "stage_ms": stage, "whole_layer": whole,
            "cpu_baseline": cpu,
        }
        if l2_cold is not None:
            out["l2_cold"] = l2_cold
        if secondary is not None:
            out["secondary"] = secondary
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
