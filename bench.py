#!/usr/bin/env python3
"""Benchmark of the routed-MoE hot path (BASELINE config 1: batch-1 decode through 40 stacked
MoE layers; a "step" is one token through the whole stack).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  `value` is tokens/s with inputs resident in HBM; `e2e` is the same loop
driven through the public provider call with the token vector copied from pinned host memory and
the result read back every step; `roofline` is the algorithmic weight bytes per token
(2 307 194 880 B = 40 x 57 679 872 B) over the measured time against the measured HBM copy
bandwidth; `cpu_baseline` times the torch-CPU statement of the reference's MoE path on this
machine's cores on a bounded sample.  `--impl reference` times only that CPU path.
Synthetic seeded weights (BF16 N(0, 0.02)) and inputs (BF16 N(0, 1)) stand in for the checkpoint.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LAYERS = 40
HIDDEN = 2048
SEED = 1234
BYTES_PER_LAYER_TOKEN = 1_048_576 + 50_331_648 + 6_295_552 + 4_096       # router, 8 experts, shared, norm
BYTES_PER_TOKEN = LAYERS * BYTES_PER_LAYER_TOKEN                          # 2 307 194 880
FALLBACK_HBM_GBS = 6650.0
# all weights of one layer: router, 256 experts (gate_up + down), shared expert, shared gate, norm
BYTES_PER_LAYER_WEIGHTS = 1_048_576 + 256 * 6_291_456 + 6_291_456 + 4_096 + 4_096
# dram__bytes_read.sum + dram__bytes_write.sum per layer of the decode kernel, from the ncu capture
# summarised in profiles/moe_decode_persistent_kernel_stack2.md (2-layer case: 115.64 MB read + 4.51 MB
# written per launch; the next layer's router rows the prediction reads are the same bytes the next
# layer reads again 15 us later, so they cost no second DRAM read)
DECODE_TRAFFIC_PER_LAYER = 60_075_000


MIN_TIMED_SECONDS = 1.0      # the K-step loop is repeated until at least this much has been timed
MAX_REPEATS = 400


def decode_config(world: int) -> dict:
    """The `config` object of the decode line; both arms (--impl ours / reference) print exactly this."""
    per_rank = 256 // max(world, 1)
    return {"workload": f"decode_b1_stack{LAYERS} (BASELINE config 1)", "layers": LAYERS,
            "hidden": HIDDEN, "experts": 256, "top_k": 8,
            "l2": "inputs larger than L2 (2.3 GB of weights per step)",
            "multi_gpu": (f"expert parallel, {per_rank} experts per GPU, per-slot down products "
                          "exchanged by peer stores over NVLink") if world > 1 else "single GPU"}


def measured_peaks() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int) -> None:
        self.device_index = device_index
        self.lines: list[str] = []
        self.process: subprocess.Popen | None = None
        self.thread: threading.Thread | None = None

    def start(self) -> None:
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.device_index), "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.process = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self) -> None:
        assert self.process is not None and self.process.stdout is not None
        for line in self.process.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.process.terminate()
        try:
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        clocks, max_clocks, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clocks.append(float(parts[1]))
                max_clocks.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None,
                "sm_max_mhz": max(max_clocks) if max_clocks else None,
                "samples": len(clocks), "reasons": sorted(reasons)}


def cpu_reference_tokens_per_second(sample_layers: int, sample_tokens: int, threads: int) -> dict:
    """Times the reference's CPU statement of the MoE path for one token per layer and extrapolates linearly
    to the 40-layer stack.  Where the reference's own torch functions are at hand (cut out of the checkout into
    oracle/_ref/ at build time) those run -- kind "reference"; otherwise the restatement in oracle/ -- kind "port"."""
    import torch

    sys.path.insert(0, str(ROOT / "oracle"))
    import reference_torch
    from __graft_entry__ import load_package

    if reference_torch.available():
        ref = reference_torch.ReferenceTorch(tokens=1)
        kind, what = "reference", "the reference's own torch functions (four_layer_mini_engine.py: router_topk, " \
                                  "expanded_routed_moe, shared_expert, rmsnorm; pure-torch CPU variant)"
    else:
        import moe_torch_ref as ref
        kind, what = "port", "the torch-CPU restatement of the reference MoE path (router, top-8, expanded bmm experts, " \
                             "shared expert)"
    synth = load_package().synth
    torch.set_num_threads(threads)
    generator = torch.Generator().manual_seed(SEED)
    layers = []
    for layer in range(sample_layers):
        weights = synth.layer_small_weights(SEED, layer)
        # timing does not depend on values: one randn block reused for all experts
        block = (torch.randn(8, 1024, HIDDEN, generator=generator) * 0.02).to(torch.bfloat16)
        weights["expert_gate_up"] = block.repeat(32, 1, 1)
        down = (torch.randn(8, HIDDEN, 512, generator=generator) * 0.02).to(torch.bfloat16)
        weights["expert_down"] = down.repeat(32, 1, 1)
        layers.append(weights)
    x = synth.activations(SEED, 1, "residual", 0)

    def one_token(x):
        for weights in layers:
            h2 = ref.rmsnorm(x, weights["post_attention_layernorm"])
            x = ref.moe_half_layer(h2, x, weights, form="expanded")["out"]
        return x

    one_token(x)                                   # warm-up
    start = time.perf_counter()
    for _ in range(sample_tokens):
        x = one_token(x)
    elapsed = time.perf_counter() - start
    per_layer = elapsed / (sample_tokens * sample_layers)
    return {"value": 1.0 / (per_layer * LAYERS), "unit": "tokens/s", "cores": threads, "kind": kind,
            "sample": f"{sample_tokens} tokens x {sample_layers} layers of {what}, per-layer time x {LAYERS}",
            "seconds": elapsed}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    warm = cpu_reference_tokens_per_second(1, max(1, min(args.warmup, 2)), threads)
    del warm
    steps = max(1, min(args.steps, 24))
    result = cpu_reference_tokens_per_second(2, steps, threads)
    value = result["value"]
    line = {
        "impl": "reference", "metric": "moe_decode_b1_tokens_per_second", "value": value,
        "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1000.0 / value, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": decode_config(args.gpus),
        "timed_tokens": steps, "note": "CPU path; bounded sample extrapolated to 40 layers",
        "cpu_baseline": {k: result[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def run_ours(args) -> None:
    import torch
    from __graft_entry__ import load_package

    package = load_package()
    synth = package.synth
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    distributed = world > 1
    if distributed:
        import torch.distributed as dist

        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=device)

    # expert parallelism: rank r holds experts [r * 256 / W, (r + 1) * 256 / W); router, shared
    # expert and norms are replicated (same generator stream on every rank)
    per_rank = 256 // world
    provider = package.MoeProvider(layers=LAYERS, max_prefill_tokens=0, world=world, rank=rank)
    keep = []
    for layer in range(LAYERS):
        weights = synth.layer_weights_cuda_fast(SEED, layer, device, rank * per_rank, (rank + 1) * per_rank)
        provider.bind_layer(layer, weights)
        keep.append(weights)
    if distributed:
        provider.ep_connect_all(dist.new_group(backend="gloo"))
    if args.decode_hot:
        # profiling aid: +20 on eight fixed experts, so every layer picks the same experts (prediction always right;
        # with few layers the touched weights stay in L2)
        provider.set_router_hooks(synth.hot_expert_bias(range(3, 256, 32)).to(device), False)
    torch.cuda.synchronize()

    x0 = synth.activations(SEED, 1, "residual", 0)[0]
    buffers = [x0.to(device), torch.empty(HIDDEN, dtype=torch.bfloat16, device=device)]

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(step_fn) -> tuple[float, int, float]:
        """Times exactly args.steps steps per repeat (barrier + synchronize on both sides, CUDA events on the
        launching stream, maximum over ranks) and repeats until MIN_TIMED_SECONDS have been timed; returns
        the median ms per step, the number of repeats and the total timed milliseconds."""
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        per_step, total = [], 0.0
        while True:
            barrier()
            start.record()
            for step in range(args.steps):
                step_fn(step)
            stop.record()
            barrier()
            ms = torch.tensor([start.elapsed_time(stop)], dtype=torch.float64, device=device)
            if distributed:
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)       # every rank sees the same figure, hence the same repeat count
            ms = float(ms.item())
            per_step.append(ms / args.steps)
            total += ms
            if total >= MIN_TIMED_SECONDS * 1000.0 or len(per_step) >= MAX_REPEATS:
                return statistics.median(per_step), len(per_step), total

    # ---- device-resident loop ----
    for step in range(args.warmup):
        provider.decode_stack(buffers[step & 1], buffers[(step + 1) & 1])
    provider.sync_metrics()
    sampler = ClockSampler(local_rank)
    sampler.start()
    offset = args.warmup & 1
    device_ms_per_step, repeats, device_total_ms = timed(
        lambda step: provider.decode_stack(buffers[(offset + step) & 1], buffers[(offset + step + 1) & 1]))
    provider.sync_metrics()

    # ---- end to end through the public call with host buffers ----
    host_in = torch.empty(HIDDEN, dtype=torch.bfloat16).pin_memory()
    host_out = torch.empty(HIDDEN, dtype=torch.bfloat16).pin_memory()
    host_in.copy_(x0)
    dev_in = torch.empty(HIDDEN, dtype=torch.bfloat16, device=device)
    dev_out = torch.empty(HIDDEN, dtype=torch.bfloat16, device=device)

    def e2e_step(_step=0):
        dev_in.copy_(host_in, non_blocking=True)
        provider.decode_stack(dev_in, dev_out)
        host_out.copy_(dev_out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        host_in.copy_(host_out)                    # the token feeds back through host memory

    for _ in range(max(3, args.warmup)):
        e2e_step()
    e2e_ms_per_step, e2e_repeats, _ = timed(e2e_step)
    clocks = sampler.stop()
    provider.sync_metrics()

    if args.decode_timeline and rank == 0:
        decode_timeline_report(provider, buffers)

    # ---- N > 1: are the ranks' results the single-GPU bits?  (outside the timed region) ----
    parity = None
    if distributed:
        parity = expert_parallel_parity(package, provider, synth, device, rank, world, dist)

    # ---- N > 1: expert-parallel prefill, T = 8192 uniform: one layer and a four-layer stack (the workload
    #      that can scale; device-timed, maximum over ranks; rank 0's stage times and exposed communication) ----
    ep_prefill = None
    if distributed and not args.no_prefill:
        provider.release()
        provider = None
        del keep
        torch.cuda.empty_cache()
        one_layer = ep_prefill_numbers(package, dist, device, world, rank, 8192, 1, "uniform", 20)
        stack = ep_prefill_numbers(package, dist, device, world, rank, 8192, 4, "uniform", 5)
        if rank == 0:
            ep_prefill = {"one_layer": one_layer, "stack4": stack,
                          "exposed_communication_ms": one_layer["exposed_communication_ms"],
                          "note": "single-GPU reference for the speed-up: the `prefill` object of the N = 1 line "
                                  "(T = 8192 Zipf) or `--workload prefill --routing uniform`"}

    if rank == 0:
        peak, peak_kind = measured_peaks()
        value = 1000.0 / device_ms_per_step        # expert parallel: all ranks work on the same token
        achieved = BYTES_PER_TOKEN / (device_ms_per_step / 1000.0) / 1.0e9
        line = {
            "metric": "moe_decode_b1_tokens_per_second", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": device_ms_per_step, "higher_is_better": True,
            # one token stream served by N GPUs: the total work is fixed as N grows
            "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": decode_config(world),
            "timing": {"repeats": repeats, "steps_per_repeat": args.steps, "timed_seconds": device_total_ms / 1000.0,
                       "statistic": "median over the repeats of (K-step loop time / K)"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak * world, "unit": "GB/s",
                         "frac": achieved / (peak * world), "traffic": DECODE_TRAFFIC_PER_LAYER * LAYERS,
                         "peak_source": peak_kind, "bytes_per_step": BYTES_PER_TOKEN},
            "e2e": {"value": 1000.0 / e2e_ms_per_step, "unit": "tokens/s",
                    "h2d_bytes_per_step": HIDDEN * 2, "d2h_bytes_per_step": HIDDEN * 2, "repeats": e2e_repeats},
            "gpu_launches": args.steps * repeats,
            "clocks": clocks,
        }
        if parity is not None:
            line["parity"] = parity
        if ep_prefill is not None:
            line["prefill"] = ep_prefill
        if world == 1 and not args.no_prefill:
            line["prefill"] = prefill_layer_numbers(package, device, 8192, 20, "zipf", weights=keep[0])
        if world == 1 and not args.no_cpu_baseline:
            baseline = cpu_reference_tokens_per_second(2, 6, os.cpu_count() or 1)
            line["cpu_baseline"] = {k: baseline[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line))
    if provider is not None:
        provider.release()
    if distributed:
        dist.destroy_process_group()


DECODE_STAMPS = ["layer entered", "input normalised", "own logits written", "all logits seen", "plan published",
                 "routed gate/up chunks consumed", "activations of all blocks packed", "block agrees to go on",
                 "first down item landed", "down products done", "output words stored", "down items consumed",
                 "producer: router/shared items issued", "producer: last blind item issued",
                 "producer: post-plan gate/up items issued", "producer: down items issued"]


def decode_timeline_report(provider, buffers) -> None:
    """One traced token (outside the timed region): for every stamp the minimum / median / maximum over all
    blocks of its time after the earliest block entered the layer, medians over the middle layers; to stderr."""
    provider.set_tracing(True)
    provider.decode_stack(buffers[0], buffers[1])
    provider.sync_metrics()
    timelines = provider.decode_block_timelines()          # [block][layer][stamp], nanoseconds
    provider.set_tracing(False)
    blocks, layers = len(timelines), len(timelines[0])
    middle = range(2, layers - 1) if layers >= 4 else range(layers)
    sys.stderr.write(f"decode timeline, {blocks} blocks, layers {middle.start}..{middle.stop - 1}: "
                     "us after the earliest block enters the layer (min / median / max over blocks)\n")
    for k, name in enumerate(DECODE_STAMPS):
        low, mid, high = [], [], []
        for layer in middle:
            base = min(timelines[b][layer][0] for b in range(blocks))
            values = sorted((timelines[b][layer][k] - base) / 1000.0 for b in range(blocks) if timelines[b][layer][k] > 0)
            if values:
                low.append(values[0]); mid.append(values[len(values) // 2]); high.append(values[-1])
        if low:
            sys.stderr.write(f"  {name:42s} {statistics.median(low):7.2f} {statistics.median(mid):7.2f} "
                             f"{statistics.median(high):7.2f}\n")


def expert_parallel_parity(package, provider, synth, device, rank: int, world: int, dist) -> dict:
    """Checks, outside any timed region, that every rank ends a decode step with the same bits and that
    these are the bits a single GPU computes (rank 0 runs the first layers alone with all 256 experts)."""
    import hashlib

    import torch

    check_layers = min(2, LAYERS)
    x = synth.activations(SEED + 1, 1, "residual", 0)[0].to(device)
    y = torch.empty_like(x)
    provider.decode_stack(x, y, first_layer=0, n_layers=check_layers)
    provider.sync_metrics()
    digest = hashlib.sha256(y.cpu().view(torch.int16).numpy().tobytes()).hexdigest()
    digests = [None] * world
    dist.all_gather_object(digests, digest)
    single_equal = None
    if rank == 0:
        single = package.MoeProvider(layers=check_layers)
        try:
            keep = []
            for layer in range(check_layers):
                weights = synth.layer_weights_cuda_fast(SEED, layer, device)
                single.bind_layer(layer, weights)
                keep.append(weights)
            z = torch.empty_like(x)
            single.decode_stack(x, z, first_layer=0, n_layers=check_layers)
            single.sync_metrics()
            single_equal = bool(torch.equal(z, y))
        finally:
            single.release()
    dist.barrier()
    return {"layers_checked": check_layers, "ranks_identical": len(set(digests)) == 1,
            "equals_single_gpu": single_equal, "sha256": digest}


PREFILL_FLOP_PER_TOKEN = 50_331_648 + 6_295_552 + 1_048_576            # routed, shared, router


def measured_tensor_peak(sustained: bool = False) -> tuple[float, str]:
    """cuBLAS BF16 peak measured on this pool: the burst figure for a kernel timed for milliseconds, the
    sustained one (seconds under the power cap) for long back-to-back stacks."""
    path = ROOT / "MEASURED_PEAKS.json"
    try:
        peaks = json.loads(path.read_text())
        if sustained:
            return float(peaks["bf16_tflops_sustained"]), "measured (sustained)"
        return float(peaks["bf16_tflops"]), "measured (burst)"
    except Exception:
        return (1400.0, "fallback (sustained)") if sustained else (1590.0, "fallback (burst)")


def apply_routing(provider, synth, device, routing: str) -> None:
    """Router hooks of the benchmark regimes: uniform (none), zipf (config 2), hot (+20 on eight fixed experts,
    config 4b), ties (logits rounded to multiples of 1/8, config 4c)."""
    if routing == "zipf":
        provider.set_router_hooks(synth.zipf_router_bias(SEED).to(device), False)
    elif routing == "hot":
        provider.set_router_hooks(synth.hot_expert_bias(range(3, 256, 32)).to(device), False)
    elif routing == "ties":
        provider.set_router_hooks(None, True)


def prefill_layer_numbers(package, device, tokens: int, iterations: int, routing: str, weights=None,
                          flags: int = 0, kernel_times_wanted: bool = False) -> dict:
    """Device-timed prefill of ONE MoE layer (BASELINE config 2: T = 8192, Zipf(1.1) router bias)."""
    import torch

    synth = package.synth
    provider = package.MoeProvider(layers=1, max_prefill_tokens=tokens, flags=flags)
    try:
        if weights is None:
            weights = synth.layer_weights_cuda_fast(SEED, 0, device)
        provider.bind_layer(0, weights)
        apply_routing(provider, synth, device, routing)
        generator = torch.Generator(device=device).manual_seed(SEED)
        h2 = torch.randn(tokens, HIDDEN, generator=generator, device=device).to(torch.bfloat16)
        resid = torch.randn(tokens, HIDDEN, generator=generator, device=device).to(torch.bfloat16)
        out = torch.empty_like(resid)
        before = provider.sync_metrics().kernel_launches
        for _ in range(3):
            provider.launch_selected_moe(post_attention=h2, residual_hidden=resid, model_layer=0, out=out)
        per_call = (provider.sync_metrics().kernel_launches - before) // 3
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(iterations):
            provider.launch_selected_moe(post_attention=h2, residual_hidden=resid, model_layer=0, out=out)
        stop.record()
        torch.cuda.synchronize()
        provider.sync_metrics()
        ms = start.elapsed_time(stop) / iterations
        kernel_times = None
        if kernel_times_wanted:
            kernel_times = prefill_kernel_times(
                lambda: provider.launch_selected_moe(post_attention=h2, residual_hidden=resid, model_layer=0, out=out))
            provider.sync_metrics()
    finally:
        provider.release()
    peak, kind = measured_tensor_peak()
    tflops = tokens * PREFILL_FLOP_PER_TOKEN / (ms * 1.0e-3) / 1.0e12
    numbers = {"workload": f"prefill_T{tokens}_1layer_{routing} (BASELINE config 2)", "tokens": tokens,
               "ms_per_layer": ms, "tokens_per_s": tokens / (ms * 1.0e-3), "achieved_tflops": tflops,
               "peak_tflops": peak, "peak_source": kind, "frac": tflops / peak, "bound": "tensor",
               "flop_per_layer": tokens * PREFILL_FLOP_PER_TOKEN, "kernel_launches_per_layer": int(per_call)}
    if kernel_times is not None:
        numbers["kernel_times"] = kernel_times
    return numbers


def prefill_kernel_times(launch_layer, layers: int = 10) -> dict:
    """Device time of every kernel inside a running layer (CUPTI activity records through torch.profiler, outside
    the timed region): per kernel the calls per layer and the mean microseconds, and the start / end of every
    kernel of the last layer relative to its first kernel.  Streams run concurrently as in production, so this
    is the timeline that an ncu launch list (serialised, cold) cannot give."""
    import torch
    from torch.profiler import ProfilerActivity, profile

    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as profiler:
        for _ in range(layers):
            launch_layer()
        torch.cuda.synchronize()
    events = sorted((e for e in profiler.events() if e.device_type.name == "CUDA"), key=lambda e: e.time_range.start)
    if not events:
        return {"note": "no CUPTI activity records"}
    totals: dict[str, list[float]] = {}
    for event in events:
        entry = totals.setdefault(event.name[:72], [0, 0.0])
        entry[0] += 1
        entry[1] += event.device_time
    last = events[-(len(events) // layers):]
    origin = last[0].time_range.start
    return {"layers": layers,
            "span_us_per_layer": (events[-1].time_range.end - events[0].time_range.start) / layers,
            "kernels": {name: {"calls_per_layer": count / layers, "mean_us": total / count}
                        for name, (count, total) in totals.items()},
            "last_layer_timeline_us": [[round(e.time_range.start - origin, 1), round(e.time_range.end - origin, 1),
                                        e.name[:48]] for e in last]}


def prefill_stack_numbers(package, device, tokens: int, layers: int, iterations: int, routing: str) -> dict:
    """Device-timed prefill through `layers` MoE layers (BASELINE config 3: T x 40 layers, norm between
    layers fused into the previous layer's combine kernel), every layer with its own weights."""
    import torch

    synth = package.synth
    provider = package.MoeProvider(layers=layers, max_prefill_tokens=tokens)
    try:
        keep = []
        for layer in range(layers):
            weights = synth.layer_weights_cuda_fast(SEED, layer, device)
            provider.bind_layer(layer, weights)
            keep.append(weights)
        apply_routing(provider, synth, device, routing)
        generator = torch.Generator(device=device).manual_seed(SEED)
        x = torch.randn(tokens, HIDDEN, generator=generator, device=device).to(torch.bfloat16)
        y = torch.empty_like(x)
        before = provider.sync_metrics().kernel_launches
        for _ in range(3):
            provider.prefill_stack(x, y, 0, layers)
        per_pass = (provider.sync_metrics().kernel_launches - before) // 3
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(iterations):
            provider.prefill_stack(x, y, 0, layers)
        stop.record()
        torch.cuda.synchronize()
        provider.sync_metrics()
        ms = start.elapsed_time(stop) / iterations
    finally:
        provider.release()
    tensor_peak, kind = measured_tensor_peak(sustained=True)      # 40 layers x several passes: a long step
    hbm_peak, _ = measured_peaks()
    tflops = tokens * PREFILL_FLOP_PER_TOKEN * layers / (ms * 1.0e-3) / 1.0e12
    # algorithmic bytes per layer: every weight once + h2, residual, output rows
    layer_bytes = BYTES_PER_LAYER_WEIGHTS + tokens * HIDDEN * 2 * 3
    gbs = layer_bytes * layers / (ms * 1.0e-3) / 1.0e9
    return {"workload": f"prefill_T{tokens}_stack{layers}_{routing} (BASELINE config 3)", "tokens": tokens,
            "layers": layers, "ms_per_pass": ms, "ms_per_layer": ms / layers, "tokens_per_s": tokens / (ms * 1.0e-3),
            "achieved_tflops": tflops, "tensor_frac": tflops / tensor_peak, "achieved_gbs": gbs,
            "hbm_frac": gbs / hbm_peak, "peak_tflops": tensor_peak, "peak_gbs": hbm_peak, "peak_source": kind,
            "kernel_launches_per_pass": int(per_pass)}


def ep_prefill_numbers(package, dist, device, world: int, rank: int, tokens: int, n_layers: int, routing: str,
                       steps: int, pipeline: int = 1) -> dict | None:
    """Expert-parallel prefill of `tokens` tokens (sharded tokens / world per GPU) through `n_layers` layers:
    device-timed ms per step (maximum over ranks), rank 0's stage times of one traced layer and the
    communication that is not hidden behind the products.  Returns the numbers on rank 0, None elsewhere."""
    import torch

    synth = package.synth
    per_rank_experts = 256 // world
    tokens_local = tokens // world
    flags = {1: 0, 2: package.provider.FLAG_EP_PIPELINE_2, 4: package.provider.FLAG_EP_PIPELINE_4}[pipeline]
    provider = package.MoeProvider(layers=n_layers, max_prefill_tokens=tokens, world=world, rank=rank, flags=flags)
    try:
        keep = []
        for layer in range(n_layers):
            weights = synth.layer_weights_cuda_fast(SEED, layer, device, rank * per_rank_experts,
                                                    (rank + 1) * per_rank_experts)
            provider.bind_layer(layer, weights)
            keep.append(weights)
        provider.ep_connect_all(dist.new_group(backend="gloo"))
        apply_routing(provider, synth, device, routing)
        generator = torch.Generator(device=device).manual_seed(SEED + rank)
        h2 = torch.randn(tokens_local, HIDDEN, generator=generator, device=device).to(torch.bfloat16)
        resid = torch.randn(tokens_local, HIDDEN, generator=generator, device=device).to(torch.bfloat16)
        out = torch.empty_like(resid)

        def one_step() -> None:
            if n_layers > 1:
                provider.prefill_stack(resid, out, 0, n_layers)          # norm + MoE half per layer (config 3 / 4)
            else:
                provider.launch_selected_moe(post_attention=h2, residual_hidden=resid, model_layer=0, out=out)

        for _ in range(3):
            one_step()
        provider.sync_metrics()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            one_step()
        stop.record()
        dist.barrier()
        torch.cuda.synchronize()
        provider.sync_metrics()
        ms = start.elapsed_time(stop) / steps
        provider.set_tracing(True)
        provider.launch_selected_moe(post_attention=h2, residual_hidden=resid, model_layer=0, out=out)
        stages = provider.ep_prefill_stages()
        times = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        ms = float(times.item())
    finally:
        provider.release()
    if rank != 0:
        return None
    peak, kind = measured_tensor_peak()
    tflops = tokens * PREFILL_FLOP_PER_TOKEN * n_layers / (ms * 1.0e-3) / 1.0e12
    exposed = sum(stages.get(name, 0.0) for name in ("routing_exchange", "dispatch", "row_return"))
    return {"workload": f"prefill_T{tokens}_{n_layers}layer_{routing} (BASELINE config 3 / 4 bucket)",
            "tokens": tokens, "layers": n_layers, "routing": routing, "tokens_per_gpu": tokens_local,
            "pipeline_parts": pipeline, "ms_per_step": ms, "ms_per_layer": ms / n_layers,
            "tokens_per_s": tokens / (ms * 1.0e-3), "achieved_tflops": tflops, "peak_tflops": peak * world,
            "peak_source": kind, "frac": tflops / (peak * world),
            "stage_ms_rank0": stages, "exposed_communication_ms": exposed,
            "exposed_communication_fraction_of_layer": exposed / (ms / n_layers),
            "multi_gpu": f"expert parallel, {per_rank_experts} experts per GPU, activations all-gathered by peer "
                         "stores beside the router, weighted rows returned by peer stores from the down "
                         "kernel's epilogue (NVLink)"}


def run_prefill_expert_parallel(args, world: int, rank: int, local_rank: int) -> None:
    """One prefill layer with tokens sharded over `world` GPUs (BASELINE config 3 per bucket)."""
    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package

    package = load_package()
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", device_id=device)
    n_layers = max(args.stack_layers, 1)
    steps = max(args.steps, 1)
    numbers = ep_prefill_numbers(package, dist, device, world, rank, args.tokens, n_layers, args.routing, steps,
                                 args.ep_pipeline)
    if rank == 0:
        print(json.dumps({
            "metric": "moe_prefill_tokens_per_second", "value": numbers["tokens_per_s"], "unit": "tokens/s",
            "n_gpus": world, "steps": steps, "warmup": 3, "ms_per_step": numbers["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": numbers["workload"], "layers": n_layers, "ms_per_layer": numbers["ms_per_layer"],
                       "routing": args.routing, "tokens_per_gpu": numbers["tokens_per_gpu"],
                       "pipeline_parts": args.ep_pipeline, "multi_gpu": numbers["multi_gpu"]},
            "roofline": {"bound": "tensor", "achieved": numbers["achieved_tflops"], "peak": numbers["peak_tflops"],
                         "unit": "TFLOP/s", "frac": numbers["frac"], "traffic": None,
                         "peak_source": numbers["peak_source"]},
            "stage_ms_rank0": numbers["stage_ms_rank0"],
            "exposed_communication_ms_rank0": numbers["exposed_communication_ms"],
        }))
    dist.destroy_process_group()


def run_lm_head(args) -> None:
    """`--workload lm_head`: certified top-1 over the reference's 248 320 x 2048 vocabulary matrix, one
    token per step.  Algorithmic bytes per step: the int8 copy once (rows x 2048) + scales, residual
    norms and logits (rows x 4 B each, logits written then read twice) + the candidates' BF16 rows."""
    import time

    import torch
    from __graft_entry__ import load_package

    package = load_package()
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    rows = 248320
    generator = torch.Generator(device=device).manual_seed(SEED)
    weight = (torch.randn(rows, HIDDEN, generator=generator, device=device) * 0.02).to(torch.bfloat16)
    hiddens = [torch.randn(HIDDEN, generator=generator, device=device).to(torch.bfloat16) for _ in range(8)]
    head = package.LmHead(weight)
    logits = torch.empty(rows, dtype=torch.float32, device=device)
    steps, warmup = max(args.steps, 1), max(args.warmup, 3)
    for i in range(warmup):
        head.launch(hiddens[i % 8], logits)
    candidates = head.result().candidate_count
    sampler = ClockSampler(device.index or 0)
    sampler.start()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for i in range(steps):
        head.launch(hiddens[i % 8], logits)
    stop.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = start.elapsed_time(stop) / steps
    result = head.result()
    # end to end: hidden from pinned host memory, the 24-byte result read back every step
    pinned = [h.cpu().pin_memory() for h in hiddens]
    staging = torch.empty(HIDDEN, dtype=torch.bfloat16, device=device)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(steps):
        staging.copy_(pinned[i % 8], non_blocking=True)
        head.launch(staging, logits)
        head.result()
    e2e_ms = (time.perf_counter() - t0) * 1.0e3 / steps
    baseline = None
    if not args.no_cpu_baseline:
        # the CPU restatement (oracle/, plain C + OpenMP) on the first tenth of the rows, scaled by ten
        sys.path.insert(0, str(ROOT / "oracle"))
        import moe_oracle

        sample = rows // 10
        q_all, scales_all, residual_all = head.views()
        w_cpu = weight[:sample].cpu()
        q_cpu, s_cpu, r_cpu = q_all[:sample].contiguous(), scales_all[:sample].contiguous(), residual_all[:sample].contiguous()
        h_cpu = hiddens[0].cpu()
        moe_oracle.lm_head_certify(w_cpu, q_cpu, s_cpu, r_cpu, h_cpu)
        t0 = time.perf_counter()
        repeats = 5
        for _ in range(repeats):
            moe_oracle.lm_head_certify(w_cpu, q_cpu, s_cpu, r_cpu, h_cpu)
        seconds = (time.perf_counter() - t0) / repeats * (rows / sample)
        baseline = {"value": 1.0 / seconds, "unit": "tokens/s", "cores": os.cpu_count() or 1, "kind": "port",
                    "sample": f"{sample} of {rows} rows x {repeats} repeats, scaled to the full vocabulary"}
    head.release()
    step_bytes = rows * HIDDEN + rows * 4 * 5 + int(candidates) * HIDDEN * 2
    peak, kind = measured_peaks()
    gbs = step_bytes / (ms * 1.0e-3) / 1.0e9
    print(json.dumps({
        "metric": "lm_head_certified_top1_tokens_per_second", "value": 1.0e3 / ms, "unit": "tokens/s",
        "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8 scan + bf16 candidates", "data": "synthetic",
        "config": {"workload": "lm_head_certified_top1 (248320 x 2048, one token per step)",
                   "l2": "inputs larger than L2 (509 MB int8 matrix per step)"},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                     "traffic": None, "peak_source": kind, "bytes_per_step": step_bytes},
        "e2e": {"value": 1.0e3 / e2e_ms, "unit": "tokens/s", "h2d_bytes_per_step": HIDDEN * 2,
                "d2h_bytes_per_step": 24},
        "candidates_last_step": int(result.candidate_count), "gpu_launches": 4 * steps, "clocks": clocks,
        **({"cpu_baseline": baseline} if baseline is not None else {})}))


def run_ingest(args) -> None:
    """`--workload ingest`: one layer's expert tensors (1.5 GiB) written as a two-lane striped image, then
    loaded with aima_moe_image_scatter_ingest; a step is one full ingest.  The roofline line is the device
    checksum kernel (reads every loaded byte once); read_gbs is file -> pinned buffer -> device."""
    import tempfile

    import torch
    from __graft_entry__ import load_package

    package = load_package()
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    image = package.StripedImage()
    generator = torch.Generator().manual_seed(SEED)
    tensors = {
        "model.language_model.layers.0.mlp.experts.gate_up_proj":
            torch.randint(-2**15, 2**15 - 1, (256, 1024, 2048), generator=generator, dtype=torch.int16),
        "model.language_model.layers.0.mlp.experts.down_proj":
            torch.randint(-2**15, 2**15 - 1, (256, 2048, 512), generator=generator, dtype=torch.int16),
    }
    names = sorted(tensors)
    steps, warmup = max(min(args.steps, 20), 1), 1
    with tempfile.TemporaryDirectory(dir=os.environ.get("AIMA_IMAGE_DIR")) as folder:
        paths = (os.path.join(folder, "lane0.bin"), os.path.join(folder, "lane1.bin"))
        plan = image.build(*paths, names, tensors)
        destinations = [torch.empty_like(tensors[name], device=device) for name in names]
        ranges = [(plan["aggregate_offset"][i], plan["payload_bytes"][i]) for i in range(len(names))]
        results = []
        for _ in range(warmup + steps):
            results.append(image.scatter_ingest(*paths, ranges, destinations, plan["lane_bytes"], chunk_bytes=32 << 20,
                                                expected=(plan["xor"], plan["sum"])))
        results = results[warmup:]
    total = results[0].bytes
    read_ms = sum(r.read_ms for r in results) / len(results)
    checksum_ms = sum(r.checksum_ms for r in results) / len(results)
    peak, kind = measured_peaks()
    gbs = total / (checksum_ms * 1.0e-3) / 1.0e9
    print(json.dumps({
        "metric": "striped_image_ingest_gigabytes_per_second", "value": total / (read_ms * 1.0e-3) / 1.0e9,
        "unit": "GB/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": read_ms + checksum_ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u64", "data": "synthetic",
        "config": {"workload": "striped_image_ingest (one layer's expert tensors, 1.5 GiB, two lanes)",
                   "direct_io_lanes": int(results[0].direct_io), "chunk_bytes": 32 << 20,
                   "l2": "inputs larger than L2 (1.6 GB per step)"},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                     "traffic": None, "peak_source": kind, "kernel": "image_checksum_kernel",
                     "bytes_per_step": int(total)},
        "read_ms": read_ms, "checksum_ms": checksum_ms, "gpu_launches": steps}))


def run_prefill(args) -> None:
    """`--workload prefill`: the one-layer T = 8192 prefill line (profiling aid and second headline)."""
    import torch
    from __graft_entry__ import load_package

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        run_prefill_expert_parallel(args, world, int(os.environ.get("RANK", "0")),
                                    int(os.environ.get("LOCAL_RANK", "0")))
        return
    package = load_package()
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    sampler = ClockSampler(device.index or 0)      # covers warm-up and the timed passes of this workload
    sampler.start()
    if args.stack_layers > 1:
        numbers = prefill_stack_numbers(package, device, args.tokens, args.stack_layers, max(args.steps, 1),
                                        args.routing)
        clocks = sampler.stop()
        tensor_bound = args.tokens >= 8192
        print(json.dumps({
            "metric": "moe_prefill_tokens_per_second", "value": numbers["tokens_per_s"], "unit": "tokens/s",
            "n_gpus": 1, "steps": args.steps, "warmup": 3, "ms_per_step": numbers["ms_per_pass"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": numbers["workload"], "routing": args.routing, "layers": args.stack_layers,
                       "l2": "inputs larger than L2 (1.6 GB of weights per layer)"},
            "roofline": {"bound": "tensor" if tensor_bound else "hbm",
                         "achieved": numbers["achieved_tflops"] if tensor_bound else numbers["achieved_gbs"],
                         "peak": numbers["peak_tflops"] if tensor_bound else numbers["peak_gbs"],
                         "unit": "TFLOP/s" if tensor_bound else "GB/s",
                         "frac": numbers["tensor_frac"] if tensor_bound else numbers["hbm_frac"],
                         "traffic": None, "peak_source": numbers["peak_source"]},
            "ms_per_layer": numbers["ms_per_layer"], "tensor_frac": numbers["tensor_frac"],
            "hbm_frac": numbers["hbm_frac"],
            "gpu_launches": numbers["kernel_launches_per_pass"] * args.steps, "clocks": clocks}))
        return
    numbers = prefill_layer_numbers(package, device, args.tokens, max(args.steps, 1), args.routing, flags=args.flags,
                                    kernel_times_wanted=args.kernel_times)
    clocks = sampler.stop()
    line = {"metric": "moe_prefill_tokens_per_second", "value": numbers["tokens_per_s"], "unit": "tokens/s",
            "n_gpus": 1, "steps": args.steps, "warmup": 3, "ms_per_step": numbers["ms_per_layer"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": {"workload": numbers["workload"], "routing": args.routing},
            "roofline": {"bound": "tensor", "achieved": numbers["achieved_tflops"], "peak": numbers["peak_tflops"],
                         "unit": "TFLOP/s", "frac": numbers["frac"], "traffic": None,
                         "peak_source": numbers["peak_source"]},
            "gpu_launches": numbers["kernel_launches_per_layer"] * args.steps, "clocks": clocks}
    if "kernel_times" in numbers:
        table = numbers["kernel_times"]
        sys.stderr.write(f"kernel times inside a running layer, {table.get('layers')} layers, "
                         f"{table.get('span_us_per_layer', 0.0):.1f} us per layer\n")
        for name, entry in table.get("kernels", {}).items():
            sys.stderr.write(f"  {entry['calls_per_layer']:4.1f} x {entry['mean_us']:8.1f} us  {name}\n")
        for begin, end, name in table.get("last_layer_timeline_us", []):
            sys.stderr.write(f"  {begin:8.1f} -> {end:8.1f}  {name}\n")
        line["kernel_times"] = {name: round(entry["mean_us"], 1) for name, entry in table.get("kernels", {}).items()}
    print(json.dumps(line))


def main() -> None:
    global LAYERS, BYTES_PER_TOKEN
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=512)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-prefill", action="store_true", help="skip the one-layer prefill sub-object")
    parser.add_argument("--layers", type=int, default=LAYERS,
                        help="stack depth; anything but 40 is a profiling aid, not the benchmark config")
    parser.add_argument("--workload", choices=["decode", "prefill", "lm_head", "ingest"], default="decode",
                        help="decode = the benchmark line; prefill = one-layer prefill line only")
    parser.add_argument("--tokens", type=int, default=8192, help="prefill tokens (--workload prefill)")
    parser.add_argument("--routing", choices=["zipf", "uniform", "hot", "ties"], default="zipf")
    parser.add_argument("--ep-pipeline", type=int, choices=[1, 2, 4], default=1,
                        help="--workload prefill on N > 1 GPUs: parts of the dispatch / products / return pipeline")
    parser.add_argument("--flags", type=int, default=0,
                        help="--workload prefill, one layer: AIMA_MOE_FLAG_* bits for A/B runs (qualification)")
    parser.add_argument("--decode-timeline", action="store_true",
                        help="decode: after the timed region, trace one token and print the all-block phase times to stderr")
    parser.add_argument("--decode-hot", action="store_true",
                        help="decode profiling aid: +20 router bias on eight fixed experts (not the benchmark config)")
    parser.add_argument("--kernel-times", action="store_true",
                        help="--workload prefill, one layer: after the timed region, record every kernel's device "
                             "time inside ten running layers (CUPTI) and print the table to stderr")
    parser.add_argument("--stack-layers", type=int, default=1,
                        help="--workload prefill: run this many layers through the stack entry point (config 3: 40)")
    args = parser.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    LAYERS = args.layers
    BYTES_PER_TOKEN = LAYERS * BYTES_PER_LAYER_TOKEN
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "prefill":
        run_prefill(args)
    elif args.workload == "lm_head":
        run_lm_head(args)
    elif args.workload == "ingest":
        run_ingest(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
