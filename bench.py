#!/usr/bin/env python3
"""Benchmark of the NVFP4 MoE layer (Gemma-4-26B-A4B shape: 128 experts, top-8,
hidden 2816, expert MLP 704) on synthetic data.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference          # CPU host path, same metric

One "step" is one pass of the whole layer (routing, permutation,
gather+quantise, grouped gate/up GEMM, GeGLU+quantise, grouped down GEMM,
ordered combine) over one batch of tokens.  N=1 runs T=8192 tokens on one
GPU; N>1 runs the expert-parallel layer over T=32768 tokens (T/N routed per
rank, experts sharded, all-to-all dispatch and combine over NCCL).
Prints ONE JSON line on rank 0.
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

E, TOPK, H, I = 128, 8, 2816, 704
FLOPS_PER_ASSIGNMENT = 2 * H * 2 * I + 2 * I * H          # 11,894,784
METRIC = "nvfp4_moe_layer_tflops"


def measured_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()) | {"source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed
    region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.lines, self.proc = [], None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={device_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, smax, reasons = [], [], set()
        chosen = [l for (t, l) in self.lines if t0 <= t <= t1 + 0.2] or [l for (_, l) in self.lines]
        for line in chosen:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def zipf_bias(alpha: float = 1.2):
    import torch
    ranks = torch.arange(1, E + 1, dtype=torch.float32)
    p = ranks.pow(-alpha)
    return (p / p.sum()).log()


def gate_up_input_scale(e: int, per_expert: bool) -> float:
    """Input scale of expert e's gate and up projections: one value for the layer (as a checkpoint
    calibrated with a layer-wide activation scale has it), or sixteen values over the experts."""
    return 6.0 / 2688 * (1.0 + (e % 16) / 64.0) if per_expert else 6.0 / 2688


def build_experts(gw, torch, device, seed=4, expert_ids=None, per_expert_scales=False):
    """The layer's experts ~ N(0, 0.02), packed to NVFP4 by the device packer;
    gate and up share one input scale per expert (they are one fused tensor in
    the checkpoint), so the layer quantises its input once per distinct scale
    among a token's experts.  Every expert has
    its own sub-seed, so a rank that owns only some experts (`expert_ids`)
    builds exactly the tensors the single-GPU run builds; the other entries
    of the returned 128-list are None."""
    experts = [None] * E
    for e in (range(E) if expert_ids is None else expert_ids):
        g = torch.Generator(device=device).manual_seed(seed * 1000003 + e)
        mats = [(torch.randn((I, H), generator=g, device=device) * 0.02).bfloat16(),
                (torch.randn((I, H), generator=g, device=device) * 0.02).bfloat16(),
                (torch.randn((H, I), generator=g, device=device) * 0.02).bfloat16()]
        scales = [gate_up_input_scale(e, per_expert_scales)] * 2 + [16.0 / 2688]
        packs = []
        for m, s in zip(mats, scales):
            w = gw.nvfp4_pack_weights(m, s)
            physical = (m.shape[0] + 127) // 128 * 128
            if physical != m.shape[0]:
                data = torch.zeros((physical, m.shape[1] // 2), dtype=torch.uint8, device=device)
                data[:m.shape[0]] = w.data
                w = gw.Nvfp4Weight(data, w.scales, w.input_scale, w.weight_scale)
            packs.append(w)
        experts[e] = tuple(packs)
    return experts


def cpu_host_path(tokens: int, steps: int, warmup: int = 0, seed: int = 11) -> dict:
    """The reference's host path for this layer on this box's host cores: dequantise the NVFP4
    expert weights (src/nvfp4_linear.cu:47-55), then per step route, FP32 matmul per expert with
    BF16 roundings, GeGLU and the ordered BF16 combine over `tokens` tokens.  The reference has no
    CPU build of this layer, so this is the CPU restatement of its arithmetic (oracle/), run with
    every host thread NumPy's BLAS takes.  The dequantised weights are kept between steps, as a CPU
    deployment would; the one-off dequantisation is timed and reported beside the per-step rate.
    Needs no GPU and does not load the CUDA library."""
    import numpy as np
    from oracle import codecs as C
    from oracle import moe as omoe
    experts = omoe.synthetic_packed_experts(seed=4)
    start = time.perf_counter()
    dense = omoe.dequantize_experts(experts)
    dequantise_s = time.perf_counter() - start
    del experts
    rng = np.random.default_rng(seed)
    ones = np.ones(E, dtype=np.float32)
    seconds = []
    for step in range(warmup + steps):
        x = C.bf16_round(rng.standard_normal((tokens, H)).astype(np.float32))
        scores = C.bf16_round(rng.standard_normal((tokens, E)).astype(np.float32))
        start = time.perf_counter()
        omoe.forward_dequantized(x, scores, ones, dense)
        if step >= warmup:
            seconds.append(time.perf_counter() - start)
    per_step = statistics.mean(seconds)
    flops = tokens * TOPK * FLOPS_PER_ASSIGNMENT
    return {"value": flops / per_step / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
            "seconds_per_step": per_step, "dequantise_seconds": dequantise_s,
            "with_dequantise_every_step": flops / (per_step + dequantise_s) / 1e12,
            "sample": (f"{tokens} tokens per step x {steps} steps of the same layer (route, FP32 matmul per expert on "
                       f"dequantised weights, GeGLU, ordered combine; NumPy/BLAS): {per_step:.2f} s per step; the "
                       f"one-off dequantisation of the 384 expert matrices took {dequantise_s:.1f} s and is not in "
                       f"`value` (`with_dequantise_every_step` includes it)")}


def run_reference_arm(args):
    """CPU arm: the host path of the reference for this layer, all host threads, no GPU."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    tokens = 1024
    result = cpu_host_path(tokens, args.steps, min(args.warmup, 1), seed=100)
    value = result["value"]
    config = workload_config(args.gpus) | {"sample_tokens_per_step": tokens}
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": result["seconds_per_step"] * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config, "gpu_launches": 0, "cpu_baseline": result,
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


INPUT_SCALE_NOTE = {
    "layer": "one gate/up input scale for the layer: a token's eight routed copies are quantised once and written eight times",
    "expert": "sixteen gate/up input scales over the experts: a token's copies are quantised per distinct scale among its experts",
}


def workload_config(n_gpus: int) -> dict:
    tokens = 8192 if n_gpus == 1 else 32768
    return {"workload": ("config 4: Gemma-4-26B-A4B MoE layer on one GPU" if n_gpus == 1 else
                         "config 5: the same layer expert-parallel, Zipf(1.2) routing bias"),
            "tokens": tokens, "experts": E, "top_k": TOPK, "hidden": H, "expert_intermediate": I,
            "weights": "NVFP4 W4A4 (E2M1 + E4M3 K16 scales + FP32 global)",
            "l2": "inputs larger than L2: 450 MB of expert weights and >400 MB of intermediates are streamed every step",
            "parallelism": "single GPU" if n_gpus == 1 else f"ep{n_gpus}"}


def one_gpu_layer_ms(gw, torch, table, expert_scales, tokens: int, zipf: bool, steps: int, warmup: int, seed: int):
    """Device-timed ms per pass of the whole layer on one GPU (inputs resident)."""
    device = expert_scales.device
    ws = gw.MoeWorkspace(tokens)
    g = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn((tokens, H), generator=g, device=device).bfloat16()
    logits = torch.randn((tokens, E), generator=g, device=device)
    if zipf:
        logits = logits + zipf_bias().to(device)
    scores = logits.bfloat16()
    y = torch.empty((tokens, H), dtype=torch.bfloat16, device=device)
    stream = torch.cuda.current_stream()
    for _ in range(warmup):
        ws.run(x, scores, expert_scales, table, y, tokens)
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    begin.record(stream)
    for _ in range(steps):
        ws.run(x, scores, expert_scales, table, y, tokens)
    end.record(stream)
    torch.cuda.synchronize()
    return begin.elapsed_time(end) / steps


def run_expert_parallel(args, world: int, rank: int, local_rank: int):
    """N > 1: config 5, the layer sharded by expert over the ranks (T = 32768
    tokens in total, T / N routed per rank, Zipf(1.2)-biased router logits)."""
    import torch
    import torch.distributed as dist
    import gewell_b200 as gw
    from gewell_b200 import expert_parallel as ep

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=device)
    config = workload_config(world)
    tokens = args.tokens or config["tokens"]
    config["tokens"] = tokens
    local_tokens = tokens // world
    g = torch.Generator(device=device).manual_seed(1000 + rank)
    if args.placement == "balanced":
        # load-aware placement from the routing histogram of a calibration batch
        # (same distribution, other seed), as a serving system keeps from earlier steps
        calibration = (torch.randn((local_tokens, E), generator=g, device=device) + zipf_bias().to(device)).bfloat16()
        chosen = calibration.float().topk(TOPK, dim=1).indices.reshape(-1)
        histogram = torch.bincount(chosen, minlength=E).float()
        dist.all_reduce(histogram)
        placement = ep.Placement.balanced(world, histogram.tolist())
    else:
        placement = getattr(ep.Placement, args.placement)(world)
    config["placement"] = args.placement
    mine = placement.local_experts(rank)
    # "home": every rank also holds the down matrices of all experts (it finishes its own tokens' rows itself)
    per_expert = args.input_scales == "expert"
    config["input_scales"] = INPUT_SCALE_NOTE[args.input_scales]
    by_id = build_experts(gw, torch, device, expert_ids=None if args.exchange == "home" else mine,
                          per_expert_scales=per_expert)
    by_position = [None] * E
    for e in mine:
        by_position[placement.physical[e]] = by_id[e]
    capacity = TOPK * tokens          # worst case: every assignment lands on one rank
    config["exchange"] = args.exchange
    if args.exchange == "home":
        config["parallelism"] = f"ep{world} for gate/up (experts sharded), down projection at the tokens' home rank (down matrices of all experts on every rank)"
    if args.exchange in ("peer", "peer_pull", "home"):
        layer = ep.PeerMemoryExpertParallelMoe(by_position, [gate_up_input_scale(e, per_expert) for e in range(E)],
                                               rank, world, local_tokens, capacity,
                                               placement=placement, send_home=args.exchange == "peer",
                                               exchange=args.sync,
                                               home_down=[w[2] for w in by_id] if args.exchange == "home" else None)
        config["sync"] = layer.exchange
        expert_ws = layer.expert_ws
    else:
        backend = ep.DeviceBackend(by_position, local_tokens, capacity)
        layer = ep.ExpertParallelMoe(backend, rank, world, local_tokens, capacity, placement=placement)
        expert_ws = backend.expert_ws
    x = torch.randn((local_tokens, H), generator=g, device=device).bfloat16()
    logits = torch.randn((local_tokens, E), generator=g, device=device) + zipf_bias().to(device)
    scores = logits.bfloat16()
    expert_scales = torch.ones(E, dtype=torch.bfloat16, device=device)
    y = torch.empty((local_tokens, H), dtype=torch.bfloat16, device=device)
    stream = torch.cuda.current_stream()

    def eager_step():
        layer.run(x, scores, expert_scales, local_tokens, out=y)

    step = eager_step

    def timed(fn, steps):
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        torch.cuda.synchronize()
        begin.record(stream)
        for _ in range(steps):
            fn()
        end.record(stream)
        torch.cuda.synchronize()
        dist.barrier()
        ms = torch.tensor([begin.elapsed_time(end) / steps], device=device)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if gw.kernel_error() != 0:
        raise SystemExit("tensor-core kernel reported an error during warm-up")
    # The step reads nothing back and keeps its mailbox epochs on the device, so it can be captured once
    # and replayed: the gaps between its dependent launches weigh more the less work a rank has.  Every rank
    # decides together (a rank that replays and a rank that launches eagerly would still meet at the barriers).
    config["launch"] = "eager"
    if args.graph and args.exchange in ("home", "peer", "peer_pull") and args.sync == "peer":
        captured = None
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                eager_step()
            captured = graph
        except Exception as error:          # noqa: BLE001  (capture is an optimisation; eager launches remain)
            print(f"rank {rank}: step not captured ({error}); launching eagerly", file=sys.stderr)
        ok = torch.tensor([1 if captured is not None else 0], device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) == 1:
            step = captured.replay
            config["launch"] = "CUDA graph replay of one step"
            for _ in range(2):
                step()
            torch.cuda.synchronize()
            if gw.kernel_error() != 0:
                raise SystemExit("tensor-core kernel reported an error during graph replay")
    sampler = ClockSampler(local_rank) if rank == 0 else None
    time.sleep(0.25)
    t0 = time.time()
    launches_before = gw.launch_count()
    ms = timed(step, args.steps)
    launches = gw.launch_count() - launches_before          # this rank's kernels inside the timed region
    if launches == 0 and config["launch"] != "eager":       # replayed: the library's launch sites ran at capture time
        before = gw.launch_count()
        eager_step()
        torch.cuda.synchronize()
        launches = (gw.launch_count() - before) * args.steps
    flops = tokens * TOPK * FLOPS_PER_ASSIGNMENT
    value = flops / (ms * 1e-3) / 1e12

    # end to end with HOST buffers: every step uploads its pinned inputs and downloads its output inside the
    # timed region; gw.HostStagedMoe overlaps the copies of neighbouring steps with the kernels
    hx, hs = x.cpu().pin_memory(), scores.cpu().pin_memory()
    hy = [torch.empty((local_tokens, H), dtype=torch.bfloat16).pin_memory() for _ in range(3)]

    def layer_pass(dx, ds, dy, rows, _stream):
        layer.run(dx, ds, expert_scales, rows, out=dy)

    runner = gw.HostStagedMoe(None, None, expert_scales, local_tokens, H, experts=E, depth=3, run=layer_pass,
                              capture=config["launch"] != "eager")
    for i in range(3):
        runner.submit(hx, hs, hy[i % 3], local_tokens)
    runner.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier()
    torch.cuda.synchronize()
    begin.record(runner.upload)
    for i in range(args.steps):
        runner.submit(hx, hs, hy[i % 3], local_tokens)
    end.record(runner.download)
    runner.synchronize()
    torch.cuda.synchronize()
    dist.barrier()
    e2e_t = torch.tensor([begin.elapsed_time(end) / args.steps], device=device)
    dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
    e2e_ms = float(e2e_t.item())
    if gw.kernel_error() != 0:
        raise SystemExit("tensor-core kernel reported an error during the host-buffer run")
    if not torch.equal(hy[(args.steps - 1) % 3], y.cpu()):
        raise SystemExit("host-buffer run and device-buffer run disagree")
    clocks = sampler.stop(t0, time.time()) if sampler else None

    # per-stage device times of this rank and the grouped GEMMs' roofline
    marks = []
    layer.timer = lambda name: marks.append((name, _record(torch, stream)))
    # the grouped GEMMs run in the owner-side workspace; with --exchange home the down GEMM runs in the routing one
    timed_workspaces = [expert_ws] + ([layer.route_ws] if args.exchange == "home" else [])
    for workspace in timed_workspaces:
        workspace.stage_timing(True)
    stage_sum, gemm_sum = {}, 0.0
    for _ in range(max(3, args.steps // 4)):
        marks.clear()
        first = _record(torch, stream)
        eager_step()           # (stage events are recorded by eager launches, not by a replayed graph)
        torch.cuda.synchronize()
        previous = first
        for name, event in marks:
            stage_sum[name] = stage_sum.get(name, 0.0) + previous.elapsed_time(event)
            previous = event
        inner = expert_ws.stage_elapsed_ms()
        gemm_sum += inner["gate_up_gemm"] + (0.0 if args.exchange == "home" else inner["down_gemm"])
        if args.exchange == "home":
            gemm_sum += layer.route_ws.stage_elapsed_ms()["down_gemm"]
    repeats = max(3, args.steps // 4)
    layer.timer = None
    for workspace in timed_workspaces:
        workspace.stage_timing(False)
    stages = {k: v / repeats for k, v in stage_sum.items()}
    rows_received = layer.rows_received() if args.exchange != "nccl" else layer.last_layout.total
    received = torch.tensor([float(rows_received), gemm_sum / repeats], device=device)
    gathered = [torch.zeros_like(received) for _ in range(world)]
    dist.all_gather(gathered, received)
    rows_per_rank = [int(t[0].item()) for t in gathered]
    gemm_ms_per_rank = [float(t[1].item()) for t in gathered]
    if rank == 0:
        peaks = measured_peaks()
        fp4_peak = 4.0 * peaks["bf16_tflops"]
        slowest = max(range(world), key=lambda r: gemm_ms_per_rank[r])
        achieved = rows_per_rank[slowest] * FLOPS_PER_ASSIGNMENT / (gemm_ms_per_rank[slowest] * 1e-3) / 1e12
        line = {"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "nvfp4 (e2m1 x e2m1, fp32 accumulate)", "data": "synthetic",
                "config": config,
                "e2e": {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                        "h2d_bytes_per_step": world * (hx.numel() + hs.numel()) * 2,
                        "d2h_bytes_per_step": world * hy[0].numel() * 2, "ms_per_step": e2e_ms,
                        "note": "uploads, kernels and downloads of consecutive steps overlap (gewell_b200.HostStagedMoe); "
                                "the layer pass of each ring slot is " + ("a CUDA graph replay" if config["launch"] != "eager" else "launched eagerly")},
                # counted by the library at its launch sites on rank 0 (every rank launches the same
                # sequence; the collectives are NCCL's and not counted)
                "gpu_launches": launches * world, "clocks": clocks,
                "roofline": {"kernel": "pair_moe_gate_up_kernel + pair_moe_down_kernel (grouped NVFP4 GEMMs on CTA pairs) on the busiest rank",
                             "bound": "tensor", "achieved": achieved, "peak": fp4_peak, "unit": "TFLOP/s",
                             "frac": achieved / fp4_peak, "traffic": None,
                             "peak_note": f"4 x the {peaks['source']} dense BF16 burst figure per GPU",
                             "rows_received_per_rank": rows_per_rank, "gemm_ms_per_rank": gemm_ms_per_rank,
                             "stage_ms_rank0": stages},
                "cpu_baseline": None}
        print(json.dumps(line))
    if args.exchange != "nccl":
        layer.close()
    dist.destroy_process_group()


def _record(torch, stream):
    event = torch.cuda.Event(enable_timing=True)
    event.record(stream)
    return event


def main():
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--tokens", type=int, default=0, help="override the token count (testing)")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--exchange", default="home", choices=["home", "peer", "peer_pull", "nccl"],
                        help="expert-parallel run: rows cross NVLink inside the dispatch/combine kernels over peer "
                             "memory (home: the owners run gate/up only and every rank fetches its rows' quantised "
                             "activations and runs the down projection itself, with the down matrices of all experts "
                             "on every rank; peer_pull: the combine kernel pulls BF16 result rows; peer: the down "
                             "GEMM's epilogue stores them into the source rank) or through NCCL all-to-all")
    parser.add_argument("--graph", type=int, default=1,
                        help="expert-parallel run over peer memory: capture one step in a CUDA graph and replay it (1), "
                             "or launch every step eagerly (0)")
    parser.add_argument("--sync", default="peer", choices=["peer", "nccl"],
                        help="expert-parallel run over peer memory: the histogram exchange and the two barriers of a "
                             "step through mailboxes in peer memory, or through NCCL (all-gather + two all-reduces)")
    parser.add_argument("--input-scales", default="layer", choices=["layer", "expert"],
                        help="gate/up input scales of the synthetic experts: one for the layer, or sixteen values over "
                             "the experts (the quantiser then repeats its work for a token's experts that differ)")
    parser.add_argument("--placement", default="balanced", choices=["contiguous", "interleaved", "balanced"],
                        help="expert placement of the expert-parallel run")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return run_reference_arm(args)

    import torch
    import gewell_b200 as gw

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        return run_expert_parallel(args, world, rank, local_rank)

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    config = workload_config(1)
    tokens = args.tokens or config["tokens"]
    config["tokens"] = tokens
    config["input_scales"] = INPUT_SCALE_NOTE[args.input_scales]
    experts = build_experts(gw, torch, device, per_expert_scales=args.input_scales == "expert")
    table = gw.ExpertTable(experts)
    ws = gw.MoeWorkspace(tokens)
    g = torch.Generator(device=device).manual_seed(1)
    x = torch.randn((tokens, H), generator=g, device=device).bfloat16()
    scores = torch.randn((tokens, E), generator=g, device=device).bfloat16()
    expert_scales = torch.ones(E, dtype=torch.bfloat16, device=device)
    y = torch.empty((tokens, H), dtype=torch.bfloat16, device=device)
    stream = torch.cuda.current_stream()

    def step():
        ws.run(x, scores, expert_scales, table, y, tokens)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if gw.kernel_error() != 0:
        raise SystemExit("tensor-core kernel reported an error during warm-up")

    sampler = ClockSampler(local_rank)
    time.sleep(0.25)
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    t0 = time.time()
    launches_before = gw.launch_count()
    begin.record(stream)
    for _ in range(args.steps):
        step()
    end.record(stream)
    torch.cuda.synchronize()
    launches = gw.launch_count() - launches_before          # counted by the library at its launch sites
    t1 = time.time()
    ms = begin.elapsed_time(end) / args.steps
    flops = tokens * TOPK * FLOPS_PER_ASSIGNMENT
    value = flops / (ms * 1e-3) / 1e12

    # End to end through the C ABI's host-buffer entry point (gw_moe_host_runner_*, wrapped by
    # gw.HostStagedMoe): every step uploads its pinned inputs and downloads the layer output inside the
    # timed region; the runner overlaps step i+1's upload and step i-1's download with step i's kernels
    # (three streams, ring of 3 device buffers).
    hx = x.cpu().pin_memory()
    hs = scores.cpu().pin_memory()
    hy = [torch.empty((tokens, H), dtype=torch.bfloat16).pin_memory() for _ in range(3)]
    runner = gw.HostStagedMoe(ws, table, expert_scales, tokens, H, experts=E, depth=3)
    torch.cuda.synchronize()

    for i in range(3):
        runner.submit(hx, hs, hy[i % 3], tokens)
    runner.synchronize()
    before_h2d, before_d2h = runner.h2d_bytes, runner.d2h_bytes
    begin.record(runner.upload)
    for i in range(args.steps):
        runner.submit(hx, hs, hy[i % 3], tokens)
    end.record(runner.download)
    runner.synchronize()
    torch.cuda.synchronize()
    if gw.kernel_error() != 0:
        raise SystemExit("tensor-core kernel reported an error during the host-buffer run")
    if not torch.equal(hy[(args.steps - 1) % 3], y.cpu()):
        raise SystemExit("host-buffer run and device-buffer run disagree")
    e2e_ms = begin.elapsed_time(end) / args.steps
    # the same call one pass at a time (submit, wait): the latency a caller sees without pipelining
    single = gw.HostStagedMoe(ws, table, expert_scales, tokens, H, experts=E, depth=1)
    single.submit(hx, hs, hy[0], tokens)
    single.synchronize()
    latencies = []
    for _ in range(min(args.steps, 10)):
        start = time.perf_counter()
        single.wait_for(single.submit(hx, hs, hy[0], tokens))
        latencies.append((time.perf_counter() - start) * 1e3)
    t2 = time.time()
    clocks = sampler.stop(t0, t2)
    e2e = {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
           "h2d_bytes_per_step": (runner.h2d_bytes - before_h2d) // args.steps,
           "d2h_bytes_per_step": (runner.d2h_bytes - before_d2h) // args.steps,
           "ms_per_step": e2e_ms, "single_pass_ms": statistics.median(latencies),
           "note": "C-ABI host-buffer runner (gw_moe_host_runner_submit): uploads, kernels and downloads of "
                   "consecutive steps overlap; single_pass_ms is one submit + wait at a time (host clock)"}
    del runner, single

    # roofline of the dominant kernel (the two grouped tcgen05 GEMMs), timed live
    # with CUDA events recorded on the launching stream between the stages
    ws.stage_timing(True)
    stage_sum = {}
    for _ in range(args.steps):
        step()
        for name, v in ws.stage_elapsed_ms().items():
            stage_sum[name] = stage_sum.get(name, 0.0) + v
    ws.stage_timing(False)
    stages = {k: v / args.steps for k, v in stage_sum.items()}
    gemm_ms = stages["gate_up_gemm"] + stages["down_gemm"]
    peaks = measured_peaks()
    fp4_peak = 4.0 * peaks["bf16_tflops"]
    achieved = flops / (gemm_ms * 1e-3) / 1e12
    roofline = {"kernel": "pair_moe_gate_up_kernel + pair_moe_down_kernel (grouped NVFP4 GEMMs on CTA pairs)", "bound": "tensor",
                "achieved": achieved, "peak": fp4_peak, "unit": "TFLOP/s", "frac": achieved / fp4_peak,
                # dram__bytes_read.sum + dram__bytes_write.sum of the two launches at this size, from the one-pass
                # ncu capture summarised in profiles/bench_moe_T8192_launch_list.md (gate/up 442.6 MB, down 483.5 MB)
                "traffic": 926.1e6 if tokens == 8192 else None, "traffic_unit": "bytes per layer pass (both launches)",
                # weights and their scales of the 128 experts once, quantised rows in and out, BF16 rows out
                "algorithmic_bytes": float(128 * (1408 * (1408 + 176) + 2816 * (352 + 44))
                                           + tokens * TOPK * ((1408 + 176) + 2 * (352 + 44) + 5632)),
                "peak_note": f"4 x the {peaks['source']} dense BF16 burst figure ({peaks['bf16_tflops']} TFLOP/s); "
                             "no FP4 GEMM peak was measured on this pool (nominal dense FP4: 9000 TFLOP/s)",
                "frac_of_nominal_fp4": achieved / 9000.0,
                "ms_per_launch": {"gate_up": stages["gate_up_gemm"], "down": stages["down_gemm"]},
                "stage_ms": stages}

    # the same layer at the expert-parallel configuration's size on this one GPU: the like-for-like
    # denominator of the multi-GPU lines (T = 32768, Zipf(1.2) routing bias)
    same_as_ep = None
    if not args.tokens:
        del ws
        ep_tokens = workload_config(2)["tokens"]
        ep_ms = one_gpu_layer_ms(gw, torch, table, expert_scales, ep_tokens, True, max(3, args.steps // 4), 3, seed=1000)
        same_as_ep = {"workload": "config 5 on one GPU (T = 32768, Zipf(1.2) bias), all 128 experts local",
                      "tokens": ep_tokens, "ms_per_step": ep_ms,
                      "value": ep_tokens * TOPK * FLOPS_PER_ASSIGNMENT / (ep_ms * 1e-3) / 1e12, "unit": "TFLOP/s"}
        if gw.kernel_error() != 0:
            raise SystemExit("tensor-core kernel reported an error during the config-5 run")

    cpu = None
    if not args.no_cpu_baseline:
        cpu = cpu_host_path(256, 1)

    line = {"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "nvfp4 (e2m1 x e2m1, fp32 accumulate)", "data": "synthetic",
            "config": config, "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
            "roofline": roofline, "cpu_baseline": cpu, "config5_on_one_gpu": same_as_ep,
            "scaling_note": "this line is config 4 (T = 8192, uniform routing); the lines at 2, 4 and 8 GPUs are config 5 "
                            "(T = 32768, Zipf(1.2) routing, total work fixed): their like-for-like one-GPU figure is "
                            "config5_on_one_gpu"}
    print(json.dumps(line))


if __name__ == "__main__":
    main()
