"""Timings of the dense-projection configurations (decode-shaped FP8, prefill-
shaped NVFP4, the small NVFP4 linear) and of the MoE layer at decode size, on
synthetic data of the published shapes.

    python bench_configs.py [--configs c1,c2,c3,moe64] [--iters 20]

Prints one JSON object per configuration.  Weights are rotated through copies
whose total size exceeds the 126 MB L2 so that every timed pass streams its
weights from HBM.  Times are CUDA-event times on the launching stream.
"""
from __future__ import annotations

import argparse
import json

import torch

import gewell_b200 as gw

L2_BYTES = 126 * 1024 * 1024


def _time(fn, iters: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(iters):
        fn(i) if fn.__code__.co_argcount else fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / iters


def _time_graph(fn, calls: int, replays: int = 10) -> float:
    """Per-call time of `calls` consecutive calls (fn(i), i = 0..calls-1) captured
    into one CUDA graph and replayed: the launch cost on the host drops out, the
    dependencies between the kernels stay."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(calls):
            fn(i)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(calls):
            fn(i)
    for _ in range(2):
        graph.replay()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(replays):
        graph.replay()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / (replays * calls)


def _copies(nbytes: int) -> int:
    return max(2, -(-2 * L2_BYTES // nbytes))


def bench_fp8_decode(rows_list=(1, 2, 8, 32, 64), n=43008, k=5376, iters=20):
    """Config 2: joined gate+up projection, E4M3 weights with per-channel scales."""
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(2)
    copies = _copies(n * k)
    weights = []
    for _ in range(copies):
        w = (torch.randn((n, k), generator=g, device=dev) * 0.02).bfloat16()
        row_scale = (w.float().abs().amax(dim=1) / 448).contiguous()
        weights.append((gw.fp8_pack_weights(w, 0.0, row_scale), row_scale))
        del w
    out = []
    for rows in rows_list:
        x = torch.randn((rows, k), generator=g, device=dev).bfloat16()
        input_scale = float(x.float().abs().max() / 448)
        plan = gw.Fp8Plan(rows, k, n, True)
        scratch = torch.empty(plan.scratch_bytes(), dtype=torch.uint8, device=dev)
        y = torch.empty((rows, n), dtype=torch.bfloat16, device=dev)
        ws = [gw.Fp8Weight(d, input_scale, 1.0, (rs * input_scale).contiguous()) for d, rs in weights]

        def run(i=0):
            plan.run(x, ws[i % copies], y, scratch)

        eager_ms = _time(run, iters)
        ms = _time_graph(run, 2 * copies)
        algorithmic = n * k + 4 * n + rows * k * 2 + rows * n * 2
        out.append({"config": "c2_fp8_decode", "rows": rows, "K": k, "N": n, "ms": ms, "eager_ms": eager_ms,
                    "timing": "CUDA-graph replay of plan.run (quantise + GEMM); eager_ms = the same calls issued one by one",
                    "algorithmic_bytes": algorithmic, "GBps": algorithmic / ms / 1e6,
                    "TFLOPs": 2.0 * rows * n * k / ms / 1e9, "weight_copies_rotated": copies,
                    "kernel_error": gw.kernel_error()})
    return out


def bench_nvfp4_linear(rows, n, k, name, iters=20, seed=3):
    """Configs 1 and 3: NVFP4 linear through the plan (quantise + GEMM)."""
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(seed)
    wbytes = n * k // 2 + n * k // 16
    copies = _copies(wbytes)
    weights = []
    for _ in range(copies):
        w = (torch.randn((n, k), generator=g, device=dev) * 0.02).bfloat16()
        weights.append(gw.nvfp4_pack_weights(w, 1.0))
        del w
    x = torch.randn((rows, k), generator=g, device=dev).bfloat16()
    input_scale = float(x.float().abs().max() / 2688)
    for w in weights:
        w.input_scale = input_scale
    plan = gw.Nvfp4Plan(rows, k, n)
    scratch = torch.empty(plan.scratch_bytes(), dtype=torch.uint8, device=dev)
    y = torch.empty((rows, n), dtype=torch.bfloat16, device=dev)

    def run(i=0):
        plan.run(x, weights[i % copies], y, scratch)

    def quantise_only(i=0):
        gw.lib.gw_nvfp4_quantize_activations(x.data_ptr(), rows, k, input_scale, 0, scratch.data_ptr(),
                                             scratch.data_ptr() + (rows * k // 2 + 255) // 256 * 256,
                                             torch.cuda.current_stream().cuda_stream)

    ms = _time(run, iters)
    qms = _time(quantise_only, iters)
    if rows <= 128:     # decode-shaped: launch cost on the host would dominate an eager loop
        ms = _time_graph(run, 2 * copies)
        qms = _time_graph(quantise_only, 2 * copies)
    algorithmic = wbytes + rows * k * 2 + rows * n * 2
    flops = 2.0 * rows * n * k
    return {"config": name, "rows": rows, "K": k, "N": n, "ms": ms, "quantise_ms": qms, "gemm_ms": ms - qms,
            "algorithmic_bytes": algorithmic, "GBps": algorithmic / ms / 1e6, "TFLOPs": flops / ms / 1e9,
            "gemm_TFLOPs": flops / max(ms - qms, 1e-6) / 1e9, "weight_copies_rotated": copies,
            "kernel_error": gw.kernel_error()}


def bench_moe(tokens, experts=None, iters=20):
    """Config 4 at decode size: bytes = NVFP4 weights of the experts that were
    touched plus activations in and out."""
    import bench as root_bench
    dev = torch.device("cuda")
    experts = experts or root_bench.build_experts(gw, torch, dev)
    table = gw.ExpertTable(experts)
    ws = gw.MoeWorkspace(max(tokens, 64))
    g = torch.Generator(device=dev).manual_seed(1)
    x = torch.randn((tokens, 2816), generator=g, device=dev).bfloat16()
    scores = torch.randn((tokens, 128), generator=g, device=dev).bfloat16()
    ones = torch.ones(128, dtype=torch.bfloat16, device=dev)
    y = torch.empty((tokens, 2816), dtype=torch.bfloat16, device=dev)
    flush = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=dev)

    def run():
        ws.run(x, scores, ones, table, y, tokens)

    run()
    torch.cuda.synchronize()
    touched = int((torch.bincount(ws.selected_experts().reshape(-1).long(), minlength=128) > 0).sum())
    # L2 flush between timed passes: 450 MB of experts do not fit anyway, the flush
    # makes the small-batch case honest
    times = []
    for _ in range(iters):
        flush.zero_()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        run()
        stop.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(stop))
    ms = sorted(times)[len(times) // 2]
    per_expert = 3 * (704 * 2816 // 2 + 704 * 176)
    algorithmic = touched * per_expert + tokens * 2816 * 2 * 2 + tokens * 128 * 2
    ws.stage_timing(True)
    run()
    stages = ws.stage_elapsed_ms()
    ws.stage_timing(False)
    return {"config": f"c4_moe_T{tokens}", "tokens": tokens, "ms": ms, "experts_touched": touched,
            "algorithmic_bytes": algorithmic, "GBps": algorithmic / ms / 1e6,
            "TFLOPs": tokens * 8 * 11894784 / ms / 1e9, "stage_ms": stages, "kernel_error": gw.kernel_error()}


def main():
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--configs", default="c1,c2,c3,moe64")
    parser.add_argument("--iters", type=int, default=20)
    args = parser.parse_args()
    wanted = args.configs.split(",")
    if "c1" in wanted:
        print(json.dumps(bench_nvfp4_linear(16, 2816, 2816, "c1_nvfp4_linear", args.iters, seed=0)), flush=True)
    if "c2" in wanted:
        for row in bench_fp8_decode(iters=args.iters):
            print(json.dumps(row), flush=True)
    if "c3" in wanted:
        print(json.dumps(bench_nvfp4_linear(4096, 5376, 21504, "c3_nvfp4_prefill", args.iters)), flush=True)
    if "c3small" in wanted:   # profiling-sized slice of config 3 (same N and K, 1024 rows)
        print(json.dumps(bench_nvfp4_linear(1024, 5376, 21504, "c3_nvfp4_prefill_rows1024", args.iters)), flush=True)
    if "c2m64" in wanted:
        for row in bench_fp8_decode(rows_list=(64,), iters=args.iters):
            print(json.dumps(row), flush=True)
    if "moe2048" in wanted:
        print(json.dumps(bench_moe(2048, iters=args.iters)), flush=True)
    if "moe64" in wanted:
        print(json.dumps(bench_moe(64, iters=args.iters)), flush=True)
    if "moe8192" in wanted:
        print(json.dumps(bench_moe(8192, iters=args.iters)), flush=True)


if __name__ == "__main__":
    main()
