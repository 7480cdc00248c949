"""MLA absorbed-decode timing on B200: microseconds per call and KV bytes streamed per second.

The operator is HBM-bound: every cached token row (576 bytes of fp8) is read once per decode step, whatever the
number of heads (<= 16) or draft positions; the algorithmic traffic of a call is batch x seq_len x 576 bytes (the
queries, outputs and split partials are a few hundred KB).  Reported: median microseconds per call over `--passes`
passes of `--iters` calls between two CUDA events, and that traffic divided by the time, next to the measured copy
bandwidth of the GPU when MEASURED_PEAKS.json is found beside the repository root.

    python amd-kernels_b200/bench_mla.py [--paged [--sequential]] [--format fnuz|fn] [--graph] [--json out.json]
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
if HERE not in sys.path:
    sys.path.insert(0, HERE)

# (batch, seq_len, q_len): decode batches of a serving engine, one long request, a speculative window
CASES = [(148, 4096, 1), (64, 8192, 1), (32, 8192, 1), (16, 32768, 1), (4, 131072, 1), (1, 131072, 1),
         (32, 8192, 4), (16, 8192, 8)]
H, LAT, ROPE, FUSED = 16, 512, 64, 576


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--paged", action="store_true", help="scatter the rows over a pool (one token per slot)")
    ap.add_argument("--sequential", action="store_true", help="with --paged: slots in token order instead of a random permutation")
    ap.add_argument("--format", default="fnuz", choices=("fnuz", "fn"))
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--passes", type=int, default=5)
    ap.add_argument("--graph", action="store_true", help="capture the call in a CUDA graph and time replays")
    ap.add_argument("--json", default="")
    args = ap.parse_args()

    import moonmath_attention as ma

    dev = torch.device("cuda:0")
    dtype = torch.float8_e4m3fnuz if args.format == "fnuz" else torch.float8_e4m3fn
    peak = None
    peaks_file = os.path.join(os.path.dirname(HERE), "MEASURED_PEAKS.json")
    if os.path.exists(peaks_file):
        peak = json.load(open(peaks_file)).get("hbm_gbs")
    results = []
    for B, S, q_len in CASES:
        g = torch.Generator(device=dev)
        g.manual_seed(42)
        kv = torch.randn(B, S, FUSED, generator=g, device=dev).to(dtype)
        shape = (B, H) if q_len == 1 else (B, q_len, H)
        q_lat = (torch.randn(*shape, LAT, generator=g, device=dev) * 3).bfloat16()
        q_pe = (torch.randn(*shape, ROPE, generator=g, device=dev) * 3).bfloat16()
        o_lat = torch.zeros_like(q_lat)
        scale, kv_scale = FUSED ** -0.5, 1.0 / 32.0
        if args.paged:
            slots = (torch.arange(B * S, device=dev) if args.sequential else torch.randperm(B * S, generator=g, device=dev)).to(torch.int32)
            pool = torch.empty(B * S, 1, FUSED, dtype=torch.uint8, device=dev)
            pool[slots.long(), 0] = kv.view(torch.uint8).view(B * S, FUSED)
            pool = pool.view(dtype)
            lens = torch.full((B,), S, dtype=torch.int32, device=dev)
            indptr = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device=dev)
            parts = ma.mla_decode_a16w8_plan_parts_q(B, S, q_len, H)
            call = lambda: ma.mla_decode_a16w8_paged_dev(q_lat, q_pe, pool, o_lat, lens, None, slots, indptr, parts, scale, kv_scale)
        elif q_len == 1:
            call = lambda: ma.mla_decode_a16w8(q_lat, q_pe, kv, o_lat, scale, kv_scale)
        elif q_len >= 4 and B <= 32:
            call = lambda: ma.mla_decode_a16w8_multiq(q_lat, q_pe, kv, o_lat, scale, kv_scale)
        else:
            continue
        for _ in range(3):
            call()
        torch.cuda.synchronize()
        assert ma.last_status()[0] == 0
        if args.graph:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                call()
            call = graph.replay
        us = []
        for _ in range(args.passes):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(args.iters):
                call()
            b.record()
            torch.cuda.synchronize()
            us.append(a.elapsed_time(b) / args.iters * 1000.0)
        t = statistics.median(us)
        gbs = B * S * FUSED / t / 1e3
        frac = f"  {100.0 * gbs / peak:5.1f} % of measured copy bandwidth" if peak else ""
        print(f"B={B:4d} S={S:7d} q_len={q_len} {'paged' if args.paged else 'slab '} {args.format}: {t:8.1f} us  {gbs:7.0f} GB/s{frac}")
        results.append({"batch": B, "seq_len": S, "q_len": q_len, "paged": args.paged, "format": args.format, "graph": args.graph, "us": t, "gbs": gbs})
        del kv
    if args.json:
        with open(args.json, "w") as f:
            json.dump(results, f, indent=1)


if __name__ == "__main__":
    main()
