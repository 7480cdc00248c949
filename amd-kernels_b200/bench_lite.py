"""LiteAttention timing on B200: time per call against the fraction of key blocks the skip list keeps.

For each shape the read lists are synthetic: every task keeps the same number of 64-key blocks, chosen as
runs of random length at random places (seeded), the pattern a learned list settles into.  The threshold is
set so low that no vote drops anything further, so every call computes exactly the named blocks; the list
written by one call is what the next call reads (directions alternate, as in `LiteAttention`).  Reported per
kept fraction: milliseconds per call (median of `--passes` passes of `--iters` calls between two CUDA events),
TFLOP/s counted on the computed blocks only (4 * B * H * Sq * kept keys * D), and the speed-up over the dense
`forward` on the same tensors.  `--uneven` makes the kept count vary from task to task and compares the
longest-first hand-out with index order (MOONMATH_LITE_PLAIN).

    python amd-kernels_b200/bench_lite.py [--shapes std,long] [--fractions 1,0.5,0.25,0.125] [--uneven]
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
if HERE not in sys.path:
    sys.path.insert(0, HERE)

SHAPES = {"std": (2, 24, 8192), "long": (2, 24, 16384), "xlong": (2, 24, 32768), "lite-test": (1, 8, 4096)}


def make_rows(tasks: int, ktiles: int, kept_per_task, rng) -> np.ndarray:
    """Read-list rows for a call with phase 1 (blocks walked upwards): pairs are read from the back."""
    rows = np.zeros((tasks, ktiles + 2), np.int16)
    for t in range(tasks):
        kept = int(kept_per_task[t])
        keep = np.zeros(ktiles, bool)
        while keep.sum() < kept:  # runs of 1-8 blocks
            start = int(rng.integers(0, ktiles))
            keep[start:start + int(rng.integers(1, 9))] = True
            over = int(keep.sum()) - kept
            if over > 0:
                keep[np.flatnonzero(keep)[:over]] = False
        marks = []
        b = 0
        while b < ktiles:
            if keep[b]:
                e = b
                while e < ktiles and keep[e]:
                    e += 1
                marks.append((b - 1, e - 1))  # range [b, e): starts one after the first marker, ends one after the second
                b = e
            else:
                b += 1
        flat = []
        for first, second in reversed(marks):  # the first range to walk is the last pair of the row
            flat += [second, first]
        rows[t, 0] = len(flat)
        rows[t, 1:1 + len(flat)] = flat
    return rows


def time_calls(fn, iters: int, passes: int) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ms = []
    for _ in range(passes):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        ms.append(a.elapsed_time(b) / iters)
    return statistics.median(ms)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="std,long")
    ap.add_argument("--fractions", default="1,0.5,0.25,0.125")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--passes", type=int, default=5)
    ap.add_argument("--uneven", action="store_true")
    ap.add_argument("--json", default="")
    args = ap.parse_args()

    import moonmath_attention as ma

    dev = torch.device("cuda:0")
    rng = np.random.default_rng(42)
    results = []
    for label in args.shapes.split(","):
        B, H, S = SHAPES[label]
        g = torch.Generator(device=dev)
        g.manual_seed(42)
        q, k, v = (torch.randn(B, S, H, 128, generator=g, device=dev).bfloat16() for _ in range(3))
        out = torch.empty_like(q)
        tile_m, tile_n = ma.LiteAttention.get_MN()
        qtiles, ktiles = (S + tile_m - 1) // tile_m, (S + tile_n - 1) // tile_n
        tasks = B * H * qtiles
        dense_ms = time_calls(lambda: ma.forward(q, k, v, out=out, layout="bshd", round_mode="rtne"), args.iters, args.passes)
        print(f"{label}: B={B} H={H} S={S}  dense forward {dense_ms:.3f} ms "
              f"({4.0 * B * H * S * S * 128 / dense_ms / 1e9:.0f} TFLOP/s)")
        for frac in (float(x) for x in args.fractions.split(",")):
            mean_kept = max(1, round(frac * ktiles))
            if args.uneven:
                kept = np.clip(rng.integers(1, 2 * mean_kept + 1, tasks), 1, ktiles)
            else:
                kept = np.full(tasks, mean_kept)
            lists = torch.zeros(2, B, H, qtiles, ktiles + 2, dtype=torch.int16, device=dev)
            lists[0] = torch.from_numpy(make_rows(tasks, ktiles, kept, rng)).view(B, H, qtiles, ktiles + 2).to(dev)
            state = {"phase": 0}

            def call():
                read, write = lists[state["phase"]], lists[1 - state["phase"]]
                state["phase"] = 1 - state["phase"]
                ma.forward_lite(q, k, v, read, write, threshold=-1000.0, phase=state["phase"], out=out,
                                layout="bshd", round_mode="rtne")

            row = {"shape": label, "fraction": frac, "kept_mean": float(kept.mean()), "dense_ms": dense_ms}
            for name, env in (("lpt", None), ("plain", "1")) if args.uneven else (("lpt", None),):
                if env:
                    os.environ["MOONMATH_LITE_PLAIN"] = env
                else:
                    os.environ.pop("MOONMATH_LITE_PLAIN", None)
                ms = time_calls(call, args.iters, args.passes)
                row[name + "_ms"] = ms
            os.environ.pop("MOONMATH_LITE_PLAIN", None)
            assert ma.last_status()[0] == 0
            flops = 4.0 * 128 * tile_n * float((kept * min(tile_m, S)).sum())  # per task: 256 rows x kept * 64 keys
            row["tflops"] = flops / row["lpt_ms"] / 1e9
            row["speedup_vs_dense"] = dense_ms / row["lpt_ms"]
            results.append(row)
            extra = f"  plain order {row['plain_ms']:.3f} ms" if args.uneven else ""
            print(f"  kept {kept.mean():7.1f}/{ktiles} blocks ({100.0 * kept.mean() / ktiles:5.1f} %): "
                  f"{row['lpt_ms']:.3f} ms  {row['tflops']:.0f} TFLOP/s on computed blocks  "
                  f"{row['speedup_vs_dense']:.2f}x dense{extra}")
    if args.json:
        with open(args.json, "w") as f:
            json.dump(results, f, indent=1)


if __name__ == "__main__":
    main()
