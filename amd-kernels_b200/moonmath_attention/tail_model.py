"""Wall-time model of the tail KV-split for a persistent grid on B200 — host arithmetic only.

B200 twin of the reference's planner tool (tools/tail_speedup.py:33-120): for a problem shape it
reports the plan the library will run (through `ma_plan_tail`, the code the kernels use) and the
speed-up the cost model predicts, and `--scan` lists the shapes that gain most.  Units are
"block times": one 128-row key block of one 256-row query task.

    python -m moonmath_attention.tail_model 2 8192 24 [--skv N] [--sms 148]
    python -m moonmath_attention.tail_model --scan
"""
from __future__ import annotations

import argparse
import math

from . import _abi

PART_OVERHEAD = 1  # kPartOverheadBlocks (csrc/tail_plan.h)
MERGE_COST = 4     # kMergeCostBlocks


def predict(batch: int, seq: int, heads: int, seq_kv: int | None = None, sms: int = 148) -> dict:
    """Plan and predicted speed-up for (batch, seq, heads[, seq_kv]) on `sms` SMs."""
    seq_kv = seq_kv or seq
    plan = _abi.plan_tail(batch, heads, seq, seq_kv, sms, 0)
    nkb, tasks = plan["nkb"], plan["tasks"]
    rounds, tail = divmod(tasks, sms)
    unit = nkb + PART_OVERHEAD
    no_split = (rounds + (1 if tail else 0)) * unit
    if plan["tail_tasks"]:
        g = plan["split"]
        span = math.ceil(plan["tail_tasks"] * g / sms) * (math.ceil(nkb / g) + PART_OVERHEAD) + MERGE_COST
        with_split = rounds * unit + span
        reason = "split"
    else:
        span, with_split = None, no_split
        reason = ("even grid" if tail == 0 else "tail >= 95% of a round" if tail > sms * 19 // 20
                  else "key sequence too short" if nkb < 8 else "no split factor beats the unsplit round")
    return dict(plan, rounds=rounds, tail=tail, span=span, gain=no_split / with_split, reason=reason)


def _fmt(info: dict) -> str:
    head = (f"nqb={info['nqb']} nkb={info['nkb']} tasks={info['tasks']} full_rounds={info['rounds']} "
            f"tail={info['tail']}")
    if info["tail_tasks"]:
        return (f"{head}\n  -> SPLIT  parts/task={info['split']}  span={info['span']}  units={info['total_units']}  "
                f"predicted speed-up = {info['gain']:.3f}x")
    return f"{head}\n  -> no split ({info['reason']})  speed-up = 1.000x"


def scan(sms: int = 148, top: int = 20) -> list[tuple]:
    res = []
    for bh in (8, 12, 16, 24, 32, 48, 64):
        for s in range(2048, 131072 + 1, 1024):
            p = predict(1, s, bh, None, sms)
            if p["gain"] > 1.0:
                res.append((p["gain"], bh, s, p["rounds"], p["tail"], p["split"]))
    res.sort(reverse=True)
    return res[:top]


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("B", type=int, nargs="?")
    ap.add_argument("S", type=int, nargs="?")
    ap.add_argument("H", type=int, nargs="?")
    ap.add_argument("--skv", type=int, default=None)
    ap.add_argument("--sms", type=int, default=148)
    ap.add_argument("--scan", action="store_true")
    a = ap.parse_args()
    if a.scan:
        print(f"{'gain':>7} {'B*H':>4} {'S':>7} {'rounds':>6} {'tail':>4} {'parts':>5}")
        for gain, bh, s, r, tail, g in scan(a.sms):
            print(f"{gain:6.3f}x {bh:4d} {s:7d} {r:6d} {tail:4d} {g:5d}")
    elif a.B and a.S and a.H:
        print(f"(B={a.B}, S={a.S}, H={a.H}" + (f", Skv={a.skv}" if a.skv else "") + f") on {a.sms} SMs")
        print(_fmt(predict(a.B, a.S, a.H, a.skv, a.sms)))
    else:
        ap.error("give B S H or --scan")


if __name__ == "__main__":
    main()
