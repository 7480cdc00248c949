"""The tail KV-split planner: structure of the unit list and the decisions at the benchmark shapes."""
import math

import pytest

import moonmath_attention as ma

SMS = 148
ROWS, KV = 256, 128


def _units(plan):
    """Expands a plan into (task, kb_begin, kb_end) the way the kernel decodes unit indices."""
    out = []
    for u in range(plan["total_units"]):
        if u < plan["full_units"]:
            out.append((u, 0, plan["nkb"]))
        else:
            v = u - plan["full_units"]
            task, g = plan["full_units"] + v // plan["split"], v % plan["split"]
            out.append((task, g * plan["nkb"] // plan["split"], (g + 1) * plan["nkb"] // plan["split"]))
    return out


SHAPES = [
    (1, 2, 256, 256), (2, 24, 8192, 8192), (2, 24, 8192, 512), (2, 24, 1000, 777), (2, 24, 1, 4097),
    (2, 24, 32768, 32768), (1, 6, 32768, 32768), (2, 8, 86016, 86016), (1, 40, 2048, 2048), (3, 5, 300, 5000),
]


@pytest.mark.parametrize("shape", SHAPES)
def test_units_cover_every_task_and_key_block_once(shape):
    B, H, Sq, Skv = shape
    p = ma.plan_tail(B, H, Sq, Skv, SMS)
    assert p["nqb"] == math.ceil(Sq / ROWS) and p["nkb"] == math.ceil(Skv / KV)
    assert p["tasks"] == p["nqb"] * B * H
    assert p["full_units"] + p["tail_tasks"] == p["tasks"]
    assert p["total_units"] == p["full_units"] + p["tail_tasks"] * p["split"]
    assert p["grid"] == min(SMS, p["total_units"])
    cover = {}
    for task, b, e in _units(p):
        assert 0 <= b < e <= p["nkb"]
        cover.setdefault(task, []).append((b, e))
    assert sorted(cover) == list(range(p["tasks"]))
    for task, spans in cover.items():
        spans.sort()
        assert spans[0][0] == 0 and spans[-1][1] == p["nkb"]
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    if p["tail_tasks"]:
        assert p["split"] >= 2 and p["full_units"] % SMS == 0
        assert p["nkb"] // p["split"] >= 2
    ws = ma.workspace_bytes(B, H, Sq, Skv, SMS)
    assert ws == 256 + p["tail_tasks"] * p["split"] * (ROWS * 128 + ROWS * 2) * 4


def test_no_tail_flag_disables_the_split():
    from moonmath_attention import _abi

    p = ma.plan_tail(2, 24, 8192, 8192, SMS, _abi.FLAG_NO_TAIL)
    assert p["tail_tasks"] == 0 and p["split"] == 1 and p["total_units"] == p["tasks"]
    assert ma.workspace_bytes(2, 24, 8192, 8192, SMS, _abi.FLAG_NO_TAIL) == 256


def test_decisions_at_benchmark_shapes():
    # headline: 1536 tasks = 10 rounds + 56 stranded -> split
    p = ma.plan_tail(2, 24, 8192, 8192, SMS)
    assert (p["tasks"], p["tail_tasks"]) == (1536, 56) and p["split"] >= 2
    # long-sequence case on one GPU and on one of eight GPUs (6 slices)
    assert ma.plan_tail(2, 24, 32768, 32768, SMS)["tail_tasks"] == 6144 % SMS
    p8 = ma.plan_tail(1, 6, 32768, 32768, SMS)
    assert p8["tasks"] == 768 and p8["tail_tasks"] == 768 % SMS and p8["split"] >= 2
    # the tail-split benchmark shape leaves a partial round, and it is split
    p = ma.plan_tail(2, 8, 86016, 86016, SMS)
    assert p["tasks"] % SMS == 48 and p["tail_tasks"] == 48 and p["split"] >= 2
    # short key/value sequences are never split
    assert ma.plan_tail(2, 24, 8192, 512, SMS)["tail_tasks"] == 0
    # even grids are never split
    assert ma.plan_tail(1, 148, 256, 4096, SMS)["tail_tasks"] == 0
    # a marginal prediction (108 stranded tasks of 32 blocks; measured slower when split) is left alone
    assert ma.plan_tail(2, 8, 4096, 4096, SMS)["tail_tasks"] == 0


def test_split_never_loses_to_no_split_in_the_model():
    """Python twin of the cost model: the chosen split's modelled span beats the unsplit last round."""
    for B, H, Sq, Skv in SHAPES:
        p = ma.plan_tail(B, H, Sq, Skv, SMS)
        if not p["tail_tasks"]:
            continue
        g, tail, nkb = p["split"], p["tail_tasks"], p["nkb"]
        span = math.ceil(tail * g / SMS) * (math.ceil(nkb / g) + 1) + 4
        assert span * 11 < (nkb + 1) * 10  # the 10 % margin of the planner
