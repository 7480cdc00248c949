"""Host-side tooling beside the hot path: the planner model and the benchmark's input patterns (CPU only)."""
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "amd-kernels_b200"))

from moonmath_attention import tail_model  # noqa: E402


def test_tail_model_matches_the_plan_the_library_runs():
    p = tail_model.predict(2, 8192, 24)
    assert (p["tasks"], p["rounds"], p["tail"]) == (1536, 10, 56)
    assert p["tail_tasks"] == 56 and p["gain"] > 1.0 and p["reason"] == "split"
    even = tail_model.predict(1, 256, 148, 4096)
    assert even["gain"] == 1.0 and even["reason"] == "even grid"
    short = tail_model.predict(2, 8192, 24, 512)
    assert short["gain"] == 1.0 and short["reason"] == "key sequence too short"
    # an under-occupied GPU gains most (the reference tool's rule of thumb, tools/tail_speedup.py:103-104)
    assert tail_model.predict(1, 5120, 8)["gain"] > 1.3


def test_scan_is_sorted_and_only_lists_wins():
    rows = tail_model.scan(top=10)
    assert len(rows) == 10 and all(r[0] > 1.0 for r in rows)
    assert [r[0] for r in rows] == sorted((r[0] for r in rows), reverse=True)


def test_benchmark_input_patterns():
    import bench_table as bt

    assert [s[0] for s in bt.SHAPES] == list(bt.REFERENCE_MS)
    cpu = torch.device("cpu")
    for pat in bt.PATTERNS:
        q, k, v = bt.make_inputs(1, 2, 256, 128, cpu, pat)
        for t in (q, k, v):
            assert t.shape == (1, 256, 2, 128) and t.dtype == torch.bfloat16 and torch.isfinite(t.float()).all()
        q2, _, _ = bt.make_inputs(1, 2, 256, 128, cpu, pat)
        assert torch.equal(q, q2)
    _, k, _ = bt.make_inputs(1, 2, 4096, 128, cpu, "realistic")
    norms = k.float().norm(dim=-1) / 128 ** 0.5
    assert 0.5 < norms.log().std().item() < 0.7  # log-normal row norms, sigma 0.6
    q, k, _ = bt.make_inputs(1, 1, 256, 128, cpu, "diag")
    assert torch.equal(q, k) and q.float().sum(-1).eq(1).all()
