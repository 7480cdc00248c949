"""CPU tests of the LiteAttention skip lists: the Python restatement (oracle/lite_oracle.py) against the values the
reference states, against the host build of the header the CUDA kernel uses, and its own round-trip properties."""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np
import pytest

from oracle import lite_oracle as lo
from oracle import oracle as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def harness(tmp_path_factory):
    so = tmp_path_factory.mktemp("lite") / "liblite_list_harness.so"
    src = os.path.join(ROOT, "tests", "native", "lite_list_harness.cpp")
    subprocess.run(["g++", "-O1", "-std=c++17", "-shared", "-fPIC", "-o", str(so), src], check=True)
    lib = ctypes.CDLL(str(so))
    lib.harness_walk.restype = ctypes.c_int
    lib.harness_kept.restype = ctypes.c_int
    lib.harness_emit.restype = None
    return lib


def c_walk(lib, row, phase):
    r = np.asarray(row, np.int16)
    cap = 4096
    blocks, closes = (ctypes.c_int * cap)(), (ctypes.c_int * cap)()
    n = lib.harness_walk(r.ctypes.data_as(ctypes.c_void_p), phase, blocks, closes, cap)
    return [(blocks[i], bool(closes[i])) for i in range(n)]


def c_emit(lib, blocks, skips, closes, width, phase, must_do=None):
    n = len(blocks)
    arr = lambda xs: (ctypes.c_int * max(n, 1))(*[int(x) for x in xs])
    out = np.zeros(width, np.int16)
    md = None if must_do is None else np.asarray(must_do, np.int16)
    lib.harness_emit(arr(blocks), arr(skips), arr(closes), n, width, phase,
                     None if md is None else md.ctypes.data_as(ctypes.c_void_p), out.ctypes.data_as(ctypes.c_void_p))
    return out.tolist()


def py_emit(blocks, skips, closes, width, phase, must_do=None):
    e, pin = lo.ListEmitter(width, phase), lo.MustDo(must_do, phase)
    for i, b in enumerate(blocks):
        e.record(b, bool(skips[i]) and not pin.forced(b), bool(closes[i]) or i + 1 == len(blocks))
    return e.finish()


# --- values the reference states ------------------------------------------------------------------------------
def test_seed_row_walks_every_block_upwards():
    # moonmath_attention/lite.py:124-127: [2, ktiles - 1, -1], read by the first call with phase 1
    for ktiles in (1, 2, 7, 64):
        row = lo.seed_row(ktiles)
        assert row[:3] == [2, ktiles - 1, -1] and len(row) == ktiles + 2
        got = lo.walk(row, 1)
        assert [b for b, _ in got] == list(range(ktiles))
        assert [c for _, c in got] == [False] * (ktiles - 1) + [True]
        assert lo.kept_blocks(row) == ktiles


def test_planner_example_of_the_reference():
    # csrc/attention_kernel.hip:1318-1319: (step +1) row = [4, 9, 5, 20, 18] -> 4 + 2 = 6 kept blocks
    row = [4, 9, 5, 20, 18]
    assert lo.kept_blocks(row) == 6
    # read from the back: first the range after marker 18 up to marker 20, then the one after 5 up to 9
    assert [b for b, _ in lo.walk(row, 1)] == [19, 20, 6, 7, 8, 9]


def test_two_directions_alternate():
    # a call that walks upwards writes what the next call reads downwards, and the other way round
    width = 34
    blocks = list(range(32))
    skips = [0 if (3 <= b < 9 or b == 20 or b >= 30) else 1 for b in blocks]
    closes = [0] * 31 + [1]
    up = py_emit(blocks, skips, closes, width, 1)
    kept_up = [b for b in blocks if not skips[b]]
    assert [b for b, _ in lo.walk(up, 0)] == kept_up[::-1]
    down_blocks = blocks[::-1]
    down = py_emit(down_blocks, [skips[b] for b in down_blocks], closes, width, 0)
    assert [b for b, _ in lo.walk(down, 1)] == kept_up
    assert lo.kept_blocks(up) == lo.kept_blocks(down) == len(kept_up)


def test_must_do_ranges_pin_blocks():
    width = 18
    blocks = list(range(16))
    skips = [1] * 16
    closes = [0] * 15 + [1]
    must = [4, 0, 2, 9, 12]  # [0, 2) and [9, 12)
    for phase, order in ((1, blocks), (0, blocks[::-1])):
        row = py_emit(order, skips, closes, width, phase, must)
        assert sorted(b for b, _ in lo.walk(row, 1 - phase)) == [0, 1, 9, 10, 11]
    assert py_emit(blocks, skips, closes, width, 1, [0])[0] == 0  # len 0: nothing pinned, nothing kept


# --- the header the CUDA kernel uses, built for the host -------------------------------------------------------
def test_header_matches_python_on_random_lists(harness):
    rng = np.random.default_rng(5)
    for trial in range(300):
        ktiles = int(rng.integers(1, 80))
        width = ktiles + 2
        phase = int(rng.integers(0, 2))
        keep = rng.random(ktiles) < rng.random()
        order = list(range(ktiles)) if phase else list(range(ktiles - 1, -1, -1))
        closes = [0] * (ktiles - 1) + [1]
        skips = [0 if keep[b] else 1 for b in order]
        must = None
        if trial % 3 == 0:
            s0 = int(rng.integers(0, ktiles)); e0 = int(rng.integers(s0, ktiles + 1))
            must = [2, s0, e0]
        row_py = py_emit(order, skips, closes, width, phase, must)
        row_c = c_emit(harness, order, skips, closes, width, phase, must)
        assert row_py == row_c
        # the next call reads it in the other direction
        w_py, w_c = lo.walk(row_py, 1 - phase), c_walk(harness, row_c, 1 - phase)
        assert w_py == w_c
        assert harness.harness_kept(np.asarray(row_c, np.int16).ctypes.data_as(ctypes.c_void_p), 1 - phase) == len(w_py)
        want = {b for b in range(ktiles) if keep[b] or (must and must[1] <= b < must[2])}
        assert {b for b, _ in w_py} == want
        # second generation: walk that list, vote again, emit, read back
        order2 = [b for b, _ in w_py]
        closes2 = [int(c) for _, c in w_py]
        keep2 = rng.random(ktiles) < 0.6
        skips2 = [0 if keep2[b] else 1 for b in order2]
        if order2:
            r2_py = py_emit(order2, skips2, closes2, width, 1 - phase)
            r2_c = c_emit(harness, order2, skips2, closes2, width, 1 - phase)
            assert r2_py == r2_c
            assert {b for b, _ in lo.walk(r2_py, phase)} == {b for b in order2 if keep2[b]}


def test_empty_and_single_block_rows(harness):
    assert lo.walk([0, 0, 0], 1) == [] and c_walk(harness, [0, 0, 0], 1) == []
    assert lo.walk(lo.seed_row(1), 1) == [(0, True)] == c_walk(harness, lo.seed_row(1), 1)


# --- the attention part of the oracle --------------------------------------------------------------------------
def _inputs(B, H, Sq, Skv, seed):
    import torch

    g = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(B, H, s, 128, generator=g).to(torch.bfloat16) for s in (Sq, Skv, Skv))
    return q, k, v


def test_compute_all_with_a_loose_threshold_is_full_attention():
    q, k, v = _inputs(1, 2, 300, 333, 3)
    ktiles = (333 + 63) // 64
    read = np.tile(np.asarray(lo.seed_row(ktiles), np.int16), (1, 2, 2, 1))
    out, write = lo.forward_lite(q.float().numpy(), k.float().numpy(), v.float().numpy(), read, -1000.0, 1)
    ref = orc.attention_fp32(q, k, v, "bhsd").numpy()
    np.testing.assert_allclose(out, ref, rtol=2e-5, atol=2e-6)
    assert all(lo.kept_blocks(write[0, h, t]) == ktiles for h in range(2) for t in range(2))
    # ... and the same downwards
    out2, write2 = lo.forward_lite(q.float().numpy(), k.float().numpy(), v.float().numpy(), write, -1000.0, 0)
    np.testing.assert_allclose(out2, ref, rtol=2e-5, atol=2e-6)
    assert [b for b, _ in lo.walk(write2[0, 0, 0], 1)] == list(range(ktiles))


def test_peaked_heads_keep_their_hot_blocks():
    # the data recipe of the reference's test (tests/test_attention.py:115-135): head h has hot keys in blocks 0..h
    import torch

    H, S = 4, 512
    g = torch.Generator().manual_seed(7)
    q, k, v = (torch.randn(1, H, S, 128, generator=g) for _ in range(3))
    scale = torch.full((H, S), 0.05)
    for h in range(H):
        scale[h, : (h + 1) * 64] = 2.0
    k = k * scale.view(1, H, S, 1)
    q, k, v = (t.to(torch.bfloat16).float().numpy() for t in (q, k, v))
    ktiles = S // 64
    read = np.tile(np.asarray(lo.seed_row(ktiles), np.int16), (1, H, 2, 1))
    phase = 0
    for step in range(3):
        phase = 1 - phase
        _, read = lo.forward_lite(q, k, v, read, -3.0, phase)
    assert [lo.kept_blocks(read[0, h, 0]) for h in range(H)] == [1, 2, 3, 4]


# --- pinned by outputs of the reference's own Python (tests/golden/make_golden_lite.py) -----------------------
def _golden():
    import os

    return np.load(os.path.join(os.path.dirname(__file__), "golden", "lite_reference.npz"))


def test_seed_rows_equal_what_the_reference_class_builds():
    """`LiteAttention._ensure` of the reference, executed on the CPU, built `seed`; the oracle's seed row and this
    library's class must build the same rows (the row count differs: 384 query rows per row there, 256 here)."""
    import torch

    import moonmath_attention as ma

    g = _golden()
    B, H, Sq, Skv = (int(x) for x in g["seed_shape_args"])
    seed = g["seed"]
    ref_m, ref_n = (int(x) for x in g["ref_tile"])
    assert ref_n == lo.KEY_BLOCK == ma.LiteAttention.get_MN()[1]
    ktiles = -(-Skv // ref_n)
    assert seed.shape == (2, B, H, -(-Sq // ref_m), ktiles + 2)
    want = np.zeros(ktiles + 2, np.int16)
    want[:3] = lo.seed_row(ktiles)[:3]
    assert np.all(seed[0] == want) and not seed[1].any()
    attn = ma.LiteAttention(threshold=-3.0)
    attn._ensure(torch.zeros(B, H, Sq, 128, dtype=torch.bfloat16), torch.zeros(B, H, Skv, 128, dtype=torch.bfloat16))
    mine = attn._skip.numpy()
    assert mine.shape == (2, B, H, -(-Sq // ma.LiteAttention.get_MN()[0]), ktiles + 2)
    assert np.all(mine[0] == want) and not mine[1].any()


def test_double_buffer_protocol_equals_the_reference_class(monkeypatch):
    """Which buffer is read, which is written and which phase the kernel is told, over three calls, as recorded
    from the reference's class with a stand-in kernel."""
    import torch

    import moonmath_attention as ma
    from moonmath_attention import _kernel

    calls = []

    def fake(q, k, v, read_list, write_list, *, threshold, phase, must_do_list=None, out=None, round_mode="rtna", layout="bhsd"):
        calls.append((read_list.data_ptr(), write_list.data_ptr(), int(phase)))
        return torch.zeros_like(q)

    monkeypatch.setattr(_kernel, "forward_lite", fake)
    q = torch.zeros(1, 2, 1000, 128, dtype=torch.bfloat16)
    k = torch.zeros(1, 2, 777, 128, dtype=torch.bfloat16)
    attn = ma.LiteAttention(threshold=-3.0)
    for _ in range(3):
        attn(q, k, k)
    buf = {attn._skip[0].data_ptr(): 0, attn._skip[1].data_ptr(): 1}
    assert [[buf[r], buf[w], ph] for r, w, ph in calls] == _golden()["protocol"].tolist()


def test_row_decoder_equals_the_reference_tests_decoder():
    from moonmath_attention.lite import kept_blocks as product_kept

    g = _golden()
    for row, kept in zip(g["sample_rows"], g["sample_kept"]):
        assert lo.kept_blocks(row) == int(kept) == product_kept(row)
        n = int(row[0])
        if n >= 2 and all(int(row[i]) != int(row[i - 1]) for i in range(n, 1, -2)):
            ascending = all(int(row[i]) < int(row[i - 1]) for i in range(n, 1, -2))
            assert len(lo.walk(row, 1 if ascending else 0)) == int(kept)


def test_vote_on_the_reference_tests_data_keeps_what_that_test_asserts():
    """The peaked tensors of the reference's skip-list test, rebuilt and hash-checked against its generator; after
    that test's number of steps at its threshold, head h must name exactly h + 1 key blocks (its assertion,
    tests/test_attention.py:209-214).  Two list rows (512 query rows) of every head are run; the block count does
    not depend on the query-row geometry."""
    from helpers import reference_peaked_inputs

    got = reference_peaked_inputs()
    if got is None:
        import pytest

        pytest.skip("this torch build draws different randn values than the one that made the fixture")
    q, k, v, g = got
    B, S, H, _ = q.shape
    rows = 2 * lo.QUERY_BLOCK
    qn, kn, vn = (t.float().numpy() for t in (q[:, :rows], k, v))
    ktiles = S // lo.KEY_BLOCK
    read = np.tile(np.asarray(lo.seed_row(ktiles), np.int16), (B, H, 2, 1))
    phase = 0
    for _ in range(int(g["peaked_steps"])):
        phase = 1 - phase
        _, read = lo.forward_lite(qn, kn, vn, read, float(g["peaked_threshold"]), phase, layout="bshd")
    for t in range(2):
        assert [lo.kept_blocks(read[0, h, t]) for h in range(H)] == g["peaked_kept_by_head"].tolist()


def test_lpt_order_is_a_permutation_heaviest_first():
    ktiles = 16
    rows = []
    rng = np.random.default_rng(1)
    for t in range(40):
        n = int(rng.integers(1, ktiles + 1))
        rows.append([2, n - 1, -1] + [0] * (ktiles - 1))
    read = np.asarray(rows, np.int16).reshape(1, 1, 40, ktiles + 2)
    order = lo.lpt_order(read, 1)
    assert sorted(order) == list(range(40))
    kept = [lo.kept_blocks(rows[t]) for t in order]
    buckets = [k * 256 // (ktiles + 1) for k in kept]
    assert buckets == sorted(buckets, reverse=True)
