"""GPU tests of LiteAttention (`forward_lite`, `LiteAttention`) through the C ABI.

The first four mirror the reference's own lite tests (tests/test_attention.py:153-214) on its shape and data
recipes; the rest compare lists (exactly) and outputs (parity criterion of the dense tests) with
oracle/lite_oracle.py and with plain attention over the named key blocks.
"""
from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

from oracle import lite_oracle as lo
from oracle import oracle as orc
from tests.helpers import assert_parity

pytestmark = pytest.mark.gpu

LITE_SHAPE = dict(B=1, H=8, S=4096)  # reference: LITE_SHAPE, tests/test_attention.py:99
LITE_STEPS = 5
LITE_THRESHOLD = -3.0


def _layout(q, k, v, layout):
    """Inputs are generated [B, S, H, D]."""
    if layout == "bhsd":
        q, k, v = (t.transpose(1, 2).contiguous() for t in (q, k, v))
    return q, k, v


def _uniform(device, layout, B, Sq, Skv, H, seed=7):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Sq, H, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(B, Skv, H, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(B, Skv, H, 128, generator=g).to(torch.bfloat16)
    return tuple(t.to(device) for t in _layout(q, k, v, layout))


def _peaked(device, layout, B, Sq, Skv, H, seed=7, hot=64):
    """Head h has large keys in its first (h + 1) * hot positions and tiny ones elsewhere, so that the vote keeps
    exactly those blocks (the recipe of the reference's test, tests/test_attention.py:115-135)."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Sq, H, 128, generator=g)
    k = torch.randn(B, Skv, H, 128, generator=g)
    v = torch.randn(B, Skv, H, 128, generator=g)
    scale = torch.full((H, Skv), 0.05)
    for h in range(H):
        scale[h, : (h + 1) * hot] = 2.0
    k = k * scale.t().reshape(1, Skv, H, 1)
    q, k, v = (t.to(torch.bfloat16) for t in (q, k, v))
    return tuple(t.to(device) for t in _layout(q, k, v, layout))


def _run(ma, q, k, v, layout, steps, must_do_list=None):
    attn = ma.LiteAttention(threshold=LITE_THRESHOLD, round_mode="rtna", layout=layout)
    out = None
    for _ in range(steps):
        out = attn(q, k, v, must_do_list=must_do_list)
    return out


def _bits(t):
    return orc.bf16_tensor_to_bits(t.cpu())


@pytest.fixture(scope="module")
def ma(cuda_device):
    import moonmath_attention

    return moonmath_attention


# --- the reference's four -----------------------------------------------------------------------------------
@pytest.mark.parametrize("layout", ["bhsd", "bshd"])
def test_lite_compute_all_matches_full_attention(ma, cuda_device, layout):
    s = LITE_SHAPE
    q, k, v = _uniform(cuda_device, layout, s["B"], s["S"], s["S"], s["H"])
    attn = ma.LiteAttention(threshold=LITE_THRESHOLD, round_mode="rtna", layout=layout)
    out = attn(q, k, v)
    ref = orc.attention_fp32(q.cpu(), k.cpu(), v.cpu(), layout)
    torch.testing.assert_close(out.float().cpu(), ref, rtol=0.05, atol=0.05)  # the reference's own bar
    wabs = orc.attention_fp32(q.cpu(), k.cpu(), v.cpu().abs(), layout)
    assert_parity(_bits(out), ref.numpy(), wabs.numpy(), "rtna", f"lite compute-all {layout}")
    assert ma.last_status()[0] == 0


def test_lite_longest_first_matches_plain_bitexact(ma, cuda_device, monkeypatch):
    s = LITE_SHAPE
    q, k, v = _peaked(cuda_device, "bshd", s["B"], s["S"], s["S"], s["H"])
    monkeypatch.delenv("MOONMATH_LITE_PLAIN", raising=False)
    lpt = _run(ma, q, k, v, "bshd", LITE_STEPS)
    monkeypatch.setenv("MOONMATH_LITE_PLAIN", "1")
    plain = _run(ma, q, k, v, "bshd", LITE_STEPS)
    assert torch.equal(lpt, plain)


def test_lite_several_tasks_per_cta_match_dense_forward(ma, cuda_device):
    """384 tasks on 148 SMs: every CTA takes several tasks from the counter, task and verdict rings wrap.  With a
    threshold nothing can reach, every call computes every block and must agree with the dense kernel."""
    B, H, S = 2, 24, 2048
    g = torch.Generator(device=cuda_device)
    g.manual_seed(5)
    q, k, v = (torch.randn(B, S, H, 128, generator=g, device=cuda_device).bfloat16() for _ in range(3))
    ref = ma.forward(q, k, v, layout="bshd", round_mode="rtne").float()
    attn = ma.LiteAttention(threshold=-1000.0, round_mode="rtne", layout="bshd")
    for _ in range(3):  # both walk directions
        out = attn(q, k, v)
        torch.cuda.synchronize()
        assert ma.last_status()[0] == 0
        assert (out.float() - ref).abs().max().item() < 2e-3
    rows = attn.read_list.cpu().numpy().reshape(-1, S // 64 + 2)
    assert (rows[:, 0] == 2).all()  # one range, all 32 key blocks


def test_lite_must_do_all_equals_compute_all(ma, cuda_device):
    s = LITE_SHAPE
    q, k, v = _peaked(cuda_device, "bshd", s["B"], s["S"], s["S"], s["H"])
    ktiles = (s["S"] + 63) // 64
    must_do_all = torch.tensor([2, 0, ktiles], dtype=torch.int16, device=cuda_device)
    ref = ma.LiteAttention(threshold=LITE_THRESHOLD, round_mode="rtna", layout="bshd")(q, k, v)
    forced = _run(ma, q, k, v, "bshd", LITE_STEPS, must_do_list=must_do_all)
    assert torch.equal(forced, ref)


def test_lite_skip_list_develops(ma, cuda_device):
    s = LITE_SHAPE
    q, k, v = _peaked(cuda_device, "bshd", s["B"], s["S"], s["S"], s["H"])
    ktiles = s["S"] // 64
    attn = ma.LiteAttention(threshold=LITE_THRESHOLD, round_mode="rtna", layout="bshd")
    attn(q, k, v)
    assert ma.lite.kept_blocks(attn.write_list[0, 0, 0]) == ktiles  # the seed it consumed
    assert ma.lite.kept_blocks(attn.read_list[0, 0, 0]) < ktiles    # the list it learned
    for _ in range(LITE_STEPS - 1):
        attn(q, k, v)
    kept = [ma.lite.kept_blocks(attn.read_list[0, h, 0]) for h in range(s["H"])]
    assert kept == list(range(1, s["H"] + 1)), kept
    assert ma.last_status()[0] == 0


# --- against the oracle ---------------------------------------------------------------------------------------
@pytest.mark.parametrize(
    "layout,B,H,Sq,Skv,hot",
    [
        ("bshd", 1, 8, 1024, 1024, 64),
        ("bhsd", 2, 3, 300, 333, 64),    # ragged query tile and ragged last key block
        ("bshd", 1, 4, 1, 4097, 640),    # one query row, 65 key blocks (odd count, last one a single key)
        ("bhsd", 1, 2, 777, 1000, 192),  # hot region ends inside a pair of blocks
    ],
)
def test_lite_lists_and_outputs_match_oracle(ma, cuda_device, layout, B, H, Sq, Skv, hot):
    q, k, v = _peaked(cuda_device, layout, B, Sq, Skv, H, seed=11, hot=hot)
    qn, kn, vn = (t.float().cpu().numpy() for t in (q, k, v))
    attn = ma.LiteAttention(threshold=LITE_THRESHOLD, round_mode="rtne", layout=layout)
    attn._ensure(q, k)
    read = attn._skip[0].cpu().numpy().copy()
    phase = 0
    for step in range(4):
        phase = 1 - phase
        ref, want = lo.forward_lite(qn, kn, vn, read, LITE_THRESHOLD, phase, layout=layout)
        wabs, _ = lo.forward_lite(qn, kn, np.abs(vn), read, LITE_THRESHOLD, phase, layout=layout)
        out = attn(q, k, v)
        got = attn.read_list.cpu().numpy()
        assert ma.last_status()[0] == 0
        assert np.array_equal(got, want), f"step {step}: written lists differ"
        assert_parity(_bits(out), ref, wabs, "rtne", f"lite step {step} {layout} {Sq}x{Skv}")
        read = want
    total = sum(lo.kept_blocks(r) for r in read.reshape(-1, read.shape[-1]))
    assert total < read.shape[0] * read.shape[1] * read.shape[2] * (read.shape[3] - 2)  # something was dropped


def test_lite_named_blocks_only(ma, cuda_device):
    """A hand-written list: the result is plain attention over exactly the named key blocks."""
    B, H, Sq, Skv = 1, 2, 256, 640
    q, k, v = _uniform(cuda_device, "bhsd", B, Sq, Skv, H, seed=3)
    named = [1, 2, 5, 9]  # ranges [1, 3), [5, 6), [9, 10)
    ktiles = Skv // 64
    for phase in (1, 0):
        row = np.zeros(ktiles + 2, np.int16)
        # pairs are read from the back; a range starts one step after its first marker and ends one step
        # after its second
        if phase:   # upwards: [1, 3), [5, 6), [9, 10)
            marks = [9, 8, 5, 4, 2, 0]
        else:       # downwards: 9, then 5, then 2 and 1
            marks = [1, 3, 5, 6, 9, 10]
        row[0] = 6
        row[1:7] = marks
        assert sorted(b for b, _ in lo.walk(row, phase)) == named
        read = torch.tensor(np.tile(row, (B, H, 1, 1)), device=cuda_device)
        write = torch.zeros_like(read)
        out = ma.forward_lite(q, k, v, read, write, threshold=-1000.0, phase=phase, round_mode="rtne")
        keys = np.concatenate([np.arange(b * 64, b * 64 + 64) for b in named])
        ks, vs = k[:, :, keys].cpu(), v[:, :, keys].cpu()
        ref = orc.attention_fp32(q.cpu(), ks, vs, "bhsd")
        wabs = orc.attention_fp32(q.cpu(), ks, vs.abs(), "bhsd")
        assert_parity(_bits(out), ref.numpy(), wabs.numpy(), "rtne", f"named blocks phase {phase}")
        # nothing can be dropped at this threshold: the written list names the same blocks
        assert sorted(b for b, _ in lo.walk(write[0, 0, 0].cpu().numpy(), 1 - phase)) == named


def test_lite_on_the_reference_tests_own_tensors(ma, cuda_device):
    """The peaked tensors of the reference's skip-list test, rebuilt and hash-checked against what its generator
    produced (tests/golden/make_golden_lite.py): after that test's steps at its threshold the list rows of head h
    that cover the query rows the reference inspects (its first 384-row tile: the first two 256-row rows here) name
    exactly h + 1 key blocks (tests/test_attention.py:209-214).  Further down a row may keep more: a block stays
    when a single query row of a voting group has no hot key scoring high, which the data makes rare, not
    impossible (the CPU oracle keeps the same extra blocks); every row keeps at least its hot blocks."""
    from tests.helpers import reference_peaked_inputs

    got = reference_peaked_inputs()
    if got is None:
        pytest.skip("this torch build draws different randn values than the one that made the fixture")
    q, k, v, g = got
    B, S, H, _ = q.shape
    attn = ma.LiteAttention(threshold=float(g["peaked_threshold"]), round_mode="rtna", layout="bshd")
    dq, dk, dv = (t.to(cuda_device) for t in (q, k, v))
    for _ in range(int(g["peaked_steps"])):
        attn(dq, dk, dv)
    torch.cuda.synchronize()
    assert ma.last_status()[0] == 0
    lists = attn.read_list.cpu().numpy()
    want = g["peaked_kept_by_head"].tolist()
    for t in range(2):
        assert [lo.kept_blocks(lists[0, h, t]) for h in range(H)] == want
    for t in range(lists.shape[2]):
        kept = [lo.kept_blocks(lists[0, h, t]) for h in range(H)]
        assert all(k >= w for k, w in zip(kept, want)), (t, kept)
        assert all(set(range(h + 1)) <= {b for b, _ in lo.walk(lists[0, h, t], 1 - attn._phase)} for h in range(H)), t  # the next call walks the other way


def test_lite_empty_list_gives_zeros_and_writes_nothing(ma, cuda_device):
    q, k, v = _uniform(cuda_device, "bhsd", 1, 256, 256, 2, seed=5)
    read = torch.zeros(1, 2, 1, 6, dtype=torch.int16, device=cuda_device)
    read[0, 1, 0, :3] = torch.tensor([2, 3, -1], dtype=torch.int16)  # head 1 computes everything
    write = torch.full_like(read, 77)
    out = ma.forward_lite(q, k, v, read, write, threshold=-3.0, phase=1)
    assert ma.last_status()[0] == 0
    assert torch.count_nonzero(out[0, 0]) == 0
    assert torch.all(write[0, 0] == 77)
    ref = ma.forward(q[:, 1:], k[:, 1:], v[:, 1:])
    assert (out[0, 1].float() - ref[0, 0].float()).abs().max() < 0.02


def test_lite_disabled_is_the_dense_forward(ma, cuda_device):
    q, k, v = _uniform(cuda_device, "bshd", 1, 512, 512, 4, seed=9)
    attn = ma.LiteAttention(enable_skipping=False, layout="bshd", round_mode="rtz")
    assert torch.equal(attn(q, k, v), ma.forward(q, k, v, layout="bshd", round_mode="rtz"))
    assert attn.read_list is None


def test_lite_state_follows_shape_and_reset(ma, cuda_device):
    attn = ma.LiteAttention(threshold=-4.0, layout="bhsd")
    q, k, v = _uniform(cuda_device, "bhsd", 1, 300, 500, 2)
    attn(q, k, v)
    assert tuple(attn.read_list.shape) == (1, 2, 2, 8 + 2)
    q2, k2, v2 = _uniform(cuda_device, "bhsd", 1, 300, 130, 2)
    attn(q2, k2, v2)  # new key length: lists rebuilt, compute-all again
    assert tuple(attn.read_list.shape) == (1, 2, 2, 3 + 2)
    attn.reset_skip_state()
    assert attn.read_list is None and attn.write_list is None
    assert ma.LiteAttention.get_MN() == (256, 64)
    with pytest.raises(ValueError):
        ma.LiteAttention(threshold=0.0)
    with pytest.raises(ValueError):
        attn.set_threshold(1.0)
    with pytest.raises(ValueError):
        ma.LiteAttention(layout="sbhd")


def test_forward_lite_argument_errors(ma, cuda_device):
    q, k, v = _uniform(cuda_device, "bhsd", 1, 256, 256, 1)
    good = torch.zeros(1, 1, 1, 6, dtype=torch.int16, device=cuda_device)
    good[..., :3] = torch.tensor([2, 3, -1], dtype=torch.int16)
    kw = dict(threshold=-3.0, phase=1)
    with pytest.raises(ValueError, match="int16"):
        ma.forward_lite(q, k, v, good.int(), good.clone(), **kw)
    with pytest.raises(ValueError, match="contiguous"):
        ma.forward_lite(q, k, v, good, torch.zeros(1, 1, 1, 12, dtype=torch.int16, device=cuda_device)[..., ::2], **kw)
    with pytest.raises(ValueError, match="same device"):
        ma.forward_lite(q, k, v, good.cpu(), good.clone(), **kw)
    with pytest.raises(ValueError, match="int16 values"):
        ma.forward_lite(q, k, v, good[..., :5].contiguous(), good.clone(), **kw)
    with pytest.raises(ValueError, match="round_mode"):
        ma.forward_lite(q, k, v, good, good.clone(), round_mode="up", **kw)
    with pytest.raises(ValueError, match="GPU-only"):
        ma.forward_lite(q.cpu(), k.cpu(), v.cpu(), good, good.clone(), **kw)
    with pytest.raises(TypeError):
        ma.forward_lite(q.float(), k, v, good, good.clone(), **kw)
    # straight at the C ABI: the reference's code 4 for missing lists, 17 for a bad threshold / phase
    lib = ma.abi.lib
    ws = torch.empty(int(lib.ma_lite_workspace_bytes(1, 1, 256)), dtype=torch.uint8, device=cuda_device)
    out = torch.empty_like(q)
    args = lambda rl, wl, thr, ph: (q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), 1, 1, 256, 256, 128, 0, 1,
                                    rl, wl, None, ctypes.c_float(thr), ph, ws.data_ptr(), ws.numel(), 0, None)
    assert lib.ma_attention_forward_lite(*args(None, good.data_ptr(), -3.0, 1)) == 4
    assert lib.ma_attention_forward_lite(*args(good.data_ptr(), good.data_ptr(), 0.5, 1)) == 17
    assert lib.ma_attention_forward_lite(*args(good.data_ptr(), good.data_ptr(), -3.0, 2)) == 17
    assert b"read_list" in lib.ma_error_string(4)
