"""Parity of the CUDA path (through the ctypes C ABI) with the CPU oracle.  Needs a B200: -m gpu."""
import hashlib
import os

import numpy as np
import pytest
import torch

from oracle import oracle as orc
from helpers import assert_parity, weighted_abs_v

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "basic_example.npz")


@pytest.fixture(scope="module")
def ma(cuda_device):
    import moonmath_attention

    return moonmath_attention


def _flags():
    from moonmath_attention import _abi

    return _abi


def gpu_forward(ma, q, k, v, layout, mode, flags=0):
    """The public call's device path with explicit C-ABI flag bits (the public call reads them from the environment)."""
    dev = torch.device("cuda:0")
    out = ma._kernel._forward_cuda(q.to(dev), k.to(dev), v.to(dev), None, mode, layout, flags)
    torch.cuda.synchronize()
    assert ma.last_status()[0] == 0
    return orc.bf16_tensor_to_bits(out)


def check_case(ma, B, H, Sq, Skv, layout, mode, flags=0, what=""):
    q, k, v = orc.make_inputs(B, H, Sq, Skv, layout)
    got = gpu_forward(ma, q, k, v, layout, mode, flags)
    ref = orc.attention_fp32(q, k, v, layout).numpy()
    wabs = weighted_abs_v(q, k, v, layout).numpy()
    precise = bool(flags & _flags().FLAG_PRECISE_P)
    return assert_parity(got, ref, wabs, mode, what or f"{(B, H, Sq, Skv)} {layout} {mode}", skv=Skv, precise=precise)


# ---- BASELINE config 1: the plumbing case ---------------------------------------------------------
@pytest.mark.parametrize("flags_name", ["pipelined", "simple", "exact_max", "precise", "precise_exact_max"])
def test_config1_bhsd_rtne(ma, flags_name):
    A = _flags()
    flags = {"pipelined": 0, "simple": A.FLAG_SIMPLE, "exact_max": A.FLAG_EXACT_MAX, "precise": A.FLAG_PRECISE_P,
             "precise_exact_max": A.FLAG_PRECISE_P | A.FLAG_EXACT_MAX}[flags_name]
    check_case(ma, 1, 2, 256, 256, "bhsd", "rtne", flags)  # the histogram of this case is pinned further down


# ---- the ULP histograms, pinned ---------------------------------------------------------------------
# The stated target is "every finite output within 1 bf16 ULP of the fp32 oracle".  A kernel that rounds the
# probabilities to bf16 (as the reference does, csrc/attention_kernel.hip:446-448) cannot meet it on outputs that
# are small next to the terms they are summed from; the precise mode (probabilities as two bf16 terms) does,
# wherever the output is not a cancellation residue.  Both distributions are pinned here so that a precision
# regression fails a test: the default mode to its measured histogram (with 15 % headroom), the precise mode to
# "at most 1 ULP" on every gated output.
ULP_CASES = {
    # name: (B, H, Sq, Skv, layout, slices checked against the oracle)
    "c1": (1, 2, 256, 256, "bhsd", None),
    "c2_slices": (2, 24, 8192, 8192, "bshd", (0, 29)),
    "c3a": (2, 24, 8192, 512, "bshd", (5, 40)),
    "c3b": (2, 24, 1000, 777, "bshd", None),
    "c3c": (2, 24, 1, 4097, "bshd", None),
}
# Measured on B200 (148 SMs; the kernel is deterministic), default mode:
#   gated frac_gt1ulp, ungated frac_gt1ulp, frac_exact, rmse for rtne / rtna, rmse for rtz
# (the gated maximum is 4..18 ULP, the ungated one ~29 000 ULP: an output of 1e-6 beside row terms of 0.1).
ULP_PINS = {
    "c1": (0.0806, 0.1184, 0.5998, 2.287e-4, 3.721e-4),
    "c2_slices": (0.0162, 0.1363, 0.5675, 4.211e-5, 6.603e-5),
    "c3a": (0.0740, 0.1251, 0.5867, 1.665e-4, 2.658e-4),
    "c3b": (0.0670, 0.1272, 0.5834, 1.366e-4, 2.175e-4),
    "c3c": (0.0262, 0.1344, 0.5710, 5.888e-5, 9.359e-5),
}


def _ulp_report(ma, name, mode, flags):
    B, H, Sq, Skv, layout, slices = ULP_CASES[name]
    if slices is None:
        q, k, v = orc.make_inputs(B, H, Sq, Skv, layout)
    else:  # only the named (batch x head) slices, as a batch of one: same values as in the full problem
        parts = [orc.make_inputs(B, H, Sq, Skv, layout, bh_range=range(s, s + 1)) for s in slices]
        hax = 2 if layout == "bshd" else 1
        q, k, v = (torch.cat([p[i] for p in parts], dim=hax).contiguous() for i in range(3))
    got = gpu_forward(ma, q, k, v, layout, mode, flags)
    ref = orc.attention_fp32(q, k, v, layout).numpy()
    wabs = weighted_abs_v(q, k, v, layout).numpy()
    precise = bool(flags & _flags().FLAG_PRECISE_P)
    return assert_parity(got, ref, wabs, mode, f"{name} {mode} flags {flags:#x}", skv=Skv, precise=precise)


@pytest.mark.parametrize("name", sorted(ULP_CASES))
@pytest.mark.parametrize("mode", orc.ROUND_MODES)
def test_ulp_histogram_default_mode_is_pinned(ma, name, mode):
    rep = _ulp_report(ma, name, mode, 0)
    gated, plain, exact, rmse_near, rmse_rtz = ULP_PINS[name]
    print(f"ULP {name} {mode} default: {rep}")
    assert rep["gated_frac_gt1ulp"] <= gated * 1.15, rep
    assert rep["frac_gt1ulp"] <= plain * 1.15, rep
    assert rep["frac_exact"] >= exact * 0.95, rep
    assert rep["rmse"] <= (rmse_rtz if mode == "rtz" else rmse_near) * 1.15, rep
    assert rep["gated_max_ulp"] <= 24, rep


@pytest.mark.parametrize("name", sorted(ULP_CASES))
@pytest.mark.parametrize("mode", orc.ROUND_MODES)
def test_ulp_histogram_precise_mode_meets_one_ulp_where_it_is_meaningful(ma, name, mode):
    rep = _ulp_report(ma, name, mode, _flags().FLAG_PRECISE_P)
    print(f"ULP {name} {mode} precise: {rep}")
    assert rep["gated_max_ulp"] <= 1, rep          # the stated bar, on every output that is not a cancellation residue
    assert rep["frac_gt1ulp"] <= 2e-3, rep         # and all but a sliver of the residues (measured 5e-4 .. 1e-3)
    assert rep["frac_exact"] >= 0.985, rep         # measured 0.991 .. 0.993 (default mode: 0.57 .. 0.60)


def test_precise_flag_through_the_public_call(ma, monkeypatch):
    # the development switches of the environment change which path runs; this test compares paths, so it runs without them
    for name in ("MOONMATH_NO_TAIL", "MOONMATH_SIMPLE", "MOONMATH_EXACT_MAX", "MOONMATH_PRECISE_P"):
        monkeypatch.delenv(name, raising=False)
    dev = torch.device("cuda:0")
    q, k, v = (t.to(dev) for t in orc.make_inputs(1, 2, 300, 400, "bhsd"))
    a = ma.forward(q, k, v, round_mode="rtne", precise=True)
    b = ma._kernel._forward_cuda(q, k, v, None, "rtne", "bhsd", _flags().FLAG_PRECISE_P)
    monkeypatch.setenv("MOONMATH_PRECISE_P", "1")
    c = ma.forward(q, k, v, round_mode="rtne")
    monkeypatch.delenv("MOONMATH_PRECISE_P")
    d = ma.forward(q, k, v, round_mode="rtne")
    torch.cuda.synchronize()
    assert torch.equal(a.view(torch.int16), b.view(torch.int16)) and torch.equal(a.view(torch.int16), c.view(torch.int16))
    assert not torch.equal(a.view(torch.int16), d.view(torch.int16))


# ---- the reference's example, against the output its own oracle lines produced ---------------------
def test_reference_example_fixture(ma):
    g = np.load(GOLDEN)
    B, H, S, D = (int(x) for x in g["shape"])
    torch.manual_seed(int(g["seed"]))
    q = torch.randn(B, H, S, D, dtype=torch.bfloat16)
    k = torch.randn(B, H, S, D, dtype=torch.bfloat16)
    v = torch.randn(B, H, S, D, dtype=torch.bfloat16)
    sha = hashlib.sha256(q.view(torch.int16).numpy().tobytes()).hexdigest()
    if sha != str(g["sha_q"]):
        pytest.skip("this torch build draws different randn values than the one that made the fixture")
    rows = g["rows"]
    wabs = weighted_abs_v(q, k, v, "bhsd")[0][:, rows, :].numpy()
    for mode in orc.ROUND_MODES:
        got = gpu_forward(ma, q, k, v, "bhsd", mode).reshape(B, H, S, D)[0][:, rows, :]
        assert_parity(got, g["ref_rows"], wabs, mode, f"basic.py fixture {mode}")


# ---- ragged lengths and cross-attention (BASELINE config 3 and edge sizes) --------------------------
EDGE = [1, 15, 16, 17, 63, 64, 65, 127, 128, 129, 255, 257]


@pytest.mark.parametrize("layout", ["bhsd", "bshd"])
def test_edge_lengths(ma, layout):
    for i, sq in enumerate(EDGE):
        skv = EDGE[(i * 5 + 3) % len(EDGE)]
        check_case(ma, 2, 3, sq, skv, layout, orc.ROUND_MODES[i % 3])


@pytest.mark.parametrize("sq,skv", [(8192, 512), (1000, 777), (1, 4097)])
def test_config3_cross_attention_ragged(ma, sq, skv):
    B, H = 2, 24
    q, k, v = orc.make_inputs(B, H, sq, skv, "bshd")
    got = gpu_forward(ma, q, k, v, "bshd", "rtne").reshape(B, sq, H, 128)
    # the CPU oracle on every slice of the two short cases, on 4 slices of the long one
    if sq <= 1000:
        ref = orc.attention_fp32(q, k, v, "bshd").numpy()
        wabs = weighted_abs_v(q, k, v, "bshd").numpy()
        assert_parity(got, ref, wabs, "rtne", f"C3 {(sq, skv)}")
    else:
        for h in (0, 7, 23):
            qs, ks, vs = (t[:, :, h:h + 1].contiguous() for t in (q, k, v))
            ref = orc.attention_fp32(qs, ks, vs, "bshd").numpy()
            wabs = weighted_abs_v(qs, ks, vs, "bshd").numpy()
            assert_parity(np.ascontiguousarray(got[:, :, h:h + 1]), ref, wabs, "rtne", f"C3 {(sq, skv)} head {h}")


# ---- the shapes of the reference's own tests (tests/test_attention.py:20-24, 68-85) ------------------
@pytest.mark.parametrize("layout", ["bshd", "bhsd"])
@pytest.mark.parametrize("shape", [(1, 4, 1024, 256), (2, 8, 4096, 512)], ids=["small", "medium"])
@pytest.mark.parametrize("cross", [False, True], ids=["self", "cross"])
def test_reference_test_shapes_sdpa_sanity(ma, shape, layout, cross):
    import torch.nn.functional as F

    B, H, S, Skv = shape
    dev = torch.device("cuda:0")
    torch.manual_seed(42)
    q = torch.randn(B, S, H, 128, dtype=torch.bfloat16, device=dev)
    kv_len = Skv if cross else S
    k = torch.randn(B, kv_len, H, 128, dtype=torch.bfloat16, device=dev)
    v = torch.randn(B, kv_len, H, 128, dtype=torch.bfloat16, device=dev)
    if layout == "bhsd":
        q, k, v = (t.transpose(1, 2).contiguous() for t in (q, k, v))
    out = ma.forward(q, k, v, round_mode="rtna", layout=layout)
    qh, kh, vh = (t.transpose(1, 2) for t in (q, k, v)) if layout == "bshd" else (q, k, v)
    ref = F.scaled_dot_product_attention(qh, kh, vh, is_causal=False)
    ref = ref.transpose(1, 2) if layout == "bshd" else ref
    torch.testing.assert_close(out.float(), ref.float(), rtol=0.05, atol=0.05)  # the reference's tolerance


# ---- rounding modes -------------------------------------------------------------------------------
def test_rounding_kernel_bit_exact_on_all_upper_halves(ma, cuda_device):
    A = _flags()
    hi = np.arange(1 << 16, dtype=np.uint32) << 16
    lows = (0x0000, 0x0001, 0x7FFF, 0x8000, 0x8001, 0xFFFF, 0x1234, 0xC000)
    x = np.concatenate([hi | lo for lo in lows]).view(np.float32)
    xd = torch.from_numpy(x.copy()).to(cuda_device)
    for mode in orc.ROUND_MODES:
        dst = torch.empty(x.size, dtype=torch.int16, device=cuda_device)
        rc = A.lib.ma_round_bf16(xd.data_ptr(), dst.data_ptr(), x.size, A.ROUND_MODE[mode],
                                 torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert np.array_equal(dst.cpu().numpy().view(np.uint16), orc.round_bf16_bits(x, mode)), mode


def test_round_modes_relate_as_the_formulas_say(ma):
    """Same inputs, three modes: truncation is never above the nearest modes and at most one ulp below."""
    q, k, v = orc.make_inputs(1, 4, 512, 512, "bshd")
    out = {m: gpu_forward(ma, q, k, v, "bshd", m).reshape(-1) for m in orc.ROUND_MODES}
    z, e, a = (out[m].astype(np.int64) & 0x7FFF for m in ("rtz", "rtne", "rtna"))
    assert np.all((e - z >= 0) & (e - z <= 1)) and np.all((a - z >= 0) & (a - z <= 1))
    assert np.count_nonzero(e != a) < e.size // 1000  # ties only
    assert np.count_nonzero(e != z) > e.size // 4


def test_deterministic_run_to_run(ma):
    q, k, v = orc.make_inputs(2, 5, 700, 900, "bhsd")
    first = gpu_forward(ma, q, k, v, "bhsd", "rtne")
    for _ in range(3):
        assert np.array_equal(gpu_forward(ma, q, k, v, "bhsd", "rtne"), first)


# ---- kernels against each other ---------------------------------------------------------------------
def test_pipelined_matches_serialised_kernel(ma):
    A = _flags()
    q, k, v = orc.make_inputs(2, 3, 640, 1111, "bshd")
    a = gpu_forward(ma, q, k, v, "bshd", "rtne", A.FLAG_EXACT_MAX | A.FLAG_NO_TAIL)
    b = gpu_forward(ma, q, k, v, "bshd", "rtne", A.FLAG_SIMPLE)
    d = orc.ulp_distance(a.reshape(-1), b.reshape(-1))
    fa, fb = orc.bf16_bits_to_f32(a.reshape(-1)), orc.bf16_bits_to_f32(b.reshape(-1))
    assert np.abs(fa - fb).max() < 2e-3 and np.count_nonzero(d > 1) < d.size // 20


def test_kv_split_agrees_with_unsplit(ma):
    """320 tasks on 148 SMs: two full rounds and a split tail; the tail's rows must satisfy the same bound."""
    A = _flags()
    B, H, S = 1, 40, 2048
    plan = ma.plan_tail(B, H, S, S, torch.cuda.get_device_properties(0).multi_processor_count)
    q, k, v = orc.make_inputs(B, H, S, S, "bhsd")
    split = gpu_forward(ma, q, k, v, "bhsd", "rtne", 0).reshape(B * H, S, 128)
    whole = gpu_forward(ma, q, k, v, "bhsd", "rtne", A.FLAG_NO_TAIL).reshape(B * H, S, 128)
    if plan["tail_tasks"]:
        first_tail_bh = plan["full_units"] // plan["nqb"]
        assert np.array_equal(split[:first_tail_bh], whole[:first_tail_bh])  # untouched tasks are bit-identical
    for bh in (0, B * H - 1):
        qs, ks, vs = orc.make_inputs(B, H, S, S, "bhsd", bh_range=range(bh, bh + 1))
        ref = orc.attention_fp32(qs, ks, vs, "bhsd").numpy()
        wabs = weighted_abs_v(qs, ks, vs, "bhsd").numpy()
        assert_parity(split[bh], ref, wabs, "rtne", f"split bh {bh}")
        assert_parity(whole[bh], ref, wabs, "rtne", f"whole bh {bh}")


def test_late_dominant_keys_force_the_exact_path(ma):
    """Scores of the last key block exceed everything before by hundreds of log2 units: the speculative
    softmax pass must notice (its exponentials would overflow) and redo the block on the exact path;
    and a slowly growing maximum exercises the deferred lazy rescale."""
    B, H, Sq, Skv = 1, 3, 384, 1024
    q, k, v = orc.make_inputs(B, H, Sq, Skv, "bhsd")
    kf = k.float()
    kf[:, 0, -128:] *= 40.0                                                          # head 0: late jump
    kf[:, 1] *= torch.linspace(0.2, 12.0, Skv).view(1, Skv, 1)                       # head 1: steady growth
    kf[:, 2, 300:428] *= 25.0                                                        # head 2: jump in the middle
    k = kf.to(torch.bfloat16)
    ref = orc.attention_fp32(q, k, v, "bhsd").numpy()
    wabs = weighted_abs_v(q, k, v, "bhsd").numpy()
    assert np.isfinite(ref).all()
    for mode, flags in (("rtne", 0), ("rtz", 0), ("rtne", _flags().FLAG_PRECISE_P)):
        got = gpu_forward(ma, q, k, v, "bhsd", mode, flags)
        # a handful of keys carries each row here: the few-keys bound applies, whatever Skv is
        assert_parity(got, ref, wabs, mode, f"late dominant keys {mode} flags {flags:#x}", skv=None, precise=flags != 0)


# ---- NaN / Inf --------------------------------------------------------------------------------------
@pytest.mark.parametrize("precise", [False, True], ids=["default", "precise"])
@pytest.mark.parametrize("mode", orc.ROUND_MODES)
def test_special_values_bit_and_position_exact(ma, mode, precise):
    """+Inf / -Inf / NaN planted in q, k or v (one tensor at a time, then all three)."""
    B, H, S = 1, 4, 1536
    flags = _flags().FLAG_PRECISE_P if precise else 0
    for which, kinds in (("q", (0, 1, 2)), ("k", (0, 1)), ("v", (0, 1, 2)), ("qkv", (0, 1, 2))):
        q, k, v = orc.make_inputs(B, H, S, S, "bshd")
        for name, t, seed in (("q", q, 11), ("k", k, 12), ("v", v, 13)):
            if name in which:
                orc.inject_specials(t, 2e-5, seed, kinds)
        got = gpu_forward(ma, q, k, v, "bshd", mode, flags)
        ref = orc.attention_fp32(q, k, v, "bshd").numpy()
        want = orc.round_bf16_bits(ref, mode)
        cls = orc.classify_special(want)
        assert cls.any(), "the case must contain non-finite outputs"
        if which != "qkv":
            assert (cls == 0).any(), "and finite ones"
        wabs = np.nan_to_num(weighted_abs_v(q, k, v, "bshd").numpy(), nan=0.0, posinf=0.0, neginf=0.0)
        assert_parity(got, ref, wabs, mode, f"specials in {which} {mode} precise={precise}", skv=S, precise=precise)
        nan = orc.classify_special(got) == 3
        assert np.all(got[nan] == 0x7FFF)  # canonical NaN in every mode
