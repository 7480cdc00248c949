"""The oracle against the reference's own fixtures and against itself (CPU only)."""
import hashlib
import os

import numpy as np
import pytest
import torch

from oracle import oracle as orc
from helpers import c_oracle_attention, load_c_oracle

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "basic_example.npz")


def _basic_inputs():
    """q, k, v of the reference's examples/basic.py:6-11 (seed 42, randn in bf16 on the CPU, in that order)."""
    g = np.load(GOLDEN)
    B, H, S, D = (int(x) for x in g["shape"])
    torch.manual_seed(int(g["seed"]))
    q = torch.randn(B, H, S, D, dtype=torch.bfloat16)
    k = torch.randn(B, H, S, D, dtype=torch.bfloat16)
    v = torch.randn(B, H, S, D, dtype=torch.bfloat16)

    def sha(t):
        return hashlib.sha256(t.contiguous().view(torch.int16).numpy().tobytes()).hexdigest()

    same = sha(q) == str(g["sha_q"]) and sha(k) == str(g["sha_k"]) and sha(v) == str(g["sha_v"])
    return g, q, k, v, same


def test_oracle_matches_reference_example_output():
    """attention_fp32 reproduces `ref` of examples/basic.py:16-17 as that script computed it."""
    g, q, k, v, same = _basic_inputs()
    if not same:
        pytest.skip("this torch build draws different randn values than the one that made the fixture")
    rows = g["rows"]
    out = orc.attention_fp32(q, k, v, "bhsd", q_block=256)
    got = out[0][:, rows, :].numpy()
    # per-slice, row-blocked evaluation changes the fp32 summation order inside the BLAS calls only
    np.testing.assert_allclose(got, g["ref_rows"], rtol=2e-5, atol=2e-6)
    full = orc.attention_fp32(q, k, v, "bhsd", q_block=1 << 20)
    np.testing.assert_allclose(full[0][:, rows, :].numpy(), g["ref_rows"], rtol=2e-5, atol=2e-6)
    # and the rounded outputs agree to the bit except where fp32 noise straddles a rounding boundary
    a = orc.round_bf16_bits(got, "rtne")
    b = orc.round_bf16_bits(g["ref_rows"], "rtne")
    assert np.count_nonzero(a != b) <= a.size // 500 and orc.ulp_distance(a, b).max() <= 1


def test_c_oracle_matches_torch_oracle():
    for layout, shape in (("bhsd", (1, 2, 70, 131)), ("bshd", (2, 3, 33, 64))):
        q, k, v = orc.make_inputs(shape[0], shape[1], shape[2], shape[3], layout)
        a = orc.attention_fp32(q, k, v, layout).numpy()
        b = c_oracle_attention(q, k, v, layout).numpy()
        np.testing.assert_allclose(a, b, rtol=3e-5, atol=3e-6)


def test_layouts_agree():
    q, k, v = orc.make_inputs(2, 3, 50, 77, "bhsd")
    a = orc.attention_fp32(q, k, v, "bhsd")
    qt, kt, vt = (t.transpose(1, 2).contiguous() for t in (q, k, v))
    b = orc.attention_fp32(qt, kt, vt, "bshd").transpose(1, 2)
    assert torch.equal(a, b)


# ---- rounding: known answers derived by hand from the bit formulas (csrc/attention_kernel.hip:110-145)
KAT = [
    # fp32 bits,   rtne,   rtna,   rtz
    (0x3F800000, 0x3F80, 0x3F80, 0x3F80),  # 1.0 exact
    (0x3F808000, 0x3F80, 0x3F81, 0x3F80),  # tie, even below: rtne down, rtna away
    (0x3F818000, 0x3F82, 0x3F82, 0x3F81),  # tie, odd below: rtne up to even
    (0x3F807FFF, 0x3F80, 0x3F80, 0x3F80),  # just under the tie
    (0x3F808001, 0x3F81, 0x3F81, 0x3F80),  # just over the tie
    (0xBF808000, 0xBF80, 0xBF81, 0xBF80),  # negative tie: away from zero grows the magnitude
    (0xBF818000, 0xBF82, 0xBF82, 0xBF81),
    (0x7F7FFFFF, 0x7F80, 0x7F80, 0x7F7F),  # largest finite: rounds to +Inf except under truncation
    (0x7F800000, 0x7F80, 0x7F80, 0x7F80),  # +Inf
    (0xFF800000, 0xFF80, 0xFF80, 0xFF80),  # -Inf
    (0x7FC00000, 0x7FFF, 0x7FFF, 0x7FFF),  # quiet NaN -> canonical
    (0xFFC00001, 0x7FFF, 0x7FFF, 0x7FFF),  # negative NaN -> canonical positive
    (0x7F800001, 0x7FFF, 0x7FFF, 0x7FFF),  # signalling NaN whose top 16 bits alone look like Inf
    (0x00000000, 0x0000, 0x0000, 0x0000),
    (0x80000000, 0x8000, 0x8000, 0x8000),  # -0 keeps its sign
    (0x00008000, 0x0000, 0x0001, 0x0000),  # subnormal tie
    (0x0000FFFF, 0x0001, 0x0001, 0x0000),
]


def test_rounding_known_answers():
    x = np.array([r[0] for r in KAT], dtype=np.uint32).view(np.float32)
    lib = load_c_oracle()
    for col, mode in enumerate(orc.ROUND_MODES, start=1):
        want = np.array([r[col] for r in KAT], dtype=np.uint16)
        assert np.array_equal(orc.round_bf16_bits(x, mode), want), mode
        dst = np.zeros(len(KAT), dtype=np.uint16)
        lib.oracle_round_bf16(x.ctypes.data, dst.ctypes.data, len(KAT), col - 1)
        assert np.array_equal(dst, want), f"C {mode}"


def test_rtne_equals_torch_cast_on_finite_values():
    rng = np.random.default_rng(1)
    u = rng.integers(0, 1 << 32, size=1 << 18, dtype=np.uint64).astype(np.uint32)
    x = u.view(np.float32)
    x = x[np.isfinite(x)]
    want = torch.from_numpy(x.copy()).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(orc.round_bf16_bits(x, "rtne"), want)


def test_rounding_properties_all_upper_halves():
    """Every 16-bit upper half with lower halves around the tie: ordering relations between the modes."""
    hi = np.arange(1 << 16, dtype=np.uint32) << 16
    for lo in (0x0000, 0x0001, 0x7FFF, 0x8000, 0x8001, 0xFFFF):
        x = (hi | lo).view(np.float32)
        fin = np.isfinite(x)
        z = orc.round_bf16_bits(x, "rtz")
        e = orc.round_bf16_bits(x, "rtne")
        a = orc.round_bf16_bits(x, "rtna")
        assert np.all((z[fin] & 0x8000) == (e[fin] & 0x8000))
        dz_e = (e[fin] & 0x7FFF).astype(np.int64) - (z[fin] & 0x7FFF)
        dz_a = (a[fin] & 0x7FFF).astype(np.int64) - (z[fin] & 0x7FFF)
        assert set(np.unique(dz_e)) <= {0, 1} and set(np.unique(dz_a)) <= {0, 1}
        if lo != 0x8000:
            assert np.array_equal(e[fin], a[fin])  # the two nearest modes differ on ties only
        nan = np.isnan(x)
        assert np.all(z[nan] == 0x7FFF) and np.all(e[nan] == 0x7FFF) and np.all(a[nan] == 0x7FFF)


def test_ulp_distance_and_ordinals():
    b = np.array([0x0000, 0x8000, 0x0001, 0x8001, 0x3F80, 0x3F81, 0xBF80], dtype=np.uint16)
    o = orc.bf16_ordinal(b)
    assert o[0] == o[1] == 0 and o[2] == 1 and o[3] == -1
    assert orc.ulp_distance(b[4:5], b[5:6])[0] == 1
    assert orc.ulp_distance(b[2:3], b[3:4])[0] == 2


def test_special_value_propagation_rules():
    """NaN / Inf travel through the oracle as IEEE arithmetic dictates (the rules the GPU tests rely on)."""
    S = 64
    q, k, v = orc.make_inputs(1, 1, S, S, "bhsd")

    def run(qq, kk, vv):
        return orc.attention_bf16_bits(qq, kk, vv, "bhsd", "rtne")[0, 0]

    def setbits(t, idx, bits):
        t = t.clone()
        t.view(torch.int16)[idx] = np.int16(np.uint16(bits).view(np.int16))
        return t

    out = run(setbits(q, (0, 0, 3, 7), 0x7FC0), k, v)  # NaN in q row 3 -> row 3 all NaN, canonical
    assert np.all(out[3] == 0x7FFF) and not np.any(orc.classify_special(np.delete(out, 3, axis=0)))
    out = run(q, setbits(k, (0, 0, 5, 9), 0x7FC0), v)  # NaN in k -> every row NaN
    assert np.all(out == 0x7FFF)
    out = run(q, k, setbits(v, (0, 0, 5, 9), 0x7FC0))  # NaN in v[5, 9] -> column 9 NaN
    assert np.all(out[:, 9] == 0x7FFF) and not np.any(orc.classify_special(np.delete(out, 9, axis=1)))
    out = run(q, k, setbits(v, (0, 0, 5, 9), 0x7F80))  # +Inf in v -> column 9 +Inf
    assert np.all(out[:, 9] == 0x7F80)
    out = run(q, setbits(k, (0, 0, 5, 9), 0x7F80), v)  # +Inf in k[5, 9]: rows with q[:, 9] > 0 are NaN
    pos = (q[0, 0, :, 9].float() > 0).numpy()
    assert np.all(out[pos] == 0x7FFF) and not np.any(orc.classify_special(out[~pos]))


def test_inject_specials_writes_exact_patterns():
    t = torch.zeros(4, 1000, dtype=torch.bfloat16)
    pos = orc.inject_specials(t, 0.01, seed=7)
    bits = orc.bf16_tensor_to_bits(t).reshape(-1)
    assert len(pos) == 40 and len(np.unique(pos)) == 40
    assert set(np.unique(bits[pos])) == {0x7F80, 0xFF80, 0x7FC0}
    assert np.count_nonzero(bits) == 40


def test_slice_seeding_is_independent_of_sharding():
    q, k, v = orc.make_inputs(2, 3, 16, 24, "bhsd")
    q2, k2, v2 = orc.make_inputs(2, 3, 16, 24, "bhsd", bh_range=range(2, 5))
    assert torch.equal(q.view(1, 6, 16, 128)[:, 2:5], q2)
    assert torch.equal(v.view(1, 6, 24, 128)[:, 2:5], v2)
