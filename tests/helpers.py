"""Shared helpers of the test-suite (test infrastructure; may use oracle/)."""
from __future__ import annotations

import ctypes
import os

import numpy as np
import torch

from oracle import oracle as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load_c_oracle() -> ctypes.CDLL:
    lib = ctypes.CDLL(os.path.join(ROOT, "oracle", "liboracle.so"))
    lib.oracle_attention_f32.restype = ctypes.c_int
    lib.oracle_attention_f32.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int] * 8
    lib.oracle_round_bf16.restype = None
    lib.oracle_round_bf16.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
    return lib


def c_oracle_attention(q, k, v, layout: str, rows: tuple[int, int] | None = None, threads: int = 8) -> torch.Tensor:
    lib = load_c_oracle()
    sax, hax = (1, 2) if layout == "bshd" else (2, 1)
    B, H, Sq, Skv = q.size(0), q.size(hax), q.size(sax), k.size(sax)
    out = torch.zeros(q.shape, dtype=torch.float32)
    qb, kb, vb = (t.contiguous().view(torch.int16) for t in (q, k, v))
    r0, r1 = rows if rows is not None else (0, Sq)
    rc = lib.oracle_attention_f32(qb.data_ptr(), kb.data_ptr(), vb.data_ptr(), out.data_ptr(), B, H, Sq, Skv,
                                  1 if layout == "bshd" else 0, r0, r1, threads)
    assert rc == 0
    return out


def weighted_abs_v(q, k, v, layout: str) -> torch.Tensor:
    """softmax(q k^T / sqrt(D)) @ |v| in fp32: the scale of the error that rounding P to bf16 can cause."""
    return orc.attention_fp32(q, k, v.abs(), layout)


def ulp_of(x: np.ndarray) -> np.ndarray:
    """Size of one bf16 unit in the last place at |x| (fp32 array), with the subnormal floor."""
    ax = np.abs(x).astype(np.float32)
    e = np.floor(np.log2(np.maximum(ax, np.float32(2.0 ** -126))))
    return np.exp2(e - 7).astype(np.float64)


# How far the rounding rule alone may put the stored value from the exact one, in ulps.
MODE_ULPS = {"rtne": 0.5, "rtna": 0.5, "rtz": 1.0}


def p_term_for(skv: int | None, precise: bool = False) -> float:
    """Factor of wabs in the parity bound.

    Rounding a probability to bf16 moves it by at most 2^-8 of itself (2^-9 on average over the
    binade).  With few keys the errors of a row can line up, so the rigorous 2^-8 is the bound; from
    128 keys on the sum behaves like the random sum it is and 2^-9 holds with room to spare (a CPU
    emulation of bf16 probabilities on the test shapes peaks at 2^-8.8 for 16 keys, 2^-9.8 for 128 and
    more).  The precise mode carries the probabilities to 16 bits: 2^-15 covers them, the approximate
    exponential (2 ulp of fp32) and the fp32 sums.
    """
    if precise:
        return 2.0 ** -15
    return 2.0 ** -8 if skv is None or skv < 128 else 2.0 ** -9


def assert_parity(got_bits: np.ndarray, ref32: np.ndarray, wabs32: np.ndarray, mode: str, what: str = "",
                  skv: int | None = None, precise: bool = False) -> dict:
    """The parity criterion of the GPU tests.

    * NaN / Inf: bit- and position-identical with the oracle's rounded output.
    * finite: |got - ref| <= (MODE_ULPS + 0.5) * ulp(ref) + p_term * wabs
      - the first term is the final rounding (plus half an ulp of slack for a
        value that sits next to a rounding boundary),
      - the second bounds what rounding the probabilities to bf16 (relative 2^-9
        each, the reference does the same: csrc/attention_kernel.hip:446-448) can
        move an output by, wabs = sum_j p_j |v_j| / l; p_term = p_term_for(skv, precise).
    Returns the comparison report (ULP histograms, plain and gated to |ref| >= 2^-7 wabs).
    """
    want_bits = orc.round_bf16_bits(ref32, mode)
    rep = orc.compare_bits(got_bits, want_bits, ref32, wabs32)
    assert rep["special_mismatch"] == 0, f"{what}: NaN/Inf mismatch {rep}"
    g = got_bits.reshape(-1)
    fin = orc.classify_special(g) == 0
    fin &= orc.classify_special(want_bits.reshape(-1)) == 0
    gf = orc.bf16_bits_to_f32(g[fin]).astype(np.float64)
    rf = ref32.reshape(-1)[fin].astype(np.float64)
    wa = wabs32.reshape(-1)[fin].astype(np.float64)
    tol = (MODE_ULPS[mode] + 0.5) * ulp_of(rf) + p_term_for(skv, precise) * wa
    bad = np.abs(gf - rf) > tol
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.size} finite outputs outside tolerance; {rep}"
    return rep


def reference_peaked_inputs():
    """The q, k, v [B, S, H, 128] (bshd) of the reference's skip-list test, rebuilt here and verified against the
    hashes that tests/golden/make_golden_lite.py took from the reference's own generator
    (tests/test_attention.py:118-138: global seed 7, three fp32 draws, head h keeps its first (h + 1) * 64 keys
    at scale 2 and the rest at 0.05, then bf16).  Returns (q, k, v, fixture) or None when this torch build
    draws other values than the one that made the fixture."""
    import hashlib

    g = np.load(os.path.join(ROOT, "tests", "golden", "lite_reference.npz"))
    B, S, H, D = (int(x) for x in g["peaked_shape"])
    state = torch.get_rng_state()
    try:
        torch.manual_seed(7)
        q = torch.randn(B, S, H, D)
        k = torch.randn(B, S, H, D)
        v = torch.randn(B, S, H, D)
    finally:
        torch.set_rng_state(state)
    scale = torch.full((H, S), 0.05)
    for h in range(H):
        scale[h, : (h + 1) * 64] = 2.0
    k = k * scale.t().view(1, S, H, 1)
    q, k, v = (t.to(torch.bfloat16) for t in (q, k, v))
    sha = [hashlib.sha256(t.contiguous().view(torch.int16).numpy().tobytes()).hexdigest() for t in (q, k, v)]
    if sha != [str(x) for x in g["peaked_sha"]]:
        return None
    return q, k, v, g
