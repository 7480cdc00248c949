"""CPU oracle for `moonmath_attention.forward` -- TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and the cpu_baseline / reference legs of
bench.py may import this module.  The product (amd-kernels_b200/) never does.

What it restates, and from where in the reference:

* the math: `softmax(q.float() @ k.float().transpose(-1, -2) / D**0.5, dim=-1) @ v.float()`
  -- the reference's own fp32 oracle, examples/basic.py:16-17.  `attention_fp32`
  evaluates exactly that expression with torch on the CPU, per (batch, head)
  slice and per block of query rows so that the S x S score matrix never
  exists for long sequences.
* the fp32 -> bf16 rounding rules of the kernel's final store,
  csrc/attention_kernel.hip:110-145:
      RTNE  (u + 0x7FFF + ((u >> 16) & 1)) >> 16
      RTNA  (u + 0x8000) >> 16
      RTZ    u >> 16
  with NaN -> 0x7FFF in every mode (hip:117-123, :135-139 for RTNE / RTNA;
  README.md:65-68 states it for all three).
* the layouts: "bhsd" [B,H,S,D] and "bshd" [B,S,H,D] (csrc/attention_kernel.hip:554-566).

Pinning: `tests/golden/basic_example.npz` holds outputs of the reference's own
examples/basic.py oracle lines, produced by running that file in this
container with a stand-in for the (unbuildable) GPU extension; see
tests/golden/make_golden.py.  The reference ships no golden vectors for the
rounding modes, NaN/Inf handling or ragged lengths (its tests compare against
bf16 SDPA at rtol = atol = 0.05, tests/test_attention.py:68-85), and its HIP
kernel cannot be compiled or run here, so those parts are pinned only by the
formulae cited above: bit-level parity with the reference binary is unpinned.
"""

from __future__ import annotations

import math

import numpy as np
import torch

HEAD_DIM = 128
ROUND_MODES = ("rtne", "rtna", "rtz")
BASE_SEED = 42  # the reference's tests and example seed with 42 (tests/test_attention.py:38, examples/basic.py:7)


# ---------------------------------------------------------------------------
# rounding
# ---------------------------------------------------------------------------
def round_bf16_bits(x: np.ndarray | torch.Tensor, mode: str) -> np.ndarray:
    """fp32 array -> uint16 bf16 bit patterns under `mode`; NaN -> 0x7FFF."""
    if isinstance(x, torch.Tensor):
        x = x.detach().cpu().contiguous().numpy()
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    if mode == "rtne":
        r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    elif mode == "rtna":
        r = (u + 0x8000) >> 16
    elif mode == "rtz":
        r = u >> 16
    else:
        raise ValueError(f"unknown rounding mode {mode!r}")
    r = (r & 0xFFFF).astype(np.uint16)
    r[np.isnan(x)] = 0x7FFF
    return r


def bits_to_bf16_tensor(bits: np.ndarray) -> torch.Tensor:
    """uint16 bit patterns -> torch.bfloat16 tensor (no float conversion on the way)."""
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16).copy()).view(torch.bfloat16)


def bf16_tensor_to_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def bf16_ordinal(bits: np.ndarray) -> np.ndarray:
    """Maps bf16 bit patterns to integers that are monotone in the value (+0 and -0 coincide)."""
    b = bits.astype(np.int64)
    mag = b & 0x7FFF
    return np.where(b & 0x8000, -mag, mag)


def ulp_distance(a_bits: np.ndarray, b_bits: np.ndarray) -> np.ndarray:
    """|ordinal(a) - ordinal(b)| in bf16 units of least precision (meaningful for finite values)."""
    return np.abs(bf16_ordinal(a_bits) - bf16_ordinal(b_bits))


def classify_special(bits: np.ndarray) -> np.ndarray:
    """0 finite, 1 +Inf, 2 -Inf, 3 NaN."""
    out = np.zeros(bits.shape, dtype=np.uint8)
    mag = bits & 0x7FFF
    out[(mag == 0x7F80) & ((bits & 0x8000) == 0)] = 1
    out[(mag == 0x7F80) & ((bits & 0x8000) != 0)] = 2
    out[mag > 0x7F80] = 3
    return out


# ---------------------------------------------------------------------------
# the attention math
# ---------------------------------------------------------------------------
def _to_bhsd(t: torch.Tensor, layout: str) -> torch.Tensor:
    if layout == "bhsd":
        return t
    if layout == "bshd":
        return t.transpose(1, 2)
    raise ValueError(f"unknown layout {layout!r}")


def attention_fp32(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, layout: str = "bhsd",
                   q_block: int = 1024, rows: slice | None = None) -> torch.Tensor:
    """fp32 softmax(q k^T / sqrt(D)) v on the CPU, returned in `layout` as float32.

    `rows` restricts the query rows that are computed (a slice along the
    sequence axis); the result then has that many rows.
    """
    qh, kh, vh = (_to_bhsd(t, layout) for t in (q, k, v))
    if rows is not None:
        qh = qh[:, :, rows, :]
    B, H, Sq, D = qh.shape
    out = torch.empty(B, H, Sq, D, dtype=torch.float32)
    for b in range(B):
        for h in range(H):
            kf = kh[b, h].float()
            vf = vh[b, h].float()
            kt = kf.transpose(-1, -2).contiguous()
            for r0 in range(0, Sq, q_block):
                qf = qh[b, h, r0:r0 + q_block].float()
                # examples/basic.py:17, verbatim in structure
                out[b, h, r0:r0 + q_block] = torch.softmax(qf @ kt / (D ** 0.5), dim=-1) @ vf
    return out if layout == "bhsd" else out.transpose(1, 2).contiguous()


def attention_bf16_bits(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, layout: str = "bhsd",
                        round_mode: str = "rtne", **kw) -> np.ndarray:
    """Oracle output as bf16 bit patterns (uint16) in `layout`."""
    return round_bf16_bits(attention_fp32(q, k, v, layout, **kw), round_mode)


# ---------------------------------------------------------------------------
# seeded inputs
# ---------------------------------------------------------------------------
def slice_seed(bh: int, which: int, base: int = BASE_SEED) -> int:
    """Seed of one [S, 128] slice: which = 0 q, 1 k, 2 v.  Independent of how slices are spread over GPUs."""
    return base * 1000003 + 3 * bh + which


def make_slice(seq: int, bh: int, which: int, base: int = BASE_SEED) -> torch.Tensor:
    """One (batch, head) slice [seq, 128]: N(0,1) drawn in fp32, then cast to bf16."""
    g = torch.Generator(device="cpu")
    g.manual_seed(slice_seed(bh, which, base))
    return torch.randn(seq, HEAD_DIM, generator=g, dtype=torch.float32).to(torch.bfloat16)


def make_inputs(batch: int, heads: int, seq_q: int, seq_kv: int, layout: str, base: int = BASE_SEED,
                bh_range: range | None = None):
    """q, k, v for the given shape; with `bh_range` only those (batch*heads) slices, stacked as a batch of 1."""
    bhs = list(bh_range) if bh_range is not None else list(range(batch * heads))

    def build(seq: int, which: int) -> torch.Tensor:
        sl = torch.stack([make_slice(seq, bh, which, base) for bh in bhs])  # [n, S, D]
        if bh_range is not None:
            t = sl.unsqueeze(0)  # [1, n, S, D]
        else:
            t = sl.view(batch, heads, seq, HEAD_DIM)
        return t.contiguous() if layout == "bhsd" else t.transpose(1, 2).contiguous()

    return build(seq_q, 0), build(seq_kv, 1), build(seq_kv, 2)


SPECIAL_BITS = (0x7F80, 0xFF80, 0x7FC0)  # +Inf, -Inf, NaN


def inject_specials(t: torch.Tensor, density: float, seed: int, kinds=(0, 1, 2)) -> np.ndarray:
    """Overwrites round(density * numel) seeded positions of a bf16 tensor, in place, with
    +Inf / -Inf / NaN bit patterns (cycled over `kinds`, indices into SPECIAL_BITS).
    Written through an int16 view: no float cast touches the patterns.  Returns the flat positions."""
    n = t.numel()
    count = max(1, int(round(density * n)))
    rng = np.random.default_rng(seed)
    pos = np.unique(rng.integers(0, n, size=2 * count + 16))
    rng.shuffle(pos)
    pos = pos[:count]
    flat = t.view(torch.int16).view(-1)
    vals = np.array([SPECIAL_BITS[kinds[i % len(kinds)]] for i in range(len(pos))], dtype=np.uint16)
    flat[torch.from_numpy(pos.astype(np.int64))] = torch.from_numpy(vals.view(np.int16))
    return pos


# ---------------------------------------------------------------------------
# comparison report
# ---------------------------------------------------------------------------
GATE = 2.0 ** -7  # an output counts as "not a cancellation residue" when |oracle| >= GATE * sum_j p_j |v_j| / l


def compare_bits(got: np.ndarray, want: np.ndarray, want_f32: np.ndarray | None = None,
                 row_scale: np.ndarray | None = None) -> dict:
    """Statistics of a bf16 result against the oracle's bf16 bits.

    special_mismatch counts positions where either side is NaN/Inf and the bit
    patterns differ (these must be bit- and position-identical); the ULP figures
    cover the positions where both are finite.

    With `row_scale` (= softmax(q k^T / sqrt(D)) @ |v| in fp32, the magnitude the terms of an output had
    before they cancelled) the report also carries the same histogram restricted to outputs that are not
    cancellation residues, |oracle| >= GATE * row_scale: `gated_n`, `gated_max_ulp`, `gated_frac_gt1ulp`.
    An output far below its row scale carries an absolute error that is many units of *its own* last
    place whatever the kernel does; the gated figures are the ones a precision change moves.
    """
    got = got.reshape(-1)
    want = want.reshape(-1)
    cg, cw = classify_special(got), classify_special(want)
    special = (cg != 0) | (cw != 0)
    special_mismatch = int(np.count_nonzero(special & (got != want)))
    fin = ~special
    d = ulp_distance(got[fin], want[fin])
    rep = {
        "n": int(got.size),
        "n_finite": int(np.count_nonzero(fin)),
        "n_special": int(np.count_nonzero(special)),
        "special_mismatch": special_mismatch,
        "max_ulp": int(d.max()) if d.size else 0,
        "frac_gt1ulp": float(np.count_nonzero(d > 1) / max(1, d.size)),
        "frac_exact": float(np.count_nonzero(d == 0) / max(1, d.size)),
    }
    gf, wf = bf16_bits_to_f32(got[fin]), bf16_bits_to_f32(want[fin])
    if want_f32 is not None:
        wf = want_f32.reshape(-1)[fin]
    err = np.abs(gf.astype(np.float64) - wf.astype(np.float64))
    rep["max_abs_err"] = float(err.max()) if err.size else 0.0
    rep["rmse"] = float(math.sqrt(float((err ** 2).mean()))) if err.size else 0.0
    if row_scale is not None and want_f32 is not None:
        scale = np.abs(np.asarray(row_scale, dtype=np.float64).reshape(-1)[fin])
        keep = np.isfinite(scale) & (np.abs(wf.astype(np.float64)) >= GATE * scale)
        dg = d[keep]
        rep["gated_n"] = int(dg.size)
        rep["gated_max_ulp"] = int(dg.max()) if dg.size else 0
        rep["gated_frac_gt1ulp"] = float(np.count_nonzero(dg > 1) / max(1, dg.size))
    return rep
