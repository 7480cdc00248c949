"""CPU oracle for `moonmath_attention.forward_lite` -- TEST INFRASTRUCTURE ONLY.

Only tests/ and __graft_entry__.smoke() may import this module; the product never does.

What it restates, and from where in the reference:

* the skip-list format and its walk (csrc/attention_kernel.hip:629-664 read cursor; moonmath_attention/lite.py:108-128
  seed): `ListCursor`, `kept_blocks`;
* the write-list emitter and the must-do ranges (hip:666-713, final length hip:1081-1084): `ListEmitter`, `MustDo`;
* the vote (hip:981-1004): a group of query rows keeps a key block when some live row's block maximum, in log2
  units, exceeds that row's reference maximum plus `threshold`; the first processed block of a task is always
  kept; a group that votes "skip" adds nothing for the block; the block leaves the written list when every
  group of the task skipped it and no must-do range pins it;
* the lazily moved reference maximum (hip:390-441, RescaleThreshold): it moves, for all rows of a group, when
  some row's block maximum exceeds it by more than tau = 8;
* the longest-first order (hip:1296-1347): `lpt_order`.

Geometry is that of the B200 kernel, not of the reference's MI300X kernel: 256 query rows per list row
(reference 384), votes per 32 rows (reference 48), key blocks of 64 (same), processed two at a time: the second
block of a pair is judged against the reference maximum as it stood before the pair (for the first pair of a
task: against the first block's own maximum).

Pinning: the list format is pinned by the values the reference states in text -- the seed row
[2, ktiles - 1, -1] (lite.py:124-127), the planner's worked example "row = [4, 9, 5, 20, 18] -> kept 6"
(hip:1318-1319) and the kept-block count of its tests (tests/test_attention.py:145-150); tests/test_lite_oracle.py
checks them.  The numerical behaviour (which blocks a given input keeps, the approximate output) is
**parity unpinned**: the reference's HIP kernel cannot be built or run here, it ships no golden lists, and its
tile geometry differs, so its lists are not comparable block for block.  The properties its tests assert
(tests/test_attention.py:153-214) are the portable part and are asserted on the GPU in tests/test_gpu_lite.py.
"""

from __future__ import annotations

import math

import numpy as np

KEY_BLOCK = 64
QUERY_BLOCK = 256
VOTE_ROWS = 32
TAU = 8.0
SCALE_LOG2E = np.float32(1.4426950408889634 / math.sqrt(128.0))


class ListCursor:
    """Read cursor over one row [len, m_1, ..., m_len] (hip:645-664)."""

    def __init__(self, row, phase: int):
        self.row = [int(x) for x in row]
        self.step = 1 if phase else -1
        self.idx = self.row[0]
        self.block = -1
        self.end = 0
        if self.idx >= 2:
            self._open()

    def _open(self):
        self.block = self.row[self.idx] + self.step
        self.end = self.row[self.idx - 1] + self.step
        self.idx -= 2

    def advance(self) -> bool:
        """Move to the next kept block; True when the block just left closed its range."""
        nxt = self.block + self.step
        if (nxt < self.end) if self.step > 0 else (nxt > self.end):
            self.block = nxt
            return False
        if self.idx >= 2:
            self._open()
        else:
            self.block = -1
        return True


def walk(row, phase: int):
    """[(block, closes_its_range), ...] in walk order."""
    cur = ListCursor(row, phase)
    out = []
    while cur.block >= 0:
        b = cur.block
        out.append((b, cur.advance()))
    return out


def kept_blocks(row) -> int:
    """Key blocks a row names (tests/test_attention.py:145-150: sum of |hi - lo| over the pairs)."""
    r = [int(x) for x in row]
    return sum(abs(r[i] - r[i - 1]) for i in range(r[0], 1, -2))


def seed_row(ktiles: int):
    """Compute-all row for a first call with phase 1 (lite.py:124-127)."""
    return [2, ktiles - 1, -1] + [0] * (ktiles - 1)


class MustDo:
    """Global force-compute ranges [len, s0, e0, ...], walked monotonically (hip:676-691)."""

    def __init__(self, lst, phase: int):
        self.lst = None if lst is None else [int(x) for x in lst]
        self.step = 1 if phase else -1
        self.ranges = (self.lst[0] >> 1) if self.lst is not None and self.lst[0] > 0 else 0
        self.cur = 0 if self.step > 0 else self.ranges - 1

    def forced(self, block: int) -> bool:
        if self.ranges == 0:
            return False
        if self.step > 0:
            while self.cur < self.ranges and block >= self.lst[2 + 2 * self.cur]:
                self.cur += 1
        else:
            while self.cur >= 0 and block < self.lst[1 + 2 * self.cur]:
                self.cur -= 1
        return 0 <= self.cur < self.ranges and self.lst[1 + 2 * self.cur] <= block < self.lst[2 + 2 * self.cur]


class ListEmitter:
    """Write-list emitter (hip:703-713): a marker at every skip <-> compute change, a closing marker when a range
    of the read list ends while computing; slot 0 receives the number of markers."""

    def __init__(self, width: int, phase: int):
        self.row = [0] * width
        self.step = 1 if phase else -1
        self.idx = 1
        self.skip = True

    def _put(self, marker: int):
        if self.idx < len(self.row):
            self.row[self.idx] = marker
            self.idx += 1

    def record(self, block: int, skip_block: bool, range_end: bool):
        if skip_block != self.skip:
            self._put(block)
            self.skip = skip_block
        if range_end:
            self.skip = True
            if not skip_block:
                self._put(block + self.step)

    def finish(self):
        self.row[0] = self.idx - 1
        return self.row


def lpt_order(read_list: np.ndarray, phase: int) -> list[int]:
    """Tasks sorted by kept blocks, 256 buckets, heaviest bucket first (hip:1296-1347); order inside a bucket is
    unspecified there (atomics) -- here: ascending task index."""
    rows = read_list.reshape(-1, read_list.shape[-1])
    ktiles = rows.shape[1] - 2
    step = 1 if phase else -1

    def bucket(row):
        kept = 0
        r = [int(x) for x in row]
        for i in range(r[0], 1, -2):
            n = (r[i - 1] - r[i]) * step
            kept += max(n, 1)
        return min(kept * 256 // (ktiles + 1), 255)

    keyed = sorted(range(rows.shape[0]), key=lambda t: (-bucket(rows[t]), t))
    return keyed


def _task(q, k, v, row, threshold, phase, must_do, write_width):
    """One task: q [rows <= 256, 128] fp32, k / v [Skv, 128] fp32.  Returns (out [rows, 128] fp32, written row or None)."""
    rows, skv = q.shape[0], k.shape[0]
    x_all = (q @ k.T).astype(np.float32) * SCALE_LOG2E  # scores in log2 units
    blocks = walk(row, phase)
    out = np.zeros((rows, 128), np.float32)
    if not blocks:
        return out, None
    groups = [(g, min(g + VOTE_ROWS, rows)) for g in range(0, QUERY_BLOCK, VOTE_ROWS)]
    m_ref = np.zeros(rows, np.float32)
    l_run = np.zeros(rows, np.float32)
    acc = np.zeros((rows, 128), np.float32)
    emit = ListEmitter(write_width, phase)
    pin = MustDo(must_do, phase)
    thr = np.float32(threshold)
    for j in range(0, len(blocks), 2):
        pair = blocks[j:j + 2]
        first = j == 0
        spans = [(b * KEY_BLOCK, min(b * KEY_BLOCK + KEY_BLOCK, skv)) for b, _ in pair]
        skip_all = [True] * len(pair)
        for g0, g1 in groups:
            if g0 >= rows:
                # a group without live rows never asks to keep a block; the first block is kept regardless
                if first:
                    skip_all[0] = False
                continue
            mx = []
            for lo, hi in spans:
                xs = x_all[g0:g1, lo:hi] if lo < hi else np.full((g1 - g0, 0), -np.inf, np.float32)
                mx.append(np.nanmax(np.where(np.isnan(xs), -np.inf, xs), axis=1, initial=-np.inf).astype(np.float32))
            ref = m_ref[g0:g1]
            keep = [first or bool(np.any((mx[0] - ref) > thr))]
            if len(pair) > 1:
                ref1 = np.where(np.isneginf(mx[0]), np.float32(0), mx[0]) if first else ref
                keep.append(bool(np.any((mx[1] - ref1) > thr)))
            for i, kp in enumerate(keep):
                if kp:
                    skip_all[i] = False
            m_blk = np.full(g1 - g0, -np.inf, np.float32)
            for i, kp in enumerate(keep):
                if kp:
                    m_blk = np.maximum(m_blk, mx[i])
            if first:
                m_ref[g0:g1] = np.where(np.isneginf(m_blk), np.float32(0), m_blk)
            elif np.any((m_blk - ref) > np.float32(TAU)):
                m_new = np.maximum(ref, m_blk)
                alpha = np.exp2(ref - m_new).astype(np.float32)
                acc[g0:g1] *= alpha[:, None]
                l_run[g0:g1] *= alpha
                m_ref[g0:g1] = m_new
            for i, kp in enumerate(keep):
                lo, hi = spans[i]
                if not kp or lo >= hi:
                    continue
                p = np.exp2(x_all[g0:g1, lo:hi] - m_ref[g0:g1, None]).astype(np.float32)
                l_run[g0:g1] += p.sum(axis=1, dtype=np.float32)
                acc[g0:g1] += p @ v[lo:hi]
        last_pair = j + 2 >= len(blocks)
        for i, (b, closes) in enumerate(pair):
            emit.record(b, skip_all[i] and not pin.forced(b), closes or (last_pair and i == len(pair) - 1))
    with np.errstate(divide="ignore", invalid="ignore"):
        out = acc / l_run[:, None]
    return out.astype(np.float32), emit.finish()


def forward_lite(q, k, v, read_list, threshold: float, phase: int, must_do=None, layout: str = "bhsd"):
    """q, k, v: float32 / bf16-valued numpy arrays in `layout`; read_list [B, H, qtiles, ktiles + 2] int16.

    Returns (out fp32 in `layout`, write_list int16 like read_list; rows of tasks with an empty read list stay 0).
    """
    q, k, v = (np.asarray(t, np.float32) for t in (q, k, v))
    if layout == "bshd":
        q, k, v = (t.transpose(0, 2, 1, 3) for t in (q, k, v))
    B, H, Sq, _ = q.shape
    read_list = np.asarray(read_list)
    qtiles, width = read_list.shape[2], read_list.shape[3]
    assert qtiles == (Sq + QUERY_BLOCK - 1) // QUERY_BLOCK
    out = np.zeros((B, H, Sq, 128), np.float32)
    write = np.zeros_like(read_list)
    for b in range(B):
        for h in range(H):
            for t in range(qtiles):
                r0, r1 = t * QUERY_BLOCK, min((t + 1) * QUERY_BLOCK, Sq)
                o, row = _task(q[b, h, r0:r1], k[b, h], v[b, h], read_list[b, h, t], threshold, phase, must_do, width)
                out[b, h, r0:r1] = o
                if row is not None:
                    write[b, h, t] = np.asarray(row, np.int16)
    if layout == "bshd":
        out = out.transpose(0, 2, 1, 3)
    return np.ascontiguousarray(out), write
