"""CPU oracle for the MLA absorbed-decode operators -- TEST INFRASTRUCTURE ONLY.

Only tests/ may import this module; the product never does.

What it restates, and from where in the reference:

* the operator: the fp32 reference of the reference's own test (tests/test_mla_decode.py:52-68): for request b
  and draft position t, with k = dequantised kv[b] * kv_scale,
      score = (q_lat[b,t] @ k[:end,:512].T + q_pe[b,t] @ k[:end,512:].T) * scale,  end = seq_len[b] - q_len + t + 1
      out   = softmax(score) @ k[:end,:512]
* the cache formats: `decode_e4m3fnuz` (AMD's e4m3-fnuz as the reference stores it, csrc/mla_decode_a16w8.hip
  unpack: bias 8, no infinities, 0x80 = NaN) and `decode_e4m3fn` (OCP e4m3: bias 7, 0x7F / 0xFF = NaN);
* the paged pool: token i of request b lives in slot kv_indices[kv_indptr[b] + i], one token per slot
  (csrc/mla_decode_a16w8_api.cpp:103-112).

Pinning: the decode tables are checked against torch's float8 dtypes for all 256 codes; the operator formula is
the one the reference's test asserts against with rel-L2 < 3e-3, and that bar is the parity bar of the GPU tests
(the reference's HIP kernels cannot run here, so there are no reference outputs to compare bit for bit).
"""
from __future__ import annotations

import numpy as np

LAT, ROPE, FUSED = 512, 64, 576
REL_L2 = 3e-3  # tests/test_mla_decode.py:25


def decode_e4m3fnuz() -> np.ndarray:
    """Value of each of the 256 byte codes of e4m3-fnuz (fp32; NaN for 0x80)."""
    out = np.zeros(256, np.float32)
    for b in range(256):
        s, e, m = b >> 7, (b >> 3) & 0xF, b & 7
        v = (m / 8.0) * 2.0 ** -7 if e == 0 else (1 + m / 8.0) * 2.0 ** (e - 8)
        out[b] = -v if s else v
    out[0x80] = np.nan
    return out


def decode_e4m3fn() -> np.ndarray:
    """Value of each of the 256 byte codes of OCP e4m3 (fp32; NaN for 0x7F and 0xFF)."""
    out = np.zeros(256, np.float32)
    for b in range(256):
        s, e, m = b >> 7, (b >> 3) & 0xF, b & 7
        v = (m / 8.0) * 2.0 ** -6 if e == 0 else (1 + m / 8.0) * 2.0 ** (e - 7)
        out[b] = -v if s else v
    out[0x7F] = out[0xFF] = np.nan
    return out


def mla_decode(q_lat, q_pe, kv_bytes, seq_lens, scale: float, kv_scale: float, fmt: str = "fnuz") -> np.ndarray:
    """q_lat [B, q_len, H, 512], q_pe [B, q_len, H, 64] fp32; kv_bytes [B, S, 576] uint8; seq_lens: B ints.

    Returns out [B, q_len, H, 512] fp32.
    """
    table = decode_e4m3fnuz() if fmt == "fnuz" else decode_e4m3fn()
    q_lat, q_pe = np.asarray(q_lat, np.float64), np.asarray(q_pe, np.float64)
    B, q_len, H, _ = q_lat.shape
    out = np.zeros((B, q_len, H, LAT), np.float32)
    for b in range(B):
        k = table[np.asarray(kv_bytes[b], np.uint8)].astype(np.float64) * kv_scale
        for t in range(q_len):
            end = int(seq_lens[b]) - q_len + t + 1
            if end <= 0:
                continue
            score = (q_lat[b, t] @ k[:end, :LAT].T + q_pe[b, t] @ k[:end, LAT:].T) * scale
            score -= score.max(axis=-1, keepdims=True)
            p = np.exp(score)
            out[b, t] = (p @ k[:end, :LAT]) / p.sum(axis=-1, keepdims=True)
    return out


def gather_pool(pool_bytes, kv_indices, kv_indptr, seq_lens) -> list:
    """Per-request [seq_len, 576] uint8 arrays out of a [slots, 576] pool."""
    return [np.asarray(pool_bytes)[np.asarray(kv_indices[kv_indptr[b]: kv_indptr[b] + seq_lens[b]])] for b in range(len(seq_lens))]


def rel_l2(out, ref) -> float:
    out, ref = np.asarray(out, np.float64), np.asarray(ref, np.float64)
    return float(np.linalg.norm(out - ref) / np.linalg.norm(ref))
