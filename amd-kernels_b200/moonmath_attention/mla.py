"""MLA (DeepSeek-V3) absorbed-decode attention on B200: bf16 queries against an fp8 KV cache ("A16W8").

The eight entry points of the reference's module (moonmath_attention/mla.py:41-186; argument checks of
csrc/mla_decode_a16w8_api.cpp:40-150 and csrc/mla_decode_a16w8_multiq_api.cpp:40-150), same names, argument
order, domains and exception types.  All of them run one kernel (`ma_mla_decode_a16w8` of the C ABI): the
reference's split into a q_len = 1 CTA shape and a resident draft window is an MI300X tuning choice, not part of
the interface; the domains (q_len 1..8 here, 4..8 for the `multiq` names, H <= 16, B <= 32 for `multiq`) are kept.

KV rows are 576 bytes: [..., :512] latent, [..., 512:576] rope, one per-tensor `kv_scale`; either a contiguous
[B, S, 576] slab or a [num_slots, 1, 576] pool with one token per slot.  `torch.float8_e4m3fnuz` (the reference's
format) and `torch.float8_e4m3fn` (the format the B200 tensor core reads) are both accepted; see
include/moonmath_attention.h for the two fnuz byte codes that are approximated.  Everything runs on the caller's
current stream, without host synchronisation; the paged entry points read their index tensors on the device only.
"""
from __future__ import annotations

import torch

from . import _abi, _kernel

__all__ = [
    "mla_decode_a16w8",
    "mla_decode_a16w8_paged_dev",
    "mla_decode_a16w8_plan_parts",
    "mla_decode_a16w8_plan_parts_capped",
    "mla_decode_a16w8_plan_parts_q",
    "mla_decode_a16w8_multiq",
    "mla_decode_a16w8_multiq_paged_dev",
    "mla_decode_a16w8_multiq_plan_parts_q",
]

_LAT, _ROPE = 512, 64
_QK = _LAT + _ROPE
_KV_FORMAT = {torch.float8_e4m3fnuz: 0, torch.float8_e4m3fn: 1}
_MAX_PARTS = 256  # MA_MLA_MAX_PARTS


def _check_q(q_lat, q_pe, o_lat, who: str, multiq: bool) -> int:
    """Layout, dtype and domain of the query / output tensors; returns q_len."""
    for t in (q_lat, q_pe, o_lat):
        if not isinstance(t, torch.Tensor):
            raise TypeError(f"{who}: q_lat/q_pe/o_lat must be torch.Tensor")
    rank = q_lat.dim()
    if multiq:
        if rank != 4:
            raise ValueError(f"{who}: q_lat must be [B,q_len,H,512] (q_len 4..8)")
    elif rank not in (3, 4):
        raise ValueError(f"{who}: q_lat must be [B,H,512] or [B,q_len,H,512]")
    if q_pe.dim() != rank or o_lat.dim() != rank:
        raise ValueError(f"{who}: q_lat/q_pe/o_lat must have the same rank")
    if any(t.dtype != torch.bfloat16 for t in (q_lat, q_pe, o_lat)):
        raise ValueError(f"{who}: q_lat/q_pe/o_lat must be bfloat16")
    if q_lat.device.type != "cuda":
        raise ValueError(f"{who}: tensors must be on a CUDA/HIP device")
    if q_pe.device != q_lat.device or o_lat.device != q_lat.device:
        raise ValueError(f"{who}: q_lat/q_pe/o_lat must be on the same device")
    if q_lat.size(-1) != _LAT or q_pe.size(-1) != _ROPE or o_lat.size(-1) != _LAT:
        raise ValueError(f"{who}: expected q_lat[...,512], q_pe[...,64], o_lat[...,512]")
    if not 1 <= q_lat.size(-2) <= 16:
        raise ValueError(f"{who}: H must be in [1,16]")
    q_len = q_lat.size(1) if rank == 4 else 1
    lo, hi = (4, 8) if multiq else (1, 8)
    if not lo <= q_len <= hi:
        raise ValueError(f"{who}: q_len must be in [{lo},{hi}]")
    if tuple(q_pe.shape[:-1]) != tuple(q_lat.shape[:-1]) or tuple(o_lat.shape) != tuple(q_lat.shape):
        raise ValueError(f"{who}: q_lat/q_pe/o_lat shapes do not match")
    if not (q_lat.is_contiguous() and q_pe.is_contiguous() and o_lat.is_contiguous()):
        raise ValueError(f"{who}: q_lat/q_pe/o_lat must be contiguous")
    return q_len


def _kv_format(kv, who: str, what: str) -> int:
    if kv.dtype not in _KV_FORMAT:
        raise ValueError(f"{who}: {what} must be float8_e4m3fnuz (or float8_e4m3fn)")
    return _KV_FORMAT[kv.dtype]


def _launch(who, q_lat, q_pe, kv, o_lat, seq_lens, rows, kv_indices, kv_indptr, q_len, seq, parts, scale, kv_scale, fmt):
    B, H = q_lat.size(0), q_lat.size(-2)
    ptr = lambda t: None if t is None else t.data_ptr()
    with torch.cuda.device(q_lat.device):
        stream = torch.cuda.current_stream(q_lat.device).cuda_stream
        ws_bytes = int(_abi.lib.ma_mla_workspace_bytes(B, q_len, parts))
        workspace = _kernel._workspace(q_lat.device, ws_bytes)
        rc = _abi.lib.ma_mla_decode_a16w8(
            q_lat.data_ptr(), q_pe.data_ptr(), kv.data_ptr(), o_lat.data_ptr(), ptr(seq_lens), ptr(rows),
            ptr(kv_indices), ptr(kv_indptr), B, H, q_len, seq, parts, float(scale), float(kv_scale), fmt,
            workspace.data_ptr(), workspace.numel(), stream,
        )
    if rc != 0:
        raise RuntimeError(f"launch_{who} returned error code {rc}: {_abi.error_string(rc)}")


def _contiguous(who, multiq, q_lat, q_pe, kv, o_lat, scale, kv_scale):
    q_len = _check_q(q_lat, q_pe, o_lat, who, multiq)
    if not multiq and q_len != 1:
        raise ValueError(f"{who}: the contiguous entry point is q_len==1 only; use {who}_paged_dev for a draft window")
    fmt = _kv_format(kv, who, "kv")
    if kv.dim() != 3 or kv.size(2) != _QK:
        raise ValueError(f"{who}: kv must be the FUSED [B,S,576] slab ([...,:512]=latent, [512:576]=rope), "
                         "not the split c_kv/k_pe pair")
    if kv.size(0) != q_lat.size(0):
        raise ValueError(f"{who}: kv batch must match q_lat batch")
    if not kv.is_contiguous():
        raise ValueError(f"{who}: kv must be contiguous")
    if kv.device != q_lat.device:
        raise ValueError(f"{who}: kv must be on the same device as q_lat")
    if multiq and q_lat.size(0) > 32:
        raise ValueError(f"{who}: B must be in [1,32]")
    B, S = q_lat.size(0), kv.size(1)
    parts = int(_abi.lib.ma_mla_plan_parts_contiguous(B, q_len, S, 0))
    _launch(who, q_lat, q_pe, kv, o_lat, None, None, None, None, q_len, S, parts, scale, kv_scale, fmt)


def _paged(who, multiq, q_lat, q_pe, kv_pool, o_lat, seq_lens, rows, kv_indices, kv_indptr, parts, scale, kv_scale):
    q_len = _check_q(q_lat, q_pe, o_lat, who, multiq)
    fmt = _kv_format(kv_pool, who, "kv_pool")
    if kv_pool.size(-1) != _QK:
        raise ValueError(f"{who}: kv_pool rows must be 576 wide ([...,:512]=c_KV, [512:576]=k_pe)")
    if not kv_pool.is_contiguous():
        raise ValueError(f"{who}: kv_pool must be contiguous")
    for name, t in (("seq_lens", seq_lens), ("kv_indices", kv_indices), ("kv_indptr", kv_indptr), ("rows", rows)):
        if t is None and name == "rows":
            continue
        if t.dtype != torch.int32:
            raise ValueError(f"{who}: seq_lens/kv_indices/kv_indptr must be int32" if name != "rows"
                             else f"{who}: rows must be int32")
        if t.device != q_lat.device or not t.is_contiguous():
            raise ValueError(f"{who}: {name} must be a contiguous tensor on the same device as q_lat")
    B = q_lat.size(0)
    if seq_lens.numel() != B or kv_indptr.numel() != B + 1 or (rows is not None and rows.numel() != B):
        raise ValueError(f"{who}: seq_lens/rows must have B entries and kv_indptr B+1")
    if multiq and B > 32:
        raise ValueError(f"{who}: B must be in [1,32]")
    if not 1 <= int(parts) <= _MAX_PARTS:
        raise ValueError(f"{who}: parts must be in [1,{_MAX_PARTS}]")
    _launch(who, q_lat, q_pe, kv_pool, o_lat, seq_lens, rows, kv_indices, kv_indptr, q_len, 0, int(parts), scale,
            kv_scale, fmt)


def mla_decode_a16w8(q_lat, q_pe, kv, o_lat, scale: float, kv_scale: float, scale_p: float = 1.0) -> None:
    """A16W8 absorbed-decode MLA (q_len = 1, H <= 16).

    q_lat [B,H,512] bf16, q_pe [B,H,64] bf16, kv [B,S,576] fp8, o_lat [B,H,512] bf16 (written in place);
    scale = softmax scale, kv_scale = per-tensor fp8 descale, scale_p unused (kept for the signature).
    """
    _contiguous("mla_decode_a16w8", False, q_lat, q_pe, kv, o_lat, scale, kv_scale)


def mla_decode_a16w8_paged_dev(q_lat, q_pe, kv_pool, o_lat, seq_lens, rows, kv_indices, kv_indptr, parts: int,
                               scale: float, kv_scale: float, scale_p: float = 1.0) -> None:
    """A16W8 absorbed-decode MLA over a paged pool, device-driven (no host read, fixed grid).

    q_lat / q_pe: bf16 [B,H,*] or [B,q_len,H,*] (q_len <= 8); position t attends KV [0, S - q_len + t], so
    `seq_lens` includes the q_len draft tokens.  kv_pool [num_slots,1,576] fp8; seq_lens [B], kv_indptr [B+1],
    kv_indices [sum(seq_lens)] int32 on the device; rows [B] int32 or None maps request -> q / out batch row;
    parts: fixed KV split (mla_decode_a16w8_plan_parts_capped, or _plan_parts_q for q_len > 1).
    """
    _paged("mla_decode_a16w8_paged_dev", False, q_lat, q_pe, kv_pool, o_lat, seq_lens, rows, kv_indices, kv_indptr,
           parts, scale, kv_scale)


def mla_decode_a16w8_plan_parts(B: int, H: int, max_seq_len: int, lat_dim: int = 512) -> int:
    """Fixed KV-split count for a graph captured at (B, H, max_seq_len)."""
    return int(_abi.lib.ma_mla_plan_parts(int(B), 1, int(max_seq_len), 0))


def mla_decode_a16w8_plan_parts_capped(B: int, H: int, max_seq_len: int, lat_dim: int = 512) -> int:
    """As plan_parts; the planner already keeps B * parts inside what the workspace is sized for."""
    return int(_abi.lib.ma_mla_plan_parts(int(B), 1, int(max_seq_len), 0))


def mla_decode_a16w8_plan_parts_q(B: int, max_seq_len: int, q_len: int = 1, H: int = 16) -> int:
    """q_len-aware KV-split count: a window of q_len positions is q_len CTAs per (request, part)."""
    return int(_abi.lib.ma_mla_plan_parts(int(B), max(1, int(q_len)), int(max_seq_len), 0))


def mla_decode_a16w8_multiq(q_lat, q_pe, kv, o_lat, scale: float, kv_scale: float, scale_p: float = 1.0) -> None:
    """A16W8 multi-query absorbed-decode MLA (q_len 4..8, H <= 16, B <= 32).

    q_lat [B,q_len,H,512], q_pe [B,q_len,H,64], o_lat like q_lat (bf16); kv [B,S,576] fp8.  Draft position t
    attends kv[:, : S - q_len + t + 1].
    """
    _contiguous("mla_decode_a16w8_multiq", True, q_lat, q_pe, kv, o_lat, scale, kv_scale)


def mla_decode_a16w8_multiq_paged_dev(q_lat, q_pe, kv_pool, o_lat, seq_lens, rows, kv_indices, kv_indptr, parts: int,
                                      scale: float, kv_scale: float, scale_p: float = 1.0) -> None:
    """A16W8 multi-query decode over a paged pool, device-driven; q_len 4..8.  Arguments as the paged q_len op."""
    _paged("mla_decode_a16w8_multiq_paged_dev", True, q_lat, q_pe, kv_pool, o_lat, seq_lens, rows, kv_indices,
           kv_indptr, parts, scale, kv_scale)


def mla_decode_a16w8_multiq_plan_parts_q(B: int, max_seq_len: int, q_len: int = 4, H: int = 16) -> int:
    """Fixed KV-split count for a multi-query graph captured at (B, max_seq_len, q_len, H)."""
    return int(_abi.lib.ma_mla_plan_parts(int(B), max(1, int(q_len)), int(max_seq_len), 0))
