"""`forward`: argument checks and the call into the C ABI.

Mirrors the reference's Python entry (moonmath_attention/_kernel.py:14-82) and
the checks of its torch binding (csrc/attention_api.cpp:134-229): same
signature, same defaults, same exception types.
"""

from __future__ import annotations

import os

import torch

from . import _abi

_SMS: dict[int, int] = {}
_LAST: dict[str, object] = {}


def _flags_from_env() -> int:
    flags = 0
    if os.environ.get("MOONMATH_NO_TAIL"):  # reference: csrc/attention_api.cpp:261
        flags |= _abi.FLAG_NO_TAIL
    if os.environ.get("MOONMATH_SIMPLE"):
        flags |= _abi.FLAG_SIMPLE
    if os.environ.get("MOONMATH_EXACT_MAX"):
        flags |= _abi.FLAG_EXACT_MAX
    flags |= int(os.environ.get("MOONMATH_FLAGS", "0"), 0)  # raw flag bits (tuning)
    return flags


def _num_sms(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _SMS:
        _SMS[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _SMS[idx]


def plan_tail(batch: int, heads: int, seq_len: int, seq_len_kv: int, num_sms: int = 148, flags: int = 0) -> dict:
    return _abi.plan_tail(batch, heads, seq_len, seq_len_kv, num_sms, flags)


def workspace_bytes(batch: int, heads: int, seq_len: int, seq_len_kv: int, num_sms: int = 148, flags: int = 0) -> int:
    return _abi.workspace_bytes(batch, heads, seq_len, seq_len_kv, num_sms, flags)


def last_status() -> list[int] | None:
    """Device status words of the most recent `forward` call (synchronises); [0, ...] when healthy."""
    ws = _LAST.get("workspace")
    if ws is None:
        return None
    return ws[:16].view(torch.int32).cpu().tolist()


def _check_tensor(t, name: str, layout: str) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be torch.Tensor; got {type(t).__name__}")
    if t.dtype != torch.bfloat16:
        raise TypeError(f"{name} must be torch.bfloat16; got dtype={t.dtype}")
    if t.dim() != 4:
        raise ValueError(f"{name} must be 4-D ({layout.upper()}); got shape={tuple(t.shape)}")


def _forward_cuda(q, k, v, out, round_mode: str, layout: str, flags: int | None):
    if round_mode not in _abi.ROUND_MODE:
        raise ValueError(f"round_mode must be 'rtna', 'rtne', or 'rtz', got '{round_mode}'")
    if layout not in _abi.LAYOUT:
        raise ValueError(f"layout must be 'bhsd' or 'bshd', got '{layout}'")
    for name, t in (("q", q), ("k", k), ("v", v)):
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
        if t.device.type != "cuda":
            raise ValueError(f"{name} must be on a CUDA device (GPU-only), got device={t.device}")
    sax, hax = (1, 2) if layout == "bshd" else (2, 1)
    B, H, Sq, D = q.size(0), q.size(hax), q.size(sax), q.size(3)
    Skv = k.size(sax)
    if D != 128:
        raise ValueError(f"head_dim must be 128, got {D}")
    if k.size(0) != B or k.size(hax) != H or k.size(3) != D:
        raise ValueError(
            f"k shape mismatch: expected batch={B}, heads={H}, head_dim={D}, got k.shape={tuple(k.shape)}"
        )
    if v.size(0) != B or v.size(hax) != H or v.size(sax) != Skv or v.size(3) != D:
        raise ValueError(f"v shape mismatch: must match k.shape, got v.shape={tuple(v.shape)}, k.shape={tuple(k.shape)}")
    if Sq <= 0 or Skv <= 0:
        raise ValueError(f"seq_len must be positive, got Sq={Sq}, Skv={Skv}")
    if q.device != k.device or q.device != v.device:
        raise ValueError("q, k, v must be on the same device")
    if out is not None:
        _check_tensor(out, "out", layout)
        if not out.is_contiguous():
            raise ValueError("out must be contiguous")
        if tuple(out.shape) != tuple(q.shape):
            raise ValueError(f"out shape must match q.shape, got out.shape={tuple(out.shape)}, q.shape={tuple(q.shape)}")
        if out.device != q.device:
            raise ValueError("out must be on the same device as q")
    else:
        out = torch.empty_like(q)

    if flags is None:
        flags = _flags_from_env()
    with torch.cuda.device(q.device):
        stream = torch.cuda.current_stream(q.device).cuda_stream
        ws_bytes = _abi.workspace_bytes(B, H, Sq, Skv, _num_sms(q.device), flags)
        # Allocated per call through the caching allocator, as the reference does
        # (csrc/attention_api.cpp:261-267); stream-ordered reuse makes that safe.
        workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
        rc = _abi.lib.ma_attention_forward(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
            B, H, Sq, Skv, D, _abi.LAYOUT[layout], _abi.ROUND_MODE[round_mode],
            workspace.data_ptr(), ws_bytes, flags, stream,
        )
    if rc != 0:
        raise RuntimeError(f"ma_attention_forward returned error code {rc}: {_abi.error_string(rc)}")
    _LAST["workspace"] = workspace
    if os.environ.get("MOONMATH_CHECK"):
        st = last_status()
        if st[0] != 0:
            raise RuntimeError(
                f"moonmath_attention kernel reported status {st[0]:#x} (site {st[1] & 0xFF:#x}, "
                f"cta {st[1] >> 8}, detail {st[2]})"
            )
    return out


def forward(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    *,
    out: torch.Tensor | None = None,
    round_mode: str = "rtna",
    layout: str = "bhsd",
    _flags: int | None = None,
) -> torch.Tensor:
    """Fused forward attention: O = softmax(QK^T / sqrt(D)) V on B200.

    Args:
        q, k, v: torch.bfloat16 tensors of shape (batch, heads, seq_len, head_dim)
                 or (batch, seq_len, heads, head_dim) depending on layout.
                 Contiguous. head_dim=128. K and V may have their own length.
                 CPU tensors are copied to cuda:0 and the result is copied back
                 (a convenience copy; the arithmetic always runs on the GPU).
        out: optional preallocated output tensor. Must match q's shape, dtype,
             device, and be contiguous. If None, a new tensor is allocated.
        round_mode: "rtna" (default; ties away from zero), "rtne", or "rtz"
            (truncation) for the final fp32 -> bf16 conversion. NaN is always 0x7FFF.
        layout: "bhsd" (default) or "bshd".

    Returns:
        torch.bfloat16 tensor of the same shape and device as q. The kernel is
        launched on the caller's current stream of q's device and not synchronised.
    """
    for name, t in (("q", q), ("k", k), ("v", v)):
        _check_tensor(t, name, layout)

    if q.device.type == "cpu":
        if k.device.type != "cpu" or v.device.type != "cpu":
            raise ValueError("q is on CPU but k or v is not; all must be on the same device")
        if not torch.cuda.is_available():
            raise RuntimeError("moonmath_attention has no CPU implementation and no CUDA device is available")
        device = torch.device("cuda:0")
        out_gpu = out.to(device) if out is not None else None
        result = _forward_cuda(q.to(device), k.to(device), v.to(device), out_gpu, round_mode, layout, _flags)
        return result.cpu()
    elif q.device.type == "cuda":
        if k.device != q.device or v.device != q.device:
            raise ValueError(f"q/k/v must be on the same device; got q={q.device}, k={k.device}, v={v.device}")
        return _forward_cuda(q, k, v, out, round_mode, layout, _flags)
    else:
        raise NotImplementedError(f"Unsupported device {q.device!r}; expected 'cpu' or 'cuda'")


def _check_list(t, name: str, device) -> None:
    # reference: check_list, csrc/attention_api.cpp:329-339 (std::invalid_argument -> ValueError)
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be torch.Tensor; got {type(t).__name__}")
    if t.dtype != torch.int16:
        raise ValueError(f"{name} must be int16, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if t.device != device:
        raise ValueError(f"{name} must be on the same device as q")


def forward_lite(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    read_list: torch.Tensor,
    write_list: torch.Tensor,
    *,
    threshold: float,
    phase: int,
    must_do_list: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
    round_mode: str = "rtna",
    layout: str = "bhsd",
) -> torch.Tensor:
    """LiteAttention forward: compute only the key blocks the skip list names, write the next list.

    Same signature as the reference's entry (moonmath_attention/_kernel.py:85-134; binding
    csrc/attention_api.cpp:287-434).  `read_list` / `write_list` are int16 CUDA tensors
    [B, H, qtiles, ktiles + 2], the two halves of the double buffer `LiteAttention` owns
    (read = skip[phase before the flip], write = the other; `phase` is the value after the flip).
    qtiles = ceil(Sq / 256), ktiles = ceil(Skv / 64): `LiteAttention.get_MN()`.  A key block is dropped
    from the written list when, for every group of 32 query rows of the tile, its largest score lies
    more than |threshold| (log2 units) below the group's rows' running maxima.

    `must_do_list` (optional): one global int16 1-D tensor [len, start0, end0, start1, end1, ...] of
    key-block ranges [start, end) that are always written as "compute".

    GPU tensors only.  The output approximates full attention (skipped blocks contribute nothing); with a
    compute-all list and a threshold no block falls under, it is full attention.
    """
    for name, t in (("q", q), ("k", k), ("v", v)):
        _check_tensor(t, name, layout)
    if round_mode not in _abi.ROUND_MODE:
        raise ValueError(f"round_mode must be 'rtna', 'rtne', or 'rtz', got '{round_mode}'")
    if layout not in _abi.LAYOUT:
        raise ValueError(f"layout must be 'bhsd' or 'bshd', got '{layout}'")
    for name, t in (("q", q), ("k", k), ("v", v)):
        if t.device.type != "cuda":
            raise ValueError(f"{name} must be on a CUDA device (GPU-only), got device={t.device}")
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
    sax, hax = (1, 2) if layout == "bshd" else (2, 1)
    B, H, Sq, D = q.size(0), q.size(hax), q.size(sax), q.size(3)
    Skv = k.size(sax)
    if D != 128:
        raise ValueError(f"head_dim must be 128, got {D}")
    if q.device != k.device or q.device != v.device:
        raise ValueError("q, k, v must be on the same device")
    if k.size(0) != B or k.size(hax) != H or k.size(3) != D or tuple(v.shape) != tuple(k.shape):
        raise ValueError(f"k / v shape mismatch: q.shape={tuple(q.shape)}, k.shape={tuple(k.shape)}, v.shape={tuple(v.shape)}")
    _check_list(read_list, "read_list", q.device)
    _check_list(write_list, "write_list", q.device)
    if must_do_list is not None:
        _check_list(must_do_list, "must_do_list", q.device)
    tile_m, tile_n = _abi.lite_tile()
    need = B * H * ((Sq + tile_m - 1) // tile_m) * ((Skv + tile_n - 1) // tile_n + 2)
    for name, t in (("read_list", read_list), ("write_list", write_list)):
        if t.numel() != need:
            raise ValueError(
                f"{name} must hold B*H*ceil(Sq/{tile_m})*(ceil(Skv/{tile_n})+2) = {need} int16 values, got {t.numel()}"
            )
    if out is not None:
        _check_tensor(out, "out", layout)
        if tuple(out.shape) != tuple(q.shape):
            raise ValueError("out shape must match q.shape")
        if out.device != q.device:
            raise ValueError("out must be on the same device as q")
        if not out.is_contiguous():
            raise ValueError("out must be contiguous")
    else:
        out = torch.empty_like(q)

    flags = _abi.FLAG_LITE_PLAIN if os.environ.get("MOONMATH_LITE_PLAIN") else 0  # csrc/attention_api.cpp:403
    with torch.cuda.device(q.device):
        stream = torch.cuda.current_stream(q.device).cuda_stream
        ws_bytes = int(_abi.lib.ma_lite_workspace_bytes(B, H, Sq))
        workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
        rc = _abi.lib.ma_attention_forward_lite(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
            B, H, Sq, Skv, D, _abi.LAYOUT[layout], _abi.ROUND_MODE[round_mode],
            read_list.data_ptr(), write_list.data_ptr(),
            must_do_list.data_ptr() if must_do_list is not None else None,
            float(threshold), int(phase), workspace.data_ptr(), ws_bytes, flags, stream,
        )
    if rc != 0:
        raise RuntimeError(f"launch_attention_forward_lite returned error code {rc}: {_abi.error_string(rc)}")
    _LAST["workspace"] = workspace
    if os.environ.get("MOONMATH_CHECK"):
        st = last_status()
        if st[0] != 0:
            raise RuntimeError(
                f"moonmath_attention lite kernel reported status {st[0]:#x} (site {st[1] & 0xFF:#x}, "
                f"cta {st[1] >> 8}, detail {st[2]})"
            )
    return out
