"""`forward`: argument checks and the call into the C ABI.

Mirrors the reference's Python entry (moonmath_attention/_kernel.py:14-82) and
the checks of its torch binding (csrc/attention_api.cpp:134-229): same
signature, same defaults, same exception types.
"""

from __future__ import annotations

import os
import threading
from collections import OrderedDict

import torch

from . import _abi

_SMS: dict[int, int] = {}

# Workspaces are kept per (device, stream, thread) and reused by later calls on the same stream: calls on
# one stream are ordered, every call rewrites what it reads (the status block is cleared first), so sharing
# is safe there and saves an allocator round trip per call.  Different streams or threads never share one.
# The reference allocates its 121 MB workspace on every call (csrc/attention_api.cpp:261-267).
_WORKSPACES: "OrderedDict[tuple[int, int, int], torch.Tensor]" = OrderedDict()
_WORKSPACE_SLOTS = 8  # least recently used entries beyond this are dropped (their memory returns to torch's allocator)


def _flags_from_env() -> int:
    flags = 0
    if os.environ.get("MOONMATH_NO_TAIL"):  # reference: csrc/attention_api.cpp:261
        flags |= _abi.FLAG_NO_TAIL
    if os.environ.get("MOONMATH_SIMPLE"):
        flags |= _abi.FLAG_SIMPLE
    if os.environ.get("MOONMATH_EXACT_MAX"):
        flags |= _abi.FLAG_EXACT_MAX
    if os.environ.get("MOONMATH_PRECISE_P"):
        flags |= _abi.FLAG_PRECISE_P
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


def _slot_key(device: torch.device) -> tuple[int, int, int]:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    return idx, int(torch.cuda.current_stream(device).cuda_stream), threading.get_ident()


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """A 256-byte aligned device buffer of at least `nbytes` for a call on the caller's current stream."""
    if torch.cuda.is_current_stream_capturing():
        # Memory allocated during a capture belongs to the graph's pool: neither take it from the cache nor put it there.
        return torch.empty(nbytes, dtype=torch.uint8, device=device)
    key = _slot_key(device)
    ws = _WORKSPACES.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 4096), dtype=torch.uint8, device=device)
        _WORKSPACES[key] = ws
    _WORKSPACES.move_to_end(key)
    while len(_WORKSPACES) > _WORKSPACE_SLOTS:
        _WORKSPACES.popitem(last=False)
    return ws


def last_status(device: torch.device | None = None) -> list[int] | None:
    """Device status words left by this thread's most recent call on the current stream of `device`
    (default: the current device); synchronises.  [0, ...] when healthy, None when there was no such call."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    ws = _WORKSPACES.get(_slot_key(device))
    if ws is None:
        return None
    return ws[:64].view(torch.int32).cpu().tolist()


def _raise_on_device_status(what: str, device: torch.device) -> None:
    st = last_status(device)
    if st is not None and st[0] != 0:
        raise RuntimeError(
            f"moonmath_attention {what} reported status {st[0]:#x} (site {st[1] & 0xFF:#x}, "
            f"cta {st[1] >> 8}, detail {st[2]})"
        )


def _check_tensor(t, name: str, layout: str) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be torch.Tensor; got {type(t).__name__}")
    if t.dtype != torch.bfloat16:
        raise TypeError(f"{name} must be torch.bfloat16; got dtype={t.dtype}")
    if t.dim() != 4:
        raise ValueError(f"{name} must be 4-D ({layout.upper()}); got shape={tuple(t.shape)}")


def _check_problem(q, k, v, out, round_mode: str, layout: str, on_gpu: bool = False):
    """The checks of the reference's binding (csrc/attention_api.cpp:160-229); returns (B, H, Sq, Skv)."""
    if round_mode not in _abi.ROUND_MODE:
        raise ValueError(f"round_mode must be 'rtna', 'rtne', or 'rtz', got '{round_mode}'")
    if layout not in _abi.LAYOUT:
        raise ValueError(f"layout must be 'bhsd' or 'bshd', got '{layout}'")
    for name, t in (("q", q), ("k", k), ("v", v)):
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
        if on_gpu and t.device.type != "cuda":
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
    return B, H, Sq, Skv


def _launch(q_ptr: int, k_ptr: int, v_ptr: int, out_ptr: int, B: int, H: int, Sq: int, Skv: int, layout: str,
            round_mode: str, flags: int, device: torch.device) -> None:
    """One `ma_attention_forward` on the current stream of `device` (which must be the current device)."""
    stream = torch.cuda.current_stream(device).cuda_stream
    ws_bytes = _abi.workspace_bytes(B, H, Sq, Skv, _num_sms(device), flags)
    workspace = _workspace(device, ws_bytes)
    rc = _abi.lib.ma_attention_forward(
        q_ptr, k_ptr, v_ptr, out_ptr, B, H, Sq, Skv, 128, _abi.LAYOUT[layout], _abi.ROUND_MODE[round_mode],
        workspace.data_ptr(), workspace.numel(), flags, stream,
    )
    if rc != 0:
        raise RuntimeError(f"ma_attention_forward returned error code {rc}: {_abi.error_string(rc)}")


def _forward_cuda(q, k, v, out, round_mode: str, layout: str, flags: int | None):
    B, H, Sq, Skv = _check_problem(q, k, v, out, round_mode, layout, on_gpu=True)
    if out is None:
        out = torch.empty_like(q)
    if flags is None:
        flags = _flags_from_env()
    with torch.cuda.device(q.device):
        _launch(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, H, Sq, Skv, layout, round_mode, flags,
                q.device)
        if os.environ.get("MOONMATH_CHECK"):
            _raise_on_device_status("kernel", q.device)
    return out


# ---------------------------------------------------------------------------
# host tensors: a three-stream pipeline over PCIe
# ---------------------------------------------------------------------------
_HOST_CHUNK_BYTES = 8 << 20  # q / out bytes one pipeline step moves (per tensor)
_SIDE_STREAMS: dict[int, tuple] = {}


def _side_streams(device: torch.device):
    idx = device.index
    if idx not in _SIDE_STREAMS:
        _SIDE_STREAMS[idx] = tuple(torch.cuda.Stream(device=device) for _ in range(3))
    return _SIDE_STREAMS[idx]


def _host_chunks(B: int, H: int, Sq: int, layout: str) -> list[tuple]:
    """Independent pieces of a problem whose q and out bytes are contiguous in host memory.

    bhsd [B,H,S,D]: (batch, head range): q, k, v and out of a few heads, each one contiguous block.
    bshd [B,S,H,D]: (batch, query-row range): k and v of the batch travel once, ahead of its first piece.
    """
    pieces = []
    if layout == "bhsd":
        per_head = Sq * 128 * 2
        nh = max(1, min(H, _HOST_CHUNK_BYTES // per_head))
        for b in range(B):
            for h0 in range(0, H, nh):
                pieces.append((b, h0, min(H, h0 + nh)))
    else:
        per_row = H * 128 * 2
        nr = max(256, (_HOST_CHUNK_BYTES // per_row) // 256 * 256)
        for b in range(B):
            for r0 in range(0, Sq, nr):
                pieces.append((b, r0, min(Sq, r0 + nr)))
    return pieces


def _forward_host(q, k, v, out, round_mode: str, layout: str, flags: int | None):
    """CPU tensors in, CPU tensor out, arithmetic on the current CUDA device (the reference's convenience,
    moonmath_attention/_kernel.py:52-67, which copies q, k, v up, runs, and copies the result down, one
    after the other).  Here the three legs overlap: the problem is cut into independent pieces
    (`_host_chunks`); one stream uploads, a second runs the kernel on each piece as soon as its inputs have
    landed, a third downloads finished pieces, so PCIe carries both directions at once and the kernels
    hide under the copies.  Pinned host tensors (`Tensor.pin_memory()`) make the copies asynchronous;
    pageable ones work, more slowly.  The result is complete when the call returns.  `out`, if given, is
    filled and returned (the reference ignores a CPU `out` and returns a new tensor)."""
    B, H, Sq, Skv = _check_problem(q, k, v, out, round_mode, layout)
    # The reference says "cuda:0"; the current device is that in a single-GPU process, and the right one in a
    # process that was given its own GPU with torch.cuda.set_device (one rank per GPU).
    device = torch.device("cuda", torch.cuda.current_device())
    if flags is None:
        flags = _flags_from_env()
    # The pieces never split their last round along KV: their kernels hide under the copies anyway, and a
    # piece's result then does not depend on how the problem was cut.
    flags |= _abi.FLAG_NO_TAIL
    if out is None:
        out = torch.empty_like(q)
    with torch.cuda.device(device):
        up, run, down = _side_streams(device)
        caller = torch.cuda.current_stream(device)
        for s in (up, run, down):
            s.wait_stream(caller)
        dq, dk, dv = (torch.empty(t.shape, dtype=t.dtype, device=device) for t in (q, k, v))
        dout = torch.empty(q.shape, dtype=q.dtype, device=device)
        last_batch = -1
        for piece in _host_chunks(B, H, Sq, layout):
            b, lo, hi = piece
            with torch.cuda.stream(up):
                if layout == "bhsd":
                    for d, h in ((dk, k), (dv, v), (dq, q)):
                        d[b, lo:hi].copy_(h[b, lo:hi], non_blocking=True)
                else:
                    if b != last_batch:
                        dk[b].copy_(k[b], non_blocking=True)
                        dv[b].copy_(v[b], non_blocking=True)
                        last_batch = b
                    dq[b, lo:hi].copy_(q[b, lo:hi], non_blocking=True)
                sent = torch.cuda.Event()
                sent.record(up)
            with torch.cuda.stream(run):
                run.wait_event(sent)
                if layout == "bhsd":
                    _launch(dq[b, lo].data_ptr(), dk[b, lo].data_ptr(), dv[b, lo].data_ptr(), dout[b, lo].data_ptr(),
                            1, hi - lo, Sq, Skv, layout, round_mode, flags, device)
                else:
                    _launch(dq[b, lo].data_ptr(), dk[b].data_ptr(), dv[b].data_ptr(), dout[b, lo].data_ptr(),
                            1, H, hi - lo, Skv, layout, round_mode, flags, device)
                done = torch.cuda.Event()
                done.record(run)
            with torch.cuda.stream(down):
                down.wait_event(done)
                out[b, lo:hi].copy_(dout[b, lo:hi], non_blocking=True)
        down.synchronize()  # the caller gets host memory: it must be complete on return
        if os.environ.get("MOONMATH_CHECK"):
            with torch.cuda.stream(run):
                _raise_on_device_status("kernel", device)
        caller.wait_stream(down)
    return out


def forward(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    *,
    out: torch.Tensor | None = None,
    round_mode: str = "rtna",
    layout: str = "bhsd",
    precise: bool = False,
) -> torch.Tensor:
    """Fused forward attention: O = softmax(QK^T / sqrt(D)) V on B200.

    Args:
        q, k, v: torch.bfloat16 tensors of shape (batch, heads, seq_len, head_dim)
                 or (batch, seq_len, heads, head_dim) depending on layout.
                 Contiguous. head_dim=128. K and V may have their own length.
                 CPU tensors are copied to the current CUDA device (cuda:0 unless the process
                 selected another) and the result is copied back (a convenience copy; the
                 arithmetic always runs on the GPU).
        out: optional preallocated output tensor. Must match q's shape, dtype,
             device, and be contiguous. If None, a new tensor is allocated.
        round_mode: "rtna" (default; ties away from zero), "rtne", or "rtz"
            (truncation) for the final fp32 -> bf16 conversion. NaN is always 0x7FFF.
        layout: "bhsd" (default) or "bshd".
        precise: not in the reference.  False: the softmax probabilities are rounded to bf16 before
            the second matrix product, as the reference does (csrc/attention_kernel.hip:446-448).
            True (or MOONMATH_PRECISE_P=1): they are carried as the sum of two bf16 terms, which brings
            the result to within one bf16 unit of the fp32 formula wherever the output is not a
            cancellation residue; costs about 40 % more time.

    Returns:
        torch.bfloat16 tensor of the same shape and device as q. The kernel is
        launched on the caller's current stream of q's device and not synchronised.
    """
    for name, t in (("q", q), ("k", k), ("v", v)):
        _check_tensor(t, name, layout)
    flags = _flags_from_env() | (_abi.FLAG_PRECISE_P if precise else 0)

    if q.device.type == "cpu":
        if k.device.type != "cpu" or v.device.type != "cpu":
            raise ValueError("q is on CPU but k or v is not; all must be on the same device")
        if not torch.cuda.is_available():
            raise RuntimeError("moonmath_attention has no CPU implementation and no CUDA device is available")
        return _forward_host(q, k, v, out, round_mode, layout, flags)
    elif q.device.type == "cuda":
        if k.device != q.device or v.device != q.device:
            raise ValueError(f"q/k/v must be on the same device; got q={q.device}, k={k.device}, v={v.device}")
        return _forward_cuda(q, k, v, out, round_mode, layout, flags)
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
        workspace = _workspace(q.device, ws_bytes)
        rc = _abi.lib.ma_attention_forward_lite(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
            B, H, Sq, Skv, D, _abi.LAYOUT[layout], _abi.ROUND_MODE[round_mode],
            read_list.data_ptr(), write_list.data_ptr(),
            must_do_list.data_ptr() if must_do_list is not None else None,
            float(threshold), int(phase), workspace.data_ptr(), workspace.numel(), flags, stream,
        )
        if rc != 0:
            raise RuntimeError(f"launch_attention_forward_lite returned error code {rc}: {_abi.error_string(rc)}")
        if os.environ.get("MOONMATH_CHECK"):
            _raise_on_device_status("lite kernel", q.device)
    return out
