"""Failure path and memory discipline of the kernels, checked without faulting anything.  Needs a B200: -m gpu.

* A bounded wait that runs out: `ma_selftest_wait_timeout` launches a CTA that waits on a barrier nobody
  arrives on, under a one-millisecond limit.  The kernel must return, leave the time-out code and the wait
  site in the status block, free its tensor memory, and leave the device fit for the next call.
* Guard words: `out` and the workspace sit between 64 KiB zones filled with a pattern; after calls whose
  tiles hang over the ends of the sequences (ragged lengths) and whose plan writes KV-split partial results,
  the zones must be untouched.  This is the stand-in for a memory checker, which is not available here.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu

GUARD = 64 << 10
PATTERN = 0x5A


@pytest.fixture(scope="module")
def abi(cuda_device):
    from moonmath_attention import _abi

    return _abi


def _status_words(ws: torch.Tensor) -> list[int]:
    return [x & 0xFFFFFFFF for x in ws[:64].view(torch.int32).cpu().tolist()]


def test_a_wait_that_runs_out_ends_the_kernel_and_reports(abi, cuda_device):
    import moonmath_attention as ma

    q, k, v = (t.to(cuda_device) for t in orc.make_inputs(1, 3, 300, 500, "bhsd"))
    before = ma.forward(q, k, v, round_mode="rtne")
    torch.cuda.synchronize()

    ws = torch.full((4096,), 0x77, dtype=torch.uint8, device=cuda_device)
    stream = torch.cuda.current_stream().cuda_stream
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    rc = abi.lib.ma_selftest_wait_timeout(1_000_000, ws.data_ptr(), ws.numel(), stream)
    t1.record()
    assert rc == 0, abi.error_string(rc)
    torch.cuda.synchronize()  # returns: the kernel ended by itself
    assert t0.elapsed_time(t1) < 200.0, "a 1 ms limit must not take longer than a few polls to notice"
    st = _status_words(ws)
    assert st[0] == abi.ERR_WAIT_TIMEOUT
    assert st[1] & 0xFF in (0x71, 0x72) and st[1] >> 8 == 0   # the site of the wait that gave up, CTA 0
    assert st[8] == 0                                          # nothing ran past a wait that never completed
    assert st[9] == 1                                          # the CTA left through its abort flag and common exit
    assert torch.all(ws[256:] == 0x77)                         # only the status block was written

    # Tensor memory was released and the context is healthy: a full 512-column allocation (the attention
    # kernel takes all of an SM's tensor memory) succeeds on every SM, and the result is what it was.
    for _ in range(2):
        after = ma.forward(q, k, v, round_mode="rtne")
        torch.cuda.synchronize()
        assert ma.last_status()[0] == 0
        assert torch.equal(after.view(torch.int16), before.view(torch.int16))


def _guarded(nbytes: int, dev) -> tuple[torch.Tensor, torch.Tensor]:
    """A device buffer with GUARD bytes of PATTERN on either side; returns (whole, payload view)."""
    pad = (-nbytes) % 256
    whole = torch.full((GUARD + nbytes + pad + GUARD,), PATTERN, dtype=torch.uint8, device=dev)
    return whole, whole[GUARD:GUARD + nbytes]


def _guards_intact(whole: torch.Tensor, nbytes: int) -> bool:
    pad = (-nbytes) % 256
    return bool(torch.all(whole[:GUARD] == PATTERN)) and bool(torch.all(whole[GUARD + nbytes + pad:] == PATTERN))


@pytest.mark.parametrize("case", [
    # (B, H, Sq, Skv, layout, flags): ragged tiles in both layouts; a plan with a KV-split tail; a single row
    (2, 3, 257, 129, "bhsd", 0),
    (2, 3, 255, 65, "bshd", 0),
    (1, 5, 1, 4097, "bshd", 0),
    (1, 40, 2048, 2048, "bhsd", 0),
    (1, 37, 512, 2304, "bshd", 0),
    (1, 40, 2048, 2048, "bhsd", 0x10),   # precise mode writes the same places
])
def test_guard_words_around_output_and_workspace_stay_intact(abi, cuda_device, case):
    B, H, Sq, Skv, layout, flags = case
    sms = torch.cuda.get_device_properties(cuda_device).multi_processor_count
    q, k, v = (t.to(cuda_device) for t in orc.make_inputs(B, H, Sq, Skv, layout))
    out_bytes = q.numel() * 2
    out_whole, out_view = _guarded(out_bytes, cuda_device)
    ws_bytes = abi.workspace_bytes(B, H, Sq, Skv, sms, flags)
    ws_whole, ws_view = _guarded(ws_bytes, cuda_device)
    assert out_view.data_ptr() % 256 == 0 and ws_view.data_ptr() % 256 == 0
    rc = abi.lib.ma_attention_forward(q.data_ptr(), k.data_ptr(), v.data_ptr(), out_view.data_ptr(), B, H, Sq, Skv, 128,
                                      abi.LAYOUT[layout], 0, ws_view.data_ptr(), ws_bytes, flags,
                                      torch.cuda.current_stream().cuda_stream)
    assert rc == 0, abi.error_string(rc)
    torch.cuda.synchronize()
    assert ws_view[:4].view(torch.int32).item() == 0
    assert _guards_intact(out_whole, out_bytes), "the kernel wrote outside `out`"
    assert _guards_intact(ws_whole, ws_bytes), "the kernel wrote outside its workspace"
    # every byte of `out` was written (no row left at the fill pattern) and equals the regular call
    import moonmath_attention as ma

    want = ma._kernel._forward_cuda(q, k, v, None, "rtne", layout, flags)
    torch.cuda.synchronize()
    assert torch.equal(out_view.view(torch.int16), want.view(torch.int16).reshape(-1))


def test_guard_words_around_the_lite_lists_and_output(abi, cuda_device):
    """LiteAttention writes a list row per task: rows, output and workspace must stay inside their buffers."""
    B, H, Sq, Skv = 1, 3, 700, 1000
    q, k, v = (t.to(cuda_device) for t in orc.make_inputs(B, H, Sq, Skv, "bhsd"))
    tile_m, tile_n = abi.lite_tile()
    qt, kt = -(-Sq // tile_m), -(-Skv // tile_n)
    n_list = B * H * qt * (kt + 2)
    rd_whole, rd = _guarded(n_list * 2, cuda_device)
    wr_whole, wr = _guarded(n_list * 2, cuda_device)
    rows = rd.view(torch.int16).view(B * H * qt, kt + 2)
    rows.zero_()
    rows[:, 0], rows[:, 1], rows[:, 2] = 2, kt - 1, -1   # the compute-all seed row, read with phase 1
    out_whole, out_view = _guarded(q.numel() * 2, cuda_device)
    ws_bytes = int(abi.lib.ma_lite_workspace_bytes(B, H, Sq))
    ws_whole, ws_view = _guarded(ws_bytes, cuda_device)
    rc = abi.lib.ma_attention_forward_lite(q.data_ptr(), k.data_ptr(), v.data_ptr(), out_view.data_ptr(), B, H, Sq, Skv,
                                           128, 0, 0, rd.data_ptr(), wr.data_ptr(), None, ctypes.c_float(-4.0), 1,
                                           ws_view.data_ptr(), ws_bytes, 0, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, abi.error_string(rc)
    torch.cuda.synchronize()
    assert ws_view[:4].view(torch.int32).item() == 0
    for whole, n in ((rd_whole, n_list * 2), (wr_whole, n_list * 2), (out_whole, q.numel() * 2), (ws_whole, ws_bytes)):
        assert _guards_intact(whole, n)
    assert np.all(wr.view(torch.int16).view(B * H * qt, kt + 2)[:, 0].cpu().numpy() >= 2)  # every task wrote a row
