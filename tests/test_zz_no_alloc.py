"""`ma_attention_forward_static`: the entry point for callers that may not allocate device memory.

Some callers of this library cannot call cudaMalloc or keep a workspace of their own: a plug-in that
is handed only its input and output buffers, code that runs inside another framework's fixed memory
pool, or a host thread for which an allocation (which may synchronise the device) is not acceptable.
For them the scratch lives in a static device array inside the library.  This file checks, through
the C ABI, that the variant gives exactly what the regular entry point gives, twice in a row (the
array keeps the previous call's contents, so the second call proves nothing stale is read), and that
a problem whose plan outgrows the array is refused before anything runs.

Collected last on purpose (file name): a run that stops at the first failure has then already run
every other test.  Needs a B200: -m gpu.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def abi(cuda_device):
    from moonmath_attention import _abi

    return _abi


def _regular(abi, q, k, v, B, H, Sq, Skv, layout, mode):
    out = torch.empty_like(q)
    sms = torch.cuda.get_device_properties(q.device).multi_processor_count
    ws_bytes = abi.workspace_bytes(B, H, Sq, Skv, sms, 0)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
    rc = abi.lib.ma_attention_forward(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, H, Sq, Skv, 128,
                                      abi.LAYOUT[layout], abi.ROUND_MODE[mode], ws.data_ptr(), ws_bytes, 0,
                                      torch.cuda.current_stream().cuda_stream)
    assert rc == 0, abi.error_string(rc)
    torch.cuda.synchronize()
    assert ws[:4].view(torch.int32).item() == 0
    return out


def _static(abi, q, k, v, B, H, Sq, Skv, layout, mode, flags=0):
    out = torch.full_like(q, float("nan"))
    stream = torch.cuda.current_stream().cuda_stream
    rc = abi.lib.ma_attention_forward_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, H, Sq, Skv,
                                             128, abi.LAYOUT[layout], abi.ROUND_MODE[mode], flags, stream)
    assert rc == 0, abi.error_string(rc)
    words = (ctypes.c_uint32 * 4)()
    assert abi.lib.ma_static_status(words, 4, stream) == 0
    assert words[0] == 0, f"device status {list(words)}"
    return out


@pytest.mark.parametrize("case", [
    (1, 40, 2048, 2048, "bhsd", "rtne"),   # two full rounds and a KV-split tail: the scratch holds partial results
    (2, 3, 300, 333, "bshd", "rtz"),       # ragged, no split: only the status block of the scratch is used
])
def test_static_scratch_variant_matches_regular_entry_point(abi, cuda_device, case):
    B, H, Sq, Skv, layout, mode = case
    sms = torch.cuda.get_device_properties(cuda_device).multi_processor_count
    plan = abi.plan_tail(B, H, Sq, Skv, sms, 0)
    if (B, H) == (1, 40):
        assert plan["tail_tasks"] > 0, "this case must use the scratch for partial results"
    assert abi.workspace_bytes(B, H, Sq, Skv, sms, 0) <= abi.STATIC_SCRATCH_BYTES
    q, k, v = (t.to(cuda_device) for t in orc.make_inputs(B, H, Sq, Skv, layout))
    want = orc.bf16_tensor_to_bits(_regular(abi, q, k, v, B, H, Sq, Skv, layout, mode))
    # two calls in a row on the same stream; between them the scratch is dirtied by a different problem
    got1 = orc.bf16_tensor_to_bits(_static(abi, q, k, v, B, H, Sq, Skv, layout, mode))
    q2, k2, v2 = (t.to(cuda_device) for t in orc.make_inputs(1, 37, 512, 2304, "bhsd", base=7))
    _static(abi, q2, k2, v2, 1, 37, 512, 2304, "bhsd", "rtna")
    got2 = orc.bf16_tensor_to_bits(_static(abi, q, k, v, B, H, Sq, Skv, layout, mode))
    # same kernels, same plan, deterministic arithmetic: the tolerance of the comparison is zero
    assert np.array_equal(got1, want)
    assert np.array_equal(got2, want)


def test_static_scratch_variant_allocates_no_device_memory(abi, cuda_device):
    """What the entry point is for: after its first call on a device (which looks the array's address up),
    further calls leave the device's free memory exactly where it was -- no cudaMalloc, no pool growth."""
    B, H, Sq, Skv, layout, mode = 1, 40, 2048, 2048, "bhsd", "rtne"
    q, k, v = (t.to(cuda_device) for t in orc.make_inputs(B, H, Sq, Skv, layout))
    out = torch.empty_like(q)
    stream = torch.cuda.current_stream().cuda_stream

    def call():
        rc = abi.lib.ma_attention_forward_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, H, Sq,
                                                 Skv, 128, abi.LAYOUT[layout], abi.ROUND_MODE[mode], 0, stream)
        assert rc == 0, abi.error_string(rc)

    call()  # set-up call
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(cuda_device)
    reserved_before = torch.cuda.memory_reserved(cuda_device)
    for _ in range(5):
        call()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(cuda_device)
    assert free_after == free_before, (free_before, free_after)
    assert torch.cuda.memory_reserved(cuda_device) == reserved_before  # torch's allocator was not asked either


def test_static_scratch_variant_refuses_plans_beyond_its_buffer(abi, cuda_device):
    """76 tasks x 256 key blocks: the planner wants ~130 MB of partial results; the variant must refuse
    before launching (the tensors are never read), and must accept the same problem without the split."""
    B, H, Sq, Skv = 1, 76, 256, 32768
    sms = torch.cuda.get_device_properties(cuda_device).multi_processor_count
    if abi.workspace_bytes(B, H, Sq, Skv, sms, 0) <= abi.STATIC_SCRATCH_BYTES:
        pytest.skip("on this device the plan fits the static buffer")
    q = torch.zeros(B, H, Sq, 128, dtype=torch.bfloat16, device=cuda_device)
    kv = torch.zeros(B, H, Skv, 128, dtype=torch.bfloat16, device=cuda_device)
    out = torch.zeros_like(q)
    stream = torch.cuda.current_stream().cuda_stream
    rc = abi.lib.ma_attention_forward_static(q.data_ptr(), kv.data_ptr(), kv.data_ptr(), out.data_ptr(), B, H, Sq,
                                             Skv, 128, 0, 0, 0, stream)
    assert rc == abi.ERR_STATIC_SCRATCH
    assert "scratch" in abi.error_string(rc)
    rc = abi.lib.ma_attention_forward_static(q.data_ptr(), kv.data_ptr(), kv.data_ptr(), out.data_ptr(), B, H, Sq,
                                             Skv, 128, 0, 0, abi.FLAG_NO_TAIL, stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.all(out == 0)  # softmax over equal scores of all-zero values
