"""Behaviour of the public call on a GPU beyond numerics: streams, `out=`, CPU tensors, concurrency.  -m gpu."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from helpers import assert_parity, weighted_abs_v

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ma(cuda_device):
    import moonmath_attention

    return moonmath_attention


def test_out_argument_is_used_and_returned(ma, cuda_device):
    q, k, v = (t.to(cuda_device) for t in orc.make_inputs(1, 2, 200, 300, "bhsd"))
    out = torch.empty_like(q)
    ret = ma.forward(q, k, v, out=out, round_mode="rtne")
    assert ret.data_ptr() == out.data_ptr()
    ref = ma.forward(q, k, v, round_mode="rtne")
    assert torch.equal(ret.view(torch.int16), ref.view(torch.int16))
    with pytest.raises(ValueError):
        ma.forward(q, k, v, out=torch.empty(1, 2, 201, 128, dtype=torch.bfloat16, device=cuda_device))
    with pytest.raises(TypeError):
        ma.forward(q, k, v, out=torch.empty_like(q, dtype=torch.float16))
    with pytest.raises(ValueError):
        ma.forward(q, k, v, out=torch.empty(1, 2, 128, 200, dtype=torch.bfloat16, device=cuda_device).transpose(2, 3))


def test_shape_errors_on_device(ma, cuda_device):
    q = torch.zeros(1, 2, 64, 128, dtype=torch.bfloat16, device=cuda_device)
    with pytest.raises(ValueError, match="head_dim"):
        ma.forward(q[..., :64].contiguous(), q[..., :64].contiguous(), q[..., :64].contiguous())
    with pytest.raises(ValueError, match="k shape"):
        ma.forward(q, torch.zeros(1, 3, 64, 128, dtype=torch.bfloat16, device=cuda_device), q)
    with pytest.raises(ValueError, match="v shape"):
        ma.forward(q, q, torch.zeros(1, 2, 65, 128, dtype=torch.bfloat16, device=cuda_device))
    with pytest.raises(ValueError, match="round_mode"):
        ma.forward(q, q, q, round_mode="nearest")
    with pytest.raises(ValueError, match="layout"):
        ma.forward(q, q, q, layout="sbhd")
    with pytest.raises(ValueError, match="contiguous"):
        ma.forward(q.transpose(1, 2), q.transpose(1, 2), q.transpose(1, 2))


def test_cpu_tensors_are_copied_to_the_gpu_and_back(ma, cuda_device):
    """The reference's convenience (moonmath_attention/_kernel.py:52-67): CPU in, CPU out, GPU arithmetic."""
    q, k, v = orc.make_inputs(1, 2, 96, 160, "bhsd")
    out = ma.forward(q, k, v, round_mode="rtne")
    assert out.device.type == "cpu" and out.dtype == torch.bfloat16
    on_gpu = ma.forward(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), round_mode="rtne").cpu()
    assert torch.equal(out.view(torch.int16), on_gpu.view(torch.int16))


@pytest.mark.parametrize("layout,shape", [("bhsd", (2, 6, 1500, 900)), ("bshd", (2, 5, 2100, 700))])
def test_host_tensor_pipeline_is_bit_identical_to_the_device_path(ma, cuda_device, layout, shape, monkeypatch):
    """Pinned CPU tensors travel in pieces over three streams (upload, kernel, download).  Each piece is an
    independent sub-problem made of whole 256-row query blocks, so the result equals the device path's bit for
    bit when neither splits its last round along KV; `out=` is filled and returned."""
    monkeypatch.setattr(ma._kernel, "_HOST_CHUNK_BYTES", 256 << 10)  # several pieces per batch at this size
    B, H, Sq, Skv = shape
    q, k, v = (t.pin_memory() for t in orc.make_inputs(B, H, Sq, Skv, layout))
    pieces = ma._kernel._host_chunks(B, H, Sq, layout)
    assert len(pieces) > 2 * B
    host_out = torch.empty_like(q).pin_memory()
    ret = ma.forward(q, k, v, out=host_out, round_mode="rtne", layout=layout)
    assert ret.data_ptr() == host_out.data_ptr() and ret.device.type == "cpu"
    monkeypatch.setenv("MOONMATH_NO_TAIL", "1")
    dev_out = ma.forward(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), round_mode="rtne", layout=layout).cpu()
    assert torch.equal(host_out.view(torch.int16), dev_out.view(torch.int16))
    # pageable tensors take the same route
    ret2 = ma.forward(q.clone(), k.clone(), v.clone(), round_mode="rtne", layout=layout)
    assert torch.equal(ret2.view(torch.int16), dev_out.view(torch.int16))


def test_runs_on_the_callers_current_stream(ma, cuda_device):
    """Work queued on a side stream before the call must be seen by the kernel (same-stream ordering),
    and the default stream must not need to be involved."""
    q, k, v = (t.to(cuda_device) for t in orc.make_inputs(1, 4, 512, 512, "bshd"))
    want = ma.forward(q, k, v, round_mode="rtne", layout="bshd")
    torch.cuda.synchronize()
    side = torch.cuda.Stream(device=cuda_device)
    q2 = torch.zeros_like(q)
    with torch.cuda.stream(side):
        big = torch.randn(64 << 20, device=cuda_device)  # keeps the stream busy for a while
        big.mul_(1.0001)
        q2.copy_(q, non_blocking=True)                   # the kernel must see this copy
        got = ma.forward(q2, k, v, round_mode="rtne", layout="bshd")
    side.synchronize()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def test_concurrent_calls_on_two_streams_do_not_interfere(ma, cuda_device):
    """No state is shared between calls (the reference keeps a static schedule and is single-stream only,
    csrc/attention_kernel.hip:1375-1378): two different problems with KV-split tails on two streams."""
    a = [t.to(cuda_device) for t in orc.make_inputs(1, 40, 2048, 2048, "bhsd")]
    b = [t.to(cuda_device) for t in orc.make_inputs(1, 37, 512, 2304, "bhsd", base=7)]
    want_a = ma.forward(*a, round_mode="rtne")
    want_b = ma.forward(*b, round_mode="rtz")
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(device=cuda_device), torch.cuda.Stream(device=cuda_device)
    for _ in range(3):
        with torch.cuda.stream(s1):
            got_a = ma.forward(*a, round_mode="rtne")
        with torch.cuda.stream(s2):
            got_b = ma.forward(*b, round_mode="rtz")
        s1.synchronize()
        s2.synchronize()
        assert torch.equal(got_a.view(torch.int16), want_a.view(torch.int16))
        assert torch.equal(got_b.view(torch.int16), want_b.view(torch.int16))


def test_workspaces_are_kept_per_stream_and_status_follows_the_stream(ma, cuda_device):
    """The package reuses one workspace per (device, stream, thread): calls on one stream share it (ordered, so
    safe), two streams never do, and `last_status()` reads the block of the current stream's latest call."""
    a = [t.to(cuda_device) for t in orc.make_inputs(1, 40, 2048, 2048, "bhsd")]   # plan with a KV-split tail
    b = [t.to(cuda_device) for t in orc.make_inputs(1, 3, 300, 300, "bhsd", base=3)]
    want_a, want_b = ma.forward(*a, round_mode="rtne"), ma.forward(*b, round_mode="rtne")
    torch.cuda.synchronize()
    ws = ma._kernel._WORKSPACES
    key_default = ma._kernel._slot_key(cuda_device)
    assert key_default in ws
    big = ws[key_default].data_ptr()
    ma.forward(*b, round_mode="rtne")                      # a smaller problem on the same stream: same buffer
    assert ws[key_default].data_ptr() == big
    side = torch.cuda.Stream(device=cuda_device)
    with torch.cuda.stream(side):
        got_a = ma.forward(*a, round_mode="rtne")
        key_side = ma._kernel._slot_key(cuda_device)
        assert key_side != key_default and ws[key_side].data_ptr() != big
        # interleave: the default stream runs the other problem while the side stream's call is in flight
        with torch.cuda.stream(torch.cuda.default_stream(cuda_device)):
            got_b = ma.forward(*b, round_mode="rtne")
        assert ma.last_status()[0] == 0                    # the side stream's block
    torch.cuda.synchronize()
    assert ma.last_status()[0] == 0                        # the default stream's block
    assert torch.equal(got_a.view(torch.int16), want_a.view(torch.int16))
    assert torch.equal(got_b.view(torch.int16), want_b.view(torch.int16))
    assert len(ws) <= ma._kernel._WORKSPACE_SLOTS


def test_forward_and_lite_replay_from_a_cuda_graph(ma, cuda_device, monkeypatch):
    """The dense call (memset, main kernel and, where the plan splits the last wave, merge; 240 tasks here) and a
    LiteAttention call keep no host state between launches: captured once, they replay bit-identically on new data."""
    monkeypatch.delenv("MOONMATH_CHECK", raising=False)  # the check synchronises after every call
    g = torch.Generator(device=cuda_device)
    g.manual_seed(9)
    q, k, v = (torch.randn(1, 1300, 40, 128, generator=g, device=cuda_device).bfloat16() for _ in range(3))
    out = torch.empty_like(q)
    lists = torch.zeros(2, 1, 40, 6, 23, dtype=torch.int16, device=cuda_device)  # ceil(1300/256) x (ceil(1300/64) + 2)
    lists[0, ..., 0], lists[0, ..., 1], lists[0, ..., 2] = 2, 20, -1
    out_lite = torch.empty_like(q)

    def calls():
        ma.forward(q, k, v, out=out, layout="bshd", round_mode="rtna")
        ma.forward_lite(q, k, v, lists[0], lists[1], threshold=-1000.0, phase=1, out=out_lite, layout="bshd", round_mode="rtna")

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        calls()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        calls()
    q.copy_(torch.randn(q.shape, generator=g, device=cuda_device).bfloat16())
    graph.replay()
    torch.cuda.synchronize()
    got, got_lite = out.clone(), out_lite.clone()
    calls()
    torch.cuda.synchronize()
    assert ma.last_status()[0] == 0
    assert torch.equal(got.view(torch.int16), out.view(torch.int16))
    assert torch.equal(got_lite.view(torch.int16), out_lite.view(torch.int16))


def test_randomised_shapes_against_the_oracle(ma):
    """Seeded sweep over batch, heads, ragged lengths, layouts and modes (small enough for the CPU oracle)."""
    rng = np.random.default_rng(2026)
    for case in range(24):
        B, H = int(rng.integers(1, 4)), int(rng.integers(1, 7))
        sq = int(rng.choice([1, 2, 31, 100, 128, 129, 255, 256, 257, 400, 513, 700]))
        skv = int(rng.choice([1, 3, 64, 65, 127, 128, 130, 300, 512, 777, 1025, 1400]))
        layout = ("bhsd", "bshd")[case % 2]
        mode = orc.ROUND_MODES[case % 3]
        q, k, v = orc.make_inputs(B, H, sq, skv, layout, base=100 + case)
        dev = torch.device("cuda:0")
        out = ma.forward(q.to(dev), k.to(dev), v.to(dev), round_mode=mode, layout=layout)
        torch.cuda.synchronize()
        ref = orc.attention_fp32(q, k, v, layout).numpy()
        wabs = weighted_abs_v(q, k, v, layout).numpy()
        assert_parity(orc.bf16_tensor_to_bits(out), ref, wabs, mode, f"case {case}: {(B, H, sq, skv, layout, mode)}",
                      skv=skv)
