"""Calls on a device other than the current one, and on two devices at once.  Needs two GPUs: -m gpu, skipped on one."""
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ma(cuda_device):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    import moonmath_attention

    return moonmath_attention


def test_tensors_on_a_non_current_device(ma):
    """The call follows the tensors' device, not the current one: workspace, stream and tensor maps belong to cuda:1."""
    assert torch.cuda.current_device() == 0
    q, k, v = orc.make_inputs(1, 40, 2048, 2048, "bhsd")  # a plan with a KV-split tail: the workspace holds partials
    want = ma.forward(q.to("cuda:0"), k.to("cuda:0"), v.to("cuda:0"), round_mode="rtne").cpu()
    got = ma.forward(q.to("cuda:1"), k.to("cuda:1"), v.to("cuda:1"), round_mode="rtne")
    assert got.device == torch.device("cuda:1") and torch.cuda.current_device() == 0
    torch.cuda.synchronize(1)
    assert ma.last_status(torch.device("cuda:1"))[0] == 0
    assert torch.equal(got.cpu().view(torch.int16), want.view(torch.int16))
    with pytest.raises(ValueError):
        ma.forward(q.to("cuda:0"), k.to("cuda:1"), v.to("cuda:0"))


def test_two_devices_run_concurrently(ma):
    """No state is shared between devices (the reference keeps one static schedule per process)."""
    a = [t.to("cuda:0") for t in orc.make_inputs(1, 40, 2048, 2048, "bhsd")]
    b = [t.to("cuda:1") for t in orc.make_inputs(1, 37, 512, 2304, "bhsd", base=7)]
    want_a, want_b = ma.forward(*a, round_mode="rtne").cpu(), ma.forward(*b, round_mode="rtz").cpu()
    for _ in range(3):
        got_a = ma.forward(*a, round_mode="rtne")
        got_b = ma.forward(*b, round_mode="rtz")
        torch.cuda.synchronize(0)
        torch.cuda.synchronize(1)
        assert torch.equal(got_a.cpu().view(torch.int16), want_a.view(torch.int16))
        assert torch.equal(got_b.cpu().view(torch.int16), want_b.view(torch.int16))


def test_host_tensors_follow_the_current_device(ma):
    """CPU tensors are computed on the process's current device (cuda:0 unless another was selected)."""
    q, k, v = (t.pin_memory() for t in orc.make_inputs(1, 4, 600, 700, "bhsd"))
    want = ma.forward(q, k, v, round_mode="rtne")
    with torch.cuda.device(1):
        got = ma.forward(q, k, v, round_mode="rtne")
        assert ma._kernel._SIDE_STREAMS.get(1) is not None
    assert got.device.type == "cpu" and torch.equal(got.view(torch.int16), want.view(torch.int16))
