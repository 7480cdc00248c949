"""`forward` keeps the reference's signature, defaults and exception types
(moonmath_attention/_kernel.py:14-82, csrc/attention_api.cpp:134-229)."""
import inspect

import pytest
import torch

import moonmath_attention as ma


def _t(*shape, dtype=torch.bfloat16):
    return torch.zeros(*shape, dtype=dtype)


def test_signature_and_defaults():
    sig = inspect.signature(ma.forward)
    names = list(sig.parameters)
    assert names[:3] == ["q", "k", "v"]
    assert sig.parameters["out"].default is None and sig.parameters["out"].kind is inspect.Parameter.KEYWORD_ONLY
    assert sig.parameters["round_mode"].default == "rtna"  # _kernel.py:20 (the code, not the README)
    assert sig.parameters["layout"].default == "bhsd"      # _kernel.py:21


def test_type_errors():
    q = _t(1, 1, 8, 128)
    with pytest.raises(TypeError):
        ma.forward([1, 2], q, q)
    with pytest.raises(TypeError):
        ma.forward(q.float(), q, q)
    with pytest.raises(TypeError):
        ma.forward(q, q, q.half())


def test_rank_error():
    q = _t(1, 1, 8, 128)
    with pytest.raises(ValueError):
        ma.forward(_t(1, 8, 128), q, q)


def test_mixed_devices():
    q = _t(1, 1, 8, 128)
    meta = torch.zeros(1, 1, 8, 128, dtype=torch.bfloat16, device="meta")
    with pytest.raises(ValueError):
        ma.forward(q, meta, q)
    with pytest.raises(NotImplementedError):
        ma.forward(meta, meta, meta)


def test_shape_and_string_validation_cuda_path():
    """The checks of the binding run before the launch; drive them with the internal entry on CPU tensors."""
    from moonmath_attention._kernel import _forward_cuda

    q = _t(1, 2, 8, 128)
    with pytest.raises(ValueError, match="round_mode"):
        _forward_cuda(q, q, q, None, "rtx", "bhsd", 0)
    with pytest.raises(ValueError, match="layout"):
        _forward_cuda(q, q, q, None, "rtne", "hbsd", 0)
    with pytest.raises(ValueError, match="contiguous"):
        _forward_cuda(q.transpose(1, 2), q, q, None, "rtne", "bhsd", 0)
    with pytest.raises(ValueError, match="CUDA device"):
        _forward_cuda(q, q, q, None, "rtne", "bhsd", 0)
