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
    # the reference's parameters in its order, then the one addition, keyword-only and off by default
    assert names == ["q", "k", "v", "out", "round_mode", "layout", "precise"]
    assert sig.parameters["precise"].default is False and sig.parameters["precise"].kind is inspect.Parameter.KEYWORD_ONLY


def test_flags_come_from_the_documented_environment_switches_only(monkeypatch):
    from moonmath_attention import _abi, _kernel

    for name in ("MOONMATH_NO_TAIL", "MOONMATH_SIMPLE", "MOONMATH_EXACT_MAX", "MOONMATH_PRECISE_P", "MOONMATH_FLAGS"):
        monkeypatch.delenv(name, raising=False)
    assert _kernel._flags_from_env() == 0
    monkeypatch.setenv("MOONMATH_FLAGS", "0x800")       # the raw-bits switch of earlier builds is gone
    assert _kernel._flags_from_env() == 0
    monkeypatch.setenv("MOONMATH_NO_TAIL", "1")
    monkeypatch.setenv("MOONMATH_PRECISE_P", "1")
    assert _kernel._flags_from_env() == _abi.FLAG_NO_TAIL | _abi.FLAG_PRECISE_P


def test_host_tensor_pieces_cover_the_problem_in_whole_query_blocks():
    """The pieces the host-tensor path cuts a problem into: disjoint, complete, contiguous in host memory, and for
    bshd made of whole 256-row query blocks (so that a piece's result does not depend on the cut)."""
    from moonmath_attention import _kernel

    for B, H, Sq, layout in ((2, 24, 8192, "bshd"), (2, 24, 8192, "bhsd"), (3, 5, 1000, "bshd"), (1, 7, 96, "bhsd"),
                             (2, 3, 1, "bshd"), (1, 1, 70000, "bhsd"), (1, 40, 300, "bhsd")):
        pieces = _kernel._host_chunks(B, H, Sq, layout)
        extent = H if layout == "bhsd" else Sq
        for b in range(B):
            mine = sorted((lo, hi) for bb, lo, hi in pieces if bb == b)
            assert mine[0][0] == 0 and mine[-1][1] == extent
            assert all(a[1] == c[0] for a, c in zip(mine, mine[1:])) and all(lo < hi for lo, hi in mine)
            if layout == "bshd":
                assert all(lo % 256 == 0 for lo, _ in mine)
        per = (Sq * 128 * 2) if layout == "bhsd" else (H * 128 * 2)
        assert all((hi - lo) * per <= max(_kernel._HOST_CHUNK_BYTES, per if layout == "bhsd" else 256 * per)
                   for _, lo, hi in pieces)


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
