"""The C ABI without a GPU: the library loads, exports what the header declares, validates arguments."""
import ctypes
import os
import re

import pytest
import torch

import moonmath_attention as ma
from moonmath_attention import _abi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "moonmath_attention.h")


def _declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ma_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported():
    syms = _declared_symbols()
    assert set(syms) == set(_abi.EXPORTS)
    lib = ctypes.CDLL(str(_abi.LIB_PATH))
    for s in syms:
        assert hasattr(lib, s), s


def test_abi_version_and_error_strings():
    assert _abi.lib.ma_abi_version() == 1
    m = re.search(r"#define MA_ABI_VERSION (\d+)", open(HEADER).read())
    assert int(m.group(1)) == _abi.ABI_VERSION
    for rc in (0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15, 16, 17, 18, 19, 1001):
        assert _abi.error_string(rc) and "unknown" not in _abi.error_string(rc)
    assert "unknown" in _abi.error_string(20)


def _call(q=16, k=16, v=16, out=16, B=1, H=1, Sq=128, Skv=128, D=128, layout=0, mode=0, ws=0, wsb=0, flags=0):
    return _abi.lib.ma_attention_forward(q, k, v, out, B, H, Sq, Skv, D, layout, mode, ws, wsb, flags, 0)


def test_argument_validation_return_codes():
    """Codes 1, 2, 3, 5 as the reference's launcher (csrc/attention_kernel.hip:1573-1576); checks run before any CUDA call."""
    assert _call(B=0) == 1 and _call(H=-1) == 1
    assert _call(Sq=0) == 2
    assert _call(Skv=0) == 5
    assert _call(D=64) == 3
    assert _call(layout=2) == 7
    assert _call(mode=3) == 8
    assert _call(q=0) == 9 and _call(out=0) == 9
    assert _call(k=24) == 10
    assert _call(B=70000) == 15


def test_undefined_flag_bits_are_refused():
    """Every flag bit an entry point does not define is an error, not a silent no-op."""
    header = open(HEADER).read()
    defined = {name: int(val, 16) for name, val in re.findall(r"#define (MA_FLAG_[A-Z_]+) (0x[0-9a-fA-F]+)", header)}
    assert defined == {"MA_FLAG_NO_TAIL": 0x1, "MA_FLAG_SIMPLE": 0x2, "MA_FLAG_EXACT_MAX": 0x8,
                       "MA_FLAG_PRECISE_P": 0x10, "MA_FLAG_LITE_PLAIN": 0x20}
    assert (_abi.FLAG_NO_TAIL, _abi.FLAG_SIMPLE, _abi.FLAG_EXACT_MAX, _abi.FLAG_PRECISE_P, _abi.FLAG_LITE_PLAIN) == \
        (0x1, 0x2, 0x8, 0x10, 0x20)
    for bad in (0x4, 0x20, 0x40, 0x800, 0xB00, 1 << 30):
        assert _call(flags=bad) == _abi.ERR_FLAGS, hex(bad)
        assert _abi.lib.ma_attention_forward_static(16, 16, 16, 16, 1, 1, 128, 128, 128, 0, 0, bad, 0) == _abi.ERR_FLAGS
    lite = lambda flags: _abi.lib.ma_attention_forward_lite(16, 16, 16, 16, 1, 1, 128, 128, 128, 0, 0, 16, 16, None,
                                                            ctypes.c_float(-3.0), 1, 0, 0, flags, None)
    assert lite(0x1) == _abi.ERR_FLAGS and lite(0x10) == _abi.ERR_FLAGS and lite(0x20) == 11  # 11: workspace missing


def test_selftest_entry_validates_its_arguments():
    f = _abi.lib.ma_selftest_wait_timeout
    assert f(1000000, None, 256, None) == 9
    assert f(1000000, 128, 256, None) == 11          # misaligned
    assert f(1000000, 256, 64, None) == 11           # too small
    assert f(0, 256, 256, None) == 15 and f(10**9, 256, 256, None) == 15  # limit out of range


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the behaviour of a machine without a GPU")
def test_no_gpu_means_an_error_not_a_fallback():
    rc = _call()
    assert rc >= 1000, "a valid call without a CUDA device must fail with a CUDA error code"
    q = torch.zeros(1, 1, 8, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        ma.forward(q, q, q)


def test_mla_cluster_capacity_domain():
    """Outside 2..8 parts or q_len 1..8 there is no cluster; without a GPU the answer is 0 as well (a query, not a launch)."""
    cap = _abi.lib.ma_mla_cluster_capacity
    assert cap(1, 0, 1) == 0 and cap(1, 0, 9) == 0 and cap(0, 0, 4) == 0 and cap(9, 1, 4) == 0
    if not torch.cuda.is_available():
        assert cap(1, 0, 4) == 0 and cap(4, 1, 2) == 0


def test_round_bf16_rejects_bad_arguments():
    assert _abi.lib.ma_round_bf16(0, 0, 0, 5, 0) == 8
    assert _abi.lib.ma_round_bf16(0, 0, 4, 0, 0) == 9


def test_lite_argument_validation_return_codes():
    """ma_attention_forward_lite: codes 1, 2, 3, 4, 5 as the reference's launcher (csrc/attention_kernel.hip:1623-1627)."""
    def call(B=1, H=1, Sq=128, Skv=128, D=128, layout=0, mode=0, rl=16, wl=16, thr=-3.0, phase=1, ws=0, wsb=0, q=16):
        return _abi.lib.ma_attention_forward_lite(q, 16, 16, 16, B, H, Sq, Skv, D, layout, mode, rl, wl, None,
                                                  ctypes.c_float(thr), phase, ws, wsb, 0, None)
    assert call(B=0) == 1 and call(Sq=0) == 2 and call(D=64) == 3 and call(Skv=0) == 5
    assert call(rl=None) == 4 and call(wl=None) == 4
    assert call(layout=3) == 7 and call(mode=5) == 8 and call(q=None) == 9 and call(q=8) == 10
    assert call(thr=0.0) == 17 and call(phase=-1) == 17 and call(Skv=64 * 40000) == 17
    assert call() == 11  # workspace is required
    assert _abi.lib.ma_lite_workspace_bytes(2, 24, 8192) == 256 + 256 + 2 * 24 * 32 * 4
    assert _abi.lite_tile() == (256, 64)
