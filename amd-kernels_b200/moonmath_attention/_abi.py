"""ctypes binding of libmoonmath_attention_sm100.so (C ABI: include/moonmath_attention.h).

Plays the part of the reference's torch/pybind module `moonmath_attention._C`
(csrc/attention_api.cpp:441-473).  Importing this module fails loudly when the
library is missing: there is no fallback implementation.
"""

from __future__ import annotations

import ctypes
import os
from pathlib import Path

LIB_NAME = "libmoonmath_attention_sm100.so"
LIB_PATH = Path(__file__).resolve().parent / LIB_NAME

ABI_VERSION = 1

LAYOUT = {"bhsd": 0, "bshd": 1}
ROUND_MODE = {"rtne": 0, "rtna": 1, "rtz": 2}

FLAG_NO_TAIL = 0x1
FLAG_SIMPLE = 0x2
FLAG_EXACT_MAX = 0x8
FLAG_PRECISE_P = 0x10
FLAG_LITE_PLAIN = 0x20

STATIC_SCRATCH_BYTES = 40 << 20  # MA_STATIC_SCRATCH_BYTES
ERR_STATIC_SCRATCH = 16
ERR_FLAGS = 19
ERR_WAIT_TIMEOUT = 0x57A17  # device status word 0 when a bounded wait gave up

# every symbol include/moonmath_attention.h declares
EXPORTS = (
    "ma_abi_version",
    "ma_error_string",
    "ma_device_sms",
    "ma_workspace_bytes",
    "ma_plan_tail",
    "ma_attention_forward",
    "ma_attention_forward_static",
    "ma_static_status",
    "ma_round_bf16",
    "ma_selftest_wait_timeout",
    "ma_lite_workspace_bytes",
    "ma_lite_tile",
    "ma_attention_forward_lite",
    "ma_mla_plan_parts",
    "ma_mla_plan_parts_contiguous",
    "ma_mla_workspace_bytes",
    "ma_mla_cluster_capacity",
    "ma_mla_decode_a16w8",
)


def _load() -> ctypes.CDLL:
    path = os.environ.get("MOONMATH_ATTENTION_LIB", str(LIB_PATH))
    if not os.path.exists(path):
        raise ImportError(
            f"moonmath_attention: {path} not found. Build it with "
            "`python amd-kernels_b200/build.py` (needs nvcc with sm_100a support)."
        )
    lib = ctypes.CDLL(path)
    c_int, c_void_p, c_size_t = ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t
    lib.ma_abi_version.restype = c_int
    lib.ma_abi_version.argtypes = []
    lib.ma_error_string.restype = ctypes.c_char_p
    lib.ma_error_string.argtypes = [c_int]
    lib.ma_device_sms.restype = c_int
    lib.ma_device_sms.argtypes = []
    lib.ma_workspace_bytes.restype = c_size_t
    lib.ma_workspace_bytes.argtypes = [c_int] * 6
    lib.ma_plan_tail.restype = c_int
    lib.ma_plan_tail.argtypes = [c_int] * 6 + [ctypes.POINTER(c_int)]
    lib.ma_attention_forward.restype = c_int
    lib.ma_attention_forward.argtypes = (
        [c_void_p] * 4 + [c_int] * 7 + [c_void_p, c_size_t, c_int, c_void_p]
    )
    lib.ma_attention_forward_static.restype = c_int
    lib.ma_attention_forward_static.argtypes = [c_void_p] * 4 + [c_int] * 8 + [c_void_p]
    lib.ma_static_status.restype = c_int
    lib.ma_static_status.argtypes = [c_void_p, c_int, c_void_p]
    lib.ma_selftest_wait_timeout.restype = c_int
    lib.ma_selftest_wait_timeout.argtypes = [ctypes.c_uint64, c_void_p, c_size_t, c_void_p]
    lib.ma_round_bf16.restype = c_int
    lib.ma_round_bf16.argtypes = [c_void_p, c_void_p, c_size_t, c_int, c_void_p]
    lib.ma_lite_workspace_bytes.restype = c_size_t
    lib.ma_lite_workspace_bytes.argtypes = [c_int] * 3
    lib.ma_lite_tile.restype = None
    lib.ma_lite_tile.argtypes = [ctypes.POINTER(c_int), ctypes.POINTER(c_int)]
    lib.ma_attention_forward_lite.restype = c_int
    lib.ma_attention_forward_lite.argtypes = (
        [c_void_p] * 4 + [c_int] * 7 + [c_void_p] * 3 + [ctypes.c_float, c_int, c_void_p, c_size_t, c_int, c_void_p]
    )
    lib.ma_mla_plan_parts.restype = c_int
    lib.ma_mla_plan_parts.argtypes = [c_int] * 4
    lib.ma_mla_plan_parts_contiguous.restype = c_int
    lib.ma_mla_plan_parts_contiguous.argtypes = [c_int] * 4
    lib.ma_mla_workspace_bytes.restype = c_size_t
    lib.ma_mla_workspace_bytes.argtypes = [c_int] * 3
    lib.ma_mla_cluster_capacity.restype = c_int
    lib.ma_mla_cluster_capacity.argtypes = [c_int] * 3
    lib.ma_mla_decode_a16w8.restype = c_int
    lib.ma_mla_decode_a16w8.argtypes = (
        [c_void_p] * 8 + [c_int] * 5 + [ctypes.c_float, ctypes.c_float, c_int, c_void_p, c_size_t, c_void_p]
    )
    if lib.ma_abi_version() != ABI_VERSION:
        raise ImportError(
            f"moonmath_attention: {path} has ABI version {lib.ma_abi_version()}, expected {ABI_VERSION}; rebuild it"
        )
    return lib


lib = _load()


def error_string(rc: int) -> str:
    return lib.ma_error_string(int(rc)).decode()


def plan_tail(batch: int, heads: int, seq_len: int, seq_len_kv: int, num_sms: int, flags: int = 0) -> dict:
    """The KV-split decision for a problem on `num_sms` SMs (host arithmetic only)."""
    arr = (ctypes.c_int * 8)()
    rc = lib.ma_plan_tail(batch, heads, seq_len, seq_len_kv, num_sms, flags, arr)
    if rc != 0:
        raise ValueError(f"ma_plan_tail: {error_string(rc)} (rc={rc})")
    keys = ("tasks", "full_units", "tail_tasks", "split", "total_units", "grid", "nqb", "nkb")
    return dict(zip(keys, arr))


def workspace_bytes(batch: int, heads: int, seq_len: int, seq_len_kv: int, num_sms: int, flags: int = 0) -> int:
    return int(lib.ma_workspace_bytes(batch, heads, seq_len, seq_len_kv, num_sms, flags))


def lite_tile() -> tuple[int, int]:
    """(query rows per skip-list row, keys per skip-list block) of the LiteAttention kernel."""
    m, n = ctypes.c_int(0), ctypes.c_int(0)
    lib.ma_lite_tile(ctypes.byref(m), ctypes.byref(n))
    return m.value, n.value
