"""Generates tests/golden/mla_reference.npz from the reference's own test helpers.

The reference checks its MLA decode kernels against `_reference`, a pure-torch fp32 formula in
tests/test_mla_decode.py:52-68, on inputs drawn by `_rand_kv` / `_rand_q` (:35-49) and, for the paged
entry points, scattered by `_paged_pool` (:75-96).  None of that needs a GPU.  This generator imports that
test module where it lies (with a stand-in for the `moonmath_attention` package, which the module imports
but these helpers never call), runs the helpers on the CPU and stores inputs and outputs, so that
oracle/mla_oracle.py can be checked against the reference's formula executed by the reference's code.
Nothing of the reference is copied.

    python tests/golden/make_golden_mla.py /path/to/reference

Stored per case (small shapes; fp8 bytes and bf16 bit patterns, no float round trip):
    kv        uint8  [B, S, 576]   the e4m3-fnuz cache bytes `_rand_kv` produced
    q_lat     uint16 [B, q_len, H, 512], q_pe uint16 [B, q_len, H, 64]   bf16 bits from `_rand_q`
    seq_lens  int64  [B]
    ref       float32 [B, q_len, H, 512]  `_reference(q_lat, q_pe, kv, seq_lens)`
and for the paged case the pool bytes, slot table and offsets `_paged_pool` made.
"""
from __future__ import annotations

import importlib.util
import sys
import types
from pathlib import Path

import numpy as np
import torch

CASES = {
    # name: (B, S, q_len or None, H, seq_lens, seed)
    "single": (1, 130, None, 3, [130], 11),
    "window": (2, 96, 4, 2, [96, 61], 23),        # ragged: the second request ends inside the slab
    "window8": (1, 80, 8, 1, [70], 31),
}


def _load_reference_test(ref_root: Path):
    stub = types.ModuleType("moonmath_attention")
    sys.modules["moonmath_attention"] = stub
    try:
        spec = importlib.util.spec_from_file_location("ref_test_mla_decode", ref_root / "tests" / "test_mla_decode.py")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    finally:
        del sys.modules["moonmath_attention"]
    return mod


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden_mla.py <checkout of the reference repository>")
    ref = _load_reference_test(Path(sys.argv[1]))
    cpu = torch.device("cpu")
    store = {"scale": np.float64(ref.SCALE), "kv_scale": np.float64(ref.KV_SCALE), "rel_l2_bar": np.float64(ref.REL_L2),
             "cases": np.array(sorted(CASES)), "torch_version": torch.__version__}
    for name, (B, S, q_len, H, seq_lens, seed) in CASES.items():
        kv = ref._rand_kv(B, S, cpu, seed)
        q_lat, q_pe, _ = ref._rand_q(B, q_len, H, cpu, seed)
        if q_len is None:
            q_lat, q_pe = q_lat.unsqueeze(1), q_pe.unsqueeze(1)
        out = ref._reference(q_lat, q_pe, kv, seq_lens)
        assert out.dtype == torch.float32 and kv.dtype == torch.float8_e4m3fnuz
        store[f"{name}/kv"] = kv.view(torch.uint8).numpy()
        store[f"{name}/q_lat"] = _bits(q_lat)
        store[f"{name}/q_pe"] = _bits(q_pe)
        store[f"{name}/seq_lens"] = np.array(seq_lens, dtype=np.int64)
        store[f"{name}/ref"] = out.numpy()
        if name == "window":
            pool, slots, indptr = ref._paged_pool(kv, seq_lens, cpu, seed)
            store[f"{name}/pool"] = pool.view(torch.uint8).numpy()
            store[f"{name}/slots"] = slots.numpy().astype(np.int32)
            store[f"{name}/indptr"] = indptr.numpy().astype(np.int32)
    out_path = Path(__file__).resolve().parent / "mla_reference.npz"
    np.savez_compressed(out_path, **store)
    print("wrote", out_path, out_path.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
