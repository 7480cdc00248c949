"""Generates tests/golden/lite_reference.npz from the reference's own Python.

The reference's LiteAttention kernel is HIP and cannot run here, but three pieces of its Python can, on the
CPU, and together they pin what the skip lists of this library must look like:

* `moonmath_attention/lite.py` (the wrapper class): executed with a stand-in for its `_kernel` module that
  records the calls.  Stored: the compute-all seed the class builds (`_ensure`, lite.py:108-128), and the
  (read buffer, write buffer, phase) sequence of three successive calls (lite.py:133-157), i.e. the double
  buffer protocol.
* `tests/test_attention.py::_kept_blocks` (:145-150): the decoder of a list row, run on sample rows,
  the planner's worked example (csrc/attention_kernel.hip:1318-1319) among them.
* `tests/test_attention.py::_lite_qkv_peaked` (:118-138): the data recipe of its skip-list test, run on the
  CPU.  The tensors are 8 MB each, so only their hashes are stored, with the shape, threshold and step count of
  that test and the kept-block count per head it asserts after those steps (1..H, :214).  A block count in
  64-key blocks does not depend on how many query rows share a list row, so it carries over to this
  library's 256-row geometry (the reference: 384).

Both reference files are executed where they lie; nothing of them is copied.

    python tests/golden/make_golden_lite.py /path/to/reference
"""
from __future__ import annotations

import hashlib
import importlib.util
import sys
import types
from pathlib import Path

import numpy as np
import torch

SAMPLE_ROWS = [
    [4, 9, 5, 20, 18],          # the planner's worked example: kept 6
    [2, 63, -1],                # a compute-all seed for 64 key blocks, walked upwards
    [2, 0, 64],                 # the same set written by a downward walk
    [6, 3, 1, 10, 7, 40, 30],
    [0, 0, 0],
    [2, 5, 4],
]


def _load(path: Path, name: str, package: str | None = None):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    if package:
        mod.__package__ = package
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def _sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.int16).numpy().tobytes()).hexdigest()


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden_lite.py <checkout of the reference repository>")
    ref_root = Path(sys.argv[1])
    calls = []

    # --- the wrapper class, with a recording stand-in for the extension-backed module --------------------
    pkg = types.ModuleType("moonmath_attention")
    pkg.__path__ = []
    kern = types.ModuleType("moonmath_attention._kernel")

    def forward_lite(q, k, v, read_list, write_list, *, threshold, phase, must_do_list=None, out=None, round_mode="rtna",
                     layout="bhsd"):
        calls.append((read_list.data_ptr(), write_list.data_ptr(), int(phase), float(threshold)))
        return torch.zeros_like(q)

    kern.forward_lite = forward_lite
    kern.forward = lambda q, k, v, **kw: torch.zeros_like(q)
    pkg._kernel = kern
    saved = {n: sys.modules.get(n) for n in ("moonmath_attention", "moonmath_attention._kernel", "moonmath_attention.lite")}
    sys.modules["moonmath_attention"] = pkg
    sys.modules["moonmath_attention._kernel"] = kern
    try:
        lite = _load(ref_root / "moonmath_attention" / "lite.py", "moonmath_attention.lite", "moonmath_attention")
        pkg.LiteAttention = lite.LiteAttention
        B, H, Sq, Skv = 1, 2, 1000, 777
        q = torch.zeros(B, H, Sq, 128, dtype=torch.bfloat16)
        k = torch.zeros(B, H, Skv, 128, dtype=torch.bfloat16)
        attn = lite.LiteAttention(threshold=-3.0)
        for _ in range(3):
            attn(q, k, k)
        skip = attn._skip
        buf = {skip[0].data_ptr(): 0, skip[1].data_ptr(): 1}
        protocol = np.array([[buf[r], buf[w], ph] for r, w, ph, _ in calls], dtype=np.int64)
        ref_m, ref_n = lite.LiteAttention.get_MN()
        # what a fresh object builds before its first call
        fresh = lite.LiteAttention(threshold=-3.0)
        fresh._ensure(q, k)
        seed = fresh._skip.numpy().copy()

        # --- the reference's test helpers ------------------------------------------------------------
        tests = _load(ref_root / "tests" / "test_attention.py", "ref_test_attention")
        kept_samples = np.array([tests._kept_blocks(torch.tensor(r, dtype=torch.int16)) for r in SAMPLE_ROWS], dtype=np.int64)
        qp, kp, vp = tests._lite_qkv_peaked(torch.device("cpu"), "bshd")
        shape = tests.LITE_SHAPE
    finally:
        for n, m in saved.items():
            if m is None:
                sys.modules.pop(n, None)
            else:
                sys.modules[n] = m

    width = max(len(r) for r in SAMPLE_ROWS)
    rows = np.zeros((len(SAMPLE_ROWS), width), dtype=np.int16)
    for i, r in enumerate(SAMPLE_ROWS):
        rows[i, :len(r)] = r
    out = Path(__file__).resolve().parent / "lite_reference.npz"
    np.savez_compressed(
        out,
        ref_tile=np.array([ref_m, ref_n], dtype=np.int64),
        seed_shape_args=np.array([B, H, Sq, Skv], dtype=np.int64),
        seed=seed,                       # int16 [2, B, H, ceil(Sq / ref_m), ceil(Skv / ref_n) + 2]
        protocol=protocol,               # per call: read buffer index, write buffer index, phase passed to the kernel
        sample_rows=rows, sample_kept=kept_samples,
        peaked_shape=np.array([shape.B, shape.S, shape.H, shape.D], dtype=np.int64),
        peaked_sha=np.array([_sha(qp), _sha(kp), _sha(vp)]),
        peaked_threshold=np.float64(tests.LITE_THRESHOLD), peaked_steps=np.int64(tests.LITE_STEPS),
        peaked_kept_by_head=np.arange(1, shape.H + 1, dtype=np.int64),   # asserted by the reference's test (:214)
        torch_version=torch.__version__,
    )
    print("wrote", out, out.stat().st_size, "bytes;", "protocol", protocol.tolist(), "kept", kept_samples.tolist(),
          "tile", (ref_m, ref_n))


if __name__ == "__main__":
    main()
