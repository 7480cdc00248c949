"""Generates tests/golden/basic_example.npz from the reference's own oracle code.

The reference's fp32 oracle for `forward` is the expression in
examples/basic.py:16-17.  That script cannot run as shipped (it calls the HIP
extension), so this generator executes the *unmodified file* with a stand-in
`moonmath_attention` module whose `forward` returns zeros, then reads the
script's own `q`, `k`, `v` and `ref` variables out of its namespace.  Nothing of
the reference is copied: its file is executed where it lies.

Run in the build container (needs the reference checkout):

    python tests/golden/make_golden.py [/path/to/reference]

Stored (small on purpose; q, k, v are regenerated from the script's seed and
verified by hash):
    rows      query rows kept
    ref_rows  fp32 oracle output ref[0, :, rows, :]            (4, len(rows), 128)
    sha_q/k/v sha256 of the bf16 bytes of q, k, v
    shape     (B, H, S, D);   seed;   torch version
"""

from __future__ import annotations

import hashlib
import runpy
import sys
import types
from pathlib import Path

import numpy as np
import torch

ROWS = [0, 1, 2, 63, 64, 127, 128, 255, 256, 511, 640, 777, 1000, 1022, 1023]


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <checkout of the reference repository>")
    ref_root = Path(sys.argv[1])
    script = ref_root / "examples" / "basic.py"
    stub = types.ModuleType("moonmath_attention")
    stub.forward = lambda q, k, v, **kw: torch.zeros_like(q)
    sys.modules["moonmath_attention"] = stub
    try:
        ns = runpy.run_path(str(script))
    finally:
        del sys.modules["moonmath_attention"]
    q, k, v, ref = ns["q"], ns["k"], ns["v"], ns["ref"]
    assert ref.dtype == torch.float32 and q.dtype == torch.bfloat16

    def sha(t: torch.Tensor) -> str:
        return hashlib.sha256(t.contiguous().view(torch.int16).numpy().tobytes()).hexdigest()

    out = Path(__file__).resolve().parent / "basic_example.npz"
    np.savez_compressed(
        out,
        rows=np.array(ROWS, dtype=np.int64),
        ref_rows=ref[0][:, ROWS, :].numpy(),
        sha_q=sha(q), sha_k=sha(k), sha_v=sha(v),
        shape=np.array(q.shape, dtype=np.int64),
        seed=np.int64(42),
        torch_version=torch.__version__,
    )
    print("wrote", out, out.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
