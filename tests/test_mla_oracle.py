"""CPU tests of the MLA oracle's cache-format tables, the planner and the argument checks of the C ABI."""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from moonmath_attention import _abi
from oracle import mla_oracle as mo


def test_fp8_tables_match_torch_for_every_code():
    codes = torch.arange(256, dtype=torch.uint8)
    for name, table, dt in (("fnuz", mo.decode_e4m3fnuz(), torch.float8_e4m3fnuz), ("fn", mo.decode_e4m3fn(), torch.float8_e4m3fn)):
        want = codes.view(dt).float().numpy()
        assert np.array_equal(np.isnan(table), np.isnan(want)), name
        ok = ~np.isnan(want)
        assert np.array_equal(table[ok], want[ok]), name


def test_fnuz_bytes_read_as_e4m3_are_twice_their_value():
    # what the kernel relies on: every finite code but the two the tensor-core format reserves for NaN
    fnuz, fn = mo.decode_e4m3fnuz(), mo.decode_e4m3fn()
    for b in range(256):
        if b in (0x80, 0x7F, 0xFF):
            continue
        assert fn[b] == 2 * fnuz[b], hex(b)
    assert fnuz[0x7F] == 240 and fnuz[0xFF] == -240 and fnuz[0x7E] == 224 and np.isnan(fnuz[0x80])


def test_oracle_is_the_softmax_formula_of_the_reference_test():
    rng = np.random.default_rng(3)
    B, q_len, H, S = 2, 3, 4, 40
    kv = torch.randn(B, S, mo.FUSED, generator=torch.Generator().manual_seed(1)).to(torch.float8_e4m3fnuz)
    q_lat = rng.standard_normal((B, q_len, H, 512)).astype(np.float32)
    q_pe = rng.standard_normal((B, q_len, H, 64)).astype(np.float32)
    out = mo.mla_decode(q_lat, q_pe, kv.view(torch.uint8).numpy(), [S, S - 5], 576 ** -0.5, 1 / 32)
    k = kv.float() / 32
    for b, slen in enumerate([S, S - 5]):
        for t in range(q_len):
            end = slen - q_len + t + 1
            score = (torch.from_numpy(q_lat[b, t]) @ k[b, :end, :512].T + torch.from_numpy(q_pe[b, t]) @ k[b, :end, 512:].T) * 576 ** -0.5
            want = torch.softmax(score, dim=-1) @ k[b, :end, :512]
            np.testing.assert_allclose(out[b, t], want.numpy(), rtol=2e-5, atol=1e-6)


def _golden():
    import os

    return np.load(os.path.join(os.path.dirname(__file__), "golden", "mla_reference.npz"))


def _bf16_bits_to_f32(bits):
    return (bits.astype(np.uint32) << 16).view(np.float32)


def test_oracle_reproduces_the_reference_tests_own_formula_on_its_own_inputs():
    """tests/golden/mla_reference.npz holds inputs drawn by the reference's `_rand_kv` / `_rand_q` and outputs of
    its `_reference` (tests/test_mla_decode.py:35-68), executed where they lie by tests/golden/make_golden_mla.py:
    the oracle must agree with them to fp32 noise, ragged lengths and every draft position included."""
    g = _golden()
    for name in g["cases"]:
        out = mo.mla_decode(_bf16_bits_to_f32(g[f"{name}/q_lat"]), _bf16_bits_to_f32(g[f"{name}/q_pe"]), g[f"{name}/kv"],
                            g[f"{name}/seq_lens"].tolist(), float(g["scale"]), float(g["kv_scale"]))
        ref = g[f"{name}/ref"]
        assert out.shape == ref.shape
        np.testing.assert_allclose(out, ref, rtol=3e-5, atol=2e-6, err_msg=str(name))
        assert mo.rel_l2(out, ref) < 1e-6


def test_pool_gather_reproduces_the_reference_tests_scatter():
    """`_paged_pool` (tests/test_mla_decode.py:75-96) scatters the rows over a shuffled pool; reading them back
    through the slot table must give the slab rows again."""
    g = _golden()
    lens = g["window/seq_lens"].tolist()
    rows = mo.gather_pool(g["window/pool"][:, 0], g["window/slots"], g["window/indptr"], lens)
    for b, n in enumerate(lens):
        assert np.array_equal(rows[b], g["window/kv"][b, :n])


def test_planner_fills_the_gpu_once_and_keeps_parts_long():
    plan = lambda B, q, S: _abi.lib.ma_mla_plan_parts(B, q, S, 148)
    assert plan(148, 1, 4096) == 1 and plan(300, 1, 4096) == 1
    assert plan(32, 1, 8192) == 4                # 148 // 32, 16 parts of four tiles available
    assert plan(16, 4, 8192) == 4                # a window of four positions is two CTAs per part
    assert plan(1, 1, 131072) == 148             # one long request still fills the GPU
    assert plan(1, 1, 131072 * 4) == 148
    assert plan(1, 1, 1000) == 2                 # 8 tiles: at least four tiles per part
    assert plan(1, 1, 100) == 1
    assert plan(0, 1, 100) == 1 and plan(1, 9, 100) == 1
    slab = lambda B, q, S: _abi.lib.ma_mla_plan_parts_contiguous(B, q, S, 148)
    assert slab(16, 4, 8192) == 4                # the contiguous launchers plan the same way
    assert slab(16, 5, 8192) == 3 and slab(148, 1, 4096) == 1 and slab(32, 1, 8192) == 4
    ws = _abi.lib.ma_mla_workspace_bytes
    assert ws(32, 1, 4) == 256 + 32 * 4 * 16 * 514 * 4
    assert ws(2, 8, 3) == 256 + 2 * 8 * 3 * 16 * 514 * 4


def test_mla_argument_validation_return_codes():
    def call(B=1, H=16, q_len=1, S=128, parts=1, fmt=0, q=16, idx=None, indptr=None, lens=None, ws=0, wsb=0):
        return _abi.lib.ma_mla_decode_a16w8(q, 16, 16, 16, lens, None, idx, indptr, B, H, q_len, S, parts,
                                            ctypes.c_float(0.04), ctypes.c_float(1.0), fmt, ws, wsb, None)
    assert call(B=0) == 1 and call(H=17) == 1 and call(H=0) == 1
    assert call(q_len=0) == 2 and call(q_len=9) == 2
    assert call(S=0) == 5 and call(idx=16) == 5          # paged needs kv_indptr and seq_lens
    assert call(parts=0) == 18 and call(parts=257) == 18 and call(fmt=2) == 18
    assert call(q=None) == 9 and call(q=8) == 10
    assert call() == 11                                    # workspace is required
    assert b"parts" in _abi.lib.ma_error_string(18)
