"""GPU tests of the MLA absorbed-decode operators through the C ABI.

The scenarios are those of the reference's tests (tests/test_mla_decode.py:97-221: fp32 reference over the same
dequantised fp8 KV, rel-L2 < 3e-3, peaked queries, end-aligned causal window, scattered paged pool, `rows`
remapping, domain errors), checked against oracle/mla_oracle.py; further cases cover what this implementation
adds or approximates (e4m3 caches, saturated fnuz codes, short and ragged sequences, every q_len, small H).
"""
from __future__ import annotations

from itertools import accumulate

import numpy as np
import pytest
import torch

from oracle import mla_oracle as mo

pytestmark = pytest.mark.gpu

LAT, ROPE, FUSED = 512, 64, 576
SCALE = FUSED ** -0.5
KV_SCALE = 1.0 / 32.0
QPEAK = 3.0
REL_L2 = mo.REL_L2


@pytest.fixture(scope="module")
def ma(cuda_device):
    import moonmath_attention

    return moonmath_attention


def _rand_kv(B, S, device, seed, dtype=torch.float8_e4m3fnuz):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(B, S, FUSED, generator=g).to(dtype).to(device)


def _rand_q(B, q_len, H, device, seed):
    g = torch.Generator().manual_seed(seed + 1)
    shape = (B, H) if q_len is None else (B, q_len, H)
    q_lat = (torch.randn(*shape, LAT, generator=g) * QPEAK).to(torch.bfloat16).to(device)
    q_pe = (torch.randn(*shape, ROPE, generator=g) * QPEAK).to(torch.bfloat16).to(device)
    return q_lat, q_pe, torch.zeros_like(q_lat)


def _oracle(q_lat, q_pe, kv, seq_lens, fmt="fnuz"):
    if q_lat.dim() == 3:
        q_lat, q_pe = q_lat.unsqueeze(1), q_pe.unsqueeze(1)
    return mo.mla_decode(q_lat.float().cpu().numpy(), q_pe.float().cpu().numpy(), kv.view(torch.uint8).cpu().numpy(),
                         seq_lens, SCALE, KV_SCALE, fmt)


def _check(ma, o_lat, ref, what=""):
    out = o_lat.float().cpu().numpy().reshape(ref.shape)
    assert ma.last_status()[0] == 0, f"{what}: device status {ma.last_status()[:3]}"
    assert not np.isnan(out).any(), what
    assert mo.rel_l2(out, ref) < REL_L2, f"{what}: rel-L2 {mo.rel_l2(out, ref):.2e}"


def _paged_pool(kv, seq_lens, device, seed):
    """Scatter the requests' rows over a shared pool in a random permutation of the slots."""
    total = sum(seq_lens)
    g = torch.Generator().manual_seed(seed + 2)
    slots = torch.randperm(total, generator=g).to(torch.int32)
    pool = torch.zeros(total, 1, FUSED, dtype=torch.uint8)
    off = 0
    for b, n in enumerate(seq_lens):
        pool[slots[off:off + n].long(), 0] = kv[b, :n].cpu().view(torch.uint8)
        off += n
    indptr = torch.tensor([0, *accumulate(seq_lens)], dtype=torch.int32)
    return pool.view(kv.dtype).to(device), slots.to(device), indptr.to(device)


# ---- the reference's scenarios ---------------------------------------------------------------------------------
def test_kernel_against_outputs_of_the_reference_tests_own_formula(ma, cuda_device):
    """The fixture holds inputs drawn and outputs computed by the reference's own test helpers
    (tests/test_mla_decode.py:35-96, run by tests/golden/make_golden_mla.py): the kernels are held to the
    reference's bar (rel-L2 < 3e-3) against those outputs directly, contiguous and through the scattered pool."""
    import os

    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "mla_reference.npz"))
    scale, kv_scale, bar = float(g["scale"]), float(g["kv_scale"]), float(g["rel_l2_bar"])
    bf16 = lambda bits: torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16).to(cuda_device)  # noqa: E731
    for name in g["cases"]:
        q_lat, q_pe = bf16(g[f"{name}/q_lat"]), bf16(g[f"{name}/q_pe"])
        B, q_len, H, _ = q_lat.shape
        lens = g[f"{name}/seq_lens"].tolist()
        kv = torch.from_numpy(g[f"{name}/kv"].copy()).view(torch.float8_e4m3fnuz).to(cuda_device)
        ref = g[f"{name}/ref"]
        o_lat = torch.zeros_like(q_lat)
        lens_dev = torch.tensor(lens, dtype=torch.int32, device=cuda_device)
        if q_len == 1 and lens == [kv.size(1)] * B:
            ma.mla_decode_a16w8(q_lat[:, 0].contiguous(), q_pe[:, 0].contiguous(), kv, o_lat[:, 0], scale, kv_scale)
            torch.cuda.synchronize()
            assert mo.rel_l2(o_lat.float().cpu().numpy(), ref) < bar, name
        if f"{name}/pool" in g.files:
            pool = torch.from_numpy(g[f"{name}/pool"].copy()).view(torch.float8_e4m3fnuz).to(cuda_device)
            slots = torch.from_numpy(g[f"{name}/slots"].copy()).to(cuda_device)
            indptr = torch.from_numpy(g[f"{name}/indptr"].copy()).to(cuda_device)
        else:  # a pool in token order: the paged entry points take any q_len in 1..8 and ragged lengths
            pool = torch.cat([kv[b, :n] for b, n in enumerate(lens)]).unsqueeze(1).contiguous()
            slots = torch.arange(sum(lens), dtype=torch.int32, device=cuda_device)
            indptr = torch.tensor([0, *accumulate(lens)], dtype=torch.int32, device=cuda_device)
        o2 = torch.zeros_like(q_lat)
        ma.mla_decode_a16w8_paged_dev(q_lat if q_len > 1 else q_lat[:, 0].contiguous(), q_pe if q_len > 1 else q_pe[:, 0].contiguous(),
                                      pool, o2 if q_len > 1 else o2[:, 0], lens_dev, None, slots, indptr, 1, scale, kv_scale)
        torch.cuda.synchronize()
        assert ma.last_status()[0] == 0
        assert mo.rel_l2(o2.float().cpu().numpy(), ref) < bar, f"{name} paged"


@pytest.mark.parametrize("H", [12, 16])
def test_single_query_matches_reference(ma, cuda_device, H):
    B, S = 2, 2048
    kv = _rand_kv(B, S, cuda_device, 11)
    q_lat, q_pe, o_lat = _rand_q(B, None, H, cuda_device, 11)
    ma.mla_decode_a16w8(q_lat, q_pe, kv, o_lat, SCALE, KV_SCALE)
    _check(ma, o_lat, _oracle(q_lat, q_pe, kv, [S] * B), f"q_len 1 H {H}")


@pytest.mark.parametrize("q_len", [4, 5, 8])
@pytest.mark.parametrize("H", [12, 16])
def test_multiq_contiguous_matches_reference(ma, cuda_device, q_len, H):
    B, S = 2, 2048
    kv = _rand_kv(B, S, cuda_device, 23)
    q_lat, q_pe, o_lat = _rand_q(B, q_len, H, cuda_device, 23)
    ma.mla_decode_a16w8_multiq(q_lat, q_pe, kv, o_lat, SCALE, KV_SCALE)
    _check(ma, o_lat, _oracle(q_lat, q_pe, kv, [S] * B), f"multiq {q_len} H {H}")


def test_multiq_causal_window_is_end_aligned(ma, cuda_device):
    """Poisoning the last q_len - 1 rows moves the last draft position and leaves the first bit-identical."""
    B, S, H, q_len = 1, 2048, 16, 4
    kv = _rand_kv(B, S, cuda_device, 31)
    q_lat, q_pe, o_lat = _rand_q(B, q_len, H, cuda_device, 31)
    ma.mla_decode_a16w8_multiq(q_lat, q_pe, kv, o_lat, SCALE, KV_SCALE)
    base = o_lat.clone()
    kv[:, S - q_len + 1:] = _rand_kv(B, q_len - 1, cuda_device, 99)
    ma.mla_decode_a16w8_multiq(q_lat, q_pe, kv, o_lat, SCALE, KV_SCALE)
    assert torch.equal(o_lat[:, 0], base[:, 0]), "position 0 read past its causal limit"
    assert not torch.equal(o_lat[:, -1], base[:, -1]), "last position missed the tail tokens"


@pytest.mark.parametrize("q_len", [4, 8])
def test_multiq_paged_matches_reference(ma, cuda_device, q_len):
    B, H = 3, 16
    seq_lens = [2048, 2064, 1024]
    S = max(seq_lens)
    kv = _rand_kv(B, S, cuda_device, 43)
    q_lat, q_pe, o_lat = _rand_q(B, q_len, H, cuda_device, 43)
    pool, kv_indices, kv_indptr = _paged_pool(kv, seq_lens, cuda_device, 43)
    lens = torch.tensor(seq_lens, dtype=torch.int32, device=cuda_device)
    parts = ma.mla_decode_a16w8_multiq_plan_parts_q(B, S, q_len, H)
    assert parts >= 1
    ma.mla_decode_a16w8_multiq_paged_dev(q_lat, q_pe, pool, o_lat, lens, None, kv_indices, kv_indptr, parts, SCALE, KV_SCALE)
    _check(ma, o_lat, _oracle(q_lat, q_pe, kv, seq_lens), f"paged multiq {q_len}")


def test_multiq_paged_rows_remaps_query_and_output(ma, cuda_device):
    B, H, q_len = 4, 16, 4
    seq_lens = [2048] * B
    kv = _rand_kv(B, seq_lens[0], cuda_device, 57)
    q_lat, q_pe, o_lat = _rand_q(B, q_len, H, cuda_device, 57)
    pool, kv_indices, kv_indptr = _paged_pool(kv, seq_lens, cuda_device, 57)
    lens = torch.tensor(seq_lens, dtype=torch.int32, device=cuda_device)
    parts = ma.mla_decode_a16w8_multiq_plan_parts_q(B, seq_lens[0], q_len, H)
    ma.mla_decode_a16w8_multiq_paged_dev(q_lat, q_pe, pool, o_lat, lens, None, kv_indices, kv_indptr, parts, SCALE, KV_SCALE)
    identity = o_lat.clone()
    rows = torch.arange(B - 1, -1, -1, dtype=torch.int32, device=cuda_device)
    o_rev = torch.zeros_like(o_lat)
    ma.mla_decode_a16w8_multiq_paged_dev(q_lat.flip(0).contiguous(), q_pe.flip(0).contiguous(), pool, o_rev, lens, rows,
                                         kv_indices, kv_indptr, parts, SCALE, KV_SCALE)
    assert torch.equal(o_rev.flip(0), identity)


@pytest.mark.parametrize("q_len", [1, 3, 9])
def test_multiq_rejects_q_len_out_of_domain(ma, cuda_device, q_len):
    kv = _rand_kv(1, 256, cuda_device, 71)
    q_lat, q_pe, o_lat = _rand_q(1, q_len, 16, cuda_device, 71)
    with pytest.raises(ValueError, match="q_len"):
        ma.mla_decode_a16w8_multiq(q_lat, q_pe, kv, o_lat, SCALE, KV_SCALE)


def test_multiq_rejects_too_many_heads(ma, cuda_device):
    kv = _rand_kv(1, 256, cuda_device, 73)
    q_lat, q_pe, o_lat = _rand_q(1, 4, 17, cuda_device, 73)
    with pytest.raises(ValueError, match="H must be"):
        ma.mla_decode_a16w8_multiq(q_lat, q_pe, kv, o_lat, SCALE, KV_SCALE)


def test_multiq_rejects_q_len_1_rank(ma, cuda_device):
    kv = _rand_kv(1, 256, cuda_device, 79)
    q_lat, q_pe, o_lat = _rand_q(1, None, 16, cuda_device, 79)
    with pytest.raises(ValueError, match=r"\[B,q_len,H,512\]"):
        ma.mla_decode_a16w8_multiq(q_lat, q_pe, kv, o_lat, SCALE, KV_SCALE)


# ---- beyond the reference's tests ------------------------------------------------------------------------------
@pytest.mark.parametrize("B,H,S", [(1, 16, 1), (1, 1, 127), (3, 5, 129), (2, 16, 1000), (5, 7, 4097)])
def test_single_query_ragged_lengths_and_few_heads(ma, cuda_device, B, H, S):
    kv = _rand_kv(B, S, cuda_device, 5)
    q_lat, q_pe, o_lat = _rand_q(B, None, H, cuda_device, 5)
    ma.mla_decode_a16w8(q_lat, q_pe, kv, o_lat, SCALE, KV_SCALE)
    _check(ma, o_lat, _oracle(q_lat, q_pe, kv, [S] * B), f"B {B} H {H} S {S}")


@pytest.mark.parametrize("q_len", [1, 2, 3, 6, 7])
@pytest.mark.parametrize("parts", [1, 3, 8, 64, 256])
def test_paged_every_window_length_and_split(ma, cuda_device, q_len, parts):
    B, H = 2, 16
    seq_lens = [700, 1301]
    kv = _rand_kv(B, max(seq_lens), cuda_device, 17)
    q_lat, q_pe, o_lat = _rand_q(B, q_len if q_len > 1 else None, H, cuda_device, 17)
    pool, kv_indices, kv_indptr = _paged_pool(kv, seq_lens, cuda_device, 17)
    lens = torch.tensor(seq_lens, dtype=torch.int32, device=cuda_device)
    ma.mla_decode_a16w8_paged_dev(q_lat, q_pe, pool, o_lat, lens, None, kv_indices, kv_indptr, parts, SCALE, KV_SCALE)
    _check(ma, o_lat, _oracle(q_lat, q_pe, kv, seq_lens), f"paged q_len {q_len} parts {parts}")


@pytest.mark.parametrize("parts", [2, 3, 4, 5, 6, 7, 8])
@pytest.mark.parametrize("q_len", [1, 4])
def test_parts_merged_inside_a_cluster_and_by_the_merge_kernel_agree(ma, cuda_device, parts, q_len):
    """Two to eight parts of a request run as one thread-block cluster and merge through shared memory while the
    device holds all clusters of the call at once; with more requests than that a merge kernel follows.  Both
    ways, on the same ragged requests (some parts of the short ones are empty), against the oracle; the two
    outputs may differ by the fp32 summation order only."""
    from moonmath_attention import _abi

    H = 16 if q_len == 1 else 8
    groups = 1 if q_len == 1 else (q_len + 1) // 2
    capacity = _abi.lib.ma_mla_cluster_capacity(q_len, 1, parts)
    assert 1 <= capacity <= 148 // parts
    few, many = 3, capacity // groups + 1       # requests: inside one wave of clusters / one more than fit
    seq_lens = [97 + 211 * (b % 7) for b in range(many)]
    kv = _rand_kv(many, max(seq_lens), cuda_device, 61)
    q_lat, q_pe, o_lat = _rand_q(many, q_len if q_len > 1 else None, H, cuda_device, 61)
    pool, kv_indices, kv_indptr = _paged_pool(kv, seq_lens, cuda_device, 61)
    lens = torch.tensor(seq_lens, dtype=torch.int32, device=cuda_device)
    ma.mla_decode_a16w8_paged_dev(q_lat, q_pe, pool, o_lat, lens, None, kv_indices, kv_indptr, parts, SCALE, KV_SCALE)
    ref = _oracle(q_lat, q_pe, kv, seq_lens)
    _check(ma, o_lat, ref, f"merge kernel, parts {parts} q_len {q_len}")
    o_few = torch.zeros_like(o_lat[:few])
    ma.mla_decode_a16w8_paged_dev(q_lat[:few].contiguous(), q_pe[:few].contiguous(), pool, o_few, lens[:few].contiguous(), None,
                                  kv_indices, kv_indptr[:few + 1].contiguous(), parts, SCALE, KV_SCALE)
    _check(ma, o_few, ref[:few], f"cluster, parts {parts} q_len {q_len}")
    diff = (o_few.float() - o_lat[:few].float()).abs().max().item()
    assert diff <= 2.0 ** -7 * o_lat[:few].float().abs().max().item()   # a bf16 rounding step at most


def test_e4m3_cache_is_read_unchanged(ma, cuda_device):
    B, S, H = 2, 1500, 16
    kv = _rand_kv(B, S, cuda_device, 29, torch.float8_e4m3fn)
    q_lat, q_pe, o_lat = _rand_q(B, None, H, cuda_device, 29)
    ma.mla_decode_a16w8(q_lat, q_pe, kv, o_lat, SCALE, KV_SCALE)
    _check(ma, o_lat, _oracle(q_lat, q_pe, kv, [S] * B, "fn"), "e4m3fn cache")


@pytest.mark.parametrize("paged", [False, True])
def test_e4m3_cache_in_a_window(ma, cuda_device, paged):
    B, S, H, q_len = 2, 1100, 16, 5
    kv = _rand_kv(B, S, cuda_device, 47, torch.float8_e4m3fn)
    q_lat, q_pe, o_lat = _rand_q(B, q_len, H, cuda_device, 47)
    if paged:
        pool, kv_indices, kv_indptr = _paged_pool(kv, [S] * B, cuda_device, 47)
        lens = torch.tensor([S] * B, dtype=torch.int32, device=cuda_device)
        ma.mla_decode_a16w8_multiq_paged_dev(q_lat, q_pe, pool, o_lat, lens, None, kv_indices, kv_indptr, 3, SCALE, KV_SCALE)
    else:
        ma.mla_decode_a16w8_multiq(q_lat, q_pe, kv, o_lat, SCALE, KV_SCALE)
    _check(ma, o_lat, _oracle(q_lat, q_pe, kv, [S] * B, "fn"), f"e4m3fn cache, window of {q_len}, paged {paged}")


@pytest.mark.parametrize("paged", [False, True])
@pytest.mark.parametrize("density,exact", [(0.0005, True), (0.005, True), (0.05, False)])
def test_saturated_fnuz_codes_are_corrected(ma, cuda_device, paged, density, exact):
    """0x7F / 0xFF are +-240 in e4m3-fnuz and NaN in the format the tensor core reads.  The kernel feeds +-224 and
    adds the rest by hand for up to 640 entries per 96-token tile: exact below that, finite and close above."""
    B, S, H = 2, 1000, 16
    kv = _rand_kv(B, S, cuda_device, 37)
    raw = kv.view(torch.uint8)
    g = torch.Generator().manual_seed(3)
    hit = (torch.rand(raw.shape, generator=g) < density).to(cuda_device)
    sign = (torch.rand(raw.shape, generator=g) < 0.5).to(cuda_device)
    raw[hit & sign] = 0x7F
    raw[hit & ~sign] = 0xFF
    kv_scale = 1.0 / 512.0  # keeps the softmax spread out although some keys are huge
    q_lat, q_pe, o_lat = _rand_q(B, None, H, cuda_device, 37)
    if paged:
        pool, kv_indices, kv_indptr = _paged_pool(kv, [S] * B, cuda_device, 37)
        lens = torch.tensor([S] * B, dtype=torch.int32, device=cuda_device)
        ma.mla_decode_a16w8_paged_dev(q_lat, q_pe, pool, o_lat, lens, None, kv_indices, kv_indptr, 2, SCALE, kv_scale)
    else:
        ma.mla_decode_a16w8(q_lat, q_pe, kv, o_lat, SCALE, kv_scale)
    out = o_lat.float().cpu().numpy().reshape(B, 1, H, LAT)
    assert ma.last_status()[0] == 0 and np.isfinite(out).all()
    qa, qb = q_lat.unsqueeze(1).float().cpu().numpy(), q_pe.unsqueeze(1).float().cpu().numpy()
    err = mo.rel_l2(out, mo.mla_decode(qa, qb, raw.cpu().numpy(), [S] * B, SCALE, kv_scale))
    assert err < (REL_L2 if exact else 0.1), err


@pytest.mark.parametrize("q_len", [4, 5])
def test_saturated_codes_in_a_window_on_a_contiguous_cache(ma, cuda_device, q_len):
    """Two draft positions share a CTA there: both must get the corrections, the rows are rewritten once, and the
    positions' last tokens (seen by one of the two only) count too."""
    B, S, H = 2, 1000, 16
    kv = _rand_kv(B, S, cuda_device, 43)
    raw = kv.view(torch.uint8)
    g = torch.Generator().manual_seed(5)
    hit = (torch.rand(raw.shape, generator=g) < 0.002).to(cuda_device)
    sign = (torch.rand(raw.shape, generator=g) < 0.5).to(cuda_device)
    raw[hit & sign] = 0x7F
    raw[hit & ~sign] = 0xFF
    raw[:, S - q_len:, 17] = 0x7F      # the tokens at the causal limits
    raw[:, S - q_len:, 530] = 0xFF
    kv_scale = 1.0 / 512.0
    q_lat, q_pe, o_lat = _rand_q(B, q_len, H, cuda_device, 43)
    ma.mla_decode_a16w8_multiq(q_lat, q_pe, kv, o_lat, SCALE, kv_scale)
    out = o_lat.float().cpu().numpy()
    assert ma.last_status()[0] == 0 and np.isfinite(out).all()
    err = mo.rel_l2(out, mo.mla_decode(q_lat.float().cpu().numpy(), q_pe.float().cpu().numpy(), raw.cpu().numpy(),
                                       [S] * B, SCALE, kv_scale))
    assert err < REL_L2, err


def test_saturated_codes_under_zero_query_columns(ma, cuda_device):
    """Saturated codes whose query column is zero in every head change no score, but still reach the output
    through V (latent columns) or not at all (rope columns)."""
    B, S, H = 2, 700, 16
    kv = _rand_kv(B, S, cuda_device, 41)
    raw = kv.view(torch.uint8)
    raw[:, ::7, 100] = 0x7F
    raw[:, 3::11, 300] = 0xFF
    raw[:, 5::13, 530] = 0x7F      # a rope column
    lens = [S, 333]
    q_lat, q_pe, o_lat = _rand_q(B, None, H, cuda_device, 41)
    q_lat[..., 100] = 0
    q_lat[..., 300] = 0
    q_pe[..., 530 - LAT] = 0
    kv_scale = 1.0 / 512.0
    pool, kv_indices, kv_indptr = _paged_pool(kv, lens, cuda_device, 41)
    lens_t = torch.tensor(lens, dtype=torch.int32, device=cuda_device)
    ma.mla_decode_a16w8_paged_dev(q_lat, q_pe, pool, o_lat, lens_t, None, kv_indices, kv_indptr, 2, SCALE, kv_scale)
    out = o_lat.float().cpu().numpy().reshape(B, 1, H, LAT)
    assert ma.last_status()[0] == 0 and np.isfinite(out).all()
    qa, qb = q_lat.unsqueeze(1).float().cpu().numpy(), q_pe.unsqueeze(1).float().cpu().numpy()
    err = mo.rel_l2(out, mo.mla_decode(qa, qb, raw.cpu().numpy(), lens, SCALE, kv_scale))
    assert err < REL_L2, err
    # the contiguous form reads whole slabs: request 0 only
    o2 = torch.zeros_like(o_lat[:1])
    ma.mla_decode_a16w8(q_lat[:1].contiguous(), q_pe[:1].contiguous(), kv[:1].contiguous(), o2, SCALE, kv_scale)
    assert ma.last_status()[0] == 0
    err = mo.rel_l2(o2.float().cpu().numpy().reshape(1, 1, H, LAT),
                    mo.mla_decode(qa[:1], qb[:1], raw[:1].cpu().numpy(), [S], SCALE, kv_scale))
    assert err < REL_L2, err


def test_random_shapes_against_the_oracle(ma, cuda_device):
    """Seeded sweep: ragged lengths down to fewer tokens than draft positions (positions without any token give
    zeros), few heads, splits larger than the number of tiles, both cache formats, pool and contiguous."""
    rng = np.random.default_rng(2024)
    for case in range(24):
        q_len = int(rng.choice([1, 2, 3, 4, 5, 7, 8]))
        B, H = int(rng.integers(1, 5)), int(rng.choice([1, 3, 8, 16]))
        fmt = "fnuz" if case % 3 else "fn"
        dtype = torch.float8_e4m3fnuz if fmt == "fnuz" else torch.float8_e4m3fn
        paged = bool(case % 2) or q_len in (2, 3)  # the contiguous window entry point takes 4..8 positions
        lens = [int(x) for x in rng.choice([1, 2, 5, 95, 96, 97, 200, 777, 1500], size=B)]
        if not paged:
            lens = [max(lens)] * B
        S = max(lens)
        kv = _rand_kv(B, S, cuda_device, 100 + case, dtype)
        q_lat, q_pe, o_lat = _rand_q(B, q_len if q_len > 1 else None, H, cuda_device, 100 + case)
        o_lat.fill_(7.0)
        if paged:
            parts = int(rng.choice([1, 2, 5, 40]))
            pool, kv_indices, kv_indptr = _paged_pool(kv, lens, cuda_device, 100 + case)
            lens_t = torch.tensor(lens, dtype=torch.int32, device=cuda_device)
            fn = ma.mla_decode_a16w8_paged_dev if q_len == 1 else ma.mla_decode_a16w8_multiq_paged_dev
            if q_len in (2, 3):
                fn = ma.mla_decode_a16w8_paged_dev
            fn(q_lat, q_pe, pool, o_lat, lens_t, None, kv_indices, kv_indptr, parts, SCALE, KV_SCALE)
        elif q_len == 1:
            ma.mla_decode_a16w8(q_lat, q_pe, kv, o_lat, SCALE, KV_SCALE)
        else:
            ma.mla_decode_a16w8_multiq(q_lat, q_pe, kv, o_lat, SCALE, KV_SCALE)
        torch.cuda.synchronize()
        assert ma.last_status()[0] == 0, (case, ma.last_status())
        want = _oracle(q_lat, q_pe, kv, lens, fmt)
        got = o_lat.float().cpu().numpy().reshape(want.shape)
        assert np.isfinite(got).all(), case
        empty = np.abs(want).reshape(want.shape[0], want.shape[1], -1).max(axis=-1) == 0  # positions without tokens
        assert (got[empty] == 0).all(), case
        err = mo.rel_l2(got, want)
        assert err < REL_L2, (case, q_len, B, H, lens, fmt, paged, err)


def test_paged_call_replays_from_a_cuda_graph(ma, cuda_device):
    """All index arrays are read on the device and the grid depends on (batch, q_len, parts) only: a captured call
    replays correctly after the lengths, the slot table and the queries have changed in place."""
    B, H, q_len, parts, S = 3, 16, 4, 3, 1500
    kv = _rand_kv(B, S, cuda_device, 61)
    q_lat, q_pe, o_lat = _rand_q(B, q_len, H, cuda_device, 61)
    lens0, lens1 = [S, 900, 1200], [700, S, 333]
    pool, idx0, indptr0 = _paged_pool(kv, lens0, cuda_device, 61)
    _, idx1, indptr1 = _paged_pool(kv, lens1, cuda_device, 62)
    kv_indices = torch.zeros(B * S, dtype=torch.int32, device=cuda_device)
    kv_indptr = torch.zeros(B + 1, dtype=torch.int32, device=cuda_device)
    lens_t = torch.zeros(B, dtype=torch.int32, device=cuda_device)
    # one pool that holds both layouts: the second permutation's rows go behind the first's
    pool1, _, _ = _paged_pool(kv, lens1, cuda_device, 62)
    both = torch.cat([pool, pool1], dim=0)

    def load(lens, idx, indptr, offset):
        lens_t.copy_(torch.tensor(lens, dtype=torch.int32))
        kv_indices[: idx.numel()] = idx + offset
        kv_indptr.copy_(indptr)

    load(lens0, idx0, indptr0, 0)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):  # warm-up outside the capture, as torch asks
        ma.mla_decode_a16w8_multiq_paged_dev(q_lat, q_pe, both, o_lat, lens_t, None, kv_indices, kv_indptr, parts, SCALE, KV_SCALE)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ma.mla_decode_a16w8_multiq_paged_dev(q_lat, q_pe, both, o_lat, lens_t, None, kv_indices, kv_indptr, parts, SCALE, KV_SCALE)
    graph.replay()
    torch.cuda.synchronize()
    _check(ma, o_lat, _oracle(q_lat, q_pe, kv, lens0), "graph replay, first lengths")
    load(lens1, idx1, indptr1, pool.shape[0])
    q_lat.copy_(_rand_q(B, q_len, H, cuda_device, 63)[0])
    graph.replay()
    torch.cuda.synchronize()
    _check(ma, o_lat, _oracle(q_lat, q_pe, kv, lens1), "graph replay, second lengths")


@pytest.mark.parametrize("parts", [1, 4, 12])
def test_calls_in_a_row_see_what_the_kernels_before_them_wrote(ma, cuda_device, parts):
    """The decode kernel is launched as a programmatic dependent of its predecessor in the stream and sets up while
    that one still runs; it must not read queries, cache rows or lengths before the predecessor has completed, and
    what follows it must see its output.  Twelve steps without any synchronisation: a torch kernel writes new
    queries, another appends a token row to the cache and a third bumps the lengths, the decode call runs, a
    torch kernel copies the output away.  Every step's copy is checked at the end.  (1 part: the kernel writes the
    output itself; 4: merge inside a cluster; 12: merge kernel.)"""
    B, H, S0, steps = 3, 16, 600, 12
    g = torch.Generator().manual_seed(5)
    kv_all = torch.randn(B, S0 + steps, FUSED, generator=g).to(torch.float8_e4m3fnuz).to(cuda_device)
    qs = [_rand_q(B, None, H, cuda_device, 100 + i)[:2] for i in range(steps)]
    total = B * (S0 + steps)
    pool = torch.zeros(total, 1, FUSED, dtype=torch.uint8, device=cuda_device)
    slots = torch.arange(total, dtype=torch.int32, device=cuda_device)                      # request b owns rows b*(S0+steps)...
    indptr = torch.arange(0, total + 1, S0 + steps, dtype=torch.int32, device=cuda_device)
    pool.view(B, S0 + steps, FUSED)[:, :S0] = kv_all.view(torch.uint8)[:, :S0]
    lens = torch.full((B,), S0, dtype=torch.int32, device=cuda_device)
    q_lat, q_pe = qs[0][0].clone(), qs[0][1].clone()
    o_lat = torch.zeros_like(q_lat)
    outs = []
    torch.cuda.synchronize()
    for i in range(steps):
        q_lat.copy_(qs[i][0])
        q_pe.copy_(qs[i][1])
        pool.view(B, S0 + steps, FUSED)[:, S0 + i] = kv_all.view(torch.uint8)[:, S0 + i]    # this step's new token
        lens.add_(1)
        ma.mla_decode_a16w8_paged_dev(q_lat, q_pe, pool.view(torch.float8_e4m3fnuz), o_lat, lens, None, slots, indptr,
                                      parts, SCALE, KV_SCALE)
        outs.append(o_lat.clone())
    torch.cuda.synchronize()
    assert ma.last_status()[0] == 0
    for i in range(steps):
        ref = _oracle(qs[i][0], qs[i][1], kv_all, [S0 + i + 1] * B)
        got = outs[i].float().cpu().numpy().reshape(ref.shape)
        assert mo.rel_l2(got, ref) < REL_L2, f"step {i}: rel-L2 {mo.rel_l2(got, ref):.2e}"


def test_status_word_is_cleared_by_the_call_itself(ma, cuda_device):
    """No memset precedes the kernel: a workspace full of stale bytes (a status word left by a failed call
    included) must not disturb the call, and its first status word must read zero afterwards."""
    from moonmath_attention import _abi

    B, H, S = 5, 16, 1000
    kv = _rand_kv(B, S, cuda_device, 71)
    q_lat, q_pe, o_lat = _rand_q(B, None, H, cuda_device, 71)
    ref = _oracle(q_lat, q_pe, kv, [S] * B)
    stream = torch.cuda.current_stream().cuda_stream
    for parts in (1, 3, 20):
        ws = torch.full((int(_abi.lib.ma_mla_workspace_bytes(B, 1, parts)),), 0xAB, dtype=torch.uint8, device=cuda_device)
        o_lat.zero_()
        rc = _abi.lib.ma_mla_decode_a16w8(q_lat.data_ptr(), q_pe.data_ptr(), kv.data_ptr(), o_lat.data_ptr(), None, None,
                                          None, None, B, H, 1, S, parts, SCALE, KV_SCALE, 0, ws.data_ptr(), ws.numel(), stream)
        assert rc == 0, _abi.error_string(rc)
        torch.cuda.synchronize()
        assert ws[:4].view(torch.int32).item() == 0
        assert mo.rel_l2(o_lat.float().cpu().numpy().reshape(ref.shape), ref) < REL_L2, parts


def test_more_requests_than_sms_run_in_several_waves(ma, cuda_device):
    """600 requests are four waves of CTAs; twice in a row, so that the second call's first wave lines up behind
    the first call's last one (dependent launch) and must still wait for all of it."""
    B, H, S = 600, 4, 200
    kv = _rand_kv(B, S, cuda_device, 83)
    q_lat, q_pe, o_lat = _rand_q(B, None, H, cuda_device, 83)
    ma.mla_decode_a16w8(q_lat, q_pe, kv, o_lat, SCALE, KV_SCALE)
    first = o_lat.clone()
    o_lat.zero_()
    ma.mla_decode_a16w8(q_lat, q_pe, kv, o_lat, SCALE, KV_SCALE)
    ref = _oracle(q_lat, q_pe, kv, [S] * B)
    _check(ma, o_lat, ref, "600 requests")
    assert torch.equal(first.view(torch.int16), o_lat.view(torch.int16))


def test_contiguous_argument_errors(ma, cuda_device):
    kv = _rand_kv(2, 256, cuda_device, 83)
    q_lat, q_pe, o_lat = _rand_q(2, None, 16, cuda_device, 83)
    with pytest.raises(ValueError, match="float8_e4m3fnuz"):
        ma.mla_decode_a16w8(q_lat, q_pe, kv.view(torch.uint8), o_lat, SCALE, KV_SCALE)
    with pytest.raises(ValueError, match="FUSED"):
        ma.mla_decode_a16w8(q_lat, q_pe, kv[..., :512].contiguous(), o_lat, SCALE, KV_SCALE)
    with pytest.raises(ValueError, match="batch"):
        ma.mla_decode_a16w8(q_lat, q_pe, kv[:1], o_lat, SCALE, KV_SCALE)
    with pytest.raises(ValueError, match="bfloat16"):
        ma.mla_decode_a16w8(q_lat.float(), q_pe, kv, o_lat, SCALE, KV_SCALE)
    with pytest.raises(ValueError, match="q_len==1 only"):
        q4 = _rand_q(2, 4, 16, cuda_device, 83)
        ma.mla_decode_a16w8(q4[0], q4[1], kv, q4[2], SCALE, KV_SCALE)
    lens = torch.tensor([256, 256], dtype=torch.int64, device=cuda_device)
    with pytest.raises(ValueError, match="int32"):
        ma.mla_decode_a16w8_paged_dev(q_lat, q_pe, kv.view(512, 1, FUSED), o_lat, lens, None, lens, lens, 1, SCALE, KV_SCALE)
