"""The multi-GPU host logic on CPU: two gloo ranks shard slices, exchange results, reduce timings."""
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

from moonmath_attention.shard import slice_range


def test_slice_ranges_partition_the_slices():
    for n in (48, 6, 7, 1, 0, 100):
        for world in (1, 2, 4, 8, 3):
            rs = [slice_range(r, world, n) for r in range(world)]
            flat = [i for r in rs for i in r]
            assert flat == list(range(n))
            assert max(len(r) for r in rs) - min(len(r) for r in rs) <= 1
    assert [len(slice_range(r, 8, 48)) for r in range(8)] == [6] * 8
    with pytest.raises(ValueError):
        slice_range(2, 2, 4)


def _worker(rank: int, world: int, port: int, n_slices: int, q):
    import torch.distributed as dist

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for p in (root, os.path.join(root, "amd-kernels_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    from moonmath_attention.shard import gather_slices, max_over_ranks, slice_range as sr
    from oracle import oracle as orc

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mine = sr(rank, world, n_slices)
        # each rank builds only its own slices (per-slice seeds) and "runs" them -- with the CPU oracle
        # standing in for the kernel, which needs a GPU
        qs, ks, vs = orc.make_inputs(1, n_slices, 40, 56, "bhsd", bh_range=mine)
        local = orc.bits_to_bf16_tensor(orc.attention_bf16_bits(qs, ks, vs, "bhsd", "rtne"))
        full = gather_slices(local, n_slices)
        t = max_over_ranks(1.0 + rank)
        dist.barrier()
        if rank == 0:
            # plain bytes: a tensor would travel as a shared-memory handle that dies with this process
            q.put((full.view(torch.int16).numpy().tobytes(), t))
    finally:
        dist.destroy_process_group()


def test_two_ranks_shard_and_gather():
    from oracle import oracle as orc

    n_slices, world = 5, 2  # uneven on purpose: ranks own 3 and 2 slices
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, world, port, n_slices, queue)) for r in range(world)]
    for p in procs:
        p.start()
    full_bits, tmax = queue.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert tmax == 2.0  # max over ranks of (1 + rank)
    q, k, v = orc.make_inputs(1, n_slices, 40, 56, "bhsd")
    want = orc.bits_to_bf16_tensor(orc.attention_bf16_bits(q, k, v, "bhsd", "rtne")).view(torch.int16)
    assert full_bits == want.numpy().tobytes()


def _failing_worker(rank: int, world: int, port: int, q):
    """Rank 1 leaves between steps (after the rendezvous, before the exchange); rank 0 must learn of it as an error."""
    import datetime

    import torch.distributed as dist

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for p in (root, os.path.join(root, "amd-kernels_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    from moonmath_attention.shard import gather_slices

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    dist.barrier()
    if rank == 1:
        os._exit(3)  # no collective of this rank is in flight
    local = torch.zeros(1, 3, 4, 128, dtype=torch.bfloat16)
    try:
        gather_slices(local, 5)
        q.put("gathered")
    except Exception as e:  # noqa: BLE001  (whatever the backend raises for a lost peer or a timeout)
        q.put("error: " + type(e).__name__)
    os._exit(0)  # the process group cannot be torn down cleanly without its peer


def test_a_rank_that_leaves_is_reported_not_waited_for():
    """Failure detection on the host (the device side has none to inject): the exchange with a rank that is gone
    ends in an exception within the process-group timeout instead of hanging."""
    world = 2
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = 31500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_failing_worker, args=(r, world, port, queue)) for r in range(world)]
    for p in procs:
        p.start()
    verdict = queue.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
    assert verdict.startswith("error"), verdict
    assert procs[1].exitcode == 3 and procs[0].exitcode == 0
