"""CPU tests of the replica-parallel plumbing with two gloo ranks (no GPU involved)."""

import os
import socket

import torch
import torch.multiprocessing as mp

from lyradiff_b200 import replicas


def test_items_partition_is_a_disjoint_cover():
    for n in (0, 1, 7, 8, 9):
        for world in (1, 2, 4, 8):
            seen = []
            for r in range(world):
                seen += replicas.items_for_rank(n, r, world)
            assert sorted(seen) == list(range(n))
    assert replicas.items_for_rank(8, 3, 4) == [3, 7]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out):
    os.environ.update({"RANK": str(rank), "LOCAL_RANK": str(rank), "WORLD_SIZE": str(world),
                       "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    assert replicas.init("gloo")
    mine = replicas.items_for_rank(8, rank, world)
    # each rank "processes" its own images; nothing is exchanged but the timing scalars
    elapsed_ms = 10.0 + 5.0 * rank
    replicas.barrier()
    worst, = replicas.max_over_ranks([elapsed_ms])
    total = replicas.sum_over_ranks(len(mine))
    out.put((rank, mine, worst, total))
    replicas.shutdown()


def test_two_gloo_ranks_agree_on_max_time_and_cover_all_items():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    items = sorted(i for _, mine, _, _ in results for i in mine)
    assert items == list(range(8))
    assert all(worst == 15.0 for _, _, worst, _ in results)   # max over ranks, seen by every rank
    assert all(total == 8.0 for _, _, _, total in results)


def test_single_process_is_a_no_op():
    assert replicas.env_rank_world()[2] >= 1
    assert replicas.max_over_ranks([3.0, 4.0]) == [3.0, 4.0]
    replicas.barrier()
