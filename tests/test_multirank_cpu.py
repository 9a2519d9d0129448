"""Host logic of the N>1 path on CPU (gloo, world_size 2), through the functions bench.py itself uses: the step's
batch is sharded into disjoint contiguous slices that cover it exactly (also when it does not divide), every rank
draws ITS slice of the seeded position stream, and the step time reported is the max over ranks."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

BATCH = 37            # odd on purpose: 19 + 18


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import bench
    from chessrl_b200 import positions
    first, count = bench.shard_bounds(BATCH, world, rank)
    pos = positions.playout_positions(count, seed=20240607, first=first, max_plies=40, fens=True)
    ms = bench.max_over_ranks(10.0 + 3 * rank, dist, torch.device("cpu"))   # each rank's own device time goes in
    gathered = [None] * world
    dist.all_gather_object(gathered, (first, count, pos["fens"]))
    if rank == 0:
        out.put((ms, gathered))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_shard_and_reduce():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    ms, gathered = q.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert ms == 13.0                                            # max over ranks, not rank 0's own 10.0
    assert [g[:2] for g in gathered] == [(0, 19), (19, 18)]      # disjoint, contiguous, complete, remainder kept
    # the two slices together are exactly the positions one process would have drawn
    from chessrl_b200 import positions
    whole = positions.playout_positions(BATCH, seed=20240607, first=0, max_plies=40, fens=True)["fens"]
    assert gathered[0][2] + gathered[1][2] == whole
    assert gathered[0][2] != gathered[1][2][:len(gathered[0][2])]


def test_shard_bounds_cover_every_batch_exactly():
    import bench
    for batch in (0, 1, 7, 64, 65536, 65537):
        for world in (1, 2, 3, 4, 8):
            spans = [bench.shard_bounds(batch, world, r) for r in range(world)]
            assert spans[0][0] == 0 and sum(c for _, c in spans) == batch
            for (f0, c0), (f1, _) in zip(spans, spans[1:]):
                assert f0 + c0 == f1
            assert max(c for _, c in spans) - min(c for _, c in spans) <= 1
    assert bench.max_over_ranks(4.5, None, torch.device("cpu")) == 4.5


def test_bench_flop_model_matches_the_published_per_position_figures():
    import bench
    assert abs(bench.flops_per_position(15, 1024, 1536, 32, True) / 1e9 - 15.937) < 1e-3
    assert abs(bench.flops_per_position(8, 256, 1024, 8, False) / 1e9 - 0.8761) < 1e-4
