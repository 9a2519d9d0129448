"""Host logic of the N>1 path on CPU (gloo, world_size 2): the batch is sharded into disjoint contiguous
slices that cover it exactly, seeds differ per rank, and the step time reported is the max over ranks."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def shard(global_batch, world, rank):
    per = global_batch // world
    return rank * per, per


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    start, per = shard(65536, world, rank)
    from chessrl_b200 import synth
    bits = synth.synthetic_legal_bits(8, 1858, seed=2000 + rank)
    ms = torch.tensor([10.0 + rank])             # stand-in for the rank's CUDA-event time
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    gathered = [None] * world
    dist.all_gather_object(gathered, (start, per, int(bits.sum())))
    if rank == 0:
        out.put((float(ms), gathered))
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
    ms, gathered = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert ms == 11.0                                            # max over ranks
    assert [g[:2] for g in gathered] == [(0, 32768), (32768, 32768)]   # disjoint, contiguous, complete
    assert gathered[0][2] != gathered[1][2]                      # per-rank seeds differ


def test_bench_flop_model_matches_the_published_per_position_figures():
    import bench
    assert abs(bench.flops_per_position(15, 1024, 1536, 32, True) / 1e9 - 15.937) < 1e-3
    assert abs(bench.flops_per_position(8, 256, 1024, 8, False) / 1e9 - 0.8761) < 1e-4
