"""Host-side logic of the multi-GPU path, exercised with world_size-2 gloo ranks on the CPU:
row partitioning, and the barrier + max-over-ranks timing reduction bench.py uses."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from nemotron_infer_b200 import chain


def test_shard_range_partitions_rows():
    for total in (0, 1, 7, 64, 65536, 65537):
        for world in (1, 2, 3, 4, 8):
            spans = [chain.shard_range(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        chain.shard_range(10, 2, 2)


def test_schedule_and_byte_model():
    s = chain.layer_schedule()
    assert (len(s), s.count("M"), s.count("-"), s.count("*")) == (42, 21, 17, 4)
    assert chain.bytes_per_token(4) == 12548 + 42 * 25088 + 21 * 36864 + 17 * 50176 == 2693380
    assert chain.bytes_per_token(8) == 2693384


def test_batch_shard_rows_do_not_depend_on_the_split():
    """bench.py splits ONE seeded batch: the rows a rank generates for [lo, hi) are the rows of the whole batch,
    for every world size, also when a shard boundary falls inside a generation block."""
    total, vocab = 2 * chain.BATCH_BLOCK_ROWS + 37, 64
    whole = chain.batch_shard(total, 0, total, "cpu", seed=3, vocab=vocab)
    assert whole["ids"].dtype == torch.int32 and int(whole["ids"].max()) < vocab and int(whole["ids"].min()) >= 0
    assert whole["y"].shape == (total, chain.D_INNER) and whole["u"].dtype == torch.bfloat16
    for world in (2, 3, 8):
        for rank in range(world):
            lo, hi = chain.shard_range(total, rank, world)
            part = chain.batch_shard(total, lo, hi, "cpu", seed=3, vocab=vocab)
            for key in ("ids", "y", "z", "u"):
                assert torch.equal(part[key], whole[key][lo:hi]), (key, world, rank)
            for a, b in zip(part["mixer_out"], whole["mixer_out"]):
                assert torch.equal(a, b[lo:hi])
            for key in ("table", "norm_w", "gated_w"):
                assert torch.equal(part[key], whole[key])
    other = chain.batch_shard(total, 0, 16, "cpu", seed=4, vocab=vocab)
    assert not torch.equal(other["y"], whole["y"][:16])
    assert chain.batch_shard(total, 5, 5, "cpu", seed=3, vocab=vocab)["y"].shape[0] == 0
    with pytest.raises(ValueError):
        chain.batch_shard(10, 4, 11, "cpu")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import bench
    total = 1001
    lo, hi = chain.shard_range(total, rank, world)
    # every rank reports its own elapsed time; the job time is the slowest rank's
    job_ms = bench.max_over_ranks(10.0 + 5.0 * rank)
    rows = bench.sum_over_ranks(hi - lo)
    q.put((rank, job_ms, rows))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_timing_reduction_and_row_count():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert [g[1] for g in got] == [15.0, 15.0]      # max over ranks, seen by every rank
    assert [g[2] for g in got] == [1001, 1001]      # shards cover every row exactly once


def _gather_main(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    # the optional output all-gather of bench.py: equal shards, concatenated in rank order = the unsharded tensor
    total, hidden = 64, 16
    full = torch.arange(total * hidden, dtype=torch.float32).reshape(total, hidden)
    lo, hi = chain.shard_range(total, rank, world)
    mine = full[lo:hi].contiguous()
    out = torch.empty(total, hidden)
    dist.all_gather_into_tensor(out, mine)
    q.put((rank, bool(torch.equal(out, full))))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_output_gather_restores_row_order():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_gather_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got == [(0, True), (1, True)]
