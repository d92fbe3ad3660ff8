"""The multi-replica host logic of bench.py on CPU ranks (gloo, world size 2): every rank is an
independent replica with its own requests, the job's step time is the slowest rank's and its
tokens are the sum over ranks.  No GPU needed."""

import os
import socket
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    import bench

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    work = bench.Workload(seed=bench.replica_seed(rank), requests=4, layers=1)
    # rank r "measures" 10 + 5 r ms for 2 steps and accepts 3 + r tokens per step
    stats = torch.tensor([10.0 + 5 * rank, 20.0 + rank, 3.0 + rank, 3.0 + rank + work.requests], dtype=torch.float64)
    dist.barrier()
    job = bench.combine_ranks(stats, world, steps=2, gather=bench.all_gather_rows)
    torch.save({"job": job, "contexts": work.contexts, "tables": work.request_tables}, Path(out_dir) / f"rank{rank}.pt")
    dist.destroy_process_group()


def test_two_replicas_combine_with_max_time_and_summed_tokens(tmp_path):
    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    results = [torch.load(tmp_path / f"rank{r}.pt", weights_only=False) for r in range(world)]
    for r in results:  # every rank computes the same whole-job numbers
        job = r["job"]
        assert job["ms_per_step"] == 15.0 / 2            # slowest rank, 2 steps
        assert job["e2e_ms_per_step"] == 21.0 / 2
        assert job["accepted_per_step"] == 3.0 + 4.0      # summed over ranks
        assert job["committed_per_step"] == 7.0 + 2 * 4
        assert abs(job["accepted_tokens_per_s"] - 7.0 / 0.0075) < 1e-6
    # replicas own different requests (different seeds), with no shared state
    assert not torch.equal(results[0]["contexts"], results[1]["contexts"])


def test_single_rank_needs_no_process_group():
    sys.path.insert(0, str(ROOT))
    import bench

    job = bench.combine_ranks(torch.tensor([8.0, 16.0, 5.0, 9.0], dtype=torch.float64), 1, steps=4)
    assert job["ms_per_step"] == 2.0 and job["accepted_tokens_per_s"] == 2500.0


def test_workload_is_deterministic_per_seed_and_tables_are_disjoint():
    sys.path.insert(0, str(ROOT))
    import bench

    a, b = bench.Workload(seed=7, requests=6, layers=1), bench.Workload(seed=7, requests=6, layers=1)
    assert torch.equal(a.contexts, b.contexts) and torch.equal(a.tables, b.tables)
    pages = (a.contexts + bench.BLOCK - 1) // bench.BLOCK
    used = torch.cat([a.request_tables[i, : int(n)] for i, n in enumerate(pages)])
    assert used.numel() == used.unique().numel() == a.total_pages      # every page owned by one request
    assert a.rows == 6 * bench.TOKENS * bench.DEPTHS
    assert int(a.lengths.max()) == int(a.contexts.max())
    assert a.algorithmic_attention_bytes() > int(a.contexts.sum()) * bench.HEADS * bench.HEAD_DIM * 4


def test_requests_are_shared_out_by_length_and_cut_into_waves_that_fit():
    sys.path.insert(0, str(ROOT))
    import bench

    g = torch.Generator().manual_seed(5)
    lengths = torch.randint(256, 2049, (1024,), generator=g).tolist()
    for world in (1, 2, 4, 8):
        shards = bench.balanced_shards(lengths, world)
        assert sorted(i for shard in shards for i in shard) == list(range(1024))      # every request exactly once
        loads = [sum(lengths[i] for i in shard) for shard in shards]
        assert max(loads) - min(loads) <= max(lengths)                                  # within one request's length
        assert max(len(s) for s in shards) - min(len(s) for s in shards) <= 1
    shard = bench.balanced_shards(lengths, 8)[3]
    per_token, extra = 768 * 1024, 512 + 7 + 16
    waves = bench.waves_under_budget(shard, lengths, extra, per_token, 110e9, 128)
    assert [i for wave in waves for i in wave] == shard                                # order kept, nothing dropped
    for wave in waves:
        assert len(wave) <= 128 and sum((lengths[i] + extra) * per_token for i in wave) <= 110e9
    assert len(waves) == 2                                                              # 128 requests of ~1.3 GB each
    # a single request larger than the budget still gets a wave of its own
    assert bench.waves_under_budget([0], [10 ** 6], 0, per_token, 1e9, 128) == [[0]]
