"""Multi-rank host logic on CPU process groups (gloo, world size 2 and 3): shard arithmetic covers every unit exactly
once, the max-over-ranks reduction returns the slowest rank's value on every rank, handle exchange keeps rank order, and
the reference arm of the benchmark prints from rank 0 only."""
import json
import os
import subprocess
import sys

import pytest
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    from metalhlo_b200 import sharding

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        rows = sharding.contiguous_shard(32768 + 5, world, rank)
        heads = sharding.contiguous_shard(8 * 32, world, rank)
        cols = sharding.column_shard(8192 * 3, world, rank) if (8192 * 3) % (world * 8) == 0 else None
        slowest = sharding.max_over_ranks(1.0 + rank, dist)
        handles = sharding.exchange_handles(bytes([rank]) * 64, dist)
        gathered = [None] * world
        dist.all_gather_object(gathered, (rows.start, rows.count, heads.start, heads.count))
        with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
            json.dump({"rows": [rows.start, rows.count], "heads": [heads.start, heads.count], "cols": [cols.start, cols.count] if cols else None,
                       "slowest": slowest, "handles": [h[0] for h in handles], "gathered": gathered}, f)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_shards_tile_the_work_and_reductions_agree(world, tmp_path):
    port = 29600 + world
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    got = [json.load(open(tmp_path / f"rank{r}.json")) for r in range(world)]
    for key, total in (("rows", 32768 + 5), ("heads", 256)):
        cursor = 0
        for r in range(world):
            start, count = got[r][key]
            assert start == cursor and count in (total // world, total // world + 1)
            cursor += count
        assert cursor == total
    if got[0]["cols"]:
        assert [g["cols"][0] for g in got] == [r * (8192 * 3 // world) for r in range(world)]
    for g in got:
        assert g["slowest"] == float(world)            # 1.0 + (world - 1): the slowest rank, seen by every rank
        assert g["handles"] == list(range(world))      # rank order preserved
        assert g["gathered"] == got[0]["gathered"]


def test_shard_requests_are_validated():
    sys.path.insert(0, ROOT)
    from metalhlo_b200 import sharding

    assert sharding.contiguous_shard(10, 4, 3) == sharding.Shard(8, 2)
    assert sharding.contiguous_shard(0, 2, 1).count == 0
    assert sharding.weak_rows(32768, 8, 7) == sharding.Shard(7 * 32768, 32768)
    with pytest.raises(ValueError):
        sharding.contiguous_shard(10, 0, 0)
    with pytest.raises(ValueError):
        sharding.contiguous_shard(10, 2, 2)
    with pytest.raises(ValueError):
        sharding.column_shard(8190, 8, 0)              # 8190 / 8 ranks is not a multiple of 8 columns


def test_reference_arm_prints_from_rank_zero_only():
    env = dict(os.environ, WORLD_SIZE="2", RANK="1", LOCAL_RANK="1")
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, env=env, timeout=300)
    assert res.returncode == 0 and res.stdout.strip() == ""
