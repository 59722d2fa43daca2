"""The N > 1 path: every rank plans its own shard with the reference's rules and no rank ever talks to another on the
data path.  Two gloo ranks on CPU build their shards, then compare notes (a host-side all_gather used only by the
test) to prove the shards are disjoint and cover everything -- the assertion datago's own multi-rank tests make with
two clients in one process (src/generator_files.rs:362-424, python/test_datago_client.py:231-284)."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, n_files, n_keys, ret):
    sys.path.insert(0, ROOT)
    import datago_b200 as dg
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        start, end = dg.rank_slice(n_files, rank, world)
        mine_files = torch.zeros(n_files, dtype=torch.int32)
        mine_files[start:end] = 1
        keys = ["%06d_%04d" % (i // 1000, i % 1000) for i in range(n_keys)]
        mine_keys = torch.tensor([1 if dg.key_rank(k, world) == rank else 0 for k in keys], dtype=torch.int32)
        files = [torch.zeros_like(mine_files) for _ in range(world)]
        ks = [torch.zeros_like(mine_keys) for _ in range(world)]
        dist.all_gather(files, mine_files)
        dist.all_gather(ks, mine_keys)
        if rank == 0:
            ret["files_cover"] = bool((torch.stack(files).sum(0) == 1).all())
            ret["keys_cover"] = bool((torch.stack(ks).sum(0) == 1).all())
            ret["key_counts"] = [int(k.sum()) for k in ks]
            ret["file_counts"] = [int(f.sum()) for f in files]
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_two_ranks_get_disjoint_covering_shards(world):
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, 1025, 3000, ret), nprocs=world, join=True)
    assert ret["files_cover"] and ret["keys_cover"]
    assert ret["file_counts"] == [513, 512]
    assert sum(ret["key_counts"]) == 3000 and min(ret["key_counts"]) > 1300
