"""The N > 1 host logic (KV-head sharding + output all-gather) on CPU ranks:
world size 2 and 4, gloo backend."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import __graft_entry__ as entry


def _worker(rank, world, port, T, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    pkg = entry.load_package()
    from sera_c_b200 import sharding
    H, Hkv, D = 64, 8, 16
    g = torch.Generator().manual_seed(0)
    q = torch.randn(T, H, D, generator=g)
    k = torch.randn(T, Hkv, D, generator=g)
    v = torch.randn(T, Hkv, D, generator=g)
    ql, kl, vl = sharding.slice_heads(q, k, v, rank, world)
    kb, kc, qb, qc = sharding.head_shard(rank, world)
    assert ql.shape == (T, H // world, D) and kl.shape == (T, Hkv // world, D)
    assert torch.equal(ql, q[:, qb:qb + qc]) and torch.equal(vl, v[:, kb:kb + kc])
    # every query head of the shard maps to a KV head of the shard
    assert all(kb <= (qb + i) // 8 < kb + kc for i in range(qc))
    # stand-in for the per-rank attention output: a function of the local heads
    out_local = ql * 2.0 + 1.0
    gathered = torch.zeros(world, T, H // world, D)
    work = sharding.all_gather_heads(out_local, gathered, async_op=True)
    work.wait()
    full = sharding.gathered_to_full(gathered)
    ok = torch.equal(full, q * 2.0 + 1.0)
    ret[rank] = bool(ok)
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_head_sharded_all_gather(world):
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29600 + world
    mp.spawn(_worker, args=(world, port, 37, ret), nprocs=world, join=True)
    assert dict(ret) == {r: True for r in range(world)}


def test_head_shard_rejects_bad_worlds():
    entry.load_package()
    from sera_c_b200 import sharding
    assert sharding.head_shard(3, 8) == (3, 1, 24, 8)
    assert sharding.head_shard(1, 2) == (4, 4, 32, 32)
    with pytest.raises(ValueError):
        sharding.head_shard(0, 3)
    with pytest.raises(ValueError):
        sharding.head_shard(2, 2)
