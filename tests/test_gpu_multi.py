"""Two-GPU test of the per-layer output exchange
(q3_suffix_attention_layer_gathered: attention into this rank's slot, copy-engine
copies into the other ranks' gathered buffers, flags): the gathered result must
equal what a single GPU holding all heads produces. Skipped with fewer than two
GPUs. Ranks are child processes, one per GPU; nothing here waits without bound."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import __graft_entry__ as entry
import _cases
import _gpu_harness as harness

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    pkg = entry.load_package()
    from sera_c_b200 import sharding
    case = harness.rounded_case(_cases.Case("multi", 200, [40, 7, 33], n_heads=16 * world,
                                            n_kv_heads=2 * world, seed=77,
                                            unit_norm_weights=False))
    P, S, H, Hkv, D = case.P, case.S, case.H, case.Hkv, case.D
    kb, kc, qb, qc = sharding.head_shard(rank, world, Hkv)
    # this rank's shard as its own case
    import copy
    local = copy.copy(case)
    local.H, local.Hkv = qc, kc
    local.q = np.ascontiguousarray(case.q[:, qb:qb + qc])
    local.k = np.ascontiguousarray(case.k[:, kb:kb + kc])
    local.v = np.ascontiguousarray(case.v[:, kb:kb + kc])
    _, rt, prefix, bset, plan = harness.run_case_native(pkg, local, return_runtime=True,
                                                        device=rank)
    pg = sharding.PeerGather(S, qc, D, torch.bfloat16, dev)
    q, k, v = (harness.dev(a[P:], torch.bfloat16, dev) for a in (local.q, local.k, local.v))
    ok = True
    with torch.cuda.stream(rt.torch_stream()):
        for it in range(3):                     # buffers are reused (depth 2)
            plan.attention_layer_gathered(1, q, k, v, pg.peers(it), it + 1)
            rt.wait_gathered(pg.peers(it), it + 1)
            rt.synchronize()
            got = pg.full(it).float().cpu().numpy()
            ref_local = torch.zeros(S, qc, D, dtype=torch.bfloat16, device=dev)
            plan.attention_layer(1, q, k, v, ref_local)
            rt.synchronize()
            gathered = torch.zeros(world, S, qc, D, dtype=torch.bfloat16, device=dev)
            sharding.all_gather_heads(ref_local, gathered)
            torch.cuda.synchronize()
            want = sharding.gathered_to_full(gathered).float().cpu().numpy()
            ok = ok and np.array_equal(got, want)
            dist.barrier()
        # the same exchange recorded as a graph with step-relative sequence
        # numbers and replayed: flags left by one replay must not satisfy the next
        rt.synchronize()
        dist.barrier()
        rt.gather_advance(3)                     # past the numbers used above
        rt.graph_begin()
        for it in range(2):
            plan.attention_layer_gathered(1, q, k, v, pg.peers(it), it + 1)
        rt.wait_gathered(pg.peers(0), 1)
        rt.wait_gathered(pg.peers(1), 2)
        rt.gather_advance(2)
        graph = rt.graph_end()
        for rep in range(3):
            pg.bufs[0].zero_(); pg.bufs[1].zero_()
            torch.cuda.synchronize()
            dist.barrier()
            graph.launch()
            rt.synchronize()
            for it in range(2):
                ok = ok and np.array_equal(pg.full(it).float().cpu().numpy(), want)
            dist.barrier()
        graph.close()
        # host-buffer variant: q/k/v from pinned host memory, this rank's rows back
        hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
        outs = [torch.zeros(S, qc, D, dtype=torch.bfloat16).pin_memory() for _ in range(4)]
        for b in pg.bufs:
            b.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        for it in range(4):                      # three staging slots and two buffers wrap
            if it >= 2:
                rt.wait_gathered(pg.peers(it), it - 1)
            plan.attention_layer_gathered_host(1, hq, hk, hv, pg.peers(it), it + 1, outs[it])
        rt.wait_gathered(pg.peers(2), 3)
        rt.wait_gathered(pg.peers(3), 4)
        rt.gather_advance(4)
        rt.synchronize()
        for it in range(4):
            ok = ok and torch.equal(outs[it], ref_local.cpu())
        ok = ok and np.array_equal(pg.full(3).float().cpu().numpy(), want)
        dist.barrier()
    ok = ok and rt.stats().device_status == 0
    ret[rank] = bool(ok)
    for o in (plan, bset, prefix):
        o.close()
    rt.close()
    dist.destroy_process_group()


def test_fused_gather_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    entry.build()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, 29711, ret), nprocs=2, join=True)
    assert dict(ret) == {0: True, 1: True}
