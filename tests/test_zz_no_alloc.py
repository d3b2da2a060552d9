"""The allocation-free decode entry point (q3_cuda_attention_decode_noalloc),
called through the C ABI, against the ordinary decode entry point and against
the CPU oracle.

Who needs it: hosts that cannot call cudaMalloc when they need attention - a
server whose arena owns the whole device heap, a process that forbids device
allocation after start-up, a plugin that must not re-enter its host's
allocator. The split-KV partials then live in a fixed array inside the library.

Collected last on purpose (file name), so that a run that stops at the first
failure has already run every other test. Runs alone or after the others.
"""
import numpy as np
import pytest
import torch

import __graft_entry__ as entry
import q3_oracle as oracle

pytestmark = pytest.mark.gpu
ATOL = 2e-3


def test_noalloc_decode_matches_decode_entry_twice():
    entry.build()
    pkg = entry.load_package()
    Hkv, H, D, layer = 2, 16, 128, 1
    ctx = np.asarray([40, 1500, 3000, 1024, 2049], np.uint32)   # multi-chunk: scratch is used
    n_pages = (ctx + 15) // 16
    total = int(n_pages.sum())
    rt = pkg.Runtime(num_layers=2, n_heads=H, n_kv_heads=Hkv, max_positions=4096,
                     max_tokens=len(ctx), num_pages=total + 3)
    g = torch.Generator(device="cuda").manual_seed(17)
    kp, vp = rt.pool()
    kp.normal_(generator=g)
    vp.normal_(generator=g)
    perm = np.random.default_rng(4).permutation(total + 3)[:total].astype(np.uint32)
    indptr = np.concatenate([[0], np.cumsum(n_pages)]).astype(np.uint32)
    q = torch.randn(len(ctx), H, D, generator=g, device="cuda").to(torch.bfloat16)
    torch.cuda.synchronize()

    # the existing entry point
    plan = pkg.DecodePlan(rt, ctx, indptr, perm)
    ref = torch.zeros(len(ctx), H, D, dtype=torch.bfloat16, device="cuda")
    plan.attention_layer(layer, q, None, None, ref)
    rt.synchronize()

    # inputs of the new entry point, all caller-owned
    i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int32)).cuda()
    d_ctx, d_ptr, d_idx = i32(ctx), i32(indptr), i32(perm)
    q_f16 = torch.zeros(len(ctx), H, D, dtype=torch.float16, device="cuda")
    rt.qknorm_rope_kvwrite(layer, q, None, None, d_ctx, None, None, q_f16)
    rt.synchronize()
    work, swb = pkg.decode_work_host(ctx)
    assert len(work) > len(ctx)                     # at least one sequence is split
    d_work, d_swb = i32(work), i32(swb)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for _ in range(2):                              # two calls in a row share the array
        out = torch.full((len(ctx), H, D), float("nan"), dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        pkg.attention_decode_noalloc(q_f16, kp[layer], vp[layer], d_ctx, d_ptr, d_idx,
                                     d_work, d_swb, out)
        torch.cuda.synchronize()
        err = (out.float() - ref.float()).abs().max().item()
        assert err <= ATOL, err
        # no bounded wait of the call gave up (the word is read and cleared)
        assert pkg.attention_decode_noalloc_status() == 0
    # ... and against the oracle (ref math: src/q3_forward.cu:218-290), fed the
    # f16 query and the f16 pages the kernel read
    scale = np.float32(1 / np.sqrt(D))
    qf = q_f16.float().cpu().numpy()
    got = out.float().cpu().numpy()
    for s, c in enumerate(ctx):
        pages = torch.from_numpy(perm[indptr[s]:indptr[s + 1]].astype(np.int64)).cuda()
        ks = np.ascontiguousarray(
            kp[layer][:, pages].permute(1, 2, 0, 3).reshape(-1, Hkv, D)[:c].float().cpu().numpy())
        vs = np.ascontiguousarray(
            vp[layer][:, pages].permute(1, 2, 0, 3).reshape(-1, Hkv, D)[:c].float().cpu().numpy())
        want = oracle.decode(np.ascontiguousarray(qf[s]), ks, vs, scale)
        half_ulp = np.abs(want) * 2.0 ** -8          # bf16 output rounding
        assert (np.maximum(np.abs(got[s] - want) - half_ulp, 0).max() <= ATOL), s
    assert torch.cuda.mem_get_info()[0] >= free_before - (1 << 20)

    # beyond the fixed scratch: refused with a clear message, nothing launched
    big = torch.zeros(2049, 4, dtype=torch.int32, device="cuda")
    with pytest.raises(pkg.Q3Error, match="exceed the fixed scratch"):
        pkg.attention_decode_noalloc(q_f16, kp[layer], vp[layer], d_ctx, d_ptr, d_idx,
                                     big, d_swb, out)
    plan.close()
    rt.close()
