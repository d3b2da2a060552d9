"""GPU parity at the sizes the benchmark numbers are quoted on.

  * one layer of the 64-layer stack workload (prefix 32768 in permuted pages,
    128 branches x 16 suffix tokens, 8 KV heads): the only shape whose shared KV
    is large enough to select the lockstep-waves schedule, checked on sampled
    rows against the oracle (ref math: src/q3_forward.cu:418-525);
  * a small batch forced onto the lockstep schedule, and onto stream-K, with
    every row compared;
  * paged decode at its full size: 256 sequences, contexts from
    numpy default_rng(1).integers(1024, 16385, 256), 8 KV heads, randomly
    permuted pages; a sample of sequences (shortest, longest, 16 others)
    against the oracle (ref math: src/q3_forward.cu:218-290).

Tolerance: max |got - oracle| <= 2e-3 absolute on fp32 output, the oracle fed
the same bf16 / f16 rounded inputs as the kernels.
"""
import numpy as np
import pytest
import torch

import __graft_entry__ as entry
import _cases
import _gpu_harness as harness
import q3_oracle as oracle

pytestmark = pytest.mark.gpu
ATOL = 2e-3


@pytest.fixture(scope="module")
def pkg():
    entry.build()
    return entry.load_package()


@pytest.mark.parametrize("page_order", ["permuted", "consecutive"])
def test_stack_layer_p32768_b128x16_sampled_rows(pkg, page_order):
    """`consecutive`: the pool's own allocation order, where the kernel fetches the
    eight pages of a key tile as one copy per half; `permuted`: one copy per page."""
    P, B, n, H, Hkv, D = 32768, 128, 16, 64, 8, 128
    S = B * n
    g = torch.Generator().manual_seed(0)
    kp = torch.randn(P, Hkv, D, generator=g).to(torch.float16)
    vp = torch.randn(P, Hkv, D, generator=g).to(torch.float16)
    q = torch.randn(S, H, D, generator=g).to(torch.bfloat16)
    k = torch.randn(S, Hkv, D, generator=g).to(torch.bfloat16)
    v = torch.randn(S, Hkv, D, generator=g).to(torch.bfloat16)
    n_pp = P // 16
    num_pages = n_pp + B + 8
    rt = pkg.Runtime(num_layers=1, n_heads=H, n_kv_heads=Hkv, max_positions=P + 64,
                     max_tokens=S, num_pages=num_pages, out_fp32=True)
    perm = (np.random.default_rng(1).permutation(num_pages) if page_order == "permuted"
            else np.arange(num_pages)).astype(np.uint32)
    rt.alloc_pages(num_pages)
    rt.free_pages(perm[n_pp:][::-1].copy())
    prefix = pkg.Prefix(rt, P, pages=perm[:n_pp])
    pk, pv = rt.pool()
    idx = torch.from_numpy(perm[:n_pp].astype(np.int64)).cuda()
    pk[0][:, idx] = kp.cuda().reshape(n_pp, 16, Hkv, D).permute(2, 0, 1, 3)
    pv[0][:, idx] = vp.cuda().reshape(n_pp, 16, Hkv, D).permute(2, 0, 1, 3)
    torch.cuda.synchronize()
    prefix.set_resident(P)
    prefix.seal()
    bset = pkg.BranchSet(prefix, B, n)
    handles = [bset.acquire() for _ in range(B)]
    plan = pkg.PackPlan(prefix, bset, [(h, n) for h in handles])

    # the schedule this shape gets: whole items in waves plus a cut tail
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    tag = np.repeat(np.arange(B, dtype=np.uint32), n)
    lp = np.tile(np.arange(n, dtype=np.uint32), B)
    summ, segs = pkg.schedule_describe(tag, lp, Hkv, P, 1, B, sms, lockstep=True)
    whole = [s for s in segs if s.partial_slot < 0]
    cut = [s for s in segs if s.partial_slot >= 0]
    assert whole and cut and summ.grid == sms
    # tokens: first / last of a 32-token tile, first / last branch, one token of a
    # cut item's tile and one of a whole item's tile (all 64 heads are compared,
    # so every KV head of each sampled token is covered)
    tokens = sorted({0, 1, 15, 16, 31, 32, S - 17, S - 1, cut[0].tok0 + 5,
                     cut[-1].tok0 + 30, whole[0].tok0 + 9, whole[-1].tok0 + 20})
    tokens = [t for t in tokens if t < S]

    out = torch.zeros(S, H, D, dtype=torch.float32, device="cuda")
    plan.attention_layer(0, q.cuda(), k.cuda(), v.cuda(), out)
    rt.synchronize()
    assert rt.stats().device_status == 0
    ifreq = oracle.inv_freq(1e6, D)
    ones = np.ones(D, np.float32)
    pos = (P + np.tile(np.arange(n), B)).astype(np.uint32)
    qn = oracle.rms_norm(q.float().numpy(), ones, 1e-6)
    kn = oracle.rms_norm(k.float().numpy(), ones, 1e-6)
    qn, kn = oracle.rope(qn, kn, 0, pos, ifreq)
    kpn, vpn, vn = kp.float().numpy(), vp.float().numpy(), v.float().numpy()
    scale = np.float32(1 / np.sqrt(D))
    worst = 0.0
    for t in tokens:
        b, l = t // n, t % n
        keys = np.concatenate([kpn, kn[b * n:b * n + l + 1]])
        vals = np.concatenate([vpn, vn[b * n:b * n + l + 1]])
        ref = oracle.attention(qn[t:t + 1], keys, vals, P + l, P + l + 1, scale)[0]
        err = float(np.abs(out[t].cpu().numpy() - ref).max())
        worst = max(worst, err)
        assert err <= ATOL, (t, err)
    print("stack layer, %d sampled tokens x 64 heads: max abs err %.3e" % (len(tokens), worst))
    # every row was written, none is far from the value range of an average of N(0,1) values
    o = out.cpu().numpy()
    assert np.isfinite(o).all() and np.abs(o).max() < 1.0 and (np.abs(o).max(axis=(1, 2)) > 0).all()
    for x in (plan, bset, prefix):
        x.close()
    rt.close()


@pytest.mark.parametrize("policy", ["lockstep", "streamk"])
def test_forced_schedule_every_row(pkg, policy):
    """20 token tiles x 8 KV heads = 160 items on 148 CTAs: under the lockstep
    policy one wave of whole items plus a cut tail."""
    case = harness.rounded_case(_cases.Case("sched", 300, [16] * 40, n_heads=64, n_kv_heads=8,
                                            seed=11, unit_norm_weights=False))
    ref = oracle.run_case(case)["out"]
    got = harness.run_case_native(pkg, case, out_fp32=True, sched_policy=policy)
    err = np.abs(got - ref).max()
    print("%s: max abs err %.3e" % (policy, err))
    assert err <= ATOL


def test_decode_256_sequences_full_size(pkg):
    Hkv, H, D = 8, 64, 128
    ctx = np.random.default_rng(1).integers(1024, 16385, 256).astype(np.uint32)
    S = len(ctx)
    n_pages = (ctx + 15) // 16
    total = int(n_pages.sum())
    rt = pkg.Runtime(num_layers=1, n_heads=H, n_kv_heads=Hkv, max_positions=16400,
                     max_tokens=S, num_pages=total + 4, out_fp32=True)
    g = torch.Generator(device="cuda").manual_seed(4)
    kp, vp = rt.pool()
    kp.normal_(generator=g)
    vp.normal_(generator=g)
    perm = np.random.default_rng(2).permutation(total + 4)[:total].astype(np.uint32)
    indptr = np.concatenate([[0], np.cumsum(n_pages)]).astype(np.uint32)
    q = torch.randn(S, H, D, generator=g, device="cuda").to(torch.bfloat16)
    torch.cuda.synchronize()
    plan = pkg.DecodePlan(rt, ctx, indptr, perm)
    out = torch.zeros(S, H, D, dtype=torch.float32, device="cuda")
    plan.attention_layer(0, q, None, None, out)
    rt.synchronize()
    assert rt.stats().device_status == 0
    got = out.cpu().numpy()
    assert np.isfinite(got).all()

    sample = sorted({int(np.argmax(ctx)), int(np.argmin(ctx)), 0, S - 1} |
                    set(int(x) for x in np.random.default_rng(3).choice(S, 16, replace=False)))
    ifreq = oracle.inv_freq(1e6, D)
    ones = np.ones(D, np.float32)
    qn = oracle.rms_norm(q.float().cpu().numpy(), ones, 1e-6)
    qn, _ = oracle.rope(qn, np.zeros((S, Hkv, D), np.float32), 0, ctx, ifreq)
    scale = np.float32(1 / np.sqrt(D))
    worst = 0.0
    for s in sample:
        c = int(ctx[s])
        pages = torch.from_numpy(perm[indptr[s]:indptr[s + 1]].astype(np.int64)).cuda()
        # pool layout [Hkv, page, 16, D] -> [tokens, Hkv, D]
        ks = np.ascontiguousarray(
            kp[0][:, pages].permute(1, 2, 0, 3).reshape(-1, Hkv, D)[:c].float().cpu().numpy())
        vs = np.ascontiguousarray(
            vp[0][:, pages].permute(1, 2, 0, 3).reshape(-1, Hkv, D)[:c].float().cpu().numpy())
        ref = oracle.decode(qn[s], ks, vs, scale)
        err = float(np.abs(got[s] - ref).max())
        worst = max(worst, err)
        assert err <= ATOL, (s, c, err)
    print("decode 256 sequences (sum ctx %d): %d sampled, max abs err %.3e"
          % (int(ctx.sum()), len(sample), worst))
    plan.close()
    rt.close()
