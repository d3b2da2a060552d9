"""GPU parity tests: every kernel of the path, called through the C ABI, against
the CPU oracle (oracle/) on the same seeded inputs.

Tolerances (stated once):
  * attention, fp32 output: max |got - oracle| <= 2e-3 absolute. The oracle is
    fed the bf16-rounded inputs the kernels are fed, so what is measured is the
    kernels' own error (f16 operands for Q, K, V, P; fp32 accumulation).
  * attention, bf16 output: the same after discounting half a bf16 ulp of the
    reference value (output rounding), normalised by max |oracle|.
  * RMSNorm + RoPE + KV write: the reference's own 1e-4 plus half an f16 ulp of
    the stored value (the cache dtype).
  * argmax of a seeded 4-candidate projection of each branch's last row is
    identical to the oracle's (stand-in for the candidate-token argmax; the
    model's LM head is not available).
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


def _candidate_argmax(out, case, seed=99):
    """Proxy for 'candidate-token argmax identical': logits = W_c . attn_out of
    each branch's last token, W_c seeded fp32 [4, H*D]."""
    if not case.S:
        return np.zeros(0, np.int64)
    g = np.random.default_rng(seed)
    W = g.standard_normal((4, case.H * case.D)).astype(np.float32)
    last = case.P + case.branch_offsets[1:].astype(np.int64) - 1
    return np.argmax(out[last].reshape(len(last), -1) @ W.T, axis=1)


@pytest.mark.parametrize("name", _cases.GOLDEN_CASES)
def test_case_fp32_output(pkg, name):
    case = harness.rounded_case(_cases.make_case(name))
    ref = oracle.run_case(case)["out"]
    got = harness.run_case_native(pkg, case, out_fp32=True)
    err = np.abs(got - ref).max()
    print("%s: max abs err %.3e (max |ref| %.2f)" % (name, err, np.abs(ref).max()))
    assert err <= ATOL
    assert np.array_equal(_candidate_argmax(got, case), _candidate_argmax(ref, case))


@pytest.mark.parametrize("name", _cases.GOLDEN_CASES + ["long_prefix"])
def test_case_with_pages_in_allocation_order(pkg, name):
    """Pages as the pool hands them out (ascending): key tiles whose eight pages
    follow one another are fetched as one copy per half, through the second
    tensor map of the pool - the path the other tests (permuted pages) do not
    take."""
    case = (harness.rounded_case(_cases.Case("long_prefix", 1500, [40, 3, 33, 17], n_heads=16,
                                             n_kv_heads=2, seed=21, unit_norm_weights=False))
            if name == "long_prefix" else harness.rounded_case(_cases.make_case(name)))
    ref = oracle.run_case(case)["out"]
    got = harness.run_case_native(pkg, case, out_fp32=True, permute_pages=False)
    assert np.abs(got - ref).max() <= ATOL
    chunked = harness.run_case_native(pkg, case, out_fp32=True, permute_pages=False,
                                      prefill_chunks=[case.P - case.P // 3, case.P // 3])
    assert np.abs(chunked - ref).max() <= ATOL


@pytest.mark.parametrize("name", _cases.GOLDEN_CASES)
def test_case_bf16_output(pkg, name):
    case = harness.rounded_case(_cases.make_case(name))
    ref = oracle.run_case(case)["out"]
    got = harness.run_case_native(pkg, case, out_fp32=False)
    assert harness.max_err_vs_bf16_oracle(got, ref) <= ATOL
    assert np.array_equal(_candidate_argmax(got, case), _candidate_argmax(ref, case))


def test_kvwrite_matches_oracle(pkg):
    """Fused QK-RMSNorm + RoPE + paged KV write against the oracle's a1 -> a2/a3."""
    case = harness.rounded_case(_cases.make_case("ragged"))
    T, H, Hkv, D = case.T, case.H, case.Hkv, case.D
    rt = pkg.Runtime(num_layers=3, n_heads=H, n_kv_heads=Hkv, max_positions=40000,
                     max_tokens=T, num_pages=64)
    layer = 2
    rt.set_qk_norm(layer, case.q_norm_w, case.k_norm_w)
    rng = np.random.default_rng(5)
    # arbitrary positions up to the large-position regime, arbitrary page slots
    pos = rng.integers(0, 39000, T).astype(np.uint32)
    pos[:4] = [0, 1, 32783, 38999]
    slots = rng.permutation(64 * 16)[:T]
    dpage, dslot = (slots // 16).astype(np.uint32), (slots % 16).astype(np.uint32)
    q, k, v = (harness.dev(a, torch.bfloat16) for a in (case.q, case.k, case.v))
    q2 = torch.zeros(T, H, D, dtype=torch.float16, device="cuda")
    i32 = torch.int32
    rt.qknorm_rope_kvwrite(layer, q, k, v, harness.dev(pos.astype(np.int32), i32),
                           harness.dev(dpage.astype(np.int32), i32),
                           harness.dev(dslot.astype(np.int32), i32), q2)
    rt.synchronize()
    kp, vp = rt.pool()
    ifreq = oracle.inv_freq(case.theta, D)
    q1 = oracle.rms_norm(case.q, case.q_norm_w, case.eps)
    k1 = oracle.rms_norm(case.k, case.k_norm_w, case.eps)
    qr, kr = oracle.rope(q1, k1, 0, pos, ifreq)

    def close(got, ref):
        tol = 1e-4 + np.abs(ref) * 2.0 ** -11
        return bool(np.all(np.abs(got - ref) <= tol))

    assert close(q2.float().cpu().numpy(), qr)
    ip = torch.from_numpy(dpage.astype(np.int64)).cuda()
    isl = torch.from_numpy(dslot.astype(np.int64)).cuda()
    gk = kp[layer][:, ip, isl].permute(1, 0, 2).float().cpu().numpy()
    gv = vp[layer][:, ip, isl].permute(1, 0, 2).float().cpu().numpy()
    assert close(gk, kr)
    assert np.array_equal(gv, case.v)        # bf16 -> f16 is exact for these values
    # other layers and unwritten slots stay zero
    assert float(kp[0].abs().max()) == 0.0 and float(vp[1].abs().max()) == 0.0
    mask = torch.ones(64 * 16, dtype=torch.bool, device="cuda")
    mask[torch.from_numpy(slots.astype(np.int64)).cuda()] = False
    assert float(kp[layer].reshape(Hkv, -1, D)[:, mask].abs().max()) == 0.0
    rt.close()


def test_chunked_prefill_equals_one_shot(pkg):
    """Shape of the reference's test 4a (tests/test_q3_forward.cu:388-483):
    prefill in pieces through the cache == one contiguous pass."""
    case = harness.rounded_case(_cases.Case("chunks", 150, [], n_heads=16, n_kv_heads=2,
                                            seed=21))
    ref = oracle.run_case(case)["out"]
    one = harness.run_case_native(pkg, case, out_fp32=True)
    parts = harness.run_case_native(pkg, case, out_fp32=True, prefill_chunks=[37, 64, 1, 48])
    assert np.abs(one - ref).max() <= ATOL
    assert np.abs(parts - ref).max() <= ATOL
    assert np.abs(parts - one).max() <= 5e-4


def test_split_prefix_suffix_equals_contiguous(pkg):
    """One branch through [prefix | suffix] equals one causal pass over P+S
    tokens (the reference's prefix+suffix equivalence, tests/test_q3_decide.cu:191-353)."""
    seg = harness.rounded_case(_cases.Case("seg", 83, [29], n_heads=16, n_kv_heads=2, seed=4))
    full = harness.rounded_case(_cases.Case("full", 112, [], n_heads=16, n_kv_heads=2, seed=4))
    full.q, full.k, full.v = seg.q, seg.k, seg.v
    a = harness.run_case_native(pkg, seg, out_fp32=True)
    b = harness.run_case_native(pkg, full, out_fp32=True)
    assert np.abs(a - b).max() <= 5e-4
    assert np.abs(a - oracle.run_case(seg)["out"]).max() <= ATOL


def test_branch_isolation_and_order(pkg):
    """tests/test_q3_decide.cu:370-511: a branch's rows do not depend on which
    other branches share the batch, nor on their order or handle."""
    base = _cases.Case("iso", 40, [7, 19, 5], n_heads=16, n_kv_heads=2, seed=8)
    base = harness.rounded_case(base)
    all3 = harness.run_case_native(pkg, base, out_fp32=True)
    P = base.P
    # branch 1 alone (rows P+7 .. P+26), under a different handle
    solo = _cases.Case("solo", 40, [19], n_heads=16, n_kv_heads=2, seed=8,
                       branch_handles=[3])
    rows = np.r_[0:P, P + 7:P + 26]
    solo.q, solo.k, solo.v = base.q[rows], base.k[rows], base.v[rows]
    alone = harness.run_case_native(pkg, solo, out_fp32=True)
    assert np.abs(alone[P:] - all3[P + 7:P + 26]).max() <= 2e-4
    # reversed order
    rev = _cases.Case("rev", 40, [5, 19, 7], n_heads=16, n_kv_heads=2, seed=8,
                      branch_handles=[2, 1, 0])
    order = np.r_[0:P, P + 26:P + 31, P + 7:P + 26, P:P + 7]
    rev.q, rev.k, rev.v = base.q[order], base.k[order], base.v[order]
    r = harness.run_case_native(pkg, rev, out_fp32=True)
    assert np.abs(r[P + 5:P + 24] - all3[P + 7:P + 26]).max() <= 2e-4
    assert np.abs(r[P:P + 5] - all3[P + 26:P + 31]).max() <= 2e-4


def test_long_suffixes_many_tiles(pkg):
    """Suffixes longer than one key tile and a prefix that is not a multiple of
    the page or tile size; more items than one CTA wave is not needed to hit
    cut items: 2 KV heads x few tiles on 148 CTAs cuts every item."""
    case = harness.rounded_case(_cases.Case("long", 1000, [300, 17, 160], n_heads=16,
                                            n_kv_heads=2, seed=31, unit_norm_weights=False))
    ref = oracle.run_case(case)["out"]
    got = harness.run_case_native(pkg, case, out_fp32=True)
    assert np.abs(got - ref).max() <= ATOL
    assert np.array_equal(_candidate_argmax(got, case), _candidate_argmax(ref, case))


def test_guard_rows_around_outputs_and_pool(pkg):
    """Stand-in for a memory checker: the attention output sits between guard
    rows filled with a sentinel, and every page of the pool that the batch does
    not own must stay zero - in the layer that ran and in the one that did not.
    The shape cuts every item into pieces (2 KV heads x few key tiles on all
    CTAs), so the partial-combination path writes the rows."""
    case = harness.rounded_case(_cases.Case("guard", 700, [130, 9, 40], n_heads=16,
                                            n_kv_heads=2, seed=13))
    got, rt, prefix, bset, plan = harness.run_case_native(pkg, case, out_fp32=True,
                                                          return_runtime=True)
    P, S, H, D = case.P, case.S, case.H, case.D
    GUARD, SENT = 64, 12345.0
    buf = torch.full((GUARD + S + GUARD, H, D), SENT, dtype=torch.float32, device="cuda")
    q, k, v = (harness.dev(a[P:], torch.bfloat16) for a in (case.q, case.k, case.v))
    torch.cuda.synchronize()
    plan.attention_layer(1, q, k, v, buf[GUARD:GUARD + S])
    rt.synchronize()
    assert rt.stats().device_status == 0
    assert bool((buf[:GUARD] == SENT).all()) and bool((buf[GUARD + S:] == SENT).all())
    assert np.array_equal(buf[GUARD:GUARD + S].cpu().numpy(), got[P:])
    kp, vp = rt.pool()
    owned = set(prefix.page_table().tolist()) | set(bset.page_table().reshape(-1).tolist())
    free = torch.tensor([i for i in range(rt.cfg.num_pages) if i not in owned],
                        dtype=torch.long, device="cuda")
    assert len(free) >= 7
    for pool in (kp, vp):
        assert float(pool[1][:, free].abs().max()) == 0.0
        assert float(pool[0].abs().max()) == 0.0
    for o in (plan, bset, prefix):
        o.close()
    rt.close()


def test_warm_path_counters(pkg):
    """Zero allocations and zero host syncs across repeated layers of a batch
    (the reference's gate, tests/test_q3_decide.cu:632-821), and repeatability."""
    case = harness.rounded_case(_cases.make_case("ragged"))
    got, rt, prefix, bset, plan = harness.run_case_native(pkg, case, return_runtime=True)
    P = case.P
    q, k, v = (harness.dev(a[P:], torch.bfloat16) for a in (case.q, case.k, case.v))
    out = torch.zeros(case.S, case.H, case.D, dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    s0 = rt.stats()
    for _ in range(3):
        plan.attention_layer(1, q, k, v, out)
    s1 = rt.stats()
    assert s1.cuda_allocations == s0.cuda_allocations
    assert s1.cuda_frees == s0.cuda_frees
    assert s1.host_syncs == s0.host_syncs
    assert s1.kernel_launches > s0.kernel_launches
    rt.synchronize()
    assert rt.stats().device_status == 0
    assert np.array_equal(out.float().cpu().numpy(), got[P:])     # bit-exact repeat
    assert prefix.kv_bytes() == 2 * 2 * ((P + 15) // 16) * 16 * case.Hkv * 128 * 2
    for o in (plan, bset, prefix):
        o.close()
    rt.close()


def test_host_buffer_entry_pipelined(pkg):
    """q3_suffix_attention_layer_host: five back-to-back calls (three staging
    slots, so slots are reused) give the same rows as the device entry."""
    case = harness.rounded_case(_cases.make_case("ragged"))
    _, rt, prefix, bset, plan = harness.run_case_native(pkg, case, return_runtime=True)
    P, S = case.P, case.S
    g = torch.Generator().manual_seed(3)
    outs_dev, outs_host, keep = [], [], []
    for i in range(5):
        q = torch.randn(S, case.H, case.D, generator=g).to(torch.bfloat16)
        k = torch.randn(S, case.Hkv, case.D, generator=g).to(torch.bfloat16)
        v = torch.randn(S, case.Hkv, case.D, generator=g).to(torch.bfloat16)
        od = torch.zeros(S, case.H, case.D, dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        plan.attention_layer(i % 2, q.cuda(), k.cuda(), v.cuda(), od)
        rt.synchronize()
        outs_dev.append(od.cpu())
        keep.append((q.pin_memory(), k.pin_memory(), v.pin_memory(),
                     torch.zeros(S, case.H, case.D, dtype=torch.bfloat16).pin_memory()))
    s0 = rt.stats()
    for i, (q, k, v, oh) in enumerate(keep):
        plan.attention_layer_host(i % 2, q, k, v, oh)
    rt.synchronize()
    for i, (_, _, _, oh) in enumerate(keep):
        assert torch.equal(oh, outs_dev[i]), i
    s1 = rt.stats()
    assert s1.host_syncs == s0.host_syncs + 1      # only the explicit synchronize
    for o in (plan, bset, prefix):
        o.close()
    rt.close()


def test_graph_replay_equals_eager(pkg):
    """q3_attn_graph_*: two layer calls recorded once and replayed; every
    replay gives the rows of the eager calls, also after the inputs changed
    in place (the graph holds pointers, not data)."""
    case = harness.rounded_case(_cases.make_case("ragged"))
    _, rt, prefix, bset, plan = harness.run_case_native(pkg, case, return_runtime=True)
    S = case.S
    g = torch.Generator().manual_seed(5)
    mk = lambda h: torch.randn(S, h, case.D, generator=g).to(torch.bfloat16).cuda()
    q, k, v = mk(case.H), mk(case.Hkv), mk(case.Hkv)
    o = [torch.zeros(S, case.H, case.D, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    e = [torch.zeros_like(o[0]) for _ in range(2)]
    host = [t.cpu().pin_memory() for t in (q, k, v, o[0])]
    torch.cuda.synchronize()
    launches0 = rt.stats().kernel_launches
    rt.graph_begin()
    plan.attention_layer(0, q, k, v, o[0])
    plan.attention_layer(1, q, k, v, o[1])
    with pytest.raises(pkg.Q3Error, match="cannot be recorded"):
        plan.attention_layer_host(0, *host)
    graph = rt.graph_end()
    rt.synchronize()
    assert rt.stats().kernel_launches == launches0      # recording runs nothing
    assert float(o[0].abs().max()) == 0.0
    for rep in range(3):
        graph.launch()
        rt.synchronize()
        plan.attention_layer(0, q, k, v, e[0])
        plan.attention_layer(1, q, k, v, e[1])
        rt.synchronize()
        assert torch.equal(o[0], e[0]) and torch.equal(o[1], e[1]), rep
        assert float(o[0].float().abs().max()) > 0.0
        q.copy_(mk(case.H)); k.copy_(mk(case.Hkv)); v.copy_(mk(case.Hkv))
        torch.cuda.synchronize()
    assert rt.stats().kernel_launches == launches0 + 3 * 4 + 3 * 4
    assert rt.stats().device_status == 0
    graph.close()
    for x in (plan, bset, prefix):
        x.close()
    rt.close()


@pytest.mark.parametrize("seed", [0, 1, 2, 3])
def test_random_ragged_batches(pkg, seed):
    """Randomly shaped batches: prefix lengths around page and tile boundaries,
    1..9 branches of 1..70 tokens under scattered handles, 1-4 KV heads."""
    rng = np.random.default_rng(100 + seed)
    P = int(rng.choice([1, 15, 16, 17, 127, 128, 129, 255, 300, 513]))
    nb = int(rng.integers(1, 10))
    lens = [int(x) for x in rng.integers(1, 71, nb)]
    handles = [int(x) for x in rng.permutation(nb + 3)[:nb]]
    hkv = int(rng.choice([1, 2, 4]))
    case = harness.rounded_case(_cases.Case("rand%d" % seed, P, lens, n_heads=8 * hkv,
                                            n_kv_heads=hkv, seed=seed,
                                            unit_norm_weights=bool(seed % 2),
                                            branch_handles=handles))
    ref = oracle.run_case(case)["out"]
    got = harness.run_case_native(pkg, case, out_fp32=True, seed=seed)
    assert np.abs(got - ref).max() <= ATOL
    assert np.array_equal(_candidate_argmax(got, case), _candidate_argmax(ref, case))


def test_suffix_at_default_cap(pkg):
    """One branch at the reference's default suffix capacity (512 tokens,
    ref: src/q3_decide.h:25) next to short ones."""
    case = harness.rounded_case(_cases.Case("cap", 64, [512, 2, 31], n_heads=8, n_kv_heads=1,
                                            seed=9))
    ref = oracle.run_case(case)["out"]
    got = harness.run_case_native(pkg, case, out_fp32=True)
    assert np.abs(got - ref).max() <= ATOL


def test_bounded_wait_reports_instead_of_hanging(pkg):
    """A device-side wait whose flag nobody sets gives up after about a second
    and reports through the status word; the context stays usable."""
    import ctypes
    rt = pkg.Runtime(num_layers=1, n_heads=8, n_kv_heads=1, max_positions=64,
                     max_tokens=16, num_pages=8)
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    buf = torch.zeros(16, dtype=torch.bfloat16, device="cuda")
    peers = pkg.GatherPeers()
    peers.n_ranks, peers.rank = 2, 0
    for r in range(2):
        peers.gathered[r] = buf.data_ptr()
        peers.flags[r] = flags.data_ptr()
    flags[0] = 5                      # rank 0 "arrived", rank 1 never does
    torch.cuda.synchronize()
    rt.wait_gathered(peers, 5)
    with pytest.raises(pkg.Q3Error, match="gave up a bounded wait"):
        rt.synchronize()
    assert rt.stats().device_status & 2
    assert int(flags.sum().item()) == 5          # the device still answers
    # the documented recovery: clear the status word and the arrival counters
    rt.reset_status()
    rt.synchronize()
    assert rt.stats().device_status == 0
    rt.close()


def test_error_paths(pkg):
    rt = pkg.Runtime(num_layers=1, n_heads=8, n_kv_heads=1, max_positions=256,
                     max_tokens=32, num_pages=12)
    prefix = pkg.Prefix(rt, 64)
    with pytest.raises(pkg.Q3Error, match="prefix is empty"):
        prefix.seal()
    x = torch.zeros(40, 8, 128, dtype=torch.bfloat16, device="cuda")
    kv = torch.zeros(40, 1, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(pkg.Q3Error, match="exceeds runtime capacity"):
        prefix.prefill_layer(0, x, kv, kv, x)
    with pytest.raises(pkg.Q3Error, match="layer out of range"):
        prefix.prefill_layer(1, x[:8], kv[:8], kv[:8], x[:8])
    with pytest.raises(pkg.Q3Error, match="not sealed"):
        bs = pkg.BranchSet(prefix, 2, 16)
        pkg.PackPlan(prefix, bs, [(0, 4)])
    prefix.set_resident(60)
    prefix.seal()
    with pytest.raises(pkg.Q3Error, match="already sealed"):
        prefix.prefill_layer(0, x[:4], kv[:4], kv[:4], x[:4])
    with pytest.raises(pkg.Q3Error, match="exceeds runtime capacity"):
        pkg.PackPlan(prefix, bs, [(0, 16), (1, 16), (0, 1)])
    with pytest.raises(pkg.Q3Error, match="page pool exhausted"):
        pkg.BranchSet(prefix, 64, 64)
    with pytest.raises(pkg.Q3Error, match="branch limit exceeded"):
        for _ in range(3):
            bs.acquire()
    bs.close()
    prefix.close()
    rt.close()


def _sampled_rows_oracle(qn, kn, vn, rows, visible, scale):
    """Oracle attention for a few query rows only: row i sees keys [0, visible[i])."""
    out = np.zeros((len(rows),) + qn.shape[1:], np.float32)
    for i, (r, n) in enumerate(zip(rows, visible)):
        out[i] = oracle.attention(qn[r:r + 1], kn, vn, n - 1, n, scale)[0]
    return out


def test_prefill_4096_sampled_rows(pkg):
    """The causal-prefill benchmark configuration at full size (4096 tokens,
    64/8 heads), checked on sampled rows, with a permuted page table."""
    T, H, Hkv, D = 4096, 64, 8, 128
    g = torch.Generator().manual_seed(0)
    q = torch.randn(T, H, D, generator=g).to(torch.bfloat16)
    k = torch.randn(T, Hkv, D, generator=g).to(torch.bfloat16)
    v = torch.randn(T, Hkv, D, generator=g).to(torch.bfloat16)
    rt = pkg.Runtime(num_layers=1, n_heads=H, n_kv_heads=Hkv, max_positions=T,
                     max_tokens=T, num_pages=300, out_fp32=True)
    perm = np.random.default_rng(1).permutation(300).astype(np.uint32)
    rt.alloc_pages(300)
    prefix = pkg.Prefix(rt, T, pages=perm[:256])
    out = torch.zeros(T, H, D, dtype=torch.float32, device="cuda")
    prefix.prefill_layer(0, q.cuda(), k.cuda(), v.cuda(), out)
    rt.synchronize()
    assert rt.stats().device_status == 0
    ifreq = oracle.inv_freq(1e6, D)
    ones = np.ones(D, np.float32)
    qn = oracle.rms_norm(q.float().numpy(), ones, 1e-6)
    kn = oracle.rms_norm(k.float().numpy(), ones, 1e-6)
    qn, kn = oracle.rope(qn, kn, 0, None, ifreq)
    rows = [0, 1, 15, 16, 31, 32, 127, 128, 129, 1000, 2047, 2048, 3333, 4080, 4095]
    ref = _sampled_rows_oracle(qn, kn, v.float().numpy(), rows, [r + 1 for r in rows],
                               np.float32(1 / np.sqrt(D)))
    got = out[rows].cpu().numpy()
    assert np.abs(got - ref).max() <= ATOL
    prefix.close()
    rt.close()


def test_cascade_8192_sampled_rows(pkg):
    """The cascade benchmark configuration at full size: resident 8192-token
    prefix in permuted pages + 64 branches x 24, checked on sampled rows."""
    P, B, n, H, Hkv, D = 8192, 64, 24, 64, 8, 128
    S = B * n
    g = torch.Generator().manual_seed(0)
    # resident prefix KV: already normalised / roped values, f16
    kp = torch.randn(P, Hkv, D, generator=g).to(torch.float16)
    vp = torch.randn(P, Hkv, D, generator=g).to(torch.float16)
    q = torch.randn(S, H, D, generator=g).to(torch.bfloat16)
    k = torch.randn(S, Hkv, D, generator=g).to(torch.bfloat16)
    v = torch.randn(S, Hkv, D, generator=g).to(torch.bfloat16)
    n_pp = P // 16
    num_pages = n_pp + B * 2 + 5
    rt = pkg.Runtime(num_layers=1, n_heads=H, n_kv_heads=Hkv, max_positions=P + 64,
                     max_tokens=S, num_pages=num_pages, out_fp32=True)
    perm = np.random.default_rng(2).permutation(num_pages).astype(np.uint32)
    rt.alloc_pages(num_pages)
    rt.free_pages(perm[n_pp:])
    prefix = pkg.Prefix(rt, P, pages=perm[:n_pp])
    pk, pv = rt.pool()
    idx = torch.from_numpy(perm[:n_pp].astype(np.int64)).cuda()
    # pool layout [L, Hkv, page, 16, D]
    pk[0][:, idx] = kp.cuda().reshape(n_pp, 16, Hkv, D).permute(2, 0, 1, 3)
    pv[0][:, idx] = vp.cuda().reshape(n_pp, 16, Hkv, D).permute(2, 0, 1, 3)
    torch.cuda.synchronize()
    prefix.set_resident(P)
    prefix.seal()
    bset = pkg.BranchSet(prefix, B, n)
    handles = [bset.acquire() for _ in range(B)]
    plan = pkg.PackPlan(prefix, bset, [(h, n) for h in handles])
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
    for t in [0, 1, 23, 24, 25, 47, 700, 1535]:
        b, lp = t // n, t % n
        keys = np.concatenate([kpn, kn[b * n:b * n + lp + 1]])
        vals = np.concatenate([vpn, vn[b * n:b * n + lp + 1]])
        ref = oracle.attention(qn[t:t + 1], keys, vals, P + lp, P + lp + 1, scale)[0]
        assert np.abs(out[t].cpu().numpy() - ref).max() <= ATOL, t
    for o in (plan, bset, prefix):
        o.close()
    rt.close()


def test_prefix_cache_across_requests(pkg):
    """q3_prefix_cache: a sealed prefix outlives its request; the second request
    with the same key skips the prefill and gets identical rows; under pressure
    the least recently used unreferenced prefix is evicted and its pages are
    reused without any allocation."""
    case = harness.rounded_case(_cases.make_case("ragged"))
    P, S = case.P, case.S
    pages = (P + 15) // 16
    # the prefix must own its pages (taken from the pool's free list) to give them back
    _, rt, prefix, bset, plan = harness.run_case_native(pkg, case, return_runtime=True,
                                                        permute_pages=False)
    g = torch.Generator().manual_seed(9)
    q = torch.randn(S, case.H, case.D, generator=g).to(torch.bfloat16).cuda()
    k = torch.randn(S, case.Hkv, case.D, generator=g).to(torch.bfloat16).cuda()
    v = torch.randn(S, case.Hkv, case.D, generator=g).to(torch.bfloat16).cuda()
    first = torch.zeros(S, case.H, case.D, dtype=torch.bfloat16, device="cuda")
    plan.attention_layer(1, q, k, v, first)
    rt.synchronize()
    cache = pkg.PrefixCache(rt, max_entries=2)
    with pytest.raises(pkg.Q3Error, match="null argument"):
        pkg._call(pkg.lib().q3_prefix_cache_insert, cache.h, 1, None)
    cache.insert(0xABCD, prefix)                      # request 1 hands its prefix over
    with pytest.raises(pkg.Q3Error, match="already cached"):
        cache.insert(0xABCD, prefix)
    cache.release(prefix)
    for o in (plan, bset):
        o.close()

    # request 2: same prompt -> hit, no prefill, same rows
    hit = cache.acquire(0xABCD, P)
    assert hit is prefix and cache.acquire(0xABCD, P + 1) is None and cache.acquire(7, P) is None
    bset2 = pkg.BranchSet(hit, len(case.branch_lens), max(case.branch_lens))
    handles = [bset2.acquire() for _ in case.branch_lens]
    plan2 = pkg.PackPlan(hit, bset2, list(zip(handles, case.branch_lens)))
    second = torch.zeros_like(first)
    plan2.attention_layer(1, q, k, v, second)
    rt.synchronize()
    assert torch.equal(first, second)
    for o in (plan2, bset2):
        o.close()
    st = cache.stats()
    assert (st.hits, st.misses, st.inserts, st.evictions, st.entries) == (1, 2, 1, 0, 1)
    assert st.pages_held == pages

    # a referenced prefix is never evicted; once released it goes when room is needed
    free0 = rt.stats().pages_free
    assert cache.make_room(free0 + 1) == 0 and cache.stats().entries == 1
    cache.release(hit)
    other = pkg.Prefix(rt, 40)
    other.set_resident(40)
    other.seal()
    cache.insert(2, other)
    cache.release(other)
    assert cache.acquire(2, 40) is other               # `other` is now the most recent
    cache.release(other)
    assert cache.make_room(rt.stats().pages_free + 1) == 1          # evicts 0xABCD (LRU)
    assert prefix.h is None and cache.acquire(0xABCD, P) is None
    assert rt.stats().pages_free == free0 - 3 + pages
    allocs = rt.stats().cuda_allocations
    reuse = pkg.Prefix(rt, P)                          # takes the freed pages from the list
    assert rt.stats().cuda_allocations == allocs
    assert set(reuse.page_table().tolist()) & set(range(rt.stats().pages_total))
    reuse.close()
    st = cache.stats()
    assert (st.evictions, st.entries, st.pages_held) == (1, 1, 3)
    cache.close()
    rt.close()
