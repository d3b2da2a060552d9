"""The layer with its q/k/v projection fused in (q3_prefix_prefill_layer_projected,
q3_suffix_attention_layer_projected): Q4_K projection whose epilogue normalises,
rotates and writes the pages, then attention - against the CPU oracles chained
the way the reference chains its steps (quantised linear, src/q3_q4_linear.cu:149;
rms_norm, rope, KV append / scatter, attention, src/q3_forward.cu:1244-1286 and
:1489-1526).

Tolerance: the projection runs with f16 operands and fp32 accumulation (the
quantisation oracle with the same operand rounding agrees to 1e-4 relative); its
fp32 result feeds the norm directly. Attention output against the oracle:
max |got - ref| <= 2e-3 x max(1, max |ref|), the bar of the other attention tests.
"""
import numpy as np
import pytest
import torch

import __graft_entry__ as entry
import _cases
import _gpu_harness as harness
import q3_oracle as oracle
import q3_quant_oracle as qo

pytestmark = pytest.mark.gpu
ATOL = 2e-3
HIDDEN = 512


@pytest.fixture(scope="module")
def pkg():
    entry.build()
    pkg = entry.load_package()
    from sera_c_b200 import q4_linear
    pkg._lin = q4_linear.Q4Linear(0, 2048, 4096, 1024)     # q3_cuda_q4k_linear_init
    pkg._q4 = q4_linear
    return pkg


def _projected_case(name, P, branch_lens, H, Hkv, seed):
    """A Case whose q, k, v are the oracle's projection of seeded activations
    through seeded Q4_K weights."""
    case = _cases.Case(name, P, branch_lens, n_heads=H, n_kv_heads=Hkv, seed=seed,
                       unit_norm_weights=False)
    rng = np.random.default_rng(seed)
    w = [qo.q4k_weight(rng, n * 128, HIDDEN) for n in (H, Hkv, Hkv)]
    x = (rng.standard_normal((case.T, HIDDEN)) * 0.02).astype(np.float32)
    x16 = x.astype(np.float16).astype(np.float32)
    q, k, v = (qo.q4k_linear(wi, x16, operands="f16").astype(np.float32) for wi in w)
    case.q = np.ascontiguousarray(q.reshape(case.T, H, 128))
    case.k = np.ascontiguousarray(k.reshape(case.T, Hkv, 128))
    case.v = np.ascontiguousarray(v.reshape(case.T, Hkv, 128))
    return case, w, x16


def _run_projected(pkg, case, w, x16, chunks=None, permute=False, tiled=False, layer=1):
    P, S, T = case.P, case.S, case.T
    n_branch = (max(case.branch_handles) + 1) if S else 0
    max_suffix = max(case.branch_lens) if S else 0
    ppb = (max_suffix + 15) // 16
    n_prefix_pages = (max(P, 1) + 15) // 16
    num_pages = n_prefix_pages + n_branch * ppb + 7
    rt = pkg.Runtime(num_layers=2, n_heads=case.H, n_kv_heads=case.Hkv,
                     max_positions=P + max_suffix + 8, max_tokens=max(P, S, 1),
                     num_pages=num_pages, out_fp32=True, rms_eps=case.eps,
                     rope_theta=case.theta, device=0)
    rt.set_qk_norm(layer, case.q_norm_w, case.k_norm_w)
    wd = [torch.from_numpy(wi).cuda() for wi in w]
    qtype = 12
    if tiled:
        packed = []
        for wi, n in zip(wd, (case.H, case.Hkv, case.Hkv)):
            geo = pkg._q4.bind_geometry(HIDDEN, n * 128)
            t, tgeo = pkg._lin.pack(geo, wi)
            packed.append(t)
            qtype = tgeo.qtype
        wd = packed
    W = pkg.qkv_weights(wd[0], wd[1], wd[2], HIDDEN, qtype)
    xd = torch.from_numpy(x16).cuda().to(torch.float16)
    out = torch.zeros(T, case.H, 128, dtype=torch.float32, device="cuda")
    if permute:
        rng = np.random.default_rng(5)
        perm = rng.permutation(num_pages).astype(np.uint32)
        rt.alloc_pages(num_pages)
        rt.free_pages(perm[n_prefix_pages:])
        prefix = pkg.Prefix(rt, max(P, 1), pages=perm[:n_prefix_pages])
    else:
        prefix = pkg.Prefix(rt, max(P, 1))
    t0 = 0
    for n in (chunks or ([P] if P else [])):
        prefix.prefill_layer_projected(layer, W, xd[t0:t0 + n], out[t0:t0 + n])
        prefix.advance(n)
        t0 += n
    plan = bset = None
    if S:
        prefix.seal()
        bset = pkg.BranchSet(prefix, n_branch, max_suffix)
        for _ in range(n_branch):
            bset.acquire()
        plan = pkg.PackPlan(prefix, bset, list(zip(case.branch_handles, case.branch_lens)))
        plan.attention_layer_projected(layer, W, xd[P:], out[P:])
    rt.synchronize()
    assert rt.stats().device_status == 0
    assert pkg._lin.status() == 0
    res = out.cpu().numpy()
    return res, (rt, prefix, bset, plan, W, xd)


def _close(objs):
    rt, prefix, bset, plan = objs[:4]
    for o in (plan, bset, prefix):
        if o is not None:
            o.close()
    rt.close()


@pytest.mark.parametrize("P,branches,H,Hkv,chunks,permute,tiled", [
    (300, [40, 9, 17], 16, 2, None, False, False),     # two token tiles of the projection
    (300, [40, 9, 17], 16, 2, [130, 170], True, False),  # chunked prefill, pages in any order
    (45, [], 8, 1, None, False, True),                  # prefill only, tiled weight order
    (19, [5, 3, 1, 18], 16, 2, None, True, True),        # ragged branches
    (600, [24] * 12, 8, 1, None, False, False),          # > 256 tokens in the suffix pass too
])
def test_projected_layers_match_the_chained_oracles(pkg, P, branches, H, Hkv, chunks, permute,
                                                    tiled):
    case, w, x16 = _projected_case("proj", P, branches, H, Hkv, seed=P + len(branches))
    ref = oracle.run_case(case)["out"]
    got, objs = _run_projected(pkg, case, w, x16, chunks, permute, tiled)
    bound = ATOL * max(1.0, float(np.abs(ref).max()))
    err = float(np.abs(got - ref).max())
    print("max abs err %.3e (bound %.3e, max |ref| %.2f)" % (err, bound, np.abs(ref).max()))
    assert err <= bound
    _close(objs)


def test_projected_equals_the_unfused_calls_up_to_the_bf16_copy(pkg):
    """Same weights and activations through q3_cuda_q4k_linear_f16 (bf16 q, k, v)
    + the plain layer entries: the two paths differ by the bf16 rounding of
    q, k, v that the fused path does not have."""
    case, w, x16 = _projected_case("proj2", 200, [30, 30], 16, 2, seed=11)
    got, objs = _run_projected(pkg, case, w, x16)
    xd = objs[5]
    qkv = []
    for wi, n in zip(w, (case.H, case.Hkv, case.Hkv)):
        geo = pkg._q4.bind_geometry(HIDDEN, n * 128)
        o = pkg._lin.linear_f16(geo, torch.from_numpy(wi).cuda(), xd, out_dtype=torch.bfloat16)
        qkv.append(o.float().cpu().numpy().reshape(case.T, n, 128))
    case.q, case.k, case.v = qkv
    unfused = harness.run_case_native(pkg, case, out_fp32=True)
    scale = max(1.0, float(np.abs(unfused).max()))
    assert float(np.abs(got - unfused).max()) <= 2e-2 * scale
    _close(objs)


def test_projected_refusals(pkg):
    case, w, x16 = _projected_case("proj3", 32, [], 8, 1, seed=3)
    rt = pkg.Runtime(num_layers=1, n_heads=8, n_kv_heads=1, max_positions=64, max_tokens=32,
                     num_pages=4, out_fp32=True, device=0)
    prefix = pkg.Prefix(rt, 32)
    wd = [torch.from_numpy(wi).cuda() for wi in w]
    xd = torch.from_numpy(x16).cuda().to(torch.float16)
    out = torch.zeros(32, 8, 128, dtype=torch.float32, device="cuda")
    W = pkg.qkv_weights(wd[0], wd[1], wd[2], HIDDEN)
    W.qtype_v = 14                                    # a Q6_K value weight
    with pytest.raises(pkg.Q3Error, match="one quantisation type"):
        prefix.prefill_layer_projected(0, W, xd, out)
    W = pkg.qkv_weights(wd[0], wd[1], wd[2], HIDDEN, qtype=14)
    with pytest.raises(pkg.Q3Error, match="must be Q4_K"):
        prefix.prefill_layer_projected(0, W, xd, out)
    W = pkg.qkv_weights(wd[0], wd[1], wd[2], 300)
    with pytest.raises(pkg.Q3Error, match="multiple of 256"):
        prefix.prefill_layer_projected(0, W, xd, out)
    prefix.close()
    rt.close()
