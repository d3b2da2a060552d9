"""GPU parity tests for the paged decode kernel and for the reference-identical
fp32 surface (part 1 of the C ABI), the latter also against the reference's own
kernels compiled for sm_100a when oracle/_ref/libq3ref.so is present."""
import ctypes

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


def _decode_setup(pkg, ctx, Hkv, seed, out_fp32=True, spare_page=False):
    """Sequences with the given context lengths in randomly permuted pages."""
    S, H, D = len(ctx), Hkv * 8, 128
    g = torch.Generator().manual_seed(seed)
    n_pages = [(c + 15) // 16 + (1 if spare_page else 0) for c in ctx]
    total = int(sum(n_pages))
    rt = pkg.Runtime(num_layers=2, n_heads=H, n_kv_heads=Hkv,
                     max_positions=int(max(ctx)) + 8, max_tokens=S, num_pages=total + 3,
                     out_fp32=out_fp32)
    perm = np.random.default_rng(seed).permutation(total + 3)[:total].astype(np.uint32)
    indptr = np.concatenate([[0], np.cumsum(n_pages)]).astype(np.uint32)
    kp, vp = rt.pool()
    keys, vals = [], []
    for s, c in enumerate(ctx):
        k = torch.randn(c, Hkv, D, generator=g).to(torch.float16)
        v = torch.randn(c, Hkv, D, generator=g).to(torch.float16)
        keys.append(k.float().numpy())
        vals.append(v.float().numpy())
        pages = torch.from_numpy(perm[indptr[s]:indptr[s + 1]].astype(np.int64))
        pad = len(pages) * 16 - c
        kk = torch.cat([k, torch.zeros(pad, Hkv, D, dtype=torch.float16)])
        vv = torch.cat([v, torch.zeros(pad, Hkv, D, dtype=torch.float16)])
        kp[1][:, pages.cuda()] = kk.cuda().reshape(-1, 16, Hkv, D).permute(2, 0, 1, 3)
        vp[1][:, pages.cuda()] = vv.cuda().reshape(-1, 16, Hkv, D).permute(2, 0, 1, 3)
    q = torch.randn(S, H, D, generator=g).to(torch.bfloat16)
    torch.cuda.synchronize()
    plan = pkg.DecodePlan(rt, np.asarray(ctx, np.uint32), indptr, perm)
    return rt, plan, q, keys, vals


def _decode_oracle(q, keys, vals, ctx, pos):
    D = q.shape[-1]
    ifreq = oracle.inv_freq(1e6, D)
    ones = np.ones(D, np.float32)
    qn = oracle.rms_norm(q.float().numpy(), ones, 1e-6)
    dummy = np.zeros((q.shape[0], keys[0].shape[1], D), np.float32)
    qn, _ = oracle.rope(qn, dummy, 0, np.asarray(pos, np.uint32), ifreq)
    scale = np.float32(1 / np.sqrt(D))
    return np.stack([oracle.decode(qn[s], keys[s][:c], vals[s][:c], scale)
                     for s, c in enumerate(ctx)])


def test_decode_ragged_contexts(pkg):
    # single-chunk, exactly one chunk, multi-chunk, page-unaligned, length 1
    ctx = [1, 15, 16, 17, 333, 1024, 1025, 2500, 4097]
    rt, plan, q, keys, vals = _decode_setup(pkg, ctx, Hkv=2, seed=3)
    out = torch.zeros(len(ctx), 16, 128, dtype=torch.float32, device="cuda")
    plan.attention_layer(1, q.cuda(), None, None, out)
    rt.synchronize()
    assert rt.stats().device_status == 0
    ref = _decode_oracle(q, keys, vals, ctx, ctx)
    assert np.abs(out.cpu().numpy() - ref).max() <= ATOL
    plan.close()
    rt.close()


def test_decode_appends_new_token(pkg):
    ctx = [5, 16, 31, 1500]
    Hkv = 1
    rt, plan, q, keys, vals = _decode_setup(pkg, ctx, Hkv=Hkv, seed=9, spare_page=True)
    g = torch.Generator().manual_seed(77)
    kn = torch.randn(len(ctx), Hkv, 128, generator=g).to(torch.bfloat16)
    vn = torch.randn(len(ctx), Hkv, 128, generator=g).to(torch.bfloat16)
    out = torch.zeros(len(ctx), 8, 128, dtype=torch.float32, device="cuda")
    plan.attention_layer(1, q.cuda(), kn.cuda(), vn.cuda(), out)
    rt.synchronize()
    ifreq = oracle.inv_freq(1e6, 128)
    ones = np.ones(128, np.float32)
    k1 = oracle.rms_norm(kn.float().numpy(), ones, 1e-6)
    _, k2 = oracle.rope(np.zeros((len(ctx), 8, 128), np.float32), k1, 0,
                        np.asarray(ctx, np.uint32), ifreq)
    keys2 = [np.concatenate([keys[s], k2[s:s + 1]]) for s in range(len(ctx))]
    vals2 = [np.concatenate([vals[s], vn.float().numpy()[s:s + 1]]) for s in range(len(ctx))]
    ref = _decode_oracle(q, keys2, vals2, [c + 1 for c in ctx], ctx)
    assert np.abs(out.cpu().numpy() - ref).max() <= ATOL
    plan.close()
    rt.close()


def test_decode_bf16_output_and_no_room_error(pkg):
    ctx = [16, 700]
    rt, plan, q, keys, vals = _decode_setup(pkg, ctx, Hkv=1, seed=5, out_fp32=False)
    out = torch.zeros(2, 8, 128, dtype=torch.bfloat16, device="cuda")
    plan.attention_layer(1, q.cuda(), None, None, out)
    rt.synchronize()
    ref = _decode_oracle(q, keys, vals, ctx, ctx)
    assert harness.max_err_vs_bf16_oracle(out.float().cpu().numpy(), ref) <= ATOL
    kn = torch.zeros(2, 1, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(pkg.Q3Error, match="no page for the new token"):
        plan.attention_layer(1, q.cuda(), kn, kn, out)   # ctx 16 fills its only page
    plan.close()
    rt.close()


# --------------------------------------------------------------------------
# part 1: the reference's fp32 primitive surface
# --------------------------------------------------------------------------

@pytest.mark.parametrize("name", ["ragged", "prefill_only", "config1"])
def test_fp32_surface_matches_oracle_and_reference(pkg, name):
    case = _cases.make_case(name)
    ifreq = oracle.inv_freq(case.theta, case.D)
    ref = oracle.run_case(case)
    mine = harness.run_case_fp32_surface(harness.fp32_surface(pkg.lib_path()), case, ifreq)
    # the reference's own tolerance for its primitives is 1e-4
    assert np.abs(mine["q2"] - ref["q2"]).max() < 1e-4
    assert np.abs(mine["k2"] - ref["k2"]).max() < 1e-4
    assert np.abs(mine["out"] - ref["out"]).max() < 1e-4
    L = harness.ref_lib()
    if L is None:
        pytest.skip("oracle/_ref/libq3ref.so not built (reference checkout absent)")
    theirs = harness.run_case_fp32_surface(L, case, ifreq)
    # The reference's kernels against the oracle: this pins the oracle. The
    # reference is built with --use_fast_math (its Makefile), so its rope uses
    # the __sinf/__cosf intrinsics, whose absolute error grows with the angle
    # (its own test stops at position 14; these cases reach position 263):
    # 5e-4 instead of its 1e-4.
    assert np.abs(theirs["q2"] - ref["q2"]).max() < 5e-4
    assert np.abs(theirs["k2"] - ref["k2"]).max() < 5e-4
    assert np.abs(theirs["out"] - ref["out"]).max() < 5e-4
    assert np.abs(theirs["out"] - mine["out"]).max() < 5e-4


@pytest.mark.parametrize("name", ["ragged", "prefill_only", "config1"])
def test_fp32_surface_through_the_tensor_core_kernel(pkg, name):
    """The same fp32 symbols after q3_cuda_attention_native_init: slabs and
    queries are converted to f16 and attention_tc_kernel runs (tolerance 2e-3:
    f16 operands); without host-readable descriptors, or after shutdown, the
    exact fp32 kernels answer."""
    case = _cases.make_case(name)
    ifreq = oracle.inv_freq(case.theta, case.D)
    ref = oracle.run_case(case)
    L = pkg.lib()
    surf = harness.fp32_surface(pkg.lib_path())
    pkg._call(L.q3_cuda_attention_native_init, 0, case.T, case.T + 64, case.H, case.Hkv)
    try:
        with pytest.raises(pkg.Q3Error, match="already initialised"):
            pkg._call(L.q3_cuda_attention_native_init, 0, 8, 8, case.H, case.Hkv)
        mine = harness.run_case_fp32_surface(surf, case, ifreq, host_descriptors=True)
        assert L.q3_cuda_attention_last_path() == b"tensor-core"
        pkg._call(L.q3_cuda_attention_native_synchronize, 0)
        err = np.abs(mine["out"] - ref["out"]).max()
        print("%s through the tensor-core kernel: max abs err %.3e" % (name, err))
        assert err <= ATOL
        if case.S:
            # device-only descriptors: the host cannot build a schedule from them
            harness.run_case_fp32_surface(surf, case, ifreq, host_descriptors=False)
            assert L.q3_cuda_attention_last_path() == b"simt"
    finally:
        L.q3_cuda_attention_native_shutdown(0)
    exact = harness.run_case_fp32_surface(surf, case, ifreq, host_descriptors=False)
    assert L.q3_cuda_attention_last_path() == b"simt"
    assert np.abs(exact["out"] - ref["out"]).max() < 1e-4
    if case.S:
        # pageable host descriptors without the tensor-core path: refused, not dereferenced
        with pytest.raises(RuntimeError, match="pageable host memory"):
            harness.run_case_fp32_surface(surf, case, ifreq, host_descriptors=True)


def test_fp32_kv_cache_split_equals_contiguous(pkg):
    """tests/test_q3_forward.cu:388-483 on the fp32 surface: T=8 one-shot vs
    prefix 4 + suffix 4 through q3_kv_cache, last token's rows."""
    L = pkg.lib()
    H, Hkv, D, T = 16, 2, 128, 8
    g = torch.Generator().manual_seed(12)
    q = torch.randn(T, H, D, generator=g).cuda()
    k = torch.randn(T, Hkv, D, generator=g).cuda()
    v = torch.randn(T, Hkv, D, generator=g).cuda()
    scale = float(1 / np.sqrt(D))
    err = ctypes.create_string_buffer(256)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    one = torch.zeros(T, H, D, device="cuda")
    assert L.q3_cuda_attention(p(q), p(k), p(v), T, H, Hkv, D, 0, None, 0, scale, p(one),
                               None, err, 256), err.value
    kv = L.q3_kv_cache_init(2, Hkv, D, 16, err, 256)
    assert kv, err.value
    # the slabs, viewed as [layer][capacity][kv_heads][D] fp32
    ks = torch.as_tensor(pkg._DevView(L.q3_kv_cache_k(kv), (2, 16, Hkv, D), "<f4"),
                         device="cuda")
    vs = torch.as_tensor(pkg._DevView(L.q3_kv_cache_v(kv), (2, 16, Hkv, D), "<f4"),
                         device="cuda")
    layer = 1
    two = torch.zeros(T, H, D, device="cuda")
    for t0, n in ((0, 4), (4, 4)):
        ln = L.q3_kv_cache_length(kv)
        assert ln == t0
        ks[layer, ln:ln + n] = k[t0:t0 + n]      # the append of run_layer
        vs[layer, ln:ln + n] = v[t0:t0 + n]
        torch.cuda.synchronize()
        assert L.q3_cuda_attention(p(q[t0:t0 + n]), p(k[t0:t0 + n]), p(v[t0:t0 + n]), n, H,
                                   Hkv, D, t0, kv, layer, scale, p(two[t0:t0 + n]), None,
                                   err, 256), err.value
        L.q3_kv_cache_advance(kv, n)
    torch.cuda.synchronize()
    assert float((one - two).abs().max()) < 1e-5
    assert L.q3_kv_cache_length(kv) == 8
    L.q3_kv_cache_reset(kv)
    assert L.q3_kv_cache_length(kv) == 0
    L.q3_kv_cache_destroy(kv)
    # invalid arguments are refused with the reference's message shape
    assert not L.q3_cuda_attention(None, p(k), p(v), T, H, Hkv, D, 0, None, 0, scale,
                                   p(one), None, err, 256)
    assert b"q3_cuda_attention: invalid argument" in err.value
