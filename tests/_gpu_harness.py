"""GPU-side helpers of the parity tests: run a Case through the native paged
path of the C ABI, and through the reference's own kernels (oracle/_ref) when
that library is present."""
import ctypes
import os

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PAGE = 16


def bf16_round(a):
    """fp32 numpy -> nearest bf16 -> fp32 numpy."""
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(torch.bfloat16) \
        .to(torch.float32).numpy()


def rounded_case(case):
    """The same case with q/k/v rounded to bf16: what the native path is fed and
    therefore what the oracle must be fed for a like-for-like comparison."""
    import copy
    c = copy.copy(case)
    c.q, c.k, c.v = bf16_round(case.q), bf16_round(case.k), bf16_round(case.v)
    return c


def max_err(got, ref):
    """max |got - ref| normalised by max |ref| (ref: fp32 oracle)."""
    return float(np.abs(got.astype(np.float64) - ref).max() / np.abs(ref).max())


def max_err_vs_bf16_oracle(got, ref):
    """Error of a bf16 output: distance to the oracle in units of max|ref|, after
    discounting half a bf16 ulp of the reference value (the output rounding
    every bf16 result carries)."""
    ref = ref.astype(np.float64)
    half_ulp = np.abs(ref) * 2.0 ** -8
    e = np.maximum(np.abs(got.astype(np.float64) - ref) - half_ulp, 0.0)
    return float(e.max() / np.abs(ref).max())


def dev(a, dtype, device="cuda"):
    return torch.from_numpy(np.ascontiguousarray(a)).to(device).to(dtype).contiguous()


def run_case_native(pkg, case, out_fp32=False, prefill_chunks=None, permute_pages=True,
                    layer=1, seed=0, return_runtime=False, device=0, sched_policy=None):
    """Prefix prefill (optionally in chunks) + packed suffix pass through the C
    ABI. Inputs are given as bf16. Returns the attention output [T,H,D] fp32."""
    P, S, T = case.P, case.S, case.T
    rng = np.random.default_rng(seed)
    n_branch = (max(case.branch_handles) + 1) if S else 0
    max_suffix = max(case.branch_lens) if S else 0
    ppb = (max_suffix + PAGE - 1) // PAGE
    n_prefix_pages = (max(P, 1) + PAGE - 1) // PAGE
    num_pages = n_prefix_pages + n_branch * ppb + 7
    rt = pkg.Runtime(num_layers=2, n_heads=case.H, n_kv_heads=case.Hkv,
                     max_positions=P + max_suffix + 8, max_tokens=max(P, S, 1),
                     num_pages=num_pages, out_fp32=out_fp32, rms_eps=case.eps,
                     rope_theta=case.theta, device=device)
    cuda = torch.device("cuda", device)
    if sched_policy is not None:
        rt.set_schedule_policy(sched_policy)
    rt.set_qk_norm(layer, case.q_norm_w, case.k_norm_w)
    odt = torch.float32 if out_fp32 else torch.bfloat16
    out = torch.zeros(T, case.H, case.D, dtype=odt, device=cuda)
    q, k, v = (dev(a, torch.bfloat16, cuda) for a in (case.q, case.k, case.v))
    if permute_pages:
        perm = rng.permutation(num_pages).astype(np.uint32)
        taken = rt.alloc_pages(num_pages)   # empty the free list; we hand out ids
        assert sorted(taken.tolist()) == list(range(num_pages))
        rt.free_pages(perm[n_prefix_pages:])
        prefix = pkg.Prefix(rt, max(P, 1), pages=perm[:n_prefix_pages])
    else:
        prefix = pkg.Prefix(rt, max(P, 1))
    torch.cuda.synchronize()
    if P:
        chunks = prefill_chunks or [P]
        assert sum(chunks) == P
        t0 = 0
        for n in chunks:
            prefix.prefill_layer(layer, q[t0:t0 + n], k[t0:t0 + n], v[t0:t0 + n],
                                 out[t0:t0 + n])
            prefix.advance(n)
            t0 += n
    plan = bset = None
    if S:
        prefix.seal()
        bset = pkg.BranchSet(prefix, n_branch, max_suffix)
        handles = [bset.acquire() for _ in range(n_branch)]
        assert handles == list(range(n_branch))
        plan = pkg.PackPlan(prefix, bset,
                            list(zip(case.branch_handles, case.branch_lens)))
        assert plan.tokens == S
        plan.attention_layer(layer, q[P:], k[P:], v[P:], out[P:])
    rt.synchronize()
    res = out.to(torch.float32).cpu().numpy()
    if return_runtime:
        return res, rt, prefix, bset, plan
    for o in (plan, bset, prefix):
        if o is not None:
            o.close()
    rt.close()
    return res


# ---------------------------------------------------------------------------
# the reference's own kernels, compiled for sm_100a (oracle/_ref/libq3ref.so)
# ---------------------------------------------------------------------------

def ref_lib():
    return fp32_surface(os.path.join(ROOT, "oracle", "_ref", "libq3ref.so"))


def fp32_surface(path):
    """ctypes view of the fp32 primitive symbols, which the reference's library
    and this repository's library both export under the same names."""
    if not os.path.exists(path):
        return None
    L = ctypes.CDLL(path)
    vp, u32, cf, sz = ctypes.c_void_p, ctypes.c_uint32, ctypes.c_float, ctypes.c_size_t
    err = [ctypes.c_char_p, sz]
    L.q3_cuda_rms_norm.argtypes = [vp, vp, u32, u32, cf, vp, vp] + err
    L.q3_cuda_rope.argtypes = [vp, vp, u32, u32, u32, u32, u32, vp, vp] + err
    L.q3_cuda_rope_positions.argtypes = [vp, vp, u32, u32, u32, u32, vp, vp, vp] + err
    L.q3_cuda_attention.argtypes = [vp, vp, vp, u32, u32, u32, u32, u32, vp, u32, cf, vp,
                                    vp] + err
    L.q3_cuda_attention_segmented.argtypes = [vp, vp, vp, u32, u32, vp, vp, u32, u32, u32,
                                              vp, vp, u32, u32, u32, u32, cf, vp, vp] + err
    for f in (L.q3_cuda_rms_norm, L.q3_cuda_rope, L.q3_cuda_rope_positions,
              L.q3_cuda_attention, L.q3_cuda_attention_segmented):
        f.restype = ctypes.c_bool
    return L


def run_case_fp32_surface(L, case, inv_freq, host_descriptors=False):
    """Drive the fp32 primitive surface (the reference's, or this library's
    part 1 - same symbols) in the reference's sequencing and slab layout
    (src/q3_forward.cu:1244-1286 and :1489-1526). L is a ctypes library."""
    P, S, T, H, Hkv, D = case.P, case.S, case.T, case.H, case.Hkv, case.D
    err = ctypes.create_string_buffer(256)

    def ck(ok, what):
        if not ok:
            raise RuntimeError("%s: %s" % (what, err.value.decode()))

    def p(t):
        return ctypes.c_void_p(t.data_ptr()) if t is not None else None

    f32 = torch.float32
    q = dev(case.q, f32)
    k = dev(case.k, f32)
    v = dev(case.v, f32)
    qw, kw = dev(case.q_norm_w, f32), dev(case.k_norm_w, f32)
    ifr = dev(inv_freq, f32)
    out = torch.zeros(T, H, D, dtype=f32, device="cuda")
    torch.cuda.synchronize()
    ck(L.q3_cuda_rms_norm(p(q), p(qw), T * H, D, case.eps, p(q), None, err, 256), "rms q")
    ck(L.q3_cuda_rms_norm(p(k), p(kw), T * Hkv, D, case.eps, p(k), None, err, 256), "rms k")
    row = Hkv * D
    if P:
        ck(L.q3_cuda_rope(p(q[:P]), p(k[:P]), P, H, Hkv, D, 0, p(ifr), None, err, 256),
           "rope")
        ck(L.q3_cuda_attention(p(q[:P]), p(k[:P]), p(v[:P]), P, H, Hkv, D, 0, None, 0,
                               float(case.scale), p(out[:P]), None, err, 256), "attention")
    if S:
        pos = dev(case.positions[P:], torch.int32)
        tb = dev(case.token_branch.astype(np.int32), torch.int32)
        tl = dev(case.token_local_pos.astype(np.int32), torch.int32)
        qs, ks, vs = q[P:], k[P:], v[P:]
        ck(L.q3_cuda_rope_positions(p(qs), p(ks), S, H, Hkv, D, p(pos), p(ifr), None, err,
                                    256), "rope positions")
        nb, cap, Lyr, layer, pcap = max(case.branch_handles) + 1, max(case.branch_lens), 2, 1, P + 3
        pk = torch.zeros(Lyr, pcap, Hkv, D, dtype=f32, device="cuda")
        pv = torch.zeros_like(pk)
        pk[layer, :P], pv[layer, :P] = k[:P], v[:P]
        sk = torch.zeros(nb, Lyr, cap, row, dtype=f32, device="cuda")
        sv = torch.zeros_like(sk)
        # the reference's scatter kernel is file-static: place rows with its formula
        tbl, tll = tb.long(), tl.long()
        sk[tbl, layer, tll] = ks.reshape(S, row)
        sv[tbl, layer, tll] = vs.reshape(S, row)
        torch.cuda.synchronize()
        if host_descriptors:
            # where the reference's own caller keeps them (src/q3_decide.cu:420-464)
            hb = np.ascontiguousarray(case.token_branch, np.uint32)
            hl = np.ascontiguousarray(case.token_local_pos, np.uint32)
            ptb, ptl = ctypes.c_void_p(hb.ctypes.data), ctypes.c_void_p(hl.ctypes.data)
        else:
            ptb, ptl = p(tb), p(tl)
        ck(L.q3_cuda_attention_segmented(p(qs), p(pk), p(pv), P, pcap, p(sk), p(sv), cap,
                                         Lyr, layer, ptb, ptl, S, H, Hkv, D,
                                         float(case.scale), p(out[P:]), None, err, 256),
           "segmented")
    torch.cuda.synchronize()
    return dict(q2=q.cpu().numpy(), k2=k.cpu().numpy(), out=out.cpu().numpy())
