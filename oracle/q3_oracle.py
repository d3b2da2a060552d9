"""ctypes wrapper around oracle/libq3oracle.so (the CPU restatement of the
reference's attention path) plus a helper that runs a whole Case through it in
the reference's own data layout: contiguous fp32 prefix slabs
[layer][capacity][kv_heads][D] and a suffix arena
[branch][layer][suffix_capacity][row] (src/q3_forward.h:213-229).

TEST INFRASTRUCTURE ONLY: imported by tests, the smoke check and the timed CPU
baseline; the shipped package never imports it.
"""
import ctypes
import os
import subprocess

import numpy as np

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_LIB = None

c_f = ctypes.POINTER(ctypes.c_float)
c_u = ctypes.POINTER(ctypes.c_uint32)
u32 = ctypes.c_uint32


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_ROOT, "oracle", "libq3oracle.so")
        src = os.path.join(_ROOT, "oracle", "q3_attn_oracle.c")
        if (not os.path.exists(path)
                or os.path.getmtime(path) < os.path.getmtime(src)):
            subprocess.check_call(["make", "-C", os.path.join(_ROOT, "oracle"),
                                   "libq3oracle.so"], stdout=subprocess.DEVNULL)
        _LIB = ctypes.CDLL(path)
        _LIB.q3o_threads.restype = ctypes.c_int
    return _LIB


def _f(a):
    assert a.dtype == np.float32 and a.flags.c_contiguous
    return a.ctypes.data_as(c_f)


def _u(a):
    if a is None:
        return None
    assert a.dtype == np.uint32 and a.flags.c_contiguous
    return a.ctypes.data_as(c_u)


def threads():
    return int(lib().q3o_threads())


def set_threads(n):
    lib().q3o_set_threads(ctypes.c_int(n))


def inv_freq(theta, head_dim):
    out = np.empty(head_dim // 2, np.float32)
    lib().q3o_inv_freq(ctypes.c_double(theta), u32(head_dim), _f(out))
    return out


def rms_norm(x, w, eps):
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty_like(x)
    width = x.shape[-1]
    lib().q3o_rms_norm(_f(x), _f(np.ascontiguousarray(w, np.float32)),
                       u32(x.size // width), u32(width), ctypes.c_float(eps), _f(out))
    return out


def rope(q, k, position_base, positions, ifreq):
    """Returns roped copies of q [T,H,D] and k [T,Hkv,D]."""
    q = np.array(q, np.float32, order="C")
    k = np.array(k, np.float32, order="C")
    T, H, D = q.shape
    pos = None if positions is None else np.ascontiguousarray(positions, np.uint32)
    lib().q3o_rope(_f(q), _f(k), u32(T), u32(H), u32(k.shape[1]), u32(D),
                   u32(position_base), _u(pos), _f(ifreq))
    return q, k


def attention(q, k_rows, v_rows, position_base, kv_length, scale):
    q = np.ascontiguousarray(q, np.float32)
    T, H, D = q.shape
    Hkv = k_rows.shape[1]
    out = np.zeros_like(q)
    lib().q3o_attention(_f(q), _f(k_rows), _f(v_rows), u32(T), u32(H), u32(Hkv),
                        u32(D), u32(position_base), u32(kv_length),
                        ctypes.c_float(scale), _f(out))
    return out


def attention_segmented(q, prefix_k, prefix_v, prefix_len, prefix_capacity,
                        suffix_k, suffix_v, suffix_capacity, suffix_num_layers,
                        suffix_layer, token_branch, token_local_pos, n_kv_heads,
                        scale):
    q = np.ascontiguousarray(q, np.float32)
    T, H, D = q.shape
    out = np.zeros_like(q)
    lib().q3o_attention_segmented(
        _f(q), _f(prefix_k), _f(prefix_v), u32(prefix_len), u32(prefix_capacity),
        _f(suffix_k), _f(suffix_v), u32(suffix_capacity), u32(suffix_num_layers),
        u32(suffix_layer), _u(token_branch), _u(token_local_pos), u32(T), u32(H),
        u32(n_kv_heads), u32(D), ctypes.c_float(scale), _f(out))
    return out


def kv_scatter(suffix_k, suffix_v, k_src, v_src, token_branch, token_local_pos,
               suffix_capacity, num_layers, layer):
    T = k_src.shape[0]
    row = k_src.shape[1] * k_src.shape[2]
    lib().q3o_kv_scatter(_f(suffix_k), _f(suffix_v), _f(k_src), _f(v_src),
                         _u(token_branch), _u(token_local_pos), u32(T), u32(row),
                         u32(suffix_capacity), u32(num_layers), u32(layer))


def decode(q, k_rows, v_rows, scale):
    """q [H,D]; k_rows, v_rows [ctx,Hkv,D]."""
    q = np.ascontiguousarray(q, np.float32)
    H, D = q.shape
    out = np.zeros_like(q)
    lib().q3o_attention_decode(_f(q), _f(k_rows), _f(v_rows), u32(k_rows.shape[0]),
                               u32(H), u32(k_rows.shape[1]), u32(D),
                               ctypes.c_float(scale), _f(out))
    return out


def run_case(case):
    """The reference's sequencing (src/q3_forward.cu:1244-1286 for the prefix,
    :1489-1526 for the packed suffix) over one Case. Returns dict with the
    normalised+roped q2/k2 [T,...] and the attention output [T,H,D]."""
    P, S, T = case.P, case.S, case.T
    ifreq = inv_freq(case.theta, case.D)
    q1 = rms_norm(case.q, case.q_norm_w, case.eps)
    k1 = rms_norm(case.k, case.k_norm_w, case.eps)
    out = np.zeros((T, case.H, case.D), np.float32)
    q2 = np.zeros_like(q1)
    k2 = np.zeros_like(k1)
    if P:
        qp, kp = rope(q1[:P], k1[:P], 0, None, ifreq)
        q2[:P], k2[:P] = qp, kp
        # KV append then attention over the cache slab (layer 0, capacity P).
        out[:P] = attention(qp, kp, np.ascontiguousarray(case.v[:P]), 0, P, case.scale)
    if S:
        qs, ks = rope(q1[P:], k1[P:], 0, case.positions[P:], ifreq)
        q2[P:], k2[P:] = qs, ks
        vs = np.ascontiguousarray(case.v[P:])
        nb = max(case.branch_handles) + 1
        cap = max(case.branch_lens)
        L, layer = 2, 1          # exercise the layer stride of both segments
        row = case.Hkv * case.D
        pcap = max(P, 1) + 3
        pk = np.zeros((L, pcap, case.Hkv, case.D), np.float32)
        pv = np.zeros_like(pk)
        pk[layer, :P], pv[layer, :P] = k2[:P], case.v[:P]
        sk = np.zeros((nb, L, cap, row), np.float32)
        sv = np.zeros_like(sk)
        kv_scatter(sk, sv, ks, vs, case.token_branch, case.token_local_pos, cap, L, layer)
        out[P:] = attention_segmented(qs, pk, pv, P, pcap, sk, sv, cap, L, layer,
                                      case.token_branch, case.token_local_pos,
                                      case.Hkv, case.scale)
    return dict(q2=q2, k2=k2, out=out)
