"""Host-side mirror of the q3attn C ABI (include/q3_attn.h) for Python callers.

The product is libq3attn.so; this module only loads it with ctypes and wraps
its handles so tests, the benchmark and a Python host can drive the path with
torch tensors as device memory. There is no CPU implementation here: if the
library is missing or no CUDA device is present, the calls fail loudly.

The directory name contains a dot, so import it through the repository's
`__graft_entry__.load_package()` (module name `sera_c_b200`).
"""
import ctypes
import os

import numpy as np

from . import _lib
from ._lib import ERRLEN, GatherPeers, Q3Error, bind, lib_path  # noqa: F401

PAGE = 16
D = 128
G = 8

_c_u32p = ctypes.POINTER(ctypes.c_uint32)


def _u32(a):
    a = np.ascontiguousarray(a, dtype=np.uint32)
    return a, a.ctypes.data_as(_c_u32p)


def qkv_weights(wq, wk, wv, hidden, qtype=12):
    """q3_qkv_weights for the *_projected layer entries: three resident
    quantised weights (torch uint8 tensors on the device), one type for all
    (12 = Q4_K in GGUF order, 12 | 1 << 16 = the tiled order)."""
    w = _lib.QkvWeights()
    w.wq, w.wk, w.wv = wq.data_ptr(), wk.data_ptr(), wv.data_ptr()
    w.qtype_q = w.qtype_k = w.qtype_v = qtype
    w.hidden = hidden
    w._keep = (wq, wk, wv)
    return w


def _ptr(t):
    """Device pointer of a torch tensor (or None)."""
    if t is None:
        return None
    assert t.is_cuda and t.is_contiguous(), "need a contiguous CUDA tensor"
    return ctypes.c_void_p(t.data_ptr())


class _DevView:
    """Exposes raw device memory owned by the library to torch."""

    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = {
            "shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False),
            "version": 2}


class AttnConfig(ctypes.Structure):
    _fields_ = [("num_layers", ctypes.c_uint32), ("n_heads", ctypes.c_uint32),
                ("n_kv_heads", ctypes.c_uint32), ("head_dim", ctypes.c_uint32),
                ("rms_eps", ctypes.c_float), ("rope_theta", ctypes.c_double),
                ("max_positions", ctypes.c_uint32), ("max_tokens", ctypes.c_uint32),
                ("num_pages", ctypes.c_uint32), ("out_fp32", ctypes.c_uint32),
                ("device", ctypes.c_int)]


class AttnStats(ctypes.Structure):
    _fields_ = [("cuda_allocations", ctypes.c_uint64), ("cuda_frees", ctypes.c_uint64),
                ("host_syncs", ctypes.c_uint64), ("kernel_launches", ctypes.c_uint64),
                ("pages_total", ctypes.c_uint64), ("pages_free", ctypes.c_uint64),
                ("pool_bytes", ctypes.c_uint64), ("workspace_bytes", ctypes.c_uint64),
                ("device_status", ctypes.c_uint32)]


class SuffixItem(ctypes.Structure):
    _fields_ = [("branch", ctypes.c_uint32), ("token_count", ctypes.c_uint32)]


class SchedSegmentInfo(ctypes.Structure):
    _fields_ = [("cta", ctypes.c_uint32), ("tok0", ctypes.c_uint32),
                ("kv_head", ctypes.c_uint32), ("tile_begin", ctypes.c_uint32),
                ("tile_end", ctypes.c_uint32), ("shared_tiles", ctypes.c_uint32),
                ("partial_slot", ctypes.c_int32)]


class SchedSummary(ctypes.Structure):
    _fields_ = [("grid", ctypes.c_uint32), ("n_segments", ctypes.c_uint32),
                ("n_cut_items", ctypes.c_uint32), ("n_slots", ctypes.c_uint32),
                ("total_key_tiles", ctypes.c_uint64)]


_LIB = None


def lib():
    global _LIB
    if _LIB is None:
        _LIB = bind(AttnConfig, AttnStats, SuffixItem, SchedSegmentInfo, SchedSummary)
    return _LIB


def _call(fn, *args):
    """Invoke an ABI function that ends with (char *error, size_t error_len)."""
    err = ctypes.create_string_buffer(ERRLEN)
    r = fn(*args, err, ERRLEN)
    failed = (r is None) or (r is False) or (isinstance(r, int) and not isinstance(r, bool) and r < 0)
    if failed:
        raise Q3Error(err.value.decode() or "%s failed" % fn.__name__)
    return r


class Runtime:
    """q3_attn_runtime: stream, geometry, KV page pool, RoPE table, workspace."""

    def __init__(self, num_layers, n_heads, n_kv_heads, max_positions, max_tokens,
                 num_pages, device=0, rms_eps=1e-6, rope_theta=1e6, head_dim=D,
                 out_fp32=False):
        self.cfg = AttnConfig(num_layers, n_heads, n_kv_heads, head_dim, rms_eps,
                              rope_theta, max_positions, max_tokens, num_pages,
                              1 if out_fp32 else 0, device)
        self.h = _call(lib().q3_attn_create, ctypes.byref(self.cfg))

    def close(self):
        if getattr(self, "h", None):
            lib().q3_attn_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_qk_norm(self, layer, q_w, k_w):
        q_w = np.ascontiguousarray(q_w, np.float32)
        k_w = np.ascontiguousarray(k_w, np.float32)
        _call(lib().q3_attn_set_qk_norm, self.h, layer,
              q_w.ctypes.data_as(ctypes.POINTER(ctypes.c_float)),
              k_w.ctypes.data_as(ctypes.POINTER(ctypes.c_float)))

    @property
    def stream_ptr(self):
        return lib().q3_attn_stream(self.h)

    def torch_stream(self):
        import torch
        return torch.cuda.ExternalStream(self.stream_ptr, device=self.cfg.device)

    def synchronize(self):
        _call(lib().q3_attn_synchronize, self.h)

    def reset_status(self):
        _call(lib().q3_attn_reset_status, self.h)

    def stats(self):
        s = AttnStats()
        lib().q3_attn_get_stats(self.h, ctypes.byref(s))
        return s

    PHASES = ("kvwrite", "attention", "gather_wait", "decode")

    def enable_timing(self, max_launches=4096):
        _call(lib().q3_attn_enable_timing, self.h, max_launches)

    def phase_times(self):
        """{phase: (summed ms, launches)} since the last call; synchronises."""
        ms = (ctypes.c_double * 4)()
        n = (ctypes.c_uint64 * 4)()
        _call(lib().q3_attn_phase_times, self.h, ms, n)
        return {name: (ms[i], int(n[i])) for i, name in enumerate(self.PHASES)}

    SCHED = {"auto": 0, "streamk": 1, "lockstep": 2}

    def set_schedule_policy(self, policy):
        _call(lib().q3_attn_set_schedule_policy, self.h, self.SCHED[policy])

    def gather_advance(self, count):
        _call(lib().q3_attn_gather_advance, self.h, count)

    def graph_begin(self):
        _call(lib().q3_attn_graph_begin, self.h)

    def graph_end(self):
        return Graph(_call(lib().q3_attn_graph_end, self.h))

    def wait_gathered(self, peers, seq):
        _call(lib().q3_attn_wait_gathered, self.h, ctypes.byref(peers), seq)

    def alloc_pages(self, n):
        out = np.empty(n, np.uint32)
        _call(lib().q3_pages_alloc, self.h, n, out.ctypes.data_as(_c_u32p))
        return out

    def free_pages(self, pages):
        a, p = _u32(pages)
        lib().q3_pages_free(self.h, p, len(a))

    def pool(self):
        """(K, V) page pools as torch f16 tensors [L, Hkv, num_pages, 16, 128]."""
        import torch
        c = self.cfg
        shape = (c.num_layers, c.n_kv_heads, c.num_pages, PAGE, D)
        k = torch.as_tensor(_DevView(lib().q3_pages_k(self.h), shape, "<f2"),
                            device="cuda:%d" % c.device)
        v = torch.as_tensor(_DevView(lib().q3_pages_v(self.h), shape, "<f2"),
                            device="cuda:%d" % c.device)
        return k, v

    def qknorm_rope_kvwrite(self, layer, q, k, v, rope_pos, dst_page, dst_slot, q_out):
        tokens = (q if q is not None else k).shape[0]
        _call(lib().q3_cuda_qknorm_rope_kvwrite, self.h, layer, _ptr(q), _ptr(k), _ptr(v),
              tokens, _ptr(rope_pos), _ptr(dst_page), _ptr(dst_slot), _ptr(q_out))


class Graph:
    """q3_attn_graph: a recorded sequence of layer calls, replayed as one launch."""

    def __init__(self, handle):
        self.h = handle

    def launch(self):
        _call(lib().q3_attn_graph_launch, self.h)

    def close(self):
        if getattr(self, "h", None):
            lib().q3_attn_graph_destroy(self.h)
            self.h = None


class Prefix:
    """q3_prefix_kv: the shared, sealed prefix (also: any single sequence)."""

    def __init__(self, rt, capacity_tokens, pages=None):
        self.rt = rt
        if pages is None:
            self.h = _call(lib().q3_prefix_create, rt.h, capacity_tokens)
        else:
            a, p = _u32(pages)
            assert len(a) >= (capacity_tokens + PAGE - 1) // PAGE
            self.h = _call(lib().q3_prefix_create_with_pages, rt.h, capacity_tokens, p)
        self.capacity = capacity_tokens

    def close(self):
        if getattr(self, "h", None):
            lib().q3_prefix_destroy(self.h)
            self.h = None

    def prefill_layer(self, layer, q, k, v, out):
        _call(lib().q3_prefix_prefill_layer, self.h, layer, _ptr(q), _ptr(k), _ptr(v),
              q.shape[0], _ptr(out))

    def prefill_layer_projected(self, layer, weights, x_f16, out):
        """q/k/v projection (three resident Q4_K weights) with norm + RoPE + page
        write as its epilogue, then attention. `weights`: qkv_weights(...)."""
        _call(lib().q3_prefix_prefill_layer_projected, self.h, layer, ctypes.byref(weights),
              _ptr(x_f16), x_f16.shape[0], _ptr(out))

    def advance(self, tokens):
        _call(lib().q3_prefix_advance, self.h, tokens)

    def set_resident(self, token_count):
        _call(lib().q3_prefix_set_resident, self.h, token_count)

    def seal(self):
        _call(lib().q3_prefix_seal, self.h)

    @property
    def token_count(self):
        return lib().q3_prefix_token_count(self.h)

    def kv_bytes(self):
        return lib().q3_prefix_kv_bytes(self.h)

    def page_table(self):
        n = (self.capacity + PAGE - 1) // PAGE
        p = lib().q3_prefix_page_table(self.h)
        return np.ctypeslib.as_array(p, shape=(n,)).copy()


class PrefixCache:
    """q3_prefix_cache: sealed prefixes kept across requests, by key."""

    def __init__(self, rt, max_entries):
        self.rt = rt
        self.h = _call(lib().q3_prefix_cache_create, rt.h, max_entries)
        self._by_handle = {}

    def acquire(self, key, token_count):
        h = lib().q3_prefix_cache_acquire(self.h, key, token_count)
        return self._by_handle.get(h) if h else None

    def insert(self, key, prefix):
        _call(lib().q3_prefix_cache_insert, self.h, key, prefix.h)
        self._by_handle[prefix.h] = prefix     # the cache owns the handle from here on

    def release(self, prefix):
        _call(lib().q3_prefix_cache_release, self.h, prefix.h)

    def make_room(self, pages_needed):
        n = lib().q3_prefix_cache_make_room(self.h, pages_needed)
        self._forget_evicted()
        return n

    def stats(self):
        st = _lib.PrefixCacheStats()
        lib().q3_prefix_cache_get_stats(self.h, ctypes.byref(st))
        return st

    def _forget_evicted(self):
        # handles the library destroyed must not be destroyed again from Python
        live = self.stats().entries
        if live < len(self._by_handle):
            for h in list(self._by_handle):
                if lib().q3_prefix_cache_holds(self.h, h) == 0:
                    self._by_handle.pop(h).h = None

    def close(self):
        if getattr(self, "h", None):
            for p in self._by_handle.values():
                p.h = None
            lib().q3_prefix_cache_destroy(self.h)
            self.h = None


class BranchSet:
    """q3_branch_set: per-branch suffix pages, taken once."""

    def __init__(self, prefix, max_branches, max_suffix_tokens):
        self.prefix = prefix
        self.h = _call(lib().q3_branch_set_create, prefix.h, max_branches,
                       max_suffix_tokens)

    def close(self):
        if getattr(self, "h", None):
            lib().q3_branch_set_destroy(self.h)
            self.h = None

    def acquire(self):
        return _call(lib().q3_branch_acquire, self.h)

    def release(self, b):
        lib().q3_branch_release(self.h, b)

    def page_table(self):
        nb = lib().q3_branch_set_max_branches(self.h)
        pp = lib().q3_branch_set_pages_per_branch(self.h)
        p = lib().q3_branch_set_page_table(self.h)
        return np.ctypeslib.as_array(p, shape=(nb, pp)).copy()

    def kv_bytes(self):
        return lib().q3_branch_set_kv_bytes(self.h)


class PackPlan:
    """q3_pack_plan: staged q3_pack_view + launch schedule of one suffix batch."""

    def __init__(self, prefix, branch_set, items):
        """items: list of (branch handle, token_count)."""
        arr = (SuffixItem * len(items))(*[SuffixItem(b, n) for b, n in items])
        self.prefix, self.set = prefix, branch_set
        self.h = _call(lib().q3_pack_plan_create, prefix.h, branch_set.h, arr, len(items))
        self.tokens = lib().q3_pack_plan_tokens(self.h)
        self.branches = len(items)

    def close(self):
        if getattr(self, "h", None):
            lib().q3_pack_plan_destroy(self.h)
            self.h = None

    def _arr(self, fn, n):
        return np.ctypeslib.as_array(fn(self.h), shape=(n,)).copy()

    def descriptors(self):
        L = lib()
        return dict(
            token_positions=self._arr(L.q3_pack_plan_token_positions, self.tokens),
            token_branch=self._arr(L.q3_pack_plan_token_branch, self.tokens),
            token_local_pos=self._arr(L.q3_pack_plan_token_local_pos, self.tokens),
            branch_offsets=self._arr(L.q3_pack_plan_branch_offsets, self.branches + 1))

    def attention_layer(self, layer, q, k, v, out):
        _call(lib().q3_suffix_attention_layer, self.h, layer, _ptr(q), _ptr(k), _ptr(v),
              _ptr(out))

    def attention_layer_projected(self, layer, weights, x_f16, out):
        """The layer with its q/k/v projection fused in (see
        Prefix.prefill_layer_projected)."""
        _call(lib().q3_suffix_attention_layer_projected, self.h, layer, ctypes.byref(weights),
              _ptr(x_f16), _ptr(out))

    def attention_layer_gathered(self, layer, q, k, v, peers, seq):
        """Attention fused with the output all-gather: `peers` is a GatherPeers
        (see sharding.PeerGather)."""
        _call(lib().q3_suffix_attention_layer_gathered, self.h, layer, _ptr(q), _ptr(k),
              _ptr(v), ctypes.byref(peers), seq)

    def attention_layer_gathered_host(self, layer, q, k, v, peers, seq, out):
        """Host-buffer variant of attention_layer_gathered: q/k/v/out are pinned
        host torch tensors; `out` receives this rank's rows."""
        _call(lib().q3_suffix_attention_layer_gathered_host, self.h, layer,
              ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(k.data_ptr()),
              ctypes.c_void_p(v.data_ptr()), ctypes.byref(peers), seq,
              ctypes.c_void_p(out.data_ptr()))

    def attention_layer_host(self, layer, q, k, v, out):
        """q/k/v/out: pinned host torch tensors."""
        _call(lib().q3_suffix_attention_layer_host, self.h, layer,
              ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(k.data_ptr()),
              ctypes.c_void_p(v.data_ptr()), ctypes.c_void_p(out.data_ptr()))


class DecodePlan:
    """q3_decode_plan: page lists and split-KV work list of a decode batch."""

    def __init__(self, rt, ctx_lens, page_indptr, page_indices):
        a, pa = _u32(ctx_lens)
        b, pb = _u32(page_indptr)
        c, pc = _u32(page_indices)
        self.rt = rt
        self.num_seqs = len(a)
        self.h = _call(lib().q3_decode_plan_create, rt.h, pa, pb, pc, len(a))

    def close(self):
        if getattr(self, "h", None):
            lib().q3_decode_plan_destroy(self.h)
            self.h = None

    def attention_layer(self, layer, q, k_new, v_new, out):
        _call(lib().q3_decode_attention_layer, self.h, layer, _ptr(q), _ptr(k_new),
              _ptr(v_new), _ptr(out))


def decode_work_host(ctx_lens):
    """q3_decode_work_host: (work [n,4] uint32, seq_work_begin [S+1] uint32)."""
    a, pa = _u32(ctx_lens)
    cap = int(sum((int(c) + 15) // 16 // 64 + 2 for c in a))
    work = np.zeros((cap, 4), np.uint32)
    swb = np.zeros(len(a) + 1, np.uint32)
    n = _call(lib().q3_decode_work_host, pa, len(a), work.ctypes.data_as(ctypes.c_void_p),
              cap, swb.ctypes.data_as(_c_u32p))
    return work[:n].copy(), swb


def attention_decode_noalloc(q_f16, k_pages, v_pages, ctx_lens, page_indptr, page_indices,
                             work, seq_work_begin, out_bf16, stream_ptr=None):
    """q3_cuda_attention_decode_noalloc: every argument is a CUDA tensor owned by
    the caller; the call allocates nothing."""
    n_kv_heads, num_pages = k_pages.shape[0], k_pages.shape[1]
    _call(lib().q3_cuda_attention_decode_noalloc, _ptr(q_f16), _ptr(k_pages), _ptr(v_pages),
          num_pages, _ptr(ctx_lens), _ptr(page_indptr), _ptr(page_indices), _ptr(work),
          work.shape[0], _ptr(seq_work_begin), q_f16.shape[0], q_f16.shape[1], n_kv_heads,
          _ptr(out_bf16), ctypes.c_void_p(stream_ptr) if stream_ptr else None)


def attention_decode_noalloc_status(stream_ptr=None):
    """q3_cuda_attention_decode_noalloc_status: reads and clears the status word
    of the allocation-free decode entry on the current device (synchronises)."""
    st = ctypes.c_uint32(0xFFFFFFFF)
    _call(lib().q3_cuda_attention_decode_noalloc_status, ctypes.byref(st),
          ctypes.c_void_p(stream_ptr) if stream_ptr else None)
    return int(st.value)


def pack_suffix_host(items, prefix_len, max_branches, max_suffix):
    """q3_pack_suffix_host: the reference's q3_decide_run packing, pure host."""
    arr = (SuffixItem * len(items))(*[SuffixItem(b, n) for b, n in items])
    total = int(sum(n for _, n in items))
    pos = np.zeros(max(total, 1), np.uint32)
    br = np.zeros(max(total, 1), np.uint32)
    lp = np.zeros(max(total, 1), np.uint32)
    off = np.zeros(len(items) + 1, np.uint32)
    n = _call(lib().q3_pack_suffix_host, arr, len(items), prefix_len, max_branches,
              max_suffix, pos.ctypes.data_as(_c_u32p), br.ctypes.data_as(_c_u32p),
              lp.ctypes.data_as(_c_u32p), off.ctypes.data_as(_c_u32p))
    return dict(tokens=int(n), token_positions=pos[:n], token_branch=br[:n],
                token_local_pos=lp[:n], branch_offsets=off)


def schedule_describe(row_tag, row_lp, n_kv_heads, shared_len, pages_per_branch,
                      n_branches, num_ctas, max_slots=1 << 20, lockstep=False):
    a, pa = _u32(row_tag)
    b, pb = _u32(row_lp)
    summ = SchedSummary()
    cap = 4 * num_ctas + 4 * ((len(a) + 31) // 32) * n_kv_heads + 16
    segs = (SchedSegmentInfo * cap)()
    _call(lib().q3_schedule_describe, len(a), n_kv_heads, shared_len, pa, pb,
          pages_per_branch, n_branches, num_ctas, max_slots, lockstep, ctypes.byref(summ),
          segs, cap)
    return summ, [segs[i] for i in range(min(cap, summ.n_segments))]
