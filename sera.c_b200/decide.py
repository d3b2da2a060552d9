"""ctypes mirror of include/q3_decide.h: q3_decide_run on the attention runtime."""
import ctypes

import numpy as np

from . import _call, lib
from ._lib import ERRLEN  # noqa: F401

MAX_CANDIDATES = 30
_u32p = ctypes.POINTER(ctypes.c_uint32)


class DecisionItem(ctypes.Structure):
    _fields_ = [("branch", ctypes.c_uint32), ("tokens", _u32p),
                ("token_count", ctypes.c_uint32), ("candidate_ids", _u32p),
                ("candidate_count", ctypes.c_uint32)]


class DecisionBatch(ctypes.Structure):
    _fields_ = [("items", ctypes.POINTER(DecisionItem)), ("count", ctypes.c_uint32)]


class DecisionResult(ctypes.Structure):
    _fields_ = [("predicted_index", ctypes.c_uint32), ("candidate_count", ctypes.c_uint32),
                ("logits", ctypes.c_float * MAX_CANDIDATES),
                ("probabilities", ctypes.c_float * MAX_CANDIDATES)]


class DecideStats(ctypes.Structure):
    _fields_ = ([(n, ctypes.c_double) for n in (
        "prefix_prefill_ms", "branch_create_ms", "suffix_forward_ms", "candidate_head_ms",
        "cold_total_ms", "warm_total_ms", "suffix_questions_per_s", "warm_ms_per_question")] +
        [(n, ctypes.c_size_t) for n in (
            "prefix_kv_bytes_physical", "expected_prefix_kv_bytes", "suffix_kv_bytes",
            "workspace_bytes", "peak_cuda_bytes")] +
        [(n, ctypes.c_uint64) for n in (
            "prefix_allocations", "prefix_bytes", "prefix_copy_calls", "prefix_copy_bytes",
            "suffix_allocations", "suffix_bytes", "cuda_allocations", "cuda_frees",
            "host_syncs", "kernel_launches_per_batch", "kernel_launches_per_question")] +
        [(n, ctypes.c_uint32) for n in (
            "batch", "suffix_tokens_total", "accuracy_matches", "accuracy_total")])


HOOK = ctypes.CFUNCTYPE(ctypes.c_bool, ctypes.c_void_p, ctypes.c_uint32, _u32p,
                        ctypes.c_uint32, ctypes.c_void_p)


class DecideModelIO(ctypes.Structure):
    _fields_ = [("num_layers", ctypes.c_uint32),
                ("q", ctypes.POINTER(ctypes.c_void_p)), ("k", ctypes.POINTER(ctypes.c_void_p)),
                ("v", ctypes.POINTER(ctypes.c_void_p)),
                ("attn_out", ctypes.POINTER(ctypes.c_void_p)),
                ("between_layers", HOOK), ("user", ctypes.c_void_p),
                ("final_hidden", ctypes.c_void_p), ("hidden_size", ctypes.c_uint32),
                ("lm_head", ctypes.c_void_p), ("lm_head_qtype", ctypes.c_uint32),
                ("vocab_size", ctypes.c_uint32)]


def _bind():
    L = lib()
    if not getattr(L, "_decide_bound", False):
        L.q3_decide_run.restype = ctypes.c_bool
        L.q3_decide_run.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                    ctypes.POINTER(DecisionBatch),
                                    ctypes.POINTER(DecideModelIO),
                                    ctypes.POINTER(DecisionResult), ctypes.POINTER(DecideStats),
                                    ctypes.c_char_p, ctypes.c_size_t]
        L.q3_decide_result_softmax.restype = None
        L.q3_decide_result_softmax.argtypes = [ctypes.POINTER(DecisionResult)]
        L._decide_bound = True
    return L


def decide_run(rt, prefix, bset, items, q, k, v, attn_out, final_hidden, lm_head, qtype,
               vocab_size, hook=None):
    """items: list of (branch, token ids, candidate ids); q/k/v/attn_out: lists of
    per-layer CUDA tensors. Returns (list of (predicted, logits, probabilities), stats)."""
    L = _bind()
    keep = []
    arr = (DecisionItem * len(items))()
    for i, (b, toks, cands) in enumerate(items):
        t = np.ascontiguousarray(toks, np.uint32)
        c = np.ascontiguousarray(cands, np.uint32)
        keep += [t, c]
        arr[i] = DecisionItem(b, t.ctypes.data_as(_u32p), len(t), c.ctypes.data_as(_u32p),
                              len(c))
    batch = DecisionBatch(arr, len(items))
    ptrs = lambda ts: (ctypes.c_void_p * len(ts))(*[t.data_ptr() for t in ts])
    io = DecideModelIO()
    io.num_layers = len(q)
    pq, pk, pv, po = ptrs(q), ptrs(k), ptrs(v), ptrs(attn_out)
    io.q, io.k, io.v, io.attn_out = pq, pk, pv, po
    io.between_layers = HOOK(hook) if hook else HOOK()
    io.user = None
    io.final_hidden = final_hidden.data_ptr()
    io.hidden_size = final_hidden.shape[1]
    io.lm_head = lm_head.data_ptr()
    io.lm_head_qtype = qtype
    io.vocab_size = vocab_size
    res = (DecisionResult * len(items))()
    st = DecideStats()
    _call(L.q3_decide_run, rt.h, prefix.h, bset.h, ctypes.byref(batch), ctypes.byref(io), res,
          ctypes.byref(st))
    out = [(r.predicted_index, np.array(r.logits[:r.candidate_count]),
            np.array(r.probabilities[:r.candidate_count])) for r in res]
    return out, st
