"""ctypes signatures for every symbol include/q3_attn.h and include/q3_q4_linear.h declare."""
import ctypes
import os

ERRLEN = 512
PKG = os.path.dirname(os.path.abspath(__file__))


class Q3Error(RuntimeError):
    """An ABI call returned false / NULL / -1; the message is the library's."""


def lib_path():
    return os.path.join(PKG, "libq3attn.so")


class LinearGeometry(ctypes.Structure):
    """q3_q4_linear_geometry"""
    _fields_ = [("M", ctypes.c_int32), ("N", ctypes.c_int32), ("K", ctypes.c_int32),
                ("qtype", ctypes.c_uint32), ("weight_bytes", ctypes.c_uint64)]


class QkvWeights(ctypes.Structure):
    """q3_qkv_weights"""
    _fields_ = [("wq", ctypes.c_void_p), ("wk", ctypes.c_void_p), ("wv", ctypes.c_void_p),
                ("qtype_q", ctypes.c_uint32), ("qtype_k", ctypes.c_uint32),
                ("qtype_v", ctypes.c_uint32), ("hidden", ctypes.c_uint32)]


class LinearStats(ctypes.Structure):
    """q3_q4_linear_stats"""
    _fields_ = [("total_ms", ctypes.c_double), ("activation_quant_ms", ctypes.c_double),
                ("kernel_ms", ctypes.c_double), ("weight_bytes", ctypes.c_uint64),
                ("activation_read_bytes", ctypes.c_uint64),
                ("activation_write_bytes", ctypes.c_uint64),
                ("kernel_launches", ctypes.c_uint64), ("cuda_allocations", ctypes.c_uint64),
                ("host_syncs", ctypes.c_uint64)]


class LinearPlanInfo(ctypes.Structure):
    """q3_q4_linear_plan_info"""
    _fields_ = [("token_tile", ctypes.c_uint32), ("tiles", ctypes.c_uint32),
                ("ctas", ctypes.c_uint32), ("tiles_per_cta_max", ctypes.c_uint32)]


def bind_linear(L):
    """Signatures of include/q3_q4_linear.h (also valid for a build of the
    reference's own q3_q4_linear, which exports part 1 under the same names)."""
    vp, u32, sz, b = ctypes.c_void_p, ctypes.c_uint32, ctypes.c_size_t, ctypes.c_bool
    err = [ctypes.c_char_p, sz]
    gp, sp = ctypes.POINTER(LinearGeometry), ctypes.POINTER(LinearStats)

    def sig(name, res, args):
        f = getattr(L, name, None)
        if f is not None:
            f.restype = res
            f.argtypes = args

    sig("q3_q4_linear_bind_geometry", b, [u32, u32, u32, gp] + err)
    sig("q3_cuda_q4k_linear_init", b, [ctypes.c_int, sz, ctypes.c_int64, ctypes.c_int64] + err)
    sig("q3_cuda_q4k_linear_workspace_bytes", sz, [])
    sig("q3_cuda_q4k_linear_set_workspace", b, [vp, sz] + err)
    sig("q3_cuda_q4k_linear_path_for_batch", ctypes.c_char_p, [sz])
    sig("q3_cuda_q4k_linear", b, [gp, vp, vp, sz, vp, vp, sp] + err)
    sig("q3_cuda_q4k_linear_read_stats", None, [sp, vp])
    sig("q3_cuda_q4k_linear_f16", b, [gp, vp, vp, sz, vp, u32, vp] + err)
    sig("q3_q4_linear_plan", b, [u32, u32, u32, ctypes.POINTER(LinearPlanInfo)] + err)
    sig("q3_q4_linear_packed_bytes", sz, [gp])
    sig("q3_cuda_q4k_linear_pack", b, [gp, vp, vp, gp, vp] + err)
    sig("q3_cuda_q4k_linear_status", b, [vp, ctypes.POINTER(u32)] + err)
    # include/q3_lmhead.h
    sig("q3_cuda_gather_last_rows", b, [vp, vp, u32, u32, vp, vp] + err)
    sig("q3_cuda_candidate_logits_batched", b,
        [vp, vp, u32, u32, u32, vp, u32, u32, vp, vp] + err)
    sig("q3_cuda_candidate_head", b,
        [vp, vp, vp, u32, u32, u32, vp, u32, u32, vp, vp, vp] + err)
    return L


class PrefixCacheStats(ctypes.Structure):
    """q3_prefix_cache_stats"""
    _fields_ = [("hits", ctypes.c_uint64), ("misses", ctypes.c_uint64),
                ("inserts", ctypes.c_uint64), ("evictions", ctypes.c_uint64),
                ("entries", ctypes.c_uint32), ("pages_held", ctypes.c_uint32)]


class GatherPeers(ctypes.Structure):
    _fields_ = [("n_ranks", ctypes.c_uint32), ("rank", ctypes.c_uint32),
                ("gathered", ctypes.c_void_p * 8), ("flags", ctypes.c_void_p * 8)]


def bind(AttnConfig, AttnStats, SuffixItem, SchedSegmentInfo, SchedSummary):
    path = lib_path()
    if not os.path.exists(path):
        raise Q3Error("libq3attn.so is not built (run python sera.c_b200/build.py); "
                      "there is no fallback path")
    L = ctypes.CDLL(path)
    vp, u32, u64, sz = ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_size_t
    fp = ctypes.POINTER(ctypes.c_float)
    up = ctypes.POINTER(ctypes.c_uint32)
    cf = ctypes.c_float
    err = [ctypes.c_char_p, sz]
    b = ctypes.c_bool

    def sig(name, res, args):
        f = getattr(L, name)
        f.restype = res
        f.argtypes = args
        return f

    bind_linear(L)
    # ---- part 1: reference surface
    sig("q3_kv_cache_init", vp, [u32, u32, u32, u32] + err)
    sig("q3_kv_cache_reserve", b, [vp, u32] + err)
    sig("q3_kv_cache_reset", None, [vp])
    sig("q3_kv_cache_destroy", None, [vp])
    sig("q3_kv_cache_length", u32, [vp])
    sig("q3_kv_cache_alias", vp, [vp, vp, u32, u32, u32, u32, u32] + err)
    sig("q3_kv_cache_advance", None, [vp, u32])
    sig("q3_kv_cache_k", vp, [vp])
    sig("q3_kv_cache_v", vp, [vp])
    sig("q3_cuda_rms_norm", b, [vp, vp, u32, u32, cf, vp, vp] + err)
    sig("q3_cuda_rope", b, [vp, vp, u32, u32, u32, u32, u32, vp, vp] + err)
    sig("q3_cuda_rope_positions", b, [vp, vp, u32, u32, u32, u32, vp, vp, vp] + err)
    sig("q3_cuda_attention", b,
        [vp, vp, vp, u32, u32, u32, u32, u32, vp, u32, cf, vp, vp] + err)
    sig("q3_cuda_attention_segmented", b,
        [vp, vp, vp, u32, u32, vp, vp, u32, u32, u32, vp, vp, u32, u32, u32, u32, cf, vp,
         vp] + err)
    sig("q3_cuda_kv_scatter", b, [vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, vp] + err)
    sig("q3_kv_bytes_for_tokens", sz, [u32, u32, u32, u32])
    sig("q3_cuda_attention_native_init", b, [ctypes.c_int, u32, u32, u32, u32] + err)
    sig("q3_cuda_attention_native_shutdown", None, [ctypes.c_int])
    sig("q3_cuda_attention_last_path", ctypes.c_char_p, [])
    sig("q3_cuda_attention_native_synchronize", b, [ctypes.c_int] + err)
    # ---- part 2: native paged path
    sig("q3_attn_create", vp, [ctypes.POINTER(AttnConfig)] + err)
    sig("q3_attn_destroy", None, [vp])
    sig("q3_attn_set_qk_norm", b, [vp, u32, fp, fp] + err)
    sig("q3_attn_stream", vp, [vp])
    sig("q3_attn_synchronize", b, [vp] + err)
    sig("q3_attn_get_stats", None, [vp, ctypes.POINTER(AttnStats)])
    sig("q3_attn_enable_timing", b, [vp, u32] + err)
    sig("q3_attn_phase_times", b, [vp, ctypes.POINTER(ctypes.c_double),
                                   ctypes.POINTER(ctypes.c_uint64)] + err)
    sig("q3_pages_alloc", b, [vp, u32, up] + err)
    sig("q3_pages_free", None, [vp, up, u32])
    sig("q3_pages_k", vp, [vp])
    sig("q3_pages_v", vp, [vp])
    sig("q3_prefix_create", vp, [vp, u32] + err)
    sig("q3_prefix_create_with_pages", vp, [vp, u32, up] + err)
    sig("q3_prefix_prefill_layer", b, [vp, u32, vp, vp, vp, u32, vp] + err)
    sig("q3_prefix_advance", b, [vp, u32] + err)
    sig("q3_prefix_set_resident", b, [vp, u32] + err)
    sig("q3_prefix_seal", b, [vp] + err)
    sig("q3_prefix_destroy", None, [vp])
    sig("q3_prefix_token_count", u32, [vp])
    sig("q3_prefix_kv_bytes", sz, [vp])
    sig("q3_prefix_copy_bytes", u64, [vp])
    sig("q3_prefix_allocations", u64, [vp])
    sig("q3_prefix_page_table", up, [vp])
    sig("q3_branch_set_create", vp, [vp, u32, u32] + err)
    sig("q3_branch_acquire", ctypes.c_int32, [vp] + err)
    sig("q3_branch_reset", None, [vp, ctypes.c_int32])
    sig("q3_branch_release", None, [vp, ctypes.c_int32])
    sig("q3_branch_set_destroy", None, [vp])
    sig("q3_branch_set_kv_bytes", sz, [vp])
    sig("q3_branch_set_max_branches", u32, [vp])
    sig("q3_branch_set_max_suffix", u32, [vp])
    sig("q3_branch_set_page_table", up, [vp])
    sig("q3_branch_set_pages_per_branch", u32, [vp])
    sig("q3_pack_suffix_host", ctypes.c_int64,
        [ctypes.POINTER(SuffixItem), u32, u32, u32, u32, up, up, up, up] + err)
    sig("q3_pack_plan_create", vp, [vp, vp, ctypes.POINTER(SuffixItem), u32] + err)
    sig("q3_pack_plan_destroy", None, [vp])
    sig("q3_pack_plan_tokens", u32, [vp])
    sig("q3_pack_plan_token_positions", up, [vp])
    sig("q3_pack_plan_token_branch", up, [vp])
    sig("q3_pack_plan_token_local_pos", up, [vp])
    sig("q3_pack_plan_branch_offsets", up, [vp])
    sig("q3_suffix_attention_layer", b, [vp, u32, vp, vp, vp, vp] + err)
    sig("q3_suffix_attention_layer_host", b, [vp, u32, vp, vp, vp, vp] + err)
    sig("q3_suffix_attention_layer_projected", b,
        [vp, u32, ctypes.POINTER(QkvWeights), vp, vp] + err)
    sig("q3_prefix_prefill_layer_projected", b,
        [vp, u32, ctypes.POINTER(QkvWeights), vp, u32, vp] + err)
    sig("q3_suffix_attention_layer_gathered_host", b,
        [vp, u32, vp, vp, vp, ctypes.POINTER(GatherPeers), u32, vp] + err)
    sig("q3_suffix_attention_layer_gathered", b,
        [vp, u32, vp, vp, vp, ctypes.POINTER(GatherPeers), u32] + err)
    sig("q3_attn_wait_gathered", b, [vp, ctypes.POINTER(GatherPeers), u32] + err)
    sig("q3_attn_gather_advance", b, [vp, u32] + err)
    sig("q3_prefix_cache_create", vp, [vp, u32] + err)
    sig("q3_prefix_cache_destroy", None, [vp])
    sig("q3_prefix_cache_acquire", vp, [vp, u64, u32])
    sig("q3_prefix_cache_insert", b, [vp, u64, vp] + err)
    sig("q3_prefix_cache_release", b, [vp, vp] + err)
    sig("q3_prefix_cache_make_room", u32, [vp, u32])
    sig("q3_prefix_cache_holds", ctypes.c_int, [vp, vp])
    sig("q3_prefix_cache_get_stats", None, [vp, ctypes.POINTER(PrefixCacheStats)])
    sig("q3_attn_graph_begin", b, [vp] + err)
    sig("q3_attn_graph_end", vp, [vp] + err)
    sig("q3_attn_graph_launch", b, [vp] + err)
    sig("q3_attn_graph_destroy", None, [vp])
    sig("q3_decode_plan_create", vp, [vp, up, up, up, u32] + err)
    sig("q3_decode_plan_destroy", None, [vp])
    sig("q3_decode_attention_layer", b, [vp, u32, vp, vp, vp, vp] + err)
    sig("q3_decode_work_host", ctypes.c_int64, [up, u32, vp, u32, up] + err)
    sig("q3_cuda_attention_decode_noalloc", b,
        [vp, vp, vp, u32, vp, vp, vp, vp, u32, vp, u32, u32, u32, vp, vp] + err)
    sig("q3_cuda_attention_decode_noalloc_status", b, [up, vp] + err)
    sig("q3_attn_reset_status", b, [vp] + err)
    sig("q3_cuda_qknorm_rope_kvwrite", b, [vp, u32, vp, vp, vp, u32, vp, vp, vp, vp] + err)
    sig("q3_schedule_describe", b,
        [u32, u32, u32, up, up, u32, u32, u32, u32, b, ctypes.POINTER(SchedSummary),
         ctypes.POINTER(SchedSegmentInfo), u32] + err)
    sig("q3_attn_set_schedule_policy", b, [vp, u32] + err)
    sig("q3_attn_version", ctypes.c_char_p, [])
    return L
