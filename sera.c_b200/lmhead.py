"""Host-side mirror of include/q3_lmhead.h: the last-row gather and the batched
selected-row LM head that consume the attention path's output at the end of the
packed decision forward (ref: src/q3_forward.cu:1866-1894, host decision
src/q3_decide.cu:517-553). Torch is used for device memory only."""
import ctypes

from . import _lib
from ._lib import Q3Error


def _L():
    from . import lib
    return lib()


def _call(fn, *args):
    err = ctypes.create_string_buffer(_lib.ERRLEN)
    if not fn(*args, err, _lib.ERRLEN):
        raise Q3Error(err.value.decode() or "%s failed" % fn.__name__)


def gather_last_rows(src, branch_offsets, stream=None):
    """q3_cuda_gather_last_rows: src [tokens, hidden] fp32, branch_offsets [B+1] int32."""
    import torch
    n = branch_offsets.numel() - 1
    out = torch.empty(n, src.shape[1], dtype=torch.float32, device=src.device)
    _call(_L().q3_cuda_gather_last_rows, src.data_ptr(), branch_offsets.data_ptr(), n,
          src.shape[1], out.data_ptr(), stream)
    return out


def candidate_logits_batched(hidden_per_branch, weight, qtype, vocab_size, candidate_ids,
                             candidate_count, stream=None):
    """q3_cuda_candidate_logits_batched -> logits [B * K] fp32."""
    import torch
    n = hidden_per_branch.shape[0]
    logits = torch.empty(n * candidate_count, dtype=torch.float32,
                         device=hidden_per_branch.device)
    _call(_L().q3_cuda_candidate_logits_batched, hidden_per_branch.data_ptr(),
          weight.data_ptr(), qtype, hidden_per_branch.shape[1], vocab_size,
          candidate_ids.data_ptr(), candidate_count, n, logits.data_ptr(), stream)
    return logits


def candidate_head(hidden_rows, branch_offsets, weight, qtype, vocab_size, candidate_ids,
                   candidate_count, stream=None):
    """q3_cuda_candidate_head -> (logits [B * K] fp32, best [B] int32)."""
    import torch
    n = branch_offsets.numel() - 1
    dev = hidden_rows.device
    logits = torch.empty(n * candidate_count, dtype=torch.float32, device=dev)
    best = torch.empty(n, dtype=torch.int32, device=dev)
    _call(_L().q3_cuda_candidate_head, hidden_rows.data_ptr(), branch_offsets.data_ptr(),
          weight.data_ptr(), qtype, hidden_rows.shape[1], vocab_size, candidate_ids.data_ptr(),
          candidate_count, n, logits.data_ptr(), best.data_ptr(), stream)
    return logits, best
