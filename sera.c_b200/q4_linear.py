"""Host-side mirror of the resident Q4_K linear (include/q3_q4_linear.h).

Same calls, in the same order, as the reference's binder and layer driver make
(ref: src/q3_forward.cu:1055-1061 init + workspace, :1214-1242 q/k/v
projections, :1289-1296 output projection): bind the geometry once per weight,
initialise once per process, attach a scratch arena, then call the linear with
device pointers. Torch is used for device memory only.
"""
import ctypes

from . import _lib
from ._lib import LinearGeometry, LinearStats, Q3Error

Q4_K, Q6_K = 12, 14
OUT_F32, OUT_BF16, OUT_F16 = 0, 1, 2


def _L():
    from . import lib
    return lib()


def _call(fn, *args):
    err = ctypes.create_string_buffer(_lib.ERRLEN)
    if not fn(*args, err, _lib.ERRLEN):
        raise Q3Error(err.value.decode() or "%s failed" % fn.__name__)


def bind_geometry(k, n, qtype=Q4_K):
    """q3_q4_linear_bind_geometry: GGUF dim0 = K (row length), dim1 = N (rows)."""
    g = LinearGeometry()
    _call(_L().q3_q4_linear_bind_geometry, qtype, k, n, ctypes.byref(g))
    return g


def plan(tokens, n_features, sm_count=148):
    """q3_q4_linear_plan: the launch shape for a batch (host arithmetic only)."""
    info = _lib.LinearPlanInfo()
    _call(_L().q3_q4_linear_plan, tokens, n_features, sm_count, ctypes.byref(info))
    return info


class Q4Linear:
    """Process-wide set-up plus the scratch arena, like the reference runtime's
    mmq arena. One instance per device."""

    def __init__(self, device, max_tokens, max_features, max_k):
        import torch
        self.torch = torch
        self.device = torch.device("cuda", device)
        _call(_L().q3_cuda_q4k_linear_init, device, max_tokens, max_features, max_k)
        nbytes = int(_L().q3_cuda_q4k_linear_workspace_bytes())
        self.arena = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=self.device)
        _call(_L().q3_cuda_q4k_linear_set_workspace, self.arena.data_ptr(), self.arena.numel())

    def linear_f32(self, geo, weight, x, out=None, stream=None, stats=None):
        """q3_cuda_q4k_linear: fp32 [tokens, K] -> fp32 [tokens, N]."""
        torch = self.torch
        tokens = x.shape[0]
        if out is None:
            out = torch.empty(tokens, geo.N, dtype=torch.float32, device=x.device)
        _call(_L().q3_cuda_q4k_linear, ctypes.byref(geo), weight.data_ptr(), x.data_ptr(),
              tokens, out.data_ptr(), stream, ctypes.byref(stats) if stats is not None else None)
        return out

    def linear_f16(self, geo, weight, x, out=None, out_dtype=None, stream=None):
        """q3_cuda_q4k_linear_f16: f16 [tokens, K] -> bf16 / f16 / fp32 [tokens, N]."""
        torch = self.torch
        if x.dtype != torch.float16:
            raise Q3Error("linear_f16 takes f16 activations")
        tokens = x.shape[0]
        if out is None:
            out = torch.empty(tokens, geo.N, dtype=out_dtype or torch.bfloat16, device=x.device)
        code = {torch.float32: OUT_F32, torch.bfloat16: OUT_BF16, torch.float16: OUT_F16}[out.dtype]
        _call(_L().q3_cuda_q4k_linear_f16, ctypes.byref(geo), weight.data_ptr(), x.data_ptr(),
              tokens, out.data_ptr(), code, stream)
        return out

    def pack(self, geo, weight, stream=None):
        """q3_cuda_q4k_linear_pack: returns (tiled weight, tiled geometry)."""
        nbytes = int(_L().q3_q4_linear_packed_bytes(ctypes.byref(geo)))
        if nbytes == 0:
            raise Q3Error("pack takes a Q4_K or Q6_K weight in GGUF order")
        tiled = self.torch.empty(nbytes, dtype=self.torch.uint8, device=weight.device)
        tg = LinearGeometry()
        _call(_L().q3_cuda_q4k_linear_pack, ctypes.byref(geo), weight.data_ptr(),
              tiled.data_ptr(), ctypes.byref(tg), stream)
        return tiled, tg

    def status(self, stream=None):
        s = ctypes.c_uint32(0)
        _call(_L().q3_cuda_q4k_linear_status, stream, ctypes.byref(s))
        return s.value

    def read_stats(self, stats):
        _L().q3_cuda_q4k_linear_read_stats(ctypes.byref(stats), None)
        return stats
