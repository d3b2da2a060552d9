"""GPU parity tests of the resident Q4_K linear through the C ABI
(include/q3_q4_linear.h) against the CPU oracle, and - where it was built -
against the reference's own MMQ/MMVQ kernels run on the same inputs.

Bars: against the oracle fed the same f16-rounded operands, relative L2 error
< 1e-4 (fp32 accumulation order is the only difference); against the exact
oracle (fp32 dequantisation, fp32 activations, double accumulation), relative
L2 error < 1e-3 and cosine > 0.99999. The reference's own test accepts 1e-2
and 0.999 (tests/test_q3_q4_linear.cu:364-372)."""
import ctypes
import os

import numpy as np
import pytest
import torch

import __graft_entry__ as entry
import q3_quant_oracle as qo

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lin():
    entry.build()
    entry.load_package()
    from sera_c_b200 import q4_linear
    return q4_linear, q4_linear.Q4Linear(0, 4096, 10240, 8192)


def _case(seed, M, N, K):
    rng = np.random.default_rng(seed)
    w = qo.q4k_weight(rng, N, K)
    x = rng.standard_normal((M, K)).astype(np.float32)
    return w, x


@pytest.mark.parametrize("M,N,K", [(1, 128, 256), (4, 256, 512), (16, 128, 1024),
                                   (17, 256, 768), (32, 1024, 5120), (33, 128, 512),
                                   (100, 384, 768), (128, 128, 256), (129, 256, 512),
                                   (300, 256, 1280), (513, 1024, 5120)])
def test_f16_entry_matches_oracle(lin, M, N, K):
    q4, L = lin
    w, x = _case(M + N + K, M, N, K)
    geo = q4.bind_geometry(K, N)
    wd = torch.from_numpy(w).cuda()
    xd = torch.from_numpy(x).cuda().to(torch.float16)
    for dt in (torch.float32, torch.bfloat16, torch.float16):
        out = L.linear_f16(geo, wd, xd, out_dtype=dt)
        assert L.status() == 0
        got = out.float().cpu().numpy()
        ref16 = qo.q4k_linear(w, x, operands="f16")
        m = qo.linear_error_metrics(got, ref16)
        tol = 1e-4 if dt == torch.float32 else (6e-3 if dt == torch.bfloat16 else 1e-3)
        assert m["rel_l2"] < tol, (dt, m)
        if dt == torch.float32:
            exact = qo.linear_error_metrics(got, qo.q4k_linear(w, x))
            assert exact["rel_l2"] < 1e-3 and exact["cos"] > 0.99999, exact


@pytest.mark.parametrize("M,N,K", [(20, 128, 256), (200, 384, 1024), (700, 1024, 2560)])
def test_tiled_weight_layout_is_bit_identical(lin, M, N, K):
    """q3_cuda_q4k_linear_pack: same bytes regrouped per (feature tile, 256-wide
    k range); the linear gives bit-identical output from either layout, and the
    tiled buffer is a permutation of the 144-byte blocks."""
    q4, L = lin
    w, x = _case(3 * M + N, M, N, K)
    geo = q4.bind_geometry(K, N)
    wd = torch.from_numpy(w).cuda()
    xd = torch.from_numpy(x).cuda().half()
    tiled, tgeo = L.pack(geo, wd)
    assert tgeo.qtype == (12 | (1 << 16)) and tgeo.N == N and tgeo.K == K
    a = L.linear_f16(geo, wd, xd, out_dtype=torch.float32)
    b = L.linear_f16(tgeo, tiled, xd, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert torch.equal(a, b)
    nsb = K // 256
    want = w.reshape(N // 128, 128, nsb, 144).transpose(0, 2, 1, 3).reshape(-1)
    assert np.array_equal(tiled.cpu().numpy().reshape(-1), want)
    assert L.status() == 0


@pytest.mark.parametrize("M,N,K", [(3, 128, 256), (70, 256, 1024), (300, 384, 768),
                                   (1000, 1024, 5120)])
def test_q6k_weight_through_the_tiled_layout(lin, M, N, K):
    """Q6_K (attn_v / ffn_down / output tensors of a Q4_K_M file): packed once
    into 224-byte slots, then the same kernel with the Q6_K conversion. Parity
    bars as for Q4_K. The GGUF order itself runs through the plain kernel
    (fp32 dequantisation: exact bars)."""
    q4, L = lin
    rng = np.random.default_rng(M + N + K)
    w = qo.q6k_random_blocks(rng, N * (K // 256)).reshape(N, -1)
    x = rng.standard_normal((M, K)).astype(np.float32)
    geo = q4.bind_geometry(K, N, qtype=q4.Q6_K)
    wd = torch.from_numpy(w).cuda()
    xd = torch.from_numpy(x).cuda().half()
    plain = L.linear_f16(geo, wd, xd, out_dtype=torch.float32).cpu().numpy()
    pm = qo.linear_error_metrics(plain, qo.quant_linear(w, 14, xd.float().cpu().numpy()))
    assert pm["rel_l2"] < 1e-5 and pm["cos"] > 0.999999, pm
    tiled, tgeo = L.pack(geo, wd)
    assert tgeo.qtype == (14 | (1 << 16)) and tiled.numel() == N * (K // 256) * 224
    slots = tiled.cpu().numpy().reshape(N // 128, K // 256, 128, 224)
    want = w.reshape(N // 128, 128, K // 256, 210).transpose(0, 2, 1, 3)
    assert np.array_equal(slots[..., :210], want) and not slots[..., 210:].any()
    got = L.linear_f16(tgeo, tiled, xd, out_dtype=torch.float32).cpu().numpy()
    assert L.status() == 0
    m16 = qo.linear_error_metrics(got, qo.quant_linear(w, 14, x, operands="f16"))
    assert m16["rel_l2"] < 1e-4, m16
    exact = qo.linear_error_metrics(got, qo.quant_linear(w, 14, x))
    assert exact["rel_l2"] < 1e-3 and exact["cos"] > 0.99999, exact


@pytest.mark.parametrize("qtype", [12, 14])
@pytest.mark.parametrize("M,N,K", [(600, 8192, 256), (600, 8192, 1024), (1500, 10240, 512)])
def test_more_tiles_than_sms(lin, qtype, M, N, K):
    """The tile kernel is persistent: with more output tiles than SMs a CTA walks
    several tiles, its rings run on across the tile boundary and the accumulator
    is drained while the next tile's operands are converted. K = 256 is the
    shortest row (4 k-steps per tile: a group crosses a tile boundary after one or
    two steps). Every output is checked."""
    q4, L = lin
    plan = q4.plan(M, N)
    assert plan.tiles > 148 and plan.tiles_per_cta_max >= 2
    rng = np.random.default_rng(M + N + K + qtype)
    nb = N * (K // 256)
    w = (qo.q4k_random_blocks(rng, nb) if qtype == 12 else qo.q6k_random_blocks(rng, nb))
    w = w.reshape(N, -1)
    x = rng.standard_normal((M, K)).astype(np.float32)
    geo = q4.bind_geometry(K, N, qtype=qtype)
    wd = torch.from_numpy(w).cuda()
    xd = torch.from_numpy(x).cuda().half()
    if qtype == 14:
        wd, geo = L.pack(geo, wd)
    got = L.linear_f16(geo, wd, xd, out_dtype=torch.float32).cpu().numpy()
    assert L.status() == 0
    ref16 = qo.quant_linear(w, qtype, x, operands="f16")
    err = np.abs(got - ref16)
    assert err.max() < 1e-3 * np.abs(ref16).max(), np.unravel_index(err.argmax(), err.shape)
    assert qo.linear_error_metrics(got, ref16)["rel_l2"] < 1e-4


def test_small_batch_path_matches_tile_kernel(lin):
    """At most 16 tokens take the mma.sync kernel (GGUF order); the same batch
    through the tiled order takes the tcgen05 kernel. Same operands, different
    summation order: equal to 1e-5 relative L2."""
    q4, L = lin
    assert q4._L().q3_cuda_q4k_linear_path_for_batch(8) == b"MMVQ"
    assert q4._L().q3_cuda_q4k_linear_path_for_batch(9) == b"TC"
    w, x = _case(77, 13, 512, 2048)
    geo = q4.bind_geometry(2048, 512)
    wd = torch.from_numpy(w).cuda()
    xd = torch.from_numpy(x).cuda().half()
    tiled, tgeo = L.pack(geo, wd)
    a = L.linear_f16(geo, wd, xd, out_dtype=torch.float32).cpu().numpy()
    b = L.linear_f16(tgeo, tiled, xd, out_dtype=torch.float32).cpu().numpy()
    m = qo.linear_error_metrics(a, b)
    assert m["rel_l2"] < 1e-5, m
    assert L.status() == 0


def test_rows_beyond_the_batch_are_untouched(lin):
    q4, L = lin
    w, x = _case(9, 70, 256, 512)
    geo = q4.bind_geometry(512, 256)
    out = torch.full((128, 256), 7.0, dtype=torch.float32, device="cuda")
    L.linear_f16(geo, torch.from_numpy(w).cuda(), torch.from_numpy(x).cuda().half(), out=out[:70])
    torch.cuda.synchronize()
    assert bool((out[70:] == 7.0).all())
    assert L.status() == 0


@pytest.mark.parametrize("M", [1, 4, 16, 200])
def test_fp32_surface_like_the_reference_test(lin, M):
    """q3_cuda_q4k_linear on the reference test's batch sizes and activation
    pattern (tests/test_q3_q4_linear.cu:226-234, 294): finite, within the bars,
    bit-exact on repetition, stats filled."""
    q4, L = lin
    N, K = 512, 2048
    w, _ = _case(11, 1, N, K)
    k = np.arange(K, dtype=np.float64)[None, :]
    t = np.arange(M, dtype=np.float64)[:, None]
    a = ((k * 17 + t * 131) % 1009) * 0.1
    x = (0.5 * np.sin(a) + 0.25 * np.cos(a * 0.37)).astype(np.float32)
    geo = q4.bind_geometry(K, N)
    wd, xd = torch.from_numpy(w).cuda(), torch.from_numpy(x).cuda()
    from sera_c_b200._lib import LinearStats
    st = LinearStats()
    out = L.linear_f32(geo, wd, xd, stats=st)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    m = qo.linear_error_metrics(got, qo.q4k_linear(w, x))
    if M <= 8:
        # the reference's small-batch arithmetic (8-bit activations): its own bar
        # against the exact product, and 1e-5 against that arithmetic done exactly
        assert m["cos"] > 0.999 and m["rel_l2"] < 0.01, m
        mq = qo.linear_error_metrics(got, qo.q4k_linear_q8(w, x))
        assert mq["rel_l2"] < 1e-5, mq
    else:
        assert m["cos"] > 0.99999 and m["rel_l2"] < 1e-3, m
    out2 = L.linear_f32(geo, wd, xd)
    torch.cuda.synchronize()
    assert torch.equal(out, out2)
    L.read_stats(st)
    assert st.weight_bytes == N * (K // 256) * 144 and st.kernel_launches == 2
    assert st.cuda_allocations == 0 and st.host_syncs == 0 and st.total_ms > 0
    assert L.status() == 0


@pytest.mark.parametrize("qtype", [12, 14])
@pytest.mark.parametrize("M,N,K", [(1, 200, 512), (8, 72, 256), (19, 1000, 1024)])
def test_gguf_order_any_feature_count(lin, qtype, M, N, K):
    """What the reference's entry point accepts and the tile kernels do not:
    Q6_K in GGUF order and feature counts off the 128 grid (ref:
    src/q3_q4_linear.cu:149-228), through both the f16 and the fp32 entry."""
    q4, L = lin
    rng = np.random.default_rng(qtype + M + N + K)
    if qtype == 12:
        w = qo.q4k_weight(rng, N, K)
    else:
        w = qo.q6k_random_blocks(rng, N * (K // 256)).reshape(N, -1)
    x = rng.standard_normal((M, K)).astype(np.float32)
    geo = q4.bind_geometry(K, N, qtype=qtype)
    wd = torch.from_numpy(w).cuda()
    xh = torch.from_numpy(x).cuda().half()
    got = L.linear_f16(geo, wd, xh, out_dtype=torch.float32).cpu().numpy()
    m = qo.linear_error_metrics(got, qo.quant_linear(w, qtype, xh.float().cpu().numpy()))
    assert m["rel_l2"] < 1e-5 and m["cos"] > 0.999999, m
    got32 = L.linear_f32(geo, wd, torch.from_numpy(x).cuda()).cpu().numpy()
    m32 = qo.linear_error_metrics(got32, qo.quant_linear(w, qtype, x))
    assert m32["rel_l2"] < 1e-3 and m32["cos"] > 0.99999, m32     # activations pass through f16
    assert L.status() == 0


def test_error_paths(lin):
    q4, L = lin
    from sera_c_b200 import Q3Error
    geo = q4.bind_geometry(512, 256)
    w = torch.zeros(256 * 2 * 144, dtype=torch.uint8, device="cuda")
    x = torch.zeros(8, 512, dtype=torch.float16, device="cuda")
    with pytest.raises(Q3Error, match="workspace"):
        big = torch.zeros(5000, 8192, dtype=torch.float32, device="cuda")
        L.linear_f32(q4.bind_geometry(8192, 256), w, big)
    with pytest.raises(Q3Error, match="multiple of 256"):
        q4.bind_geometry(500, 256)
    assert geo.weight_bytes == 256 * 2 * 144


def test_against_reference_kernels(lin):
    """The reference's own Q4_K linear (Q8_1 activation quantisation + MMVQ /
    MMQ), compiled unchanged for sm_100a, on the same inputs: this library must
    be the closer to the exact oracle. On these synthetic inputs (uniformly
    random quants, N(0,1) activations) the reference's Q8_1 activation
    quantisation alone costs about 1 % relative L2 error, so its own bar
    (1 %, stated for model weights) is widened to 3 % for it here."""
    path = os.path.join(ROOT, "oracle", "_ref", "libq3q4ref.so")
    if not os.path.exists(path):
        pytest.skip("reference Q4_K linear not built (make -C oracle refq4)")
    q4, L = lin
    from sera_c_b200 import _lib
    R = _lib.bind_linear(ctypes.CDLL(path))
    err = ctypes.create_string_buffer(512)
    assert R.q3_cuda_q4k_linear_init(0, 512, 1024, 2048, err, 512), err.value
    arena = torch.empty(max(int(R.q3_cuda_q4k_linear_workspace_bytes()), 256),
                        dtype=torch.uint8, device="cuda")
    assert R.q3_cuda_q4k_linear_set_workspace(arena.data_ptr(), arena.numel(), err, 512), err.value
    N, K = 1024, 2048
    for M in (1, 5, 8, 16, 64, 300):
        w, x = _case(100 + M, M, N, K)
        geo = q4.bind_geometry(K, N)
        wd, xd = torch.from_numpy(w).cuda(), torch.from_numpy(x).cuda()
        ref_out = torch.zeros(M, N, dtype=torch.float32, device="cuda")
        assert R.q3_cuda_q4k_linear(ctypes.byref(geo), wd.data_ptr(), xd.data_ptr(), M,
                                    ref_out.data_ptr(), None, None, err, 512), err.value
        torch.cuda.synchronize()
        ours = L.linear_f32(geo, wd, xd)
        torch.cuda.synchronize()
        exact = qo.q4k_linear(w, x)
        mr = qo.linear_error_metrics(ref_out.cpu().numpy(), exact)
        mo = qo.linear_error_metrics(ours.cpu().numpy(), exact)
        assert mr["cos"] > 0.999 and mr["rel_l2"] < 0.03, (M, mr)
        if M <= 8:
            # same arithmetic as the reference's MMVQ path: the two results agree
            # to fp32 summation order (and the odd x/d tie under its fast-math build)
            both = qo.linear_error_metrics(ours.cpu().numpy(), ref_out.cpu().numpy())
            assert both["rel_l2"] < 1e-4, (M, both)
        else:
            assert mo["rel_l2"] < 1e-3 and mo["rel_l2"] < mr["rel_l2"], (M, mo, mr)
