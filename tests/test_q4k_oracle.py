"""CPU tests of the Q4_K oracle (oracle/q3_quant_oracle.py): bit-exact against
values produced by the reference's own C dequantisation (committed fixture),
the reference test's hand-derived first-nibble check, and - when the reference
library was built here - a larger random comparison."""
import ctypes
import os

import numpy as np
import pytest

import q3_quant_oracle as qo

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = os.path.join(ROOT, "tests", "golden", "q4k_dequant_ref.npz")


def test_dequant_matches_reference_fixture_bit_exactly():
    g = np.load(GOLD)
    got = qo.q4k_dequantize(g["blocks"])
    assert got.dtype == np.float32 and got.shape == g["values"].shape
    assert np.array_equal(got.view(np.uint32), g["values"].view(np.uint32))


def test_first_nibble_by_hand():
    # ref: tests/test_q3_q4_linear.cu:95-107
    g = np.load(GOLD)
    for b, vals in zip(g["blocks"][:6], g["values"].reshape(-1, 256)):
        d = float(b[0:2].copy().view(np.float16)[0])
        dmin = float(b[2:4].copy().view(np.float16)[0])
        sc, mn = int(b[4] & 63), int(b[8] & 63)
        expected = d * sc * int(b[16] & 0xF) - dmin * mn
        assert abs(expected - float(vals[0])) < 1e-3


def test_element_order_and_split_scale_fields():
    """One block with a single non-zero quant at a time: low nibbles of byte l of
    group j are element 64j+l, high nibbles element 64j+32+l; sub-blocks 4..7
    take their 6-bit scale from two bytes."""
    blk = np.zeros((1, 144), np.uint8)
    blk[0, 0:2] = np.asarray([1.0], np.float16).view(np.uint8)       # d = 1, dmin = 0
    scales = np.zeros(12, np.uint8)
    want_sc = [1, 2, 3, 4, 37, 38, 39, 40]
    for i, sc in enumerate(want_sc):
        if i < 4:
            scales[i] |= sc & 63
        else:
            scales[i + 4] |= sc & 0xF
            scales[i - 4] |= (sc >> 4) << 6
    blk[0, 4:16] = scales
    for j in range(4):
        for l in (0, 13, 31):
            for hi in (0, 1):
                b = blk.copy()
                b[0, 16 + 32 * j + l] = 5 << (4 * hi)
                v = qo.q4k_dequantize(b)
                e = 64 * j + 32 * hi + l
                assert v[e] == 5.0 * want_sc[2 * j + hi]
                assert np.count_nonzero(v) == 1


def test_dequant_matches_reference_library_on_random_blocks():
    path = os.path.join(ROOT, "oracle", "_ref", "libq3quant_ref.so")
    if not os.path.exists(path):
        pytest.skip("reference dequantisation not built here (make -C oracle refquant)")
    lib = ctypes.CDLL(path)
    lib.q3_quant_dequantize_row.restype = ctypes.c_bool
    lib.q3_quant_dequantize_row.argtypes = [ctypes.c_uint32, ctypes.c_void_p, ctypes.c_size_t,
                                            ctypes.c_void_p, ctypes.c_size_t, ctypes.c_char_p,
                                            ctypes.c_size_t]
    blocks = qo.q4k_random_blocks(np.random.default_rng(7), 2000)
    out = np.zeros(2000 * 256, np.float32)
    err = ctypes.create_string_buffer(256)
    assert lib.q3_quant_dequantize_row(12, blocks.ctypes.data, 2000, out.ctypes.data, out.size,
                                       err, 256), err.value
    assert np.array_equal(qo.q4k_dequantize(blocks).view(np.uint32), out.view(np.uint32))


def test_f16_operand_model_is_close_to_exact():
    blocks = qo.q4k_random_blocks(np.random.default_rng(3), 64)
    exact = qo.q4k_dequantize(blocks).astype(np.float64)
    f16 = qo.q4k_dequantize_f16_operands(blocks).astype(np.float64)
    assert np.abs(f16 - exact).max() <= 2e-3 * np.abs(exact).max()


def test_linear_oracle_small():
    rng = np.random.default_rng(5)
    w = qo.q4k_weight(rng, 8, 512)
    x = rng.standard_normal((3, 512)).astype(np.float32)
    out = qo.q4k_linear(w, x)
    deq = qo.q4k_dequantize(w).reshape(8, 512).astype(np.float64)
    for t in range(3):
        for n in range(8):
            assert abs(out[t, n] - float(np.dot(deq[n], x[t].astype(np.float64)))) < 1e-9
    m = qo.linear_error_metrics(qo.q4k_linear(w, x, operands="f16"), out)
    assert m["rel_l2"] < 2e-3 and m["cos"] > 0.99999


def test_q6k_dequant_matches_reference_fixture_bit_exactly():
    g = np.load(os.path.join(ROOT, "tests", "golden", "q6k_dequant_ref.npz"))
    got = qo.q6k_dequantize(g["blocks"])
    assert np.array_equal(got.view(np.uint32), g["values"].view(np.uint32))


def test_candidate_head_oracle_small():
    rng = np.random.default_rng(1)
    w = qo.q6k_random_blocks(rng, 6 * 2).reshape(6, -1)
    rows = rng.standard_normal((5, 512)).astype(np.float32)
    offs = np.asarray([0, 2, 5], np.int32)
    last = qo.gather_last_rows(rows, offs)
    assert np.array_equal(last, rows[[1, 4]])
    ids = np.asarray([0, 5, 3, 3], np.int32)
    out = qo.candidate_logits_batched(last, w, 14, ids, 2)
    deq = qo.q6k_dequantize(w).reshape(6, 512).astype(np.float64)
    assert abs(out[1] - float(deq[5] @ rows[1].astype(np.float64))) < 1e-9
    assert abs(out[2] - float(deq[3] @ rows[4].astype(np.float64))) < 1e-9


def test_q6k_f16_operand_model_is_close_to_exact():
    blocks = qo.q6k_random_blocks(np.random.default_rng(4), 64)
    exact = qo.q6k_dequantize(blocks).astype(np.float64)
    f16 = qo.q6k_dequantize_f16_operands(blocks).astype(np.float64)
    assert np.abs(f16 - exact).max() <= 2e-3 * np.abs(exact).max()


def test_q8_activation_model():
    """Q8_1 quantisation and the integer dot: error against the exact product is
    at the level the reference accepts (1 %); an all-zero block quantises to zero."""
    rng = np.random.default_rng(8)
    w = qo.q4k_weight(rng, 16, 1024)
    x = rng.standard_normal((3, 1024)).astype(np.float32)
    x[1, 64:96] = 0.0
    q, d8 = qo.q8_1_quantize(x)
    assert np.abs(q).max() == 127 and not q[1, 64:96].any() and d8[1, 2] == 0.0
    assert np.abs(q * np.repeat(d8, 32, axis=1) - x).max() <= 0.51 * d8.max() * 1.001
    m = qo.linear_error_metrics(qo.q4k_linear_q8(w, x), qo.q4k_linear(w, x))
    assert m["rel_l2"] < 0.02 and m["cos"] > 0.999
