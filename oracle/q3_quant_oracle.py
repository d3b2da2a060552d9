"""CPU oracle of the Q4_K weight format and the Q4_K linear (test infrastructure).

This file restates, in numpy, the block semantics the reference uses for its
resident Q4_K linears and the CPU check its own test applies to them. It is a
checker: only tests, the smoke entry and the benchmark's CPU-baseline /
reference arm may import it. The product path never does.

Followed reference code (by path inside the reference project):
  src/q3_quant.h:24-33      block layout: 144 bytes = d (f16), dmin (f16),
                            scales[12] (6-bit scale/min pairs), qs[128]
  src/q3_quant.c:18-42      half -> float
  src/q3_quant.c:44-55      scale/min unpack of sub-block `index` (0..7)
  src/q3_quant.c:57-76      element order: per 64 elements 32 bytes of qs, low
                            nibbles are elements 0..31, high nibbles 32..63;
                            value = d*scale*q - dmin*min in fp32
  tests/test_q3_q4_linear.cu:236-272  the linear check: dequantise the whole
                            weight, dot in double, out[token][feature]
  tests/test_q3_q4_linear.cu:340-372  its acceptance: cosine > 0.999 and
                            relative L2 error < 1 % against that CPU result
Pinned by tests/golden/q4k_dequant_ref.npz, which holds outputs of the
reference's own q3_quant_dequantize_row compiled from its source.
"""
import numpy as np

QK_K = 256
Q4_K_BLOCK_BYTES = 144
Q4_K_TYPE = 12       # GGML type ids, src/q3_quant.h:19-22
Q6_K_TYPE = 14


def _as_blocks(blocks):
    b = np.ascontiguousarray(blocks, dtype=np.uint8)
    if b.size % Q4_K_BLOCK_BYTES:
        raise ValueError("Q4_K data must be a whole number of 144-byte blocks")
    return b.reshape(-1, Q4_K_BLOCK_BYTES)


def q4k_fields(blocks):
    """Unpack [n,144] bytes into d, dmin (float32 [n]), scale, min (uint8 [n,8])
    and the 4-bit quants in element order (uint8 [n,256])."""
    b = _as_blocks(blocks)
    d = b[:, 0:2].copy().view(np.float16).astype(np.float32)[:, 0]
    dmin = b[:, 2:4].copy().view(np.float16).astype(np.float32)[:, 0]
    s = b[:, 4:16]
    sc = np.empty((b.shape[0], 8), np.uint8)
    mn = np.empty((b.shape[0], 8), np.uint8)
    for i in range(8):
        if i < 4:
            sc[:, i] = s[:, i] & 63
            mn[:, i] = s[:, i + 4] & 63
        else:
            sc[:, i] = (s[:, i + 4] & 0xF) | ((s[:, i - 4] >> 6) << 4)
            mn[:, i] = (s[:, i + 4] >> 4) | ((s[:, i] >> 6) << 4)
    qs = b[:, 16:144].reshape(-1, 4, 32)
    q = np.empty((b.shape[0], 4, 64), np.uint8)
    q[:, :, :32] = qs & 0xF
    q[:, :, 32:] = qs >> 4
    return d, dmin, sc, mn, q.reshape(-1, QK_K)


def q4k_dequantize(blocks):
    """fp32 values exactly as the reference's scalar loop produces them:
    (d*scale)*q - (dmin*min), every step in fp32."""
    d, dmin, sc, mn, q = q4k_fields(blocks)
    d1 = (d[:, None] * sc.astype(np.float32)).astype(np.float32)        # [n,8]
    m1 = (dmin[:, None] * mn.astype(np.float32)).astype(np.float32)
    d1 = np.repeat(d1, 32, axis=1)
    m1 = np.repeat(m1, 32, axis=1)
    return (d1 * q.astype(np.float32) - m1).astype(np.float32).reshape(-1)


def q4k_dequantize_f16_operands(blocks):
    """The rounding the tensor-core kernel applies when it turns a block into
    f16 MMA operands: per sub-block scale and offset rounded to f16, then one
    fused multiply-add per element rounded to f16. Used for tight parity
    checks (the comparison then isolates indexing and accumulation)."""
    d, dmin, sc, mn, q = q4k_fields(blocks)
    d1 = (d[:, None] * sc.astype(np.float32)).astype(np.float16).astype(np.float64)
    m1 = (dmin[:, None] * mn.astype(np.float32)).astype(np.float16).astype(np.float64)
    d1 = np.repeat(d1, 32, axis=1)
    m1 = np.repeat(m1, 32, axis=1)
    return (d1 * q.astype(np.float64) - m1).astype(np.float16).reshape(-1)


def q4k_random_blocks(rng, n_blocks, d_max=0.004, dmin_max=0.02):
    """Synthetic Q4_K blocks: random scales, mins and quants; d and dmin drawn so
    that the dequantised weights are O(0.1) like trained projection weights."""
    b = rng.integers(0, 256, (n_blocks, Q4_K_BLOCK_BYTES), dtype=np.uint8)
    d = (rng.random(n_blocks) * d_max + d_max * 0.1).astype(np.float16)
    dmin = (rng.random(n_blocks) * dmin_max * 0.1).astype(np.float16)
    b[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    b[:, 2:4] = dmin.view(np.uint8).reshape(-1, 2)
    return b


def q4k_weight(rng, n_features, k):
    """A [n_features, k] weight as Q4_K bytes, row-major rows of k/256 blocks."""
    if k % QK_K:
        raise ValueError("K must be a multiple of 256")
    return q4k_random_blocks(rng, n_features * (k // QK_K)).reshape(
        n_features, (k // QK_K) * Q4_K_BLOCK_BYTES)


def q4k_linear(weight_bytes, x, operands="fp32"):
    """out[token][feature] = sum_k W[feature][k] * x[token][k] in double.
    operands = "fp32": W dequantised as the reference does, x as given.
    operands = "f16":  W and x rounded the way the tensor-core kernel feeds them."""
    n = weight_bytes.shape[0]
    if operands == "fp32":
        w = q4k_dequantize(weight_bytes).reshape(n, -1).astype(np.float64)
        xx = np.asarray(x, np.float32).astype(np.float64)
    elif operands == "f16":
        w = q4k_dequantize_f16_operands(weight_bytes).reshape(n, -1).astype(np.float64)
        xx = np.asarray(x, np.float32).astype(np.float16).astype(np.float64)
    else:
        raise ValueError(operands)
    return xx @ w.T


# --------------------------------------------------------------------------
# Q6_K (the output.weight of a Q4_K_M file) and the selected-row LM head
# --------------------------------------------------------------------------
Q6_K_BLOCK_BYTES = 210


def q6k_dequantize(blocks):
    """fp32 values of Q6_K blocks as the reference's scalar loop produces them
    (src/q3_quant.c:78-103): per block ql[128] low nibbles, qh[64] high 2 bits,
    scales[16] int8, d (f16); per half of 128 elements and l in 0..31
        q1 = (ql[l]    & 15 | (qh[l]      & 3) << 4) - 32 -> element l
        q2 = (ql[l+32] & 15 | (qh[l] >> 2 & 3) << 4) - 32 -> element l + 32
        q3 = (ql[l]   >> 4  | (qh[l] >> 4 & 3) << 4) - 32 -> element l + 64
        q4 = (ql[l+32] >> 4 | (qh[l] >> 6 & 3) << 4) - 32 -> element l + 96
    value = d * scale[is + 0/2/4/6] * q with is = l / 16; the products are
    formed left to right in fp32."""
    b = np.ascontiguousarray(blocks, dtype=np.uint8)
    if b.size % Q6_K_BLOCK_BYTES:
        raise ValueError("Q6_K data must be a whole number of 210-byte blocks")
    b = b.reshape(-1, Q6_K_BLOCK_BYTES)
    n = b.shape[0]
    ql = b[:, 0:128].reshape(n, 2, 64).astype(np.int32)
    qh = b[:, 128:192].reshape(n, 2, 32).astype(np.int32)
    sc = b[:, 192:208].copy().view(np.int8).reshape(n, 2, 8).astype(np.float32)
    d = b[:, 208:210].copy().view(np.float16).astype(np.float32)[:, 0]
    out = np.empty((n, 2, 128), np.float32)
    l = np.arange(32)
    is_ = l // 16
    for q, (lo, shift_q, nib_hi, sc_off) in enumerate(
            [(0, 0, False, 0), (32, 2, False, 2), (0, 4, True, 4), (32, 6, True, 6)]):
        low = ql[:, :, lo:lo + 32]
        low = (low >> 4) if nib_hi else (low & 0xF)
        val = (low | (((qh >> shift_q) & 3) << 4)) - 32
        scale = sc[:, :, is_ + sc_off]
        t = (d[:, None, None] * scale).astype(np.float32)
        out[:, :, 32 * q:32 * q + 32] = (t * val.astype(np.float32)).astype(np.float32)
    return out.reshape(-1)


def q6k_dequantize_f16_operands(blocks):
    """The rounding the tensor-core kernel applies to a Q6_K block: per 16
    elements scale = f16(d * sc), element = f16((q - 32) * scale)."""
    b = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1, Q6_K_BLOCK_BYTES)
    exact_q = np.empty((b.shape[0], 2, 128), np.float64)
    n = b.shape[0]
    ql = b[:, 0:128].reshape(n, 2, 64).astype(np.int32)
    qh = b[:, 128:192].reshape(n, 2, 32).astype(np.int32)
    sc = b[:, 192:208].copy().view(np.int8).reshape(n, 2, 8).astype(np.float32)
    d = b[:, 208:210].copy().view(np.float16).astype(np.float32)[:, 0]
    is_ = np.arange(32) // 16
    out = np.empty((n, 2, 128), np.float16)
    for q, (lo, shift_q, nib_hi, sc_off) in enumerate(
            [(0, 0, False, 0), (32, 2, False, 2), (0, 4, True, 4), (32, 6, True, 6)]):
        low = ql[:, :, lo:lo + 32]
        low = (low >> 4) if nib_hi else (low & 0xF)
        val = ((low | (((qh >> shift_q) & 3) << 4)) - 32).astype(np.float64)
        scale = (d[:, None, None] * sc[:, :, is_ + sc_off]).astype(np.float16).astype(np.float64)
        out[:, :, 32 * q:32 * q + 32] = (scale * val).astype(np.float16)
    return out.reshape(-1)


def quant_linear(weight_bytes, qtype, x, operands="fp32"):
    """out[token][feature] in double for a Q4_K or Q6_K weight [features, row bytes];
    operands as in q4k_linear."""
    n = weight_bytes.shape[0]
    if operands == "fp32":
        f = q4k_dequantize if qtype == Q4_K_TYPE else q6k_dequantize
        xx = np.asarray(x, np.float32).astype(np.float64)
    else:
        f = q4k_dequantize_f16_operands if qtype == Q4_K_TYPE else q6k_dequantize_f16_operands
        xx = np.asarray(x, np.float32).astype(np.float16).astype(np.float64)
    return xx @ f(weight_bytes).reshape(n, -1).astype(np.float64).T


def q6k_random_blocks(rng, n_blocks, d_max=0.002):
    b = rng.integers(0, 256, (n_blocks, Q6_K_BLOCK_BYTES), dtype=np.uint8)
    d = (rng.random(n_blocks) * d_max + d_max * 0.1).astype(np.float16)
    b[:, 208:210] = d.view(np.uint8).reshape(-1, 2)
    return b


def dequantize_rows(weight_bytes, qtype):
    """[rows, row_bytes] quantised rows -> [rows, K] fp32."""
    rows = weight_bytes.shape[0]
    f = q4k_dequantize if qtype == Q4_K_TYPE else q6k_dequantize
    return f(weight_bytes).reshape(rows, -1)


def gather_last_rows(src, branch_offsets):
    """out[b] = src[branch_offsets[b+1] - 1]  (src/q3_forward.cu:553-564)."""
    idx = np.asarray(branch_offsets[1:], np.int64) - 1
    return np.asarray(src)[idx]


def candidate_logits_batched(hidden_per_branch, weight_bytes, qtype, candidate_ids,
                             candidate_count):
    """logits[b*K + c] = dot(row(candidate_ids[b*K + c]), hidden_per_branch[b]) in
    double (the reference sums fp32 products in a tree: src/q3_forward.cu:566-607)."""
    ids = np.asarray(candidate_ids, np.int64)
    w = dequantize_rows(weight_bytes[ids], qtype).astype(np.float64)
    h = np.asarray(hidden_per_branch, np.float32).astype(np.float64)
    b = np.arange(ids.size) // candidate_count
    return np.einsum("ik,ik->i", w, h[b])


# --------------------------------------------------------------------------
# The reference's small-batch arithmetic: 8-bit activations, integer dots
# --------------------------------------------------------------------------
def q8_1_quantize(x):
    """Per 32 elements: d = max|x| / 127 (fp32), q = round-half-away(x / d) as
    int8 (0 when the block is all zero); the scale that enters the dot product
    is d rounded to f16 (it is stored as a half next to the block sum). The
    reference does this before its MMVQ / MMQ kernels (src/q3_q4_linear.h:6-14;
    it vendors the ggml quantiser for it). Returns (q int32 [tokens, K],
    d8 float64 [tokens, K/32])."""
    x = np.asarray(x, np.float32)
    t, k = x.shape
    xb = x.reshape(t, k // 32, 32)
    amax = np.abs(xb).max(axis=2)
    d = (amax / np.float32(127.0)).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        r = (xb / d[:, :, None]).astype(np.float32)
    q = np.where(amax[:, :, None] == 0, 0, np.sign(r) * np.floor(np.abs(r) + np.float32(0.5)))
    return (q.reshape(t, k).astype(np.int32),
            d.astype(np.float16).astype(np.float64))


def q4k_linear_q8(weight_bytes, x):
    """out[token][feature] = sum over blocks of
         d * sum_i d8_i * sc_i * (q4 . q8)_i  -  dmin * sum_i d8_i * m_i * sum(q8)_i
    over the eight 32-element sub-blocks i, in double: the arithmetic of the
    reference's Q4_K x Q8_1 dot product, exact in the integers."""
    n = weight_bytes.shape[0]
    d, dmin, sc, mn, q4 = q4k_fields(weight_bytes)            # per block
    nb = d.shape[0] // n                                      # blocks per row
    q8, d8 = q8_1_quantize(x)
    t = q8.shape[0]
    q4 = q4.reshape(n, nb, 8, 32).astype(np.int64)
    q8 = q8.reshape(t, nb, 8, 32).astype(np.int64)
    d8 = d8.reshape(t, nb, 8)
    dots = np.einsum("nbie,tbie->tnbi", q4, q8)               # exact integers
    sums = q8.sum(axis=3)                                     # [t, nb, 8]
    scd = sc.reshape(n, nb, 8).astype(np.float64)
    mnd = mn.reshape(n, nb, 8).astype(np.float64)
    dd = d.reshape(n, nb).astype(np.float64)
    dm = dmin.reshape(n, nb).astype(np.float64)
    part_d = np.einsum("tnbi,nbi,tbi->tnb", dots.astype(np.float64), scd, d8)
    part_m = np.einsum("tbi,nbi,tbi->tnb", sums.astype(np.float64), mnd, d8)
    return (part_d * dd[None] - part_m * dm[None]).sum(axis=2)


def linear_error_metrics(got, ref):
    """The figures the reference's test prints and checks."""
    got = np.asarray(got, np.float64).reshape(-1)
    ref = np.asarray(ref, np.float64).reshape(-1)
    e = got - ref
    return {
        "max_abs": float(np.abs(e).max()),
        "rel_l2": float(np.sqrt((e * e).sum()) / (np.sqrt((ref * ref).sum()) + 1e-30)),
        "cos": float((got * ref).sum() /
                     (np.sqrt((got * got).sum()) * np.sqrt((ref * ref).sum()) + 1e-30)),
    }
