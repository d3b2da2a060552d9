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
