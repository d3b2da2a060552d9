"""Generate the Q4_K dequantisation fixture from the reference's own C code.

    make -C oracle refquant        # compiles the reference's src/q3_quant.c as it lies
    python tests/golden/make_golden_q4k.py

Writes tests/golden/q4k_dequant_ref.npz: a handful of 144-byte Q4_K blocks and
the fp32 values the reference's q3_quant_dequantize_row returns for them
(src/q3_quant.c:105-129). Blocks: 6 with every byte random (all scale/min bit
patterns, including the 6-bit fields split over two bytes), 1 all zero, 1 with
all fields at their maximum. The reference's test applies one hand-derived
check to its own oracle (tests/test_q3_q4_linear.cu:95-107: first nibble =
d*(scales[0]&63)*(qs[0]&15) - dmin*(scales[4]&63)); the same check is repeated
in tests/test_oracle_golden.py on these blocks.
"""
import ctypes
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def main():
    lib = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libq3quant_ref.so"))
    lib.q3_quant_dequantize_row.restype = ctypes.c_bool
    lib.q3_quant_dequantize_row.argtypes = [ctypes.c_uint32, ctypes.c_void_p, ctypes.c_size_t,
                                            ctypes.c_void_p, ctypes.c_size_t,
                                            ctypes.c_char_p, ctypes.c_size_t]
    rng = np.random.default_rng(20240)
    blocks = rng.integers(0, 256, (8, 144), dtype=np.uint8)
    # finite, moderate f16 scales (random exponent bytes would give inf/nan)
    for i in range(6):
        blocks[i, 0:2] = np.asarray([rng.random() * 0.01 + 1e-4], np.float16).view(np.uint8)
        blocks[i, 2:4] = np.asarray([rng.random() * 0.05], np.float16).view(np.uint8)
    blocks[6] = 0
    blocks[7] = 255
    blocks[7, 0:2] = np.asarray([0.5], np.float16).view(np.uint8)
    blocks[7, 2:4] = np.asarray([2.0], np.float16).view(np.uint8)
    out = np.zeros(8 * 256, np.float32)
    err = ctypes.create_string_buffer(256)
    ok = lib.q3_quant_dequantize_row(12, blocks.ctypes.data, 8, out.ctypes.data, out.size,
                                     err, 256)
    assert ok, err.value
    path = os.path.join(HERE, "q4k_dequant_ref.npz")
    np.savez(path, blocks=blocks, values=out)
    print(path, os.path.getsize(path), "bytes")

    # Q6_K (210-byte blocks; ref: src/q3_quant.c:78-103): 5 random + all-zero + all-ones
    b6 = rng.integers(0, 256, (7, 210), dtype=np.uint8)
    for i in range(5):
        b6[i, 208:210] = np.asarray([rng.random() * 0.01 + 1e-4], np.float16).view(np.uint8)
    b6[5] = 0
    b6[6] = 255
    b6[6, 208:210] = np.asarray([0.25], np.float16).view(np.uint8)
    out6 = np.zeros(7 * 256, np.float32)
    ok = lib.q3_quant_dequantize_row(14, b6.ctypes.data, 7, out6.ctypes.data, out6.size, err, 256)
    assert ok, err.value
    path = os.path.join(HERE, "q6k_dequant_ref.npz")
    np.savez(path, blocks=b6, values=out6)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
