"""Golden vectors from the reference's OWN CUDA kernels.

oracle/_ref/libq3ref.so is the reference's src/q3_forward.cu compiled for
sm_100a (oracle/Makefile, target `ref`). This script runs its primitives
(q3_cuda_rms_norm, q3_cuda_rope[_positions], q3_cuda_attention,
q3_cuda_attention_segmented) on a GPU over the seeded cases of tests/_cases.py
and stores a subset of the results, so that the CPU-only test suite can pin the
oracle against the reference itself. Needs a GPU:

    python tests/golden/make_golden_refkernels.py [output_dir]

Outputs refkernels_case_*.npz (default: this directory).
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(HERE)), "oracle"))
import _cases  # noqa: E402
import _gpu_harness as harness  # noqa: E402
import q3_oracle  # noqa: E402


def main():
    out_dir = sys.argv[1] if len(sys.argv) > 1 else HERE
    L = harness.ref_lib()
    assert L is not None, "build oracle/_ref first (make -C oracle ref)"
    for name in _cases.GOLDEN_CASES:
        case = _cases.make_case(name)
        r = harness.run_case_fp32_surface(L, case, q3_oracle.inv_freq(case.theta, case.D))
        rows = np.asarray(case.golden_rows, np.int64)
        heads = np.asarray(case.golden_heads, np.int64)
        kvh = np.unique(heads // (case.H // case.Hkv))
        path = os.path.join(out_dir, "refkernels_case_%s.npz" % name)
        np.savez(path, rows=rows, heads=heads, kv_heads=kvh,
                 q2=r["q2"][rows][:, heads], k2=r["k2"][rows][:, kvh],
                 out=r["out"][rows][:, heads],
                 input_sha256=np.array(case.input_sha256()),
                 built=np.array("src/q3_forward.cu, nvcc -O3 --use_fast_math, sm_100a, B200"))
        print(name, "->", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
