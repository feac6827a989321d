"""Regenerates the frozen vectors under tests/golden/ from the CPU oracle.

The reference is Rust and cannot be run where this repository is built, so these files freeze
the oracle's output AFTER the oracle passed the reference's known-answer tests
(tests/test_oracle_golden.py). They guard against later drift of the oracle itself.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

import fixtures as F  # noqa: E402
from oracle import oracle as O  # noqa: E402


def main():
    scales = [8, 16, 24, 32, 40, 48, 56, 64, 72, 80, 88, 96]
    qs = bytes((i * 3) % 256 for i in range(128))
    raw = F.f16_bytes(0.1) + F.f16_bytes(0.05) + bytes(scales) + qs
    d = O.dequantize(np.frombuffer(raw, dtype=np.uint8), O.Q4K, 256)
    np.save(os.path.join(HERE, "q4k_scale_fixture.npy"), d)
    # dequantised conformance fixtures at their smallest shapes + a GEMV of each
    out = {}
    for name, ty, (n, k), rows, _tol, seed in F.CONFORMANCE_CASES[:6]:
        raw = F.GEN[ty]((n, k))
        out[name + "_deq"] = O.dequantize(raw, ty, n * k)
        x = F.deterministic_input((rows, k), seed)
        O.set_threads(1)
        out[name + "_y"] = O.q_mat_mul(x, raw, ty, n, k)
        O.set_threads(0)
    np.savez(os.path.join(HERE, "conformance_small.npz"), **out)


if __name__ == "__main__":
    main()
