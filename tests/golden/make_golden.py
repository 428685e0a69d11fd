"""Regenerates tests/golden/qmatmul_small.npz from the CPU oracle.

    python tests/golden/make_golden.py

The reference (Rust) cannot be built or imported where this repository is developed, so these
vectors are outputs of the oracle restatement, frozen: once committed they detect any later
drift of the oracle, the NumPy twin, the library's host quantizer and the CUDA kernels, all
of which are compared against them.  Inputs are seeded; shapes include a ragged K and a
partial codebook block.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle as orc  # noqa: E402
from helpers import normal  # noqa: E402

CASES = [  # name, M, K, N, sigma
    ("aligned", 3, 64, 16, 0.02),
    ("ragged", 2, 45, 7, 0.02),
    ("wide", 1, 256, 40, 0.015),
]


def main():
    out = {}
    for ci, (name, m, k, n, sigma) in enumerate(CASES):
        w_kn = normal(100 + ci, (k, n), sigma)
        x = normal(200 + ci, (m, k), 1.0)
        bias = normal(300 + ci, (n,), 0.01)
        out[f"{name}/w_kn"], out[f"{name}/x"], out[f"{name}/bias"] = w_kn, x, bias
        for fmt, fname in orc.FMT_NAMES.items():
            q = orc.quantize_kn(fmt, w_kn)
            p = f"{name}/{fname}"
            out[p + "/words"] = q.words
            out[p + "/scales"] = q.scales
            out[p + "/zeros"] = q.zeros
            if q.codebook is not None:
                out[p + "/codebook"] = q.codebook
            out[p + "/dequant"] = orc.dequant(q)
            out[p + "/out_plain"] = orc.qmatmul(q, x)
            out[p + "/out_bias_gelu"] = orc.qmatmul(q, x, bias, orc.EPI_GELU)
            out[p + "/out_silu"] = orc.qmatmul(q, x, None, orc.EPI_SILU)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "qmatmul_small.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
