"""Writes tests/golden/golden.json: digests and sample values of the oracle's output on seeded
inputs.  The reference holds no golden vectors for this path, so these are regression pins of
the oracle itself (which the known-answer tests anchor), not vectors from the reference.

Run from the repository root:  python tests/golden/make_golden.py
"""
import hashlib
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from nvfp4_gemm_b200.inputs import generate_input  # noqa: E402
from oracle import nvfp4_oracle as O  # noqa: E402

CASES = [
    dict(m=128, n=256, k=256, l=1, seed=1111),      # the CPU-runnable configuration
    dict(m=128, n=128, k=1024, l=2, seed=1111),
    dict(m=64, n=1, k=512, l=2, seed=1111),         # GEMV form
    dict(m=32, n=128, k=16384, l=1, seed=1111),     # long K: values near the fp16 limit
]


def main():
    out = []
    for case in CASES:
        data = generate_input(case["m"], case["n"], case["k"], case["l"], case["seed"], device="cpu")
        a, b, sfa, sfb = O.tensors_to_numpy(data)
        c = O.ref_gemm(a, b, sfa, sfb, accumulate="f64")
        flat = c.reshape(-1).view(np.uint16)
        step = max(1, flat.size // 16)
        rec = dict(case)
        rec["a_sha256"] = hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()
        rec["c_sha256"] = hashlib.sha256(np.ascontiguousarray(c).tobytes()).hexdigest()
        rec["samples"] = [[int(i), int(flat[i])] for i in range(0, flat.size, step)]
        out.append(rec)
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden.json"), "w") as f:
        json.dump({"generator": "tests/golden/make_golden.py", "cases": out}, f, indent=1)


if __name__ == "__main__":
    main()
