"""Writes tests/golden/ref_cublaslt.json: outputs of the REFERENCE's own code on seeded inputs.

The reference's cuBLASLt submission (sub_cub.py:48-143,165-169), compiled from its own source
by ``oracle/build_ref.py``, is run on a B200 on the inputs ``nvfp4_gemm_b200.inputs`` generates
for config 0 (128 x 256 x 256), the reference's test shapes (task.yml:41-51) and its
benchmark shapes (task.yml:53-56).  For each case the file keeps the SHA-256 of the fp16 output
(negative zeros folded into +0 first), 64 sampled values as bit patterns, and the digest of ``a``
so that a drift of the input generator is told apart from a drift of the arithmetic.  These are
vectors produced by the reference; ``tests/test_oracle_cpu.py`` holds the CPU oracle to them.

Needs a GPU:   python tests/golden/make_ref_golden.py [--out tests/golden/ref_cublaslt.json]
"""
import argparse
import hashlib
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

CASES = [  # (m, n, k, l, seed)
    (128, 256, 256, 1, 1111),                                   # config 0, task.yml:42
    (128, 1536, 7168, 1, 1111), (128, 3072, 1536, 1, 1111), (256, 7168, 256, 1, 1111), (256, 7168, 2048, 1, 1111),
    (2304, 4608, 7168, 1, 1111), (384, 7168, 2304, 1, 1111), (512, 512, 7168, 1, 1111), (512, 4096, 512, 1, 1111),
    (512, 1536, 7168, 1, 1111),                                 # task.yml:43-51
    (128, 7168, 16384, 1, 1111), (128, 4096, 7168, 1, 1111), (128, 7168, 2048, 1, 1111),   # task.yml:54-56
    (128, 256, 256, 1, 7), (256, 512, 2048, 1, 3),              # further seeds
]


def canonical_bits(c: np.ndarray) -> np.ndarray:
    """fp16 bit patterns in [m, n, l] index order with -0 folded into +0."""
    bits = np.ascontiguousarray(c).view(np.uint16).copy()
    bits[bits == 0x8000] = 0
    return bits


def digest(c: np.ndarray) -> str:
    return hashlib.sha256(canonical_bits(c).tobytes()).hexdigest()


def sample_indices(size: int):
    return [int(i) for i in np.linspace(0, size - 1, 64).astype(np.int64)]


def main():
    import torch

    from nvfp4_gemm_b200.inputs import generate_input
    from oracle import build_ref

    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_cublaslt.json"))
    args = ap.parse_args()
    reference_kernel = build_ref.load()
    records = []
    for (m, n, k, l, seed) in CASES:
        data = generate_input(m, n, k, l, seed, device="cuda")
        data[6].view(torch.int16).fill_(0x7fff)
        out = reference_kernel(data)
        torch.cuda.synchronize()
        c = out.cpu().numpy()
        flat = canonical_bits(c).reshape(-1)
        a_bytes = np.ascontiguousarray(data[0].view(torch.uint8).cpu().numpy()).tobytes()
        records.append(dict(m=m, n=n, k=k, l=l, seed=seed, a_sha256=hashlib.sha256(a_bytes).hexdigest(), c_sha256=digest(c),
                            samples=[[i, int(flat[i])] for i in sample_indices(flat.size)]))
        print(f"{m}x{n}x{k}x{l} seed {seed}: {records[-1]['c_sha256'][:16]}", flush=True)
    with open(args.out, "w") as f:
        json.dump({"generator": "tests/golden/make_ref_golden.py",
                   "producer": "reference sub_cub.py custom_kernel (cuBLASLt block-scaled FP4), NVIDIA B200",
                   "torch": torch.__version__, "cuda": torch.version.cuda, "cases": records}, f, indent=1)


if __name__ == "__main__":
    main()
