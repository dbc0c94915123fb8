"""The oracle against hand-computable answers, independent decoders and its own C restatement."""
import json
import os

import numpy as np
import pytest
import torch

from nvfp4_gemm_b200.inputs import generate_input

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_e2m1_table_matches_format_definition(oracle):
    # sign | 2-bit exponent (bias 1) | 1-bit mantissa
    for code in range(16):
        s, e, m = code >> 3, (code >> 1) & 3, code & 1
        v = (m * 0.5) if e == 0 else (1 + m * 0.5) * 2.0 ** (e - 1)
        assert oracle.E2M1_LUT[code] == (-v if s else v)


def test_e4m3_decode_matches_torch(oracle):
    t = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).to(torch.float32).numpy()
    mine = oracle.E4M3_LUT
    assert np.array_equal(np.isnan(t), np.isnan(mine))
    ok = ~np.isnan(t)
    assert np.array_equal(t[ok], mine[ok])
    # the scale bytes of the synthetic distribution: 2^u, u in [-3, 3]
    for u in range(-3, 4):
        assert mine[(u + 7) << 3] == 2.0 ** u


def test_known_answer_single_block(oracle):
    # one row each, K = 64: A = all 1.5 (code 3), B = all -2 (code 0xC), scales 2 and 0.5
    K = 64
    a = np.full((1, K // 2, 1), 0x33, np.uint8)
    b = np.full((1, K // 2, 1), 0xCC, np.uint8)
    sfa = np.full((1, K // 16, 1), (1 + 7) << 3, np.uint8)
    sfb = np.full((1, K // 16, 1), (-1 + 7) << 3, np.uint8)
    c = oracle.ref_gemm(a, b, sfa, sfb)
    assert c[0, 0, 0] == np.float16(64 * 1.5 * -2.0 * 2 * 0.5)
    assert oracle.ref_gemm_c(a, b, sfa, sfb)[0, 0, 0] == c[0, 0, 0]


def test_known_answer_nibble_order_and_block_scales(oracle):
    # element k of A is non-zero only at k = 17 (high nibble of byte 8, second scale block)
    K = 64
    a = np.zeros((1, K // 2, 1), np.uint8)
    a[0, 8, 0] = 0x70          # high nibble = code 7 = 6.0 at k = 17
    b = np.zeros((1, K // 2, 1), np.uint8)
    b[0, 8, 0] = 0x21          # k = 16 -> 0.5, k = 17 -> 1.0
    sfa = np.full((1, 4, 1), 0x38, np.uint8)
    sfb = np.full((1, 4, 1), 0x38, np.uint8)
    sfa[0, 1, 0] = (2 + 7) << 3    # block 1 scaled by 4
    sfa[0, 0, 0] = (3 + 7) << 3    # block 0 scale must not matter
    assert oracle.ref_gemm(a, b, sfa, sfb)[0, 0, 0] == np.float16(6.0 * 1.0 * 4.0)
    assert oracle.ref_gemm_c(a, b, sfa, sfb)[0, 0, 0] == np.float16(24.0)


def test_fp16_overflow_goes_to_inf(oracle):
    K = 1024
    a = np.full((1, K // 2, 1), 0x77, np.uint8)   # 6.0
    b = np.full((1, K // 2, 1), 0x77, np.uint8)
    sf = np.full((1, K // 16, 1), (3 + 7) << 3, np.uint8)  # 8
    c = oracle.ref_gemm(a, b, sf, sf)
    assert np.isposinf(c[0, 0, 0])
    assert np.isposinf(oracle.ref_gemm_c(a, b, sf, sf)[0, 0, 0])
    b[:] = 0xFF                                   # -6.0
    assert np.isneginf(oracle.ref_gemm_c(a, b, sf, sf)[0, 0, 0])


def test_permuted_layout_formula(oracle):
    # atoms of 512 bytes: 32 rows x (4 row-groups x 4 scales), K-major inside a 128-row block
    rows, cols = 256, 8
    sf = np.arange(rows * cols, dtype=np.uint32).reshape(rows, cols, 1)
    flat = oracle.permute_sf((sf % 251).astype(np.uint8))
    assert flat.size == 2 * 2 * 512
    for (r, c) in [(0, 0), (1, 0), (31, 3), (32, 0), (127, 3), (128, 0), (200, 5), (255, 7)]:
        off = (r // 128) * 2 * 512 + (c // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + (c % 4)
        assert flat[off] == (r * cols + c) % 251
    back = oracle.unpermute_sf(flat, rows, cols, 1)
    assert np.array_equal(back[:, :, 0], (sf[:, :, 0] % 251).astype(np.uint8))


def test_generator_matches_contract(oracle):
    m, n, k, l = 128, 256, 256, 2
    a, b, sfa, sfb, sfap, sfbp, c = generate_input(m, n, k, l, 1111, device="cpu")
    assert a.shape == (m, k // 2, l) and a.stride() == (k // 2, 1, m * k // 2)
    assert b.shape == (n, k // 2, l) and sfa.shape == (m, k // 16, l) and sfb.shape == (n, k // 16, l)
    assert sfap.shape == (32, 4, 1, 4, k // 64, l)
    assert sfap.stride() == (16, 4, (k // 64) * 512, 1, 512, (k // 64) * 512)
    assert sfbp.shape == (32, 4, 2, 4, k // 64, l)
    assert c.shape == (m, n, l) and c.stride() == (n, 1, m * n) and c.dtype == torch.float16
    # the permuted tensor's memory is the oracle's permutation of the plain one
    for plain, perm in ((sfa, sfap), (sfb, sfbp)):
        mem = torch.as_strided(perm.view(torch.uint8), (perm.numel(),), (1,)).numpy()
        assert np.array_equal(mem, oracle.permute_sf(plain.view(torch.uint8).numpy()))
    # distribution: scales are 2^u, u in [-3, 3]
    vals = set(np.unique(sfa.view(torch.uint8).numpy()).tolist())
    assert vals <= {(u + 7) << 3 for u in range(-3, 4)}


@pytest.mark.parametrize("shape", [(128, 256, 256, 1), (64, 128, 512, 2), (130, 192, 1024, 1)])
def test_c_oracle_equals_numpy_oracle(oracle, shape):
    m, n, k, l = shape
    data = generate_input(m, n, k, l, 7, device="cpu")
    a, b, sfa, sfb = oracle.tensors_to_numpy(data)
    ref = oracle.ref_gemm(a, b, sfa, sfb)
    assert np.array_equal(ref.view(np.uint16), oracle.ref_gemm_c(a, b, sfa, sfb).view(np.uint16))
    # reading the permuted scales gives the same answer
    pa, pb = oracle.permute_sf(sfa), oracle.permute_sf(sfb)
    assert np.array_equal(ref.view(np.uint16), oracle.ref_gemm_c(a, b, pa, pb, permuted_sf=True).view(np.uint16))
    assert np.array_equal(ref.view(np.uint16), oracle.ref_gemm_from_permuted(a, b, pa, pb).view(np.uint16))


def test_fp32_accumulation_is_exact_for_the_configured_distribution(oracle):
    data = generate_input(64, 64, 16384, 1, 1111, device="cpu")
    a, b, sfa, sfb = oracle.tensors_to_numpy(data)
    c32 = oracle.ref_gemm(a, b, sfa, sfb)
    c64 = oracle.ref_gemm(a, b, sfa, sfb, accumulate="f64")
    assert np.array_equal(c32.view(np.uint16), c64.view(np.uint16))


def test_general_scales_within_tolerance_of_f64(oracle):
    # arbitrary e4m3 scales (not powers of two): fp32 accumulation is no longer exact but stays
    # far inside the operator's tolerance
    rng = np.random.default_rng(3)
    m, n, k = 32, 48, 2048
    a = rng.integers(0, 256, (m, k // 2, 1), dtype=np.uint8)
    b = rng.integers(0, 256, (n, k // 2, 1), dtype=np.uint8)
    sfa = rng.integers(0x28, 0x48, (m, k // 16, 1), dtype=np.uint8)
    sfb = rng.integers(0x28, 0x48, (n, k // 16, 1), dtype=np.uint8)
    c32 = oracle.ref_gemm_c(a, b, sfa, sfb).astype(np.float32)
    c64 = oracle.ref_gemm(a, b, sfa, sfb, accumulate="f64").astype(np.float32)
    np.testing.assert_allclose(c32, c64, rtol=1e-3, atol=1e-3)


def test_golden_vectors(oracle):
    with open(os.path.join(GOLDEN, "golden.json")) as f:
        golden = json.load(f)
    for case in golden["cases"]:
        data = generate_input(case["m"], case["n"], case["k"], case["l"], case["seed"], device="cpu")
        a, b, sfa, sfb = oracle.tensors_to_numpy(data)
        c = oracle.ref_gemm_c(a, b, sfa, sfb)
        import hashlib
        assert hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest() == case["a_sha256"], "generator drifted"
        assert hashlib.sha256(np.ascontiguousarray(c).tobytes()).hexdigest() == case["c_sha256"], case
        flat = c.reshape(-1)
        for idx, bits in case["samples"]:
            assert int(flat.view(np.uint16)[idx]) == bits


def _reference_cases():
    with open(os.path.join(GOLDEN, "ref_cublaslt.json")) as f:
        return json.load(f)["cases"]


@pytest.mark.parametrize("case", _reference_cases(), ids=lambda c: f"{c['m']}x{c['n']}x{c['k']}x{c['l']}-seed{c['seed']}")
def test_oracle_reproduces_the_reference_submissions_outputs(oracle, case):
    """tests/golden/ref_cublaslt.json holds outputs of the reference's own cuBLASLt submission
    (sub_cub.py:48-143,165-169) run on a B200 on this repository's seeded inputs
    (tests/golden/make_ref_golden.py): the CPU oracle must give the same fp16 bits."""
    import hashlib
    m, n, k, l = case["m"], case["n"], case["k"], case["l"]
    data = generate_input(m, n, k, l, case["seed"], device="cpu")
    a, b, sfa, sfb = oracle.tensors_to_numpy(data)
    assert hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest() == case["a_sha256"], "input generator drifted"
    if 2.0 * m * n * k > 4e10:
        # the full oracle would take too long here: the rows the fixture's samples fall into
        idx = np.array([i for i, _ in case["samples"]], dtype=np.int64)
        rows = np.unique(idx // (n * l))
        c = oracle.ref_gemm_c(a[rows], b, sfa[rows], sfb)
        bits = np.ascontiguousarray(c).view(np.uint16).copy()
        bits[bits == 0x8000] = 0
        pos = {int(r): i for i, r in enumerate(rows)}
        for i, want in case["samples"]:
            r, rest = divmod(i, n * l)
            assert int(bits[pos[r]].reshape(-1)[rest]) == want, (case["m"], case["n"], case["k"], i)
        return
    c = oracle.ref_gemm_c(a, b, sfa, sfb)
    bits = np.ascontiguousarray(c).view(np.uint16).copy()
    bits[bits == 0x8000] = 0          # the fixture folds -0 into +0
    flat = bits.reshape(-1)
    for i, want in case["samples"]:
        assert int(flat[i]) == want, (m, n, k, i)
    assert hashlib.sha256(bits.tobytes()).hexdigest() == case["c_sha256"]


def test_quantizer_roundtrip(oracle):
    rng = np.random.default_rng(0)
    x = rng.standard_normal((8, 256)).astype(np.float32) * 3
    packed, sf = oracle.quantize_rows(x)
    back = oracle.dequantize(packed, sf)
    # e2m1 has a relative step of at most 1/3 between neighbours; block max maps near 6
    assert np.all(np.abs(back - x) <= np.maximum(np.abs(x) * 0.34, 0.3 * np.abs(x).reshape(8, 16, 16).max(-1).repeat(16, -1)))
    # a block whose maximum is 6 x (a representable scale) is reproduced exactly
    vals = oracle.E2M1_LUT[rng.integers(0, 16, (4, 64))] * np.float32(0.25)
    vals[:, ::16] = 6 * 0.25
    p2, s2 = oracle.quantize_rows(vals)
    assert np.array_equal(oracle.dequantize(p2, s2), vals)
