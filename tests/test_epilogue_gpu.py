"""GPU parity of the GEMM's extended epilogue -- bias, activation, NVFP4 re-quantised output --
against the CPU oracle, through the C ABI.  The reference writes the plain fp16 cast only
(sub_cub.py:98-104); the definition checked here is oracle.ref_epilogue / ref_requantize."""
import numpy as np
import pytest
import torch

from helpers import assert_bit_exact, assert_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def sub(lib):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from nvfp4_gemm_b200 import submission
    return submission


def _bias(n, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(n, generator=g) * 64).half()


# (shape, kernel configuration): CTA-pair 256-wide and 128-wide tiles, one-CTA tiles, stream-K with
# shared tiles (grid), cluster split-K, ragged M, batches
CASES = [
    ((512, 1024, 1024, 1), dict()),
    ((300, 768, 1536, 2), dict()),
    ((384, 640, 2048, 1), dict()),                    # n not a multiple of 256: 128-wide pair tiles
    ((128, 512, 4096, 1), dict(split_k=1, grid=6)),   # shared tiles: partials summed, then the epilogue
    ((100, 1024, 4096, 1), dict()),                   # decode shape: cluster split-K
    ((256, 512, 1024, 1), dict(cta_group=1, tile_n=256)),
    ((640, 512, 2048, 1), dict(grid=4)),
]


@pytest.mark.parametrize("activation", ["none", "relu"])
@pytest.mark.parametrize("shape,kw", CASES)
def test_bias_and_activation_fp16_bit_exact(sub, oracle, shape, kw, activation):
    from nvfp4_gemm_b200.inputs import generate_input
    m, n, k, l = shape
    data = generate_input(m, n, k, l, 31)
    bias = _bias(n, 5)
    data[6].view(torch.int16).fill_(0x7fff)
    out = sub.gemm_epilogue(data, bias=bias.cuda(), activation=activation, **kw)
    sub.check_status()
    a, b, sfa, sfb = oracle.tensors_to_numpy(data)
    exp = oracle.ref_epilogue(oracle.ref_gemm_f32(a, b, sfa, sfb), bias.numpy(), activation)
    assert_bit_exact(out, exp, what=f"{shape} {activation} {sub.last_kernel()}")


@pytest.mark.parametrize("shape,kw", CASES)
def test_nvfp4_output_equals_quantised_fp16_output(sub, oracle, shape, kw):
    """Packed values and scales (plain and permuted) against the oracle; and the fused result is
    what nvfp4_quantize makes of the unfused fp16 output."""
    from nvfp4_gemm_b200.inputs import generate_input
    m, n, k, l = shape
    data = generate_input(m, n, k, l, 32)
    bias = _bias(n, 6)
    packed, sf, sf_perm = sub.gemm_epilogue(data[:6] + (None,), bias=bias.cuda(), activation="relu", nvfp4_out=True, **kw)
    sub.check_status()
    a, b, sfa, sfb = oracle.tensors_to_numpy(data)
    c16 = oracle.ref_epilogue(oracle.ref_gemm_f32(a, b, sfa, sfb), bias.numpy(), "relu")
    exp_packed, exp_sf = oracle.ref_requantize(c16)
    got_packed = packed.view(torch.uint8).cpu().numpy()
    got_sf = sf.view(torch.uint8).cpu().numpy()
    assert np.array_equal(got_sf, exp_sf), f"{shape}: scales differ ({sub.last_kernel()})"
    assert np.array_equal(got_packed, exp_packed), f"{shape}: packed values differ ({sub.last_kernel()})"
    # the permuted copy says the same as the plain one, padding rows are zero
    flat = torch.as_strided(sf_perm.view(torch.uint8), (sf_perm.numel(),), (1,)).cpu().numpy()
    assert np.array_equal(flat, oracle.permute_sf(exp_sf).reshape(-1))


def test_fused_output_feeds_the_next_gemm(sub, oracle):
    """Two layers: the first GEMM's NVFP4 output is the second GEMM's a / sfa / sfa_permuted."""
    from nvfp4_gemm_b200.inputs import generate_input
    m, n1, k1, n2 = 256, 1024, 2048, 512
    d1 = generate_input(m, n1, k1, 1, 41)
    d2 = generate_input(m, n2, n1, 1, 42)               # only its b / sfb are used
    packed, sf, sf_perm = sub.gemm_epilogue(d1[:6] + (None,), activation="relu", nvfp4_out=True)
    out = sub.custom_kernel((packed, d2[1], sf, d2[3], sf_perm, d2[5], d2[6]))
    sub.check_status()
    a, b, sfa, sfb = oracle.tensors_to_numpy(d1)
    p1, s1 = oracle.ref_requantize(oracle.ref_epilogue(oracle.ref_gemm_f32(a, b, sfa, sfb), None, "relu"))
    _, b2, _, sfb2 = oracle.tensors_to_numpy(d2)
    exp = oracle.ref_gemm(p1, b2, s1, sfb2, accumulate="f64")
    # arbitrary scales now: the operator's stated tolerance
    assert_close(out, exp, rtol=1e-3, atol=1e-3, what="two fused layers")


def test_silu_within_tolerance(sub, oracle):
    from nvfp4_gemm_b200.inputs import generate_input
    m, n, k, l = 256, 512, 256, 1
    data = generate_input(m, n, k, l, 33)
    out = sub.gemm_epilogue(data, activation="silu")
    sub.check_status()
    a, b, sfa, sfb = oracle.tensors_to_numpy(data)
    exp = oracle.ref_epilogue(oracle.ref_gemm_f32(a, b, sfa, sfb), None, "silu")
    assert_close(out, exp, rtol=2e-3, atol=2e-3, what="silu")


def test_epilogue_argument_checks(sub, lib):
    from nvfp4_gemm_b200 import _lib
    from nvfp4_gemm_b200.inputs import generate_input
    data = generate_input(128, 256, 256, 1, 1)
    p = sub.make_problem(data)
    epi = _lib.Epilogue()
    epi.activation = 7
    assert lib.nvfp4_gemm_epilogue(p, None, epi, None) == _lib.NVFP4_ERR_INVALID_ARGUMENT
    epi.activation, epi.output = 0, _lib.OUT_NVFP4        # no output buffers given
    assert lib.nvfp4_gemm_epilogue(p, None, epi, None) == _lib.NVFP4_ERR_INVALID_ARGUMENT
    assert lib.nvfp4_gemm_epilogue(p, None, None, None) == _lib.NVFP4_ERR_INVALID_ARGUMENT
