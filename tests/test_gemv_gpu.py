"""GPU parity of the CUDA-core GEMV against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from helpers import assert_bit_exact, assert_close, expected_fp16

pytestmark = pytest.mark.gpu

# task_gemv.yml:41-51, plus ragged M / K not a multiple of the unrolled stride / single row
SHAPES = [(128, 256, 1), (128, 1536, 1), (128, 3072, 1), (256, 7168, 1), (2432, 4608, 2), (384, 7168, 2), (512, 512, 2),
          (512, 4096, 2), (512, 1536, 2), (1, 64, 1), (131, 1600, 3), (7, 192, 2)]


@pytest.fixture(scope="module")
def sub(lib):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from nvfp4_gemm_b200 import submission
    return submission


@pytest.mark.parametrize("shape", SHAPES)
def test_gemv_matches_oracle_bit_exact(sub, oracle, shape):
    from nvfp4_gemm_b200.inputs import generate_input
    m, k, l = shape
    data = generate_input(m, 1, k, l, 1111)
    data[6].view(torch.int16).fill_(0x7fff)
    out = sub.custom_kernel(data)
    torch.cuda.synchronize()
    assert sub.last_kernel().startswith("gemv")
    assert_bit_exact(out, expected_fp16(oracle, data), what=f"gemv {shape}")


# config 2 (7168 x 16384, l = 4) and the shapes the reference's GEMV task is timed on (task_gemv.yml:54-57)
@pytest.mark.parametrize("shape", [(7168, 16384, 4), (7168, 16384, 1), (4096, 7168, 8), (7168, 2048, 4)])
def test_gemv_benchmark_shapes(sub, oracle, shape):
    from nvfp4_gemm_b200.inputs import generate_input
    m, k, l = shape
    data = generate_input(m, 1, k, l, 1111)
    data[6].view(torch.int16).fill_(0x7fff)
    out = sub.custom_kernel(data)
    torch.cuda.synchronize()
    assert_bit_exact(out, expected_fp16(oracle, data), what=f"gemv {shape}")


def test_gemv_general_scales_within_tolerance(sub, oracle):
    from nvfp4_gemm_b200.inputs import generate_input, SF_DTYPE
    m, k, l = 256, 4096, 2
    a, b, _, _, sfap, sfbp, c = generate_input(m, 1, k, l, 9)
    g = torch.Generator().manual_seed(11)
    sfa = torch.randint(0x20, 0x58, (l, m, k // 16), dtype=torch.uint8, generator=g).cuda().permute(1, 2, 0).view(SF_DTYPE)
    sfb = torch.randint(0x20, 0x58, (l, 1, k // 16), dtype=torch.uint8, generator=g).cuda().permute(1, 2, 0).view(SF_DTYPE)
    data = (a, b, sfa, sfb, sfap, sfbp, c)
    out = sub.custom_kernel(data)
    torch.cuda.synchronize()
    an, bn, san, sbn = oracle.tensors_to_numpy(data)
    assert_close(out, oracle.ref_gemm(an, bn, san, sbn, accumulate="f64"), rtol=1e-3, atol=1e-3, what="gemv general scales")


@pytest.mark.parametrize("rows_per_warp", [1, 2, 4])
@pytest.mark.parametrize("warps_per_cta", [1, 2, 4])
def test_every_gemv_launch_shape_gives_the_same_bits(sub, oracle, lib, rows_per_warp, warps_per_cta):
    """Ragged M (not a multiple of rows per CTA), K that is not a multiple of the unrolled stride."""
    from nvfp4_gemm_b200 import _lib
    from nvfp4_gemm_b200.inputs import generate_input
    data = generate_input(131, 1, 4160, 3, 77)
    data[6].view(torch.int16).fill_(0x7fff)
    problem = sub.make_problem(data)
    _lib.check(lib.nvfp4_gemv_config(problem, rows_per_warp, warps_per_cta, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert sub.last_kernel() == f"gemv_warp_r{rows_per_warp}_w{warps_per_cta}"
    assert_bit_exact(data[6], expected_fp16(oracle, data), what=f"gemv r{rows_per_warp} w{warps_per_cta}")


def test_gemv_config_rejects_unknown_launch_shapes(sub, lib):
    from nvfp4_gemm_b200 import _lib
    from nvfp4_gemm_b200.inputs import generate_input
    problem = sub.make_problem(generate_input(128, 1, 256, 1, 1))
    assert lib.nvfp4_gemv_config(problem, 3, 0, None) == _lib.NVFP4_ERR_INVALID_ARGUMENT
    assert lib.nvfp4_gemv_config(problem, 0, 8, None) == _lib.NVFP4_ERR_INVALID_ARGUMENT
