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


def test_gemv_benchmark_shape(sub, oracle):
    from nvfp4_gemm_b200.inputs import generate_input
    m, k, l = 7168, 16384, 4
    data = generate_input(m, 1, k, l, 1111)
    out = sub.custom_kernel(data)
    torch.cuda.synchronize()
    assert_bit_exact(out, expected_fp16(oracle, data), what="gemv 7168x16384x4")


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
