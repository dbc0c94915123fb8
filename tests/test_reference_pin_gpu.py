"""Pins on a GPU against the reference's own code: its cuBLASLt submission (sub_cub.py:48-143,
bound by custom_kernel at sub_cub.py:165-169), compiled from the reference's source by
oracle/build_ref.py, runs on the same seeded inputs as the CPU oracle and as this library, and all
three must agree bit for bit (the products are exact in fp32, so no tolerance is needed)."""
import numpy as np
import pytest
import torch

from helpers import assert_bit_exact, expected_fp16

pytestmark = pytest.mark.gpu

# config 0 and the reference's test shapes (task.yml:41-51); the largest is compared on sampled rows
SHAPES = [(128, 256, 256), (128, 1536, 7168), (128, 3072, 1536), (256, 7168, 256), (256, 7168, 2048), (384, 7168, 2304),
          (512, 512, 7168), (512, 4096, 512), (512, 1536, 7168)]


@pytest.fixture(scope="module")
def reference_kernel(lib):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from oracle import build_ref
    if not build_ref.available():
        pytest.skip("oracle/_ref is not built (python oracle/build_ref.py, where the reference checkout is)")
    return build_ref.load()


@pytest.mark.parametrize("shape", SHAPES)
def test_oracle_and_library_match_the_reference_submission(reference_kernel, oracle, shape):
    from nvfp4_gemm_b200 import submission
    from nvfp4_gemm_b200.inputs import generate_input
    m, n, k = shape
    data = generate_input(m, n, k, 1, 1111)
    data[6].view(torch.int16).fill_(0x7fff)
    ref_out = reference_kernel(data).clone()
    torch.cuda.synchronize()
    assert_bit_exact(ref_out, expected_fp16(oracle, data), what=f"oracle vs reference sub_cub {shape}")
    ours = submission.custom_kernel(data[:6] + (torch.empty_like(data[6]),))
    submission.check_status()
    assert_bit_exact(ours, ref_out.cpu().numpy(), what=f"library vs reference sub_cub {shape}")


def test_largest_test_shape_and_benchmark_shapes_against_the_reference(reference_kernel, oracle):
    """2304 x 4608 x 7168 (task.yml:47) and the three benchmark shapes (task.yml:54-56): the
    library against the reference on the whole output, the oracle on sampled rows."""
    from nvfp4_gemm_b200 import submission
    from nvfp4_gemm_b200.inputs import generate_input
    for (m, n, k) in [(2304, 4608, 7168), (128, 7168, 16384), (128, 4096, 7168), (128, 7168, 2048)]:
        data = generate_input(m, n, k, 1, 1111)
        ref_out = reference_kernel(data).clone()
        ours = submission.custom_kernel(data[:6] + (torch.empty_like(data[6]),))
        submission.check_status()
        assert_bit_exact(ours, ref_out.cpu().numpy(), what=f"library vs reference sub_cub {(m, n, k)}")
        rows = np.sort(np.random.default_rng(4).choice(m, min(m, 32), replace=False))
        a, b, sfa, sfb = oracle.tensors_to_numpy(data)
        exp = oracle.ref_gemm_c(a[rows], b, sfa[rows], sfb)
        assert_bit_exact(ref_out[torch.from_numpy(rows).cuda()], exp, what=f"oracle vs reference sub_cub {(m, n, k)}")
