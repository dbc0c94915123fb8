"""GPU checks of the data-movement kernels beside the matmul: the column-block re-layout used
after the multi-GPU all-gather and the plain -> permuted scale converter."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cuda_lib(lib):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return lib


@pytest.mark.parametrize("rows,n_local,blocks,pad", [(256, 128, 2, 0), (300, 3584, 8, 0), (77, 264, 3, 16), (1, 8, 1, 0)])
def test_interleave_column_blocks(cuda_lib, rows, n_local, blocks, pad):
    from nvfp4_gemm_b200 import _lib
    src = torch.randn((blocks, rows, n_local), device="cuda").half()
    stride = blocks * n_local + pad
    dst = torch.full((rows, stride), -1.0, dtype=torch.float16, device="cuda")
    _lib.check(cuda_lib.nvfp4_interleave_column_blocks(src.data_ptr(), dst.data_ptr(), rows, n_local, blocks, stride,
                                                       torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert torch.equal(dst[:, :blocks * n_local], src.permute(1, 0, 2).reshape(rows, -1))
    if pad:
        assert torch.all(dst[:, blocks * n_local:] == -1.0)          # padding columns untouched
    assert cuda_lib.nvfp4_interleave_column_blocks(src.data_ptr(), dst.data_ptr(), rows, 12, blocks, stride, None) == _lib.NVFP4_ERR_INVALID_ARGUMENT


@pytest.mark.parametrize("rows,k,l", [(128, 256, 1), (300, 1024, 2), (1, 64, 1), (7168, 16384, 1)])
def test_permute_scales_matches_the_layout_formula(cuda_lib, oracle, rows, k, l):
    from nvfp4_gemm_b200 import _lib
    plain = torch.randint(0, 256, (l, rows, k // 16), dtype=torch.uint8, device="cuda")
    per_batch = ((rows + 127) // 128) * (k // 64) * 512
    perm = torch.full((l * per_batch,), 0xAB, dtype=torch.uint8, device="cuda")
    _lib.check(cuda_lib.nvfp4_permute_scales(plain.data_ptr(), perm.data_ptr(), rows, k, l, k // 16, rows * (k // 16), per_batch,
                                             torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    exp = oracle.permute_sf(plain.permute(1, 2, 0).cpu().numpy())
    assert np.array_equal(perm.cpu().numpy(), exp)
