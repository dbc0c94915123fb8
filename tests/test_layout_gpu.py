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


@pytest.mark.parametrize("rows,k,l", [(128, 256, 1), (300, 1024, 2), (1, 64, 1), (4096, 7168, 1)])
def test_unpermute_scales_inverts_permute(cuda_lib, oracle, rows, k, l):
    from nvfp4_gemm_b200 import _lib
    plain = torch.randint(0, 256, (l, rows, k // 16), dtype=torch.uint8, device="cuda")
    per_batch = ((rows + 127) // 128) * (k // 64) * 512
    perm_np = np.ascontiguousarray(oracle.permute_sf(plain.permute(1, 2, 0).cpu().numpy())).reshape(-1)
    perm = torch.from_numpy(perm_np).cuda()
    back = torch.full((l, rows, k // 16 + 4), 0xCD, dtype=torch.uint8, device="cuda")      # padded rows: stride > k/16
    _lib.check(cuda_lib.nvfp4_unpermute_scales(perm.data_ptr(), back.data_ptr(), rows, k, l, k // 16 + 4, rows * (k // 16 + 4), per_batch,
                                               torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert torch.equal(back[:, :, :k // 16], plain)
    assert torch.all(back[:, :, k // 16:] == 0xCD)


def test_scale_layout_validator_counts_and_locates_differences(cuda_lib):
    from nvfp4_gemm_b200 import _lib
    from nvfp4_gemm_b200.inputs import generate_input
    from nvfp4_gemm_b200.submission import check_scale_layouts
    data = generate_input(300, 256, 1024, 2, 9)
    check_scale_layouts(data)                                   # what the generator makes agrees
    a, b, sfa, sfb, sfa_perm, sfb_perm, c = data
    sfa_u8 = sfa.view(torch.uint8)
    # flip two scales of the plain tensor: (row 200, column 5, batch 1) and (row 17, column 60, batch 1)
    sfa_u8[200, 5, 1] ^= 0x10
    sfa_u8[17, 60, 1] ^= 0x01
    result = torch.zeros(2, dtype=torch.int64, device="cuda")
    _lib.check(cuda_lib.nvfp4_compare_scale_layouts(sfa.data_ptr(), sfa_perm.data_ptr(), 300, 1024, 2, sfa.stride(0), sfa.stride(2),
                                                    sfa_perm.stride(5), result.data_ptr(), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert int(result[0]) == 2
    assert int(result[1]) == (1 * 300 + 17) * 64 + 60
    with pytest.raises(ValueError, match="sfa and sfa_permuted differ in 2 scale"):
        check_scale_layouts(data)
    sfa_u8[200, 5, 1] ^= 0x10
    sfa_u8[17, 60, 1] ^= 0x01
    # the padding rows of the permuted atoms (rows 300..383) are not part of the comparison
    flat = torch.as_strided(sfa_perm.view(torch.uint8), (sfa_perm.numel(),), (1,))
    flat[(2 * 16 + 0) * 512 + 31 * 16 + 3 * 4 + 0] ^= 0xFF        # row 383 of row block 2, first scale of atom 0
    check_scale_layouts(data)
    assert cuda_lib.nvfp4_compare_scale_layouts(sfa.data_ptr(), sfa_perm.data_ptr(), 300, 1024, 2, sfa.stride(0), sfa.stride(2),
                                                sfa_perm.stride(5), None, None) == _lib.NVFP4_ERR_INVALID_ARGUMENT
