"""GPU parity of the NVFP4 quantiser (the producer of the operator's inputs) against the oracle's
statement of it, and a round trip through the GEMM."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cuda_lib(lib):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return lib


def _quantize(cuda_lib, x):
    from nvfp4_gemm_b200 import _lib
    rows, k = x.shape
    packed = torch.empty((rows, k // 2), dtype=torch.uint8, device="cuda")
    sf = torch.empty((rows, k // 16), dtype=torch.uint8, device="cuda")
    perm = torch.full((((rows + 127) // 128) * (k // 64) * 512,), 0xEE, dtype=torch.uint8, device="cuda")
    _lib.check(cuda_lib.nvfp4_quantize(x.data_ptr(), int(x.dtype == torch.bfloat16), packed.data_ptr(), sf.data_ptr(), perm.data_ptr(),
                                       rows, k, x.stride(0), k // 2, k // 16, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return packed, sf, perm


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,k", [(128, 256), (300, 1024), (1, 64), (4096, 7168)])
def test_quantizer_matches_oracle_bit_for_bit(cuda_lib, oracle, dtype, rows, k):
    g = torch.Generator().manual_seed(rows + k)
    x = (torch.randn((rows, k), generator=g) * torch.exp(torch.randn((rows, 1), generator=g))).to(dtype)
    x[0, :16] = 0                                   # an all-zero block
    x[-1, 20] = -0.0                                # a negative zero keeps its sign bit in the code
    x[-1, -16:] = 1000.0 if dtype == torch.float16 else 1e6   # saturating scale / elements
    packed, sf, perm = _quantize(cuda_lib, x.cuda())
    exp_packed, exp_sf = oracle.quantize_rows(x.float().numpy())
    assert np.array_equal(sf.cpu().numpy(), exp_sf)
    assert np.array_equal(packed.cpu().numpy(), exp_packed)
    assert np.array_equal(perm.cpu().numpy(), oracle.permute_sf(exp_sf[:, :, None]))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_quantizer_with_outputs_that_only_allow_narrow_stores(cuda_lib, oracle, dtype):
    """Codes 8 bytes off a 16-byte boundary and scale rows with an odd stride: the kernel falls back
    from its 16-byte / 4-byte stores to 8-byte / single-byte ones."""
    from nvfp4_gemm_b200 import _lib
    rows, k = 200, 512
    g = torch.Generator().manual_seed(5)
    x = (torch.randn((rows, k), generator=g) * 3).to(dtype).cuda()
    packed_buf = torch.zeros((rows * (k // 2 + 8) + 8,), dtype=torch.uint8, device="cuda")
    packed = packed_buf[8:]                                   # 8-byte aligned only, row stride k/2 + 8
    sf_buf = torch.zeros((rows * (k // 16 + 1) + 1,), dtype=torch.uint8, device="cuda")
    sf = sf_buf[1:]                                           # odd base address, odd row stride
    perm = torch.full((((rows + 127) // 128) * (k // 64) * 512,), 0xEE, dtype=torch.uint8, device="cuda")
    _lib.check(cuda_lib.nvfp4_quantize(x.data_ptr(), int(dtype == torch.bfloat16), packed.data_ptr(), sf.data_ptr(), perm.data_ptr(),
                                       rows, k, x.stride(0), k // 2 + 8, k // 16 + 1, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    exp_packed, exp_sf = oracle.quantize_rows(x.float().cpu().numpy())
    got_packed = packed[: rows * (k // 2 + 8)].view(rows, k // 2 + 8)[:, : k // 2].cpu().numpy()
    got_sf = sf[: rows * (k // 16 + 1)].view(rows, k // 16 + 1)[:, : k // 16].cpu().numpy()
    assert np.array_equal(got_packed, exp_packed)
    assert np.array_equal(got_sf, exp_sf)
    assert np.array_equal(perm.cpu().numpy(), oracle.permute_sf(exp_sf[:, :, None]))
    assert int(packed_buf[:8].sum()) == 0 and int(sf_buf[0]) == 0          # nothing written in front of the buffers


def _e4m3_positive():
    vals = []
    for byte in range(1, 127):
        e, m = (byte >> 3) & 15, byte & 7
        vals.append((m / 8) * 2.0 ** -6 if e == 0 else (1 + m / 8) * 2.0 ** (e - 7))
    return np.array(vals, dtype=np.float32)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_quantizer_on_rounding_ties_and_their_neighbours(cuda_lib, oracle, dtype):
    """Every e4m3 scale, with elements on each e2m1 rounding threshold times the scale and one step of
    the input type either side: the cases a division that is not correctly rounded would get wrong."""
    scales = _e4m3_positive()
    ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)
    rows = []
    for s in scales:
        on = torch.tensor(ties * s).to(dtype)
        if not torch.isfinite(on.float()).all():
            continue
        bits = on.view(torch.int16)
        block = torch.cat([on, (bits + 1).view(dtype), (bits - 1).view(dtype)])         # 21 values
        signs = torch.tensor([1.0, -1.0] * 11)[:21].to(dtype)
        for part in (block[:15], block[6:21]):
            row = torch.zeros(64, dtype=dtype)
            row[:15] = part * signs[:15]
            row[15] = 6.0 * float(s)                                                    # pins the block's scale to s
            row[16:31] = part
            row[31] = -6.0 * float(s)
            rows.append(row)
    x = torch.stack(rows)
    assert torch.isfinite(x.float()).all()
    packed, sf, _ = _quantize(cuda_lib, x.cuda())
    exp_packed, exp_sf = oracle.quantize_rows(x.float().numpy())
    assert np.array_equal(sf.cpu().numpy(), exp_sf)
    assert np.array_equal(packed.cpu().numpy(), exp_packed)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_quantizer_saturates_infinities_and_huge_values(cuda_lib, oracle, dtype):
    x = torch.zeros((2, 64), dtype=dtype)
    x[0, 0], x[0, 1], x[0, 2], x[0, 3] = float("inf"), float("-inf"), 3.0, 60000.0
    x[0, 18], x[0, 19], x[0, 20] = 448.0 * 5, 448.0 * 5.5, 65504.0 if dtype == torch.float16 else 3e38
    x[1, 5], x[1, 6] = (65504.0, -1.0) if dtype == torch.float16 else (-1e30, 1e20)
    packed, sf, _ = _quantize(cuda_lib, x.cuda())
    exp_packed, exp_sf = oracle.quantize_rows(x.float().numpy())
    assert np.array_equal(sf.cpu().numpy(), exp_sf)
    assert np.array_equal(packed.cpu().numpy(), exp_packed)


def test_quantize_then_gemm_approximates_the_fp32_product(cuda_lib, oracle):
    from nvfp4_gemm_b200 import submission
    from nvfp4_gemm_b200.inputs import FP4_DTYPE, SF_DTYPE
    m, n, k = 256, 512, 2048
    g = torch.Generator().manual_seed(0)
    a = torch.randn((m, k), generator=g).half().cuda()
    b = torch.randn((n, k), generator=g).half().cuda()
    pa, sa, ppa = _quantize(cuda_lib, a)
    pb, sb, ppb = _quantize(cuda_lib, b)
    c = torch.empty((1, m, n), dtype=torch.float16, device="cuda").permute(1, 2, 0)

    def perm_view(p, rows):
        return p.view(1, (rows + 127) // 128, k // 64, 32, 4, 4).permute(3, 4, 1, 5, 2, 0).view(SF_DTYPE)

    data = (pa.view(1, m, k // 2).permute(1, 2, 0).view(FP4_DTYPE), pb.view(1, n, k // 2).permute(1, 2, 0).view(FP4_DTYPE),
            sa.view(1, m, k // 16).permute(1, 2, 0).view(SF_DTYPE), sb.view(1, n, k // 16).permute(1, 2, 0).view(SF_DTYPE),
            perm_view(ppa, m), perm_view(ppb, n), c)
    out = submission.custom_kernel(data)
    submission.check_status()
    # exact against the oracle on the quantised operands ...
    exp = oracle.ref_gemm(pa.cpu().numpy()[:, :, None], pb.cpu().numpy()[:, :, None], sa.cpu().numpy()[:, :, None], sb.cpu().numpy()[:, :, None], accumulate="f64")
    np.testing.assert_allclose(out.cpu().numpy().astype(np.float32), exp.astype(np.float32), rtol=1e-3, atol=1e-3)
    # ... and close to the unquantised product (4-bit operands: a few percent of the output scale)
    ref = (a.float() @ b.float().t()).cpu().numpy()
    err = np.abs(out[:, :, 0].float().cpu().numpy() - ref)
    assert err.mean() < 0.25 * np.abs(ref).mean() + 0.5, (err.mean(), np.abs(ref).mean())
