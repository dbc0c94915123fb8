"""GPU parity of the tensor-core GEMM against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from helpers import assert_bit_exact, assert_close, expected_fp16

pytestmark = pytest.mark.gpu

# (m, n, k, l): the reference's test shapes (task.yml:41-51) ...
TASK_SHAPES = [
    (128, 256, 256, 1), (128, 1536, 7168, 1), (128, 3072, 1536, 1), (256, 7168, 256, 1), (256, 7168, 2048, 1),
    (384, 7168, 2304, 1), (512, 512, 7168, 1), (512, 4096, 512, 1), (512, 1536, 7168, 1),
]
# ... plus ragged M, batched L, N that only fits the 128-wide tile, and a single k-tile
EXTRA_SHAPES = [(1, 128, 256, 1), (130, 384, 512, 1), (300, 768, 1536, 2), (128, 128, 256, 3), (257, 640, 1024, 2)]
# ... and mid-size shapes on either side of the launch code's choices: whole tiles on fewer CTA pairs
# than the device has, two waves of whole tiles, 128-wide single-CTA tiles for an odd number of
# 128-row blocks
MID_SHAPES = [(768, 4096, 4096, 1), (1024, 7168, 4096, 1), (640, 7168, 7168, 1), (1536, 4096, 4096, 1)]


@pytest.fixture(scope="module")
def sub(lib):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from nvfp4_gemm_b200 import submission
    return submission


@pytest.mark.parametrize("shape", TASK_SHAPES + EXTRA_SHAPES + MID_SHAPES)
def test_custom_kernel_matches_oracle_bit_exact(sub, oracle, shape):
    from nvfp4_gemm_b200.inputs import generate_input
    m, n, k, l = shape
    data = generate_input(m, n, k, l, 1111)
    data[6].view(torch.int16).fill_(0x7fff)        # NaN canary: every element must be written
    out = sub.custom_kernel(data)
    sub.check_status()
    assert out is data[6]
    # integer-valued products and power-of-two scales: fp32 accumulation is exact, so is parity
    assert_bit_exact(out, expected_fp16(oracle, data), what=f"{shape} {sub.last_kernel()}")


VARIANTS = [  # (cta_group, tile_n, epilogue, split_k)
    (1, 128, 1, 1), (1, 128, 2, 1), (1, 256, 1, 1), (1, 256, 2, 1),     # one CTA per tile, stream-K
    (2, 128, 1, 1), (2, 128, 2, 1), (2, 256, 1, 1), (2, 256, 2, 1), (2, 256, 3, 1),   # CTA pair per 256-row tile
]


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("shape,grid", [((128, 512, 4096, 1), 6), ((300, 768, 1536, 2), 0), ((512, 1024, 1024, 1), 10),
                                        ((256, 256, 256, 1), 0), ((640, 512, 2048, 1), 4)])
def test_every_kernel_variant_and_split_pattern(sub, oracle, variant, shape, grid):
    from nvfp4_gemm_b200.inputs import generate_input
    cta_group, tile_n, epilogue, split_k = variant
    m, n, k, l = shape
    data = generate_input(m, n, k, l, 7)
    data[6].view(torch.int16).fill_(0x7fff)
    kw = dict(tile_n=tile_n, epilogue=epilogue, grid=grid, cta_group=cta_group, split_k=split_k)
    sub.gemm(data, **kw)
    sub.check_status()
    assert_bit_exact(data[6], expected_fp16(oracle, data), what=f"{shape} {sub.last_kernel()} grid={grid}")
    # run it again: the per-tile counters must have been left at zero by the previous launch
    data[6].view(torch.int16).fill_(0x7fff)
    sub.gemm(data, **kw)
    sub.check_status()
    assert_bit_exact(data[6], expected_fp16(oracle, data), what=f"second launch {shape}")


@pytest.mark.parametrize("split_k,tile_n", [(2, 0), (4, 0), (4, 256), (8, 0)])
@pytest.mark.parametrize("shape", [(128, 256, 2048, 1), (77, 512, 2304, 2), (128, 512, 2048, 1), (1, 256, 2048, 1), (200, 256, 2048, 1)])
def test_cluster_split_k(sub, oracle, split_k, tile_n, shape):
    """K split across a cluster, partial sums exchanged through distributed shared memory."""
    from nvfp4_gemm_b200.inputs import generate_input
    m, n, k, l = shape
    data = generate_input(m, n, k, l, 21)
    data[6].view(torch.int16).fill_(0x7fff)
    sub.gemm(data, split_k=split_k, tile_n=tile_n)
    sub.check_status()
    assert sub.last_kernel().startswith(f"gemm_splitk{split_k}")
    assert_bit_exact(data[6], expected_fp16(oracle, data), what=f"{shape} {sub.last_kernel()}")


def test_largest_reference_test_shape(sub, oracle):
    from nvfp4_gemm_b200.inputs import generate_input
    m, n, k, l = 2304, 4608, 7168, 1                 # task.yml:47
    data = generate_input(m, n, k, l, 1111)
    out = sub.custom_kernel(data)
    sub.check_status()
    # the full oracle would take minutes: check 96 sampled rows against all columns
    rows = np.random.default_rng(0).choice(m, 96, replace=False)
    a, b, sfa, sfb = oracle.tensors_to_numpy(data)
    exp = oracle.ref_gemm_c(a[rows], b, sfa[rows], sfb)
    assert_bit_exact(out[torch.from_numpy(rows).cuda()], exp, what="2304x4608x7168 sampled rows")


# The shapes the reference task is timed on (task.yml:53-56), whole output against the oracle.
@pytest.mark.parametrize("shape", [(128, 7168, 16384, 1), (128, 4096, 7168, 1), (128, 7168, 2048, 1)])
def test_benchmark_shapes_match_oracle_bit_exact(sub, oracle, shape):
    from nvfp4_gemm_b200.inputs import generate_input
    m, n, k, l = shape
    data = generate_input(m, n, k, l, 1111)
    data[6].view(torch.int16).fill_(0x7fff)
    out = sub.custom_kernel(data)
    sub.check_status()
    assert_bit_exact(out, expected_fp16(oracle, data), what=f"{shape} {sub.last_kernel()}")


def test_largest_configuration_on_one_gpu_sampled(sub, oracle):
    """8192 x 28672 x 8192, the job the multi-GPU path partitions, whole on one GPU: sampled rows
    against the oracle over sampled columns (every 128-column block boundary region is hit), and
    the all-ones canary shows that every element was written."""
    from nvfp4_gemm_b200.inputs import generate_input
    m, n, k, l = 8192, 28672, 8192, 1
    data = generate_input(m, n, k, l, 1111)
    data[6].view(torch.int16).fill_(0x7fff)
    out = sub.custom_kernel(data)
    sub.check_status()
    assert int((out.view(torch.int16) == 0x7fff).sum().item()) == 0
    rng = np.random.default_rng(8)
    rows = np.sort(rng.choice(m, 48, replace=False))
    cols = np.sort(np.concatenate([rng.choice(n, 1024, replace=False), np.arange(0, n, 3584), np.arange(3583, n, 3584)]))
    cols = np.unique(cols)
    a, b, sfa, sfb = oracle.tensors_to_numpy(data)
    exp = oracle.ref_gemm_c(a[rows], b[cols], sfa[rows], sfb[cols])
    got = out[torch.from_numpy(rows).cuda()][:, torch.from_numpy(cols).cuda()]
    assert_bit_exact(got, exp, what="C4 sampled block on one GPU")


def test_gemms_on_two_streams_do_not_share_scratch(sub, oracle, lib):
    """Two persistent GEMMs whose tiles are shared between workers (so both use the partial-tile
    scratch and the tile counters) overlap on two streams: each stream has its own scratch set, so
    both results are exact, over several rounds."""
    from nvfp4_gemm_b200.inputs import generate_input
    shapes = [(256, 1024, 8192, 1), (384, 768, 6144, 1)]
    datas = [generate_input(m, n, k, l, 40 + i) for i, (m, n, k, l) in enumerate(shapes)]
    exps = [expected_fp16(oracle, d) for d in datas]
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    torch.cuda.synchronize()
    for rnd in range(6):
        for d in datas:
            d[6].view(torch.int16).fill_(0x7fff)
        torch.cuda.synchronize()
        for s, d in zip(streams, datas):
            with torch.cuda.stream(s):
                for _ in range(3):
                    sub.gemm(d, tile_n=128, epilogue=1, cta_group=1, split_k=1, grid=40)   # stream-K, tiles shared by workers
        torch.cuda.synchronize()
        for s in streams:
            with torch.cuda.stream(s):
                sub.check_status()
        for d, e, shp in zip(datas, exps, shapes):
            assert_bit_exact(d[6], e, what=f"round {rnd} {shp}")
    for s in streams:
        assert lib.nvfp4_release_stream(s.cuda_stream) == 0


def test_general_scales_within_stated_tolerance(sub, oracle):
    """Arbitrary e4m3 scales and values: not exact any more, must stay inside rtol = atol = 1e-3."""
    from nvfp4_gemm_b200.inputs import generate_input, permute_scale_factors, SF_DTYPE
    m, n, k, l = 256, 512, 2048, 1
    a, b, sfa, sfb, _, _, c = generate_input(m, n, k, l, 3)
    g = torch.Generator().manual_seed(5)
    sfa_u8 = torch.randint(0x20, 0x58, (l, m, k // 16), dtype=torch.uint8, generator=g).cuda()
    sfb_u8 = torch.randint(0x20, 0x58, (l, n, k // 16), dtype=torch.uint8, generator=g).cuda()
    data = (a, b, sfa_u8.permute(1, 2, 0).view(SF_DTYPE), sfb_u8.permute(1, 2, 0).view(SF_DTYPE),
            permute_scale_factors(sfa_u8).view(SF_DTYPE), permute_scale_factors(sfb_u8).view(SF_DTYPE), c)
    out = sub.custom_kernel(data)
    sub.check_status()
    an, bn, san, sbn = oracle.tensors_to_numpy(data)
    exp64 = oracle.ref_gemm(an, bn, san, sbn, accumulate="f64")
    assert_close(out, exp64, rtol=1e-3, atol=1e-3, what="general scales")


def test_decode_shape_full_size_properties(sub, oracle):
    """128 x 7168 x 16384: sampled columns against the oracle, overflow pattern, and exact linearity
    (doubling every scale of A doubles C, including the values that overflow to inf)."""
    from nvfp4_gemm_b200.inputs import generate_input
    m, n, k, l = 128, 7168, 16384, 1
    data = generate_input(m, n, k, l, 1111)
    out = sub.custom_kernel(data).clone()
    sub.check_status()
    cols = np.sort(np.random.default_rng(1).choice(n, 256, replace=False))
    a, b, sfa, sfb = oracle.tensors_to_numpy(data)
    exp = oracle.ref_gemm_c(a, b[cols], sfa, sfb[cols])
    assert_bit_exact(out[:, torch.from_numpy(cols).cuda()], exp, what="C1 sampled columns")
    # linearity: +1 on every exponent of SFA (byte + 8)
    a_t, b_t, sfa_t, sfb_t, sfap_t, sfbp_t, c_t = data
    sfap2 = (sfap_t.view(torch.uint8) + 8).view(sfap_t.dtype)
    out2 = sub.custom_kernel((a_t, b_t, sfa_t, sfb_t, sfap2, sfbp_t, torch.empty_like(c_t)))
    sub.check_status()
    assert torch.equal(out2.float(), (out.float() * 2).half().float())


def test_prefill_shape_full_size_sampled(sub, oracle):
    from nvfp4_gemm_b200.inputs import generate_input
    m, n, k, l = 4096, 7168, 7168, 1
    data = generate_input(m, n, k, l, 1111)
    out = sub.custom_kernel(data)
    sub.check_status()
    rng = np.random.default_rng(2)
    rows = np.sort(rng.choice(m, 64, replace=False))
    cols = np.sort(rng.choice(n, 512, replace=False))
    a, b, sfa, sfb = oracle.tensors_to_numpy(data)
    exp = oracle.ref_gemm_c(a[rows], b[cols], sfa[rows], sfb[cols])
    got = out[torch.from_numpy(rows).cuda()][:, torch.from_numpy(cols).cuda()]
    assert_bit_exact(got, exp, what="C3 sampled block")
    # checksum of checksums: column sums of C equal (sum of dequantised A rows) . B^T in fp64
    aq = oracle.dequantize(a[:, :, 0], sfa[:, :, 0]).astype(np.float64).sum(axis=0)
    bq = oracle.dequantize(b[cols[:64], :, 0], sfb[cols[:64], :, 0]).astype(np.float64)
    want = bq @ aq
    have = out[:, torch.from_numpy(cols[:64]).cuda(), 0].double().sum(dim=0).cpu().numpy()
    np.testing.assert_allclose(have, want, rtol=2e-3, atol=2000.0)  # 4096 fp16-rounded addends of magnitude ~1e4 per column


def test_back_to_back_launches_respect_stream_order(sub, oracle, lib):
    """The GEMM is launched with programmatic stream serialisation, so its set-up may overlap the
    kernel before it.  Its inputs and output must still behave as if the launches ran one after
    the other: (1) a producer kernel (the quantiser) rewrites A and its scales in place right
    before each GEMM, with no synchronisation in between; (2) consecutive GEMMs write the same C."""
    from nvfp4_gemm_b200 import _lib
    from nvfp4_gemm_b200.inputs import FP4_DTYPE, SF_DTYPE, generate_input
    m, n, k = 128, 1024, 4096                          # a cluster split-K decode shape
    stream = torch.cuda.current_stream().cuda_stream
    base = generate_input(m, n, k, 1, 5)
    g = torch.Generator().manual_seed(3)
    xs = [(torch.randn((m, k), generator=g) * (i + 1)).half().cuda() for i in range(4)]
    packed = torch.zeros((m, k // 2), dtype=torch.uint8, device="cuda")
    sf = torch.zeros((m, k // 16), dtype=torch.uint8, device="cuda")
    perm = torch.zeros((k // 64 * 512,), dtype=torch.uint8, device="cuda")
    a = packed.view(1, m, k // 2).permute(1, 2, 0).view(FP4_DTYPE)
    sfa = sf.view(1, m, k // 16).permute(1, 2, 0).view(SF_DTYPE)
    sfa_perm = perm.view(1, 1, k // 64, 32, 4, 4).permute(3, 4, 1, 5, 2, 0).view(SF_DTYPE)
    outs = [torch.empty((1, m, n), dtype=torch.float16, device="cuda").permute(1, 2, 0) for _ in xs]
    shared_c = torch.empty((1, m, n), dtype=torch.float16, device="cuda").permute(1, 2, 0)
    for x, c in zip(xs, outs):                         # no synchronisation inside this loop
        _lib.check(lib.nvfp4_quantize(x.data_ptr(), 0, packed.data_ptr(), sf.data_ptr(), perm.data_ptr(), m, k, x.stride(0), k // 2,
                                      k // 16, stream))
        sub.custom_kernel((a, base[1], sfa, base[3], sfa_perm, base[5], c))
        sub.custom_kernel((a, base[1], sfa, base[3], sfa_perm, base[5], shared_c))
    torch.cuda.synchronize()
    sub.check_status()
    assert sub.last_kernel().startswith("gemm_splitk")
    # the same launches again, each waited for before the next: the kernels are deterministic, so
    # any difference means a launch saw another launch's inputs or was overwritten out of order
    for i, (x, c) in enumerate(zip(xs, outs)):
        _lib.check(lib.nvfp4_quantize(x.data_ptr(), 0, packed.data_ptr(), sf.data_ptr(), perm.data_ptr(), m, k, x.stride(0), k // 2,
                                      k // 16, stream))
        torch.cuda.synchronize()
        exp = torch.empty_like(c)
        sub.custom_kernel((a, base[1], sfa, base[3], sfa_perm, base[5], exp))
        torch.cuda.synchronize()
        assert torch.equal(c.view(torch.int16), exp.view(torch.int16)), f"launch {i} read inputs of another launch"
        assert not torch.equal(exp.view(torch.int16), outs[(i + 1) % len(outs)].view(torch.int16))   # the inputs do differ
    assert torch.equal(shared_c.view(torch.int16), outs[-1].view(torch.int16))


def _padded_like(t, pad_bytes):
    """The same [rows, cols, L] values inside a wider allocation: row stride cols + pad, batch
    stride rows * (cols + pad) + pad (element size 1 byte; fp16 for c is handled by the caller)."""
    rows, cols, l = t.shape
    raw = t.view(torch.uint8) if t.element_size() == 1 else t
    row_stride = cols + pad_bytes
    batch_stride = rows * row_stride + pad_bytes
    if raw.dtype == torch.uint8:
        store = torch.full((l * batch_stride + pad_bytes,), 0x5A, dtype=torch.uint8, device=t.device)
    else:   # fp16 output: a NaN bit pattern no result can have marks the padding
        store = torch.full((l * batch_stride + pad_bytes,), 0x7E01, dtype=torch.int16, device=t.device).view(torch.float16)
    view = torch.as_strided(store, (rows, cols, l), (row_stride, 1, batch_stride))
    view.copy_(raw)
    return view.view(t.dtype) if t.element_size() == 1 else view


@pytest.mark.parametrize("shape", [(300, 512, 1024, 2), (128, 1024, 4096, 1), (64, 1, 2048, 3)])
def test_operands_and_output_with_padded_strides(sub, oracle, shape):
    """Rows and batches that are not densely packed (views into wider buffers): the strides of the
    C ABI's problem description are honoured by the tensor maps, the GEMV's pointers and the stores."""
    from nvfp4_gemm_b200.inputs import generate_input
    m, n, k, l = shape
    a, b, sfa, sfb, sfa_perm, sfb_perm, c = generate_input(m, n, k, l, 21)
    data = (_padded_like(a, 64), _padded_like(b, 32), _padded_like(sfa, 16), _padded_like(sfb, 8), sfa_perm, sfb_perm, _padded_like(c, 24))
    data[6].fill_(1.0)
    out = sub.custom_kernel(data)
    torch.cuda.synchronize()
    sub.check_status()
    assert_bit_exact(out, expected_fp16(oracle, (a, b, sfa, sfb, sfa_perm, sfb_perm, c)), what=f"padded strides {shape}")
    store = data[6].untyped_storage()
    whole = torch.empty(0, dtype=torch.int16, device="cuda").set_(store)
    assert int((whole == 0x7E01).sum().item()) == whole.numel() - m * n * l       # nothing outside C was written
