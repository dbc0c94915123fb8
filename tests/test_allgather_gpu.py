"""The GEMM whose epilogue also stores into other GPUs' outputs, exercised on ONE GPU: the
"peers" are further buffers on the same device, which checks every store path (TMA store of whole
tiles, vector stores of finished shared tiles) and that nothing outside this rank's column block
is touched.  The 2..8-GPU run itself is `bench.py --gpus N`, which checks parity against the
oracle on rank 0."""
import ctypes

import numpy as np
import pytest
import torch

from helpers import assert_bit_exact

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cuda_lib(lib):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return lib


@pytest.mark.parametrize("tma_peers", [0, 7])      # peers served by the epilogue warps' stores / by tensor stores
@pytest.mark.parametrize("m,n_local,k,blocks,rank,n_peers", [(512, 512, 1024, 2, 1, 1), (300, 256, 2048, 4, 2, 3), (128, 256, 4096, 2, 0, 1),
                                                            (1024, 1024, 512, 8, 5, 7)])
def test_gemm_stores_its_column_block_into_every_peer_buffer(cuda_lib, oracle, m, n_local, k, blocks, rank, n_peers, tma_peers):
    from nvfp4_gemm_b200 import _lib
    from nvfp4_gemm_b200.inputs import generate_input
    from nvfp4_gemm_b200.submission import make_problem

    n_total = n_local * blocks
    data = generate_input(m, n_local, k, 1, 31)
    outs = [torch.full((1, m, n_total), float("nan"), dtype=torch.float16, device="cuda").permute(1, 2, 0) for _ in range(1 + n_peers)]
    begin = rank * n_local
    problem = make_problem(tuple(data[:6]) + (outs[0][:, begin:begin + n_local],))
    peers = (ctypes.c_void_p * n_peers)(*[o.data_ptr() + begin * 2 for o in outs[1:]])
    previous = cuda_lib.nvfp4_set_peer_tma_limit(tma_peers)
    try:
        _lib.check(cuda_lib.nvfp4_gemm_allgather(problem, None, peers, n_peers, torch.cuda.current_stream().cuda_stream))
        _lib.check(cuda_lib.nvfp4_check_status(torch.cuda.current_stream().cuda_stream))
    finally:
        cuda_lib.nvfp4_set_peer_tma_limit(previous)
    a, b, sfa, sfb = oracle.tensors_to_numpy(data)
    exp = oracle.ref_gemm_c(a, b, sfa, sfb)
    for i, o in enumerate(outs):
        assert_bit_exact(o[:, begin:begin + n_local], exp, what=f"destination {i}")
        rest = torch.cat([o[:, :begin], o[:, begin + n_local:]], dim=1)
        assert torch.isnan(rest.float()).all(), f"destination {i}: columns outside the block were written"


def test_allgather_entry_point_rejects_bad_peer_lists(cuda_lib):
    from nvfp4_gemm_b200 import _lib
    from nvfp4_gemm_b200.inputs import generate_input
    from nvfp4_gemm_b200.submission import make_problem
    data = generate_input(256, 256, 512, 1, 1)
    p = make_problem(data)
    assert cuda_lib.nvfp4_gemm_allgather(p, None, None, 2, None) == _lib.NVFP4_ERR_INVALID_ARGUMENT
    arr = (ctypes.c_void_p * 8)(*[data[6].data_ptr()] * 8)
    assert cuda_lib.nvfp4_gemm_allgather(p, None, arr, 8, None) == _lib.NVFP4_ERR_INVALID_ARGUMENT
    arr[0] = data[6].data_ptr() + 2
    assert cuda_lib.nvfp4_gemm_allgather(p, None, arr, 1, None) == _lib.NVFP4_ERR_INVALID_ARGUMENT


@pytest.mark.parametrize("m,n_local,blocks,rank,row0,rows", [(512, 512, 4, 1, 0, 512), (300, 256, 8, 5, 128, 172), (64, 128, 2, 0, 7, 13)])
def test_copy_kernel_pulls_the_other_ranks_column_blocks_and_nothing_else(cuda_lib, m, n_local, blocks, rank, row0, rows):
    """One GPU stands in for all ranks: `blocks` full-size outputs, each holding only its own column
    block; the pull into output `rank` must bring rows [row0, row0 + rows) of every other block."""
    from nvfp4_gemm_b200 import _lib
    n_total = n_local * blocks
    g = torch.Generator(device="cuda").manual_seed(5)
    outs = []
    for r in range(blocks):
        o = torch.zeros((m, n_total), dtype=torch.float16, device="cuda")
        o[:, r * n_local:(r + 1) * n_local] = torch.randn((m, n_local), generator=g, device="cuda", dtype=torch.float16)
        outs.append(o)
    before = outs[rank].clone()
    peers = [r for r in range(blocks) if r != rank]
    src = (ctypes.c_void_p * len(peers))(*[outs[r].data_ptr() + r * n_local * 2 for r in peers])
    dst = (ctypes.c_void_p * len(peers))(*[outs[rank].data_ptr() + r * n_local * 2 for r in peers])
    _lib.check(cuda_lib.nvfp4_copy_column_blocks(dst, src, len(peers), row0, rows, n_local, n_total, 0, 0, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    exp = before.clone()
    for r in peers:
        exp[row0:row0 + rows, r * n_local:(r + 1) * n_local] = outs[r][row0:row0 + rows, r * n_local:(r + 1) * n_local]
    assert torch.equal(outs[rank].view(torch.int16), exp.view(torch.int16))


def test_copy_kernel_rejects_bad_arguments(cuda_lib):
    from nvfp4_gemm_b200 import _lib
    t = torch.zeros((64, 256), dtype=torch.float16, device="cuda")
    one = (ctypes.c_void_p * 1)(t.data_ptr())
    odd = (ctypes.c_void_p * 1)(t.data_ptr() + 2)
    assert cuda_lib.nvfp4_copy_column_blocks(one, one, 0, 0, 64, 128, 256, 0, 0, None) == _lib.NVFP4_ERR_INVALID_ARGUMENT
    assert cuda_lib.nvfp4_copy_column_blocks(one, one, 8, 0, 64, 128, 256, 0, 0, None) == _lib.NVFP4_ERR_INVALID_ARGUMENT
    assert cuda_lib.nvfp4_copy_column_blocks(one, odd, 1, 0, 64, 128, 256, 0, 0, None) == _lib.NVFP4_ERR_INVALID_ARGUMENT
    assert cuda_lib.nvfp4_copy_column_blocks(one, one, 1, 0, 64, 100, 256, 0, 0, None) == _lib.NVFP4_ERR_INVALID_ARGUMENT
    assert cuda_lib.nvfp4_copy_column_blocks(one, one, 1, 0, 64, 512, 256, 0, 0, None) == _lib.NVFP4_ERR_INVALID_ARGUMENT


def test_copy_kernel_pushes_one_block_into_every_peer_output(cuda_lib):
    from nvfp4_gemm_b200 import _lib
    m, n_local, blocks, rank, row0, rows = 200, 384, 4, 2, 40, 97
    n_total = n_local * blocks
    mine = torch.randn((m, n_total), device="cuda", dtype=torch.float16)
    outs = [torch.full((m, n_total), float("nan"), dtype=torch.float16, device="cuda") for _ in range(blocks - 1)]
    src = (ctypes.c_void_p * len(outs))(*[mine.data_ptr() + rank * n_local * 2] * len(outs))
    dst = (ctypes.c_void_p * len(outs))(*[o.data_ptr() + rank * n_local * 2 for o in outs])
    _lib.check(cuda_lib.nvfp4_copy_column_blocks(dst, src, len(outs), row0, rows, n_local, n_total, 3, 1, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    for o in outs:
        blk = o[row0:row0 + rows, rank * n_local:(rank + 1) * n_local]
        assert torch.equal(blk.view(torch.int16), mine[row0:row0 + rows, rank * n_local:(rank + 1) * n_local].view(torch.int16))
        assert int(torch.isnan(o.float()).sum().item()) == m * n_total - rows * n_local
