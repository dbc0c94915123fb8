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


@pytest.mark.parametrize("m,n_local,k,blocks,rank,n_peers", [(512, 512, 1024, 2, 1, 1), (300, 256, 2048, 4, 2, 3), (128, 256, 4096, 2, 0, 1),
                                                            (1024, 1024, 512, 8, 5, 7)])
def test_gemm_stores_its_column_block_into_every_peer_buffer(cuda_lib, oracle, m, n_local, k, blocks, rank, n_peers):
    from nvfp4_gemm_b200 import _lib
    from nvfp4_gemm_b200.inputs import generate_input
    from nvfp4_gemm_b200.submission import make_problem

    n_total = n_local * blocks
    data = generate_input(m, n_local, k, 1, 31)
    outs = [torch.full((1, m, n_total), float("nan"), dtype=torch.float16, device="cuda").permute(1, 2, 0) for _ in range(1 + n_peers)]
    begin = rank * n_local
    problem = make_problem(tuple(data[:6]) + (outs[0][:, begin:begin + n_local],))
    peers = (ctypes.c_void_p * n_peers)(*[o.data_ptr() + begin * 2 for o in outs[1:]])
    _lib.check(cuda_lib.nvfp4_gemm_allgather(problem, None, peers, n_peers, torch.cuda.current_stream().cuda_stream))
    _lib.check(cuda_lib.nvfp4_check_status(torch.cuda.current_stream().cuda_stream))
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
