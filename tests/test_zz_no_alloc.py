"""nvfp4_gemm_static_scratch: the GEMM entry point for callers that cannot allocate.

Some users of this library run where cudaMalloc is off limits at call time: beside a thread
that is capturing a CUDA graph in global mode, inside a service whose own pool already owns
all free HBM, or in a loop that must never wait on the allocator.  For them the library keeps
the persistent kernel's partial-tile scratch in a fixed 8 MiB device array.  This file checks
that entry point against nvfp4_gemm() through the C ABI.  It is collected last on purpose, and
passes both on its own in a fresh process and after the rest of the suite.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run_both(lib, shape, seed, workers):
    from nvfp4_gemm_b200 import _lib
    from nvfp4_gemm_b200.inputs import generate_input
    from nvfp4_gemm_b200.submission import make_problem

    m, n, k, l = shape
    data = generate_input(m, n, k, l, seed)
    stream = torch.cuda.current_stream().cuda_stream

    ref = torch.full_like(data[6], float("nan"))
    p_ref = make_problem(data[:6] + (ref,))
    # the existing entry point, forced onto the same persistent 128-wide kernel family
    _lib.check(lib.nvfp4_gemm(p_ref, _lib.GemmConfig(128, 1, 0, 1, 1), stream))

    out = torch.full_like(data[6], float("nan"))
    p_new = make_problem(data[:6] + (out,))
    _lib.check(lib.nvfp4_gemm_static_scratch(p_new, workers, stream))
    torch.cuda.synchronize()
    return ref, out


@pytest.fixture(scope="module")
def cuda_lib(lib):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return lib


def test_static_scratch_gemm_matches_the_allocating_entry_point_twice_in_a_row(cuda_lib):
    # Shapes whose tiles are shared between workers, so the fixed scratch really is used; the
    # second call follows the first on the same stream and must not see its leftovers.
    for call, (shape, seed, workers) in enumerate([((128, 512, 8192, 1), 5, 0), ((300, 384, 4096, 2), 6, 7)]):
        ref, out = _run_both(cuda_lib, shape, seed, workers)
        # same tolerance as the other parity tests: the fp16 bit patterns are equal
        assert torch.equal(ref.view(torch.int16), out.view(torch.int16)), f"call {call}: outputs differ for {shape}"
        assert not torch.isnan(out.float()).any()
        # a wait that ran out inside this variant is reported through the same status call
        assert cuda_lib.nvfp4_check_status(torch.cuda.current_stream().cuda_stream) == 0


def test_static_scratch_gemm_matches_the_oracle_and_allocates_nothing(cuda_lib, oracle):
    """The property the entry point exists for: once its first call on the device is over, a call
    leaves the device's free memory and the library's own scratch accounting exactly as they
    were -- and the result is the oracle's, bit for bit."""
    from helpers import assert_bit_exact, expected_fp16
    from nvfp4_gemm_b200 import _lib
    from nvfp4_gemm_b200.inputs import generate_input
    from nvfp4_gemm_b200.submission import make_problem

    stream = torch.cuda.current_stream().cuda_stream
    data = generate_input(200, 640, 4096, 1, 9)
    problem = make_problem(data)
    _lib.check(cuda_lib.nvfp4_gemm_static_scratch(problem, 0, stream))      # first call on the device: one-time set-up
    torch.cuda.synchronize()
    data[6].view(torch.int16).fill_(0x7fff)
    free_before, lib_bytes_before = torch.cuda.mem_get_info()[0], cuda_lib.nvfp4_scratch_bytes()
    _lib.check(cuda_lib.nvfp4_gemm_static_scratch(problem, 0, stream))
    _lib.check(cuda_lib.nvfp4_gemm_static_scratch(problem, 5, stream))
    assert cuda_lib.nvfp4_check_status(stream) == 0
    assert torch.cuda.mem_get_info()[0] == free_before
    assert cuda_lib.nvfp4_scratch_bytes() == lib_bytes_before
    assert_bit_exact(data[6], expected_fp16(oracle, data), what="static scratch vs oracle")


def test_static_scratch_gemm_rejects_more_workers_than_it_has_slots_for(cuda_lib):
    from nvfp4_gemm_b200 import _lib
    from nvfp4_gemm_b200.inputs import generate_input
    from nvfp4_gemm_b200.submission import make_problem

    data = generate_input(128, 256, 1024, 1, 1)
    rc = cuda_lib.nvfp4_gemm_static_scratch(make_problem(data), 65, None)
    assert rc == _lib.NVFP4_ERR_INVALID_ARGUMENT
    assert "at most 64" in cuda_lib.nvfp4_last_error().decode()
    bad = make_problem(data)
    bad.k = 300
    assert cuda_lib.nvfp4_gemm_static_scratch(bad, 0, None) == _lib.NVFP4_ERR_INVALID_ARGUMENT
