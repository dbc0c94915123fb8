"""Peer pointers through the C ABI alone (nvfp4_comm_export / open / close): a second process maps
this process's output buffer and pushes a column block into it with the library's copy kernel.
Both processes use the one GPU; neither kernel waits for the other."""
import ctypes
import multiprocessing as mp

import pytest
import torch

pytestmark = pytest.mark.gpu

ROWS, N_TOTAL, N_LOCAL, BLOCK = 96, 1024, 256, 2      # the peer writes column block 2


def _peer(handle_bytes, offset, conn):
    try:
        import torch as t
        from nvfp4_gemm_b200 import _lib
        lib = _lib.load()
        t.cuda.set_device(0)
        handle = (ctypes.c_uint8 * _lib.COMM_HANDLE_BYTES).from_buffer_copy(handle_bytes)
        remote = ctypes.c_void_p()
        _lib.check(lib.nvfp4_comm_open(handle, offset, ctypes.byref(remote)))
        mine = t.arange(ROWS * N_TOTAL, dtype=t.float32, device="cuda").remainder(2039).half().view(ROWS, N_TOTAL)
        src = (ctypes.c_void_p * 1)(mine.data_ptr() + BLOCK * N_LOCAL * 2)
        dst = (ctypes.c_void_p * 1)(remote.value + BLOCK * N_LOCAL * 2)
        _lib.check(lib.nvfp4_copy_column_blocks(dst, src, 1, 0, ROWS, N_LOCAL, N_TOTAL, 0, 0, None))
        t.cuda.synchronize()
        _lib.check(lib.nvfp4_comm_close(remote, offset))
        conn.send("ok")
    except Exception as e:  # noqa: BLE001
        conn.send(f"peer failed: {e!r}")


def test_a_second_process_pushes_into_an_exported_buffer(lib):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from nvfp4_gemm_b200 import _lib
    c = torch.zeros((ROWS, N_TOTAL), dtype=torch.float16, device="cuda")
    handle = (ctypes.c_uint8 * _lib.COMM_HANDLE_BYTES)()
    offset = ctypes.c_int64()
    _lib.check(lib.nvfp4_comm_export(c.data_ptr(), handle, ctypes.byref(offset)))
    torch.cuda.synchronize()
    ctx = mp.get_context("spawn")
    parent, child = ctx.Pipe()
    proc = ctx.Process(target=_peer, args=(bytes(handle), offset.value, child))
    proc.start()
    assert parent.poll(120), "the peer process did not answer"
    msg = parent.recv()
    proc.join(30)
    assert msg == "ok", msg
    torch.cuda.synchronize()
    want = torch.arange(ROWS * N_TOTAL, dtype=torch.float32, device="cuda").remainder(2039).half().view(ROWS, N_TOTAL)
    lo, hi = BLOCK * N_LOCAL, (BLOCK + 1) * N_LOCAL
    assert torch.equal(c[:, lo:hi], want[:, lo:hi])
    assert int(c[:, :lo].abs().sum().item()) == 0 and int(c[:, hi:].abs().sum().item()) == 0     # nothing else was touched


def test_comm_argument_checks(lib):
    from nvfp4_gemm_b200 import _lib
    off = ctypes.c_int64()
    assert lib.nvfp4_comm_export(None, None, ctypes.byref(off)) == _lib.NVFP4_ERR_INVALID_ARGUMENT
    out = ctypes.c_void_p()
    assert lib.nvfp4_comm_open(None, 0, ctypes.byref(out)) == _lib.NVFP4_ERR_INVALID_ARGUMENT
    assert lib.nvfp4_comm_close(None, 0) == _lib.NVFP4_ERR_INVALID_ARGUMENT
