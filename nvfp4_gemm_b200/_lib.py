"""ctypes binding of ``libnvfp4_b200.so`` (the C ABI in ``include/nvfp4_b200.h``).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int, c_int32, c_int64, c_size_t, c_uint64, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libnvfp4_b200.so"

NVFP4_OK = 0
NVFP4_ERR_INVALID_ARGUMENT = -1
NVFP4_ERR_CUDA = -2
NVFP4_ERR_DEVICE_TIMEOUT = -3
NVFP4_ERR_UNSUPPORTED = -4

EXPORTED_SYMBOLS = (
    "nvfp4_gemm", "nvfp4_gemv", "nvfp4_matmul", "nvfp4_check_status", "nvfp4_set_wait_timeout_ns",
    "nvfp4_selftest_bounded_wait", "nvfp4_scratch_bytes", "nvfp4_launch_count", "nvfp4_last_kernel",
    "nvfp4_shutdown", "nvfp4_last_error", "nvfp4_version", "nvfp4_plan_units", "nvfp4_gemm_static_scratch",
    "nvfp4_interleave_column_blocks", "nvfp4_permute_scales", "nvfp4_gemm_allgather", "nvfp4_quantize", "nvfp4_copy_2d", "nvfp4_copy_column_blocks",
    "nvfp4_unpermute_scales", "nvfp4_compare_scale_layouts", "nvfp4_gemv_config", "nvfp4_release_stream",
    "nvfp4_gemm_epilogue", "nvfp4_plan_tile", "nvfp4_plan_segment", "nvfp4_plan_work_split", "nvfp4_plan_tile_shape", "nvfp4_set_peer_tma_limit", "nvfp4_comm_export", "nvfp4_comm_open", "nvfp4_comm_close",
)
COMM_HANDLE_BYTES = 64

ACT_NONE, ACT_RELU, ACT_SILU = 0, 1, 2
OUT_FP16, OUT_NVFP4 = 0, 1


class Nvfp4Error(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"nvfp4_b200 error {code}: {message}")
        self.code = code


class Problem(ctypes.Structure):
    """Mirror of ``struct nvfp4_problem``."""
    _fields_ = [
        ("a", c_void_p), ("b", c_void_p), ("sfa", c_void_p), ("sfb", c_void_p),
        ("sfa_perm", c_void_p), ("sfb_perm", c_void_p), ("c", c_void_p),
        ("m", c_int32), ("n", c_int32), ("k", c_int32), ("l", c_int32),
        ("a_row_stride", c_int64), ("a_batch_stride", c_int64),
        ("b_row_stride", c_int64), ("b_batch_stride", c_int64),
        ("sfa_row_stride", c_int64), ("sfa_batch_stride", c_int64),
        ("sfb_row_stride", c_int64), ("sfb_batch_stride", c_int64),
        ("sfa_perm_batch_stride", c_int64), ("sfb_perm_batch_stride", c_int64),
        ("c_row_stride", c_int64), ("c_batch_stride", c_int64),
    ]


class GemmConfig(ctypes.Structure):
    """Mirror of ``struct nvfp4_gemm_config``."""
    _fields_ = [("tile_n", c_int32), ("epilogue", c_int32), ("grid", c_int32), ("cta_group", c_int32),
                ("split_k", c_int32), ("raster", c_int32)]


class Epilogue(ctypes.Structure):
    """Mirror of ``struct nvfp4_epilogue``."""
    _fields_ = [
        ("bias", c_void_p), ("activation", c_int32), ("output", c_int32),
        ("out_packed", c_void_p), ("out_sf", c_void_p), ("out_sf_perm", c_void_p),
        ("out_packed_row_stride", c_int64), ("out_packed_batch_stride", c_int64),
        ("out_sf_row_stride", c_int64), ("out_sf_batch_stride", c_int64),
        ("out_sf_perm_batch_stride", c_int64), ("out_sf_perm_block_stride", c_int64),
    ]


_lib = None


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m nvfp4_gemm_b200.build` "
            "(there is no CPU or PyTorch fallback for this operator)")
    lib = ctypes.CDLL(str(LIB_PATH))
    lib.nvfp4_gemm.argtypes = [ctypes.POINTER(Problem), ctypes.POINTER(GemmConfig), c_void_p]
    lib.nvfp4_gemm.restype = c_int
    lib.nvfp4_gemm_epilogue.argtypes = [ctypes.POINTER(Problem), ctypes.POINTER(GemmConfig), ctypes.POINTER(Epilogue), c_void_p]
    lib.nvfp4_gemm_epilogue.restype = c_int
    lib.nvfp4_gemm_static_scratch.argtypes = [ctypes.POINTER(Problem), c_int, c_void_p]
    lib.nvfp4_gemm_static_scratch.restype = c_int
    lib.nvfp4_interleave_column_blocks.argtypes = [c_void_p, c_void_p, c_int64, c_int32, c_int32, c_int64, c_void_p]
    lib.nvfp4_interleave_column_blocks.restype = c_int
    lib.nvfp4_gemm_allgather.argtypes = [ctypes.POINTER(Problem), ctypes.POINTER(GemmConfig), ctypes.POINTER(c_void_p), c_int, c_void_p]
    lib.nvfp4_gemm_allgather.restype = c_int
    lib.nvfp4_unpermute_scales.argtypes = [c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int64, c_int64, c_int64, c_void_p]
    lib.nvfp4_unpermute_scales.restype = c_int
    lib.nvfp4_compare_scale_layouts.argtypes = [c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int64, c_int64, c_int64, c_void_p, c_void_p]
    lib.nvfp4_compare_scale_layouts.restype = c_int
    lib.nvfp4_copy_column_blocks.argtypes = [ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p), c_int32, c_int64, c_int64, c_int32,
                                             c_int64, c_int32, c_int32, c_void_p]
    lib.nvfp4_copy_column_blocks.restype = c_int
    lib.nvfp4_copy_2d.argtypes = [c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64, c_void_p]
    lib.nvfp4_copy_2d.restype = c_int
    lib.nvfp4_quantize.argtypes = [c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int64, c_int64, c_int64, c_void_p]
    lib.nvfp4_quantize.restype = c_int
    lib.nvfp4_permute_scales.argtypes = [c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int64, c_int64, c_int64, c_void_p]
    lib.nvfp4_permute_scales.restype = c_int
    lib.nvfp4_gemv.argtypes = [ctypes.POINTER(Problem), c_void_p]
    lib.nvfp4_gemv.restype = c_int
    lib.nvfp4_gemv_config.argtypes = [ctypes.POINTER(Problem), c_int, c_int, c_void_p]
    lib.nvfp4_gemv_config.restype = c_int
    lib.nvfp4_matmul.argtypes = [ctypes.POINTER(Problem), c_void_p]
    lib.nvfp4_matmul.restype = c_int
    lib.nvfp4_release_stream.argtypes = [c_void_p]
    lib.nvfp4_release_stream.restype = c_int
    lib.nvfp4_check_status.argtypes = [c_void_p]
    lib.nvfp4_check_status.restype = c_int
    lib.nvfp4_set_wait_timeout_ns.argtypes = [c_uint64]
    lib.nvfp4_set_wait_timeout_ns.restype = c_uint64
    lib.nvfp4_selftest_bounded_wait.argtypes = [c_void_p]
    lib.nvfp4_selftest_bounded_wait.restype = c_int
    lib.nvfp4_scratch_bytes.argtypes = []
    lib.nvfp4_scratch_bytes.restype = c_size_t
    lib.nvfp4_plan_units.argtypes = [c_int, c_int, c_int, ctypes.POINTER(c_int), ctypes.POINTER(c_int),
                                     ctypes.POINTER(c_int), c_int]
    lib.nvfp4_plan_units.restype = c_int
    lib.nvfp4_comm_export.argtypes = [c_void_p, c_void_p, ctypes.POINTER(c_int64)]
    lib.nvfp4_comm_export.restype = c_int
    lib.nvfp4_comm_open.argtypes = [c_void_p, c_int64, ctypes.POINTER(c_void_p)]
    lib.nvfp4_comm_open.restype = c_int
    lib.nvfp4_comm_close.argtypes = [c_void_p, c_int64]
    lib.nvfp4_comm_close.restype = c_int
    lib.nvfp4_plan_tile.argtypes = [c_int] * 7 + [ctypes.POINTER(c_int)] * 3
    lib.nvfp4_plan_tile.restype = c_int
    lib.nvfp4_plan_work_split.argtypes = [ctypes.c_int64, c_int, c_int, ctypes.POINTER(c_int), ctypes.POINTER(c_int)]
    lib.nvfp4_plan_work_split.restype = c_int
    lib.nvfp4_plan_tile_shape.argtypes = [c_int] * 5 + [ctypes.POINTER(c_int)] * 2
    lib.nvfp4_plan_tile_shape.restype = c_int
    lib.nvfp4_set_peer_tma_limit.argtypes = [c_int]
    lib.nvfp4_set_peer_tma_limit.restype = c_int
    lib.nvfp4_plan_segment.argtypes = [c_int] * 5 + [ctypes.POINTER(c_int)] * 2
    lib.nvfp4_plan_segment.restype = c_int
    lib.nvfp4_launch_count.argtypes = []
    lib.nvfp4_launch_count.restype = c_uint64
    lib.nvfp4_last_kernel.argtypes = []
    lib.nvfp4_last_kernel.restype = c_char_p
    lib.nvfp4_shutdown.argtypes = []
    lib.nvfp4_shutdown.restype = None
    lib.nvfp4_last_error.argtypes = []
    lib.nvfp4_last_error.restype = c_char_p
    lib.nvfp4_version.argtypes = []
    lib.nvfp4_version.restype = c_char_p
    _lib = lib
    return lib


def check(rc: int) -> None:
    if rc != NVFP4_OK:
        raise Nvfp4Error(rc, load().nvfp4_last_error().decode())
