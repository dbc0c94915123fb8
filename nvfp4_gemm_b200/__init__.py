"""B200-native NVFP4 block-scaled matmul behind the reference's ``custom_kernel(data)`` API."""
from .task import TestSpec, input_t, output_t  # noqa: F401

__all__ = ["TestSpec", "input_t", "output_t"]
