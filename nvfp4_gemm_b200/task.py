"""Operator API types, mirroring the reference's task.py:4-10."""
from typing import TypedDict, TypeVar

import torch

input_t = TypeVar(
    "input_t",
    bound=tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor],
)
output_t = TypeVar("output_t", bound=torch.Tensor)


class TestSpec(TypedDict):
    m: int
    n: int
    k: int
    l: int
    seed: int
