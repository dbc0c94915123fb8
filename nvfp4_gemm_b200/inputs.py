"""Synthetic inputs with the reference's tensor contract.

The leaderboard harness that generated inputs for the reference
(``generate_input`` in the ``reference.py`` named at task.yml:5) is not part of
the reference repository, so seeded synthetic tensors stand in for it.  They
follow every layout fact the reference pins:

* ``a`` [M, K/2, L], ``b`` [N, K/2, L]: ``float4_e2m1fn_x2`` (two nibbles per
  byte), strides (K/2, 1, rows*K/2) -- template.py:9-22, ref.txt:31;
* ``sfa`` [M, K/16, L], ``sfb`` [N, K/16, L]: ``float8_e4m3fn``;
* ``sfa_permuted`` [32, 4, rest_m, 4, rest_k, L] with strides
  (16, 4, rest_k*512, 1, 512, rest_m*rest_k*512) -- ref.txt:31, s_128t.py:554-562;
* ``c`` [M, N, L] fp16, strides (N, 1, M*N) -- submission.py:507-509.

Value distribution: every nibble uniform over the 16 e2m1 codes, every scale
2^u with u uniform in [-3, 3].
"""
from __future__ import annotations

import torch

from .task import TestSpec

FP4_DTYPE = torch.float4_e2m1fn_x2
SF_DTYPE = torch.float8_e4m3fn


def ceil_div(a: int, b: int) -> int:
    return (a + b - 1) // b


def permute_scale_factors(sf_u8: torch.Tensor) -> torch.Tensor:
    """Plain scale bytes [L, rows, K/16] (uint8) -> the six-dimensional permuted view
    [32, 4, rest_rows, 4, rest_k, L] whose memory is 512-byte atoms of 128 rows x 4 scales
    (ref.txt:31).  Rows are zero-padded to a multiple of 128."""
    L, rows, cols = sf_u8.shape
    if cols % 4:
        raise ValueError("K must be a multiple of 64")
    rest_r, rest_k = ceil_div(rows, 128), cols // 4
    padded = torch.zeros((L, rest_r * 128, cols), dtype=torch.uint8, device=sf_u8.device)
    padded[:, :rows] = sf_u8
    # row = rr*128 + r4*32 + r32 ; col = kk*4 + k4  ->  memory order [L][rr][kk][r32][r4][k4]
    mem = padded.view(L, rest_r, 4, 32, rest_k, 4).permute(0, 1, 4, 3, 2, 5).contiguous()
    # logical order (r32, r4, rr, k4, kk, L)
    return mem.permute(3, 4, 1, 5, 2, 0)


def _random_fp4(rows: int, k: int, l: int, gen: torch.Generator, device) -> torch.Tensor:
    raw = torch.randint(0, 256, (l, rows, k // 2), dtype=torch.uint8, generator=gen, device="cpu")
    return raw.to(device).permute(1, 2, 0).view(FP4_DTYPE)


def _random_sf(rows: int, k: int, l: int, gen: torch.Generator, device):
    u = torch.randint(-3, 4, (l, rows, k // 16), dtype=torch.int32, generator=gen, device="cpu")
    sf_u8 = ((u + 7) << 3).to(torch.uint8).to(device)           # e4m3 (bias 7) encoding of 2^u
    plain = sf_u8.permute(1, 2, 0).view(SF_DTYPE)
    permuted = permute_scale_factors(sf_u8).view(SF_DTYPE)
    return plain, permuted


def generate_input(m: int, n: int, k: int, l: int, seed: int, device="cuda"):
    """Build the 7-tuple (a, b, sfa, sfb, sfa_permuted, sfb_permuted, c).  ``n == 1`` gives the
    GEMV form (task_gemv.yml:18-22): b is [1, K/2, L] and c is [M, 1, L]."""
    if k % 64:
        raise ValueError("K must be a multiple of 64")
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    a = _random_fp4(m, k, l, gen, device)
    b = _random_fp4(n, k, l, gen, device)
    sfa, sfa_perm = _random_sf(m, k, l, gen, device)
    sfb, sfb_perm = _random_sf(n, k, l, gen, device)
    c = torch.empty((l, m, n), dtype=torch.float16, device=device).permute(1, 2, 0)
    return a, b, sfa, sfb, sfa_perm, sfb_perm, c


def generate_from_spec(spec: TestSpec, device="cuda"):
    return generate_input(spec["m"], spec["n"], spec["k"], spec["l"], spec["seed"], device=device)
