"""The operator entry point, with the reference's signature (template.py:4-25):

    custom_kernel(data) -> c,   data = (a, b, sfa, sfb, sfa_permuted, sfb_permuted, c)

``c`` is pre-allocated by the caller, written in place and returned (template.py:20).
``b.shape[0] == 1`` selects the GEMV (same tuple positions, old_files/1.py:697-698); every
other shape goes to the tensor-core GEMM, which reads the permuted scale tensors like
s_128t.py:605-609.  The work is enqueued on torch's current CUDA stream and not waited for.
All compute happens in the CUDA library behind the C ABI; there is no PyTorch or CPU path.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import GemmConfig, Nvfp4Error, Problem
from .task import input_t, output_t


def _batch_stride(t: torch.Tensor, dim: int = 2) -> int:
    return t.stride(dim) if t.shape[dim] > 1 else 0


def make_problem(data: input_t) -> Problem:
    """Translate the 7-tuple into the C ABI's ``nvfp4_problem`` (pointers, sizes, strides)."""
    a, b, sfa, sfb, sfa_perm, sfb_perm, c = data
    m, k_bytes, l = a.shape
    n = b.shape[0]
    if b.shape[1] != k_bytes or b.shape[2] != l:
        raise ValueError(f"a {tuple(a.shape)} and b {tuple(b.shape)} disagree on k or l")
    if c is not None and tuple(c.shape) != (m, n, l):
        raise ValueError(f"c has shape {tuple(c.shape)}, expected {(m, n, l)}")
    if a.stride(1) != 1 or b.stride(1) != 1 or (c is not None and c.stride(1) != 1 and n > 1):
        raise ValueError("a, b must be K-major (stride 1 along k) and c row-major")
    if a.element_size() != 1 or b.element_size() != 1 or (c is not None and c.dtype != torch.float16) or any(
            t is not None and t.element_size() != 1 for t in (sfa, sfb, sfa_perm, sfb_perm)):
        raise ValueError("expected packed fp4 (1 byte per 2 values), 1-byte scales and fp16 output")
    p = Problem()
    p.a, p.b, p.c = a.data_ptr(), b.data_ptr(), (c.data_ptr() if c is not None else None)
    p.sfa = sfa.data_ptr() if sfa is not None else None
    p.sfb = sfb.data_ptr() if sfb is not None else None
    p.sfa_perm = sfa_perm.data_ptr() if sfa_perm is not None else None
    p.sfb_perm = sfb_perm.data_ptr() if sfb_perm is not None else None
    p.m, p.n, p.k, p.l = m, n, 2 * k_bytes, l
    p.a_row_stride, p.a_batch_stride = a.stride(0), _batch_stride(a)
    p.b_row_stride, p.b_batch_stride = (b.stride(0) if n > 1 else k_bytes), _batch_stride(b)
    if sfa is not None:
        p.sfa_row_stride, p.sfa_batch_stride = sfa.stride(0), _batch_stride(sfa)
    if sfb is not None:
        p.sfb_row_stride, p.sfb_batch_stride = (sfb.stride(0) if n > 1 else k_bytes // 8), _batch_stride(sfb)
    # permuted scales: [32, 4, rest_rows, 4, rest_k, L]; the batch is the last dimension
    p.sfa_perm_batch_stride = _batch_stride(sfa_perm, 5) if sfa_perm is not None else 0
    p.sfb_perm_batch_stride = _batch_stride(sfb_perm, 5) if sfb_perm is not None else 0
    if c is not None:
        p.c_row_stride, p.c_batch_stride = c.stride(0), _batch_stride(c)
    return p


def _require_cuda(data: input_t) -> None:
    if not all(t.is_cuda for t in data if t is not None):
        raise ValueError("custom_kernel needs CUDA tensors (there is no CPU fallback)")


_problem_cache: dict = {}


def _layout_key(t) -> tuple:
    """Everything of a tensor that make_problem() reads: address, shape and strides (None-safe)."""
    return (0, (), ()) if t is None else (t.data_ptr(), tuple(t.shape), tuple(t.stride()))


def _cached_problem(data: input_t) -> Problem:
    """make_problem() is ~40 attribute reads; harnesses call with the same tensors over and over,
    so remember the translated struct by the address, shape and strides of all seven tensors (a
    recycled address with another layout is a different key)."""
    key = tuple(_layout_key(t) for t in data)
    hit = _problem_cache.get(key)
    if hit is None:
        _require_cuda(data)
        if len(_problem_cache) > 256:
            _problem_cache.clear()
        hit = _problem_cache[key] = make_problem(data)
    return hit


def custom_kernel(data: input_t) -> output_t:
    lib = _lib.load()
    problem = _cached_problem(data)
    dev = data[0].device
    stream = torch.cuda.current_stream(dev).cuda_stream
    if torch.cuda.current_device() == dev.index:
        _lib.check(lib.nvfp4_matmul(problem, stream))
    else:
        with torch.cuda.device(dev):
            _lib.check(lib.nvfp4_matmul(problem, stream))
    return data[6]


def gemm(data: input_t, tile_n: int = 0, epilogue: int = 0, grid: int = 0, cta_group: int = 0,
         split_k: int = 0, raster: int = 0) -> output_t:
    """The GEMM with an explicit kernel configuration (tests and tuning)."""
    lib = _lib.load()
    _require_cuda(data)
    problem = make_problem(data)
    cfg = GemmConfig(tile_n, epilogue, grid, cta_group, split_k, raster)
    stream = torch.cuda.current_stream(data[0].device).cuda_stream
    with torch.cuda.device(data[0].device):
        _lib.check(lib.nvfp4_gemm(problem, cfg, stream))
    return data[6]


_ACTIVATIONS = {"none": _lib.ACT_NONE, "relu": _lib.ACT_RELU, "silu": _lib.ACT_SILU}


def gemm_epilogue(data: input_t, bias=None, activation: str = "none", nvfp4_out: bool = False, tile_n: int = 0, grid: int = 0,
                  cta_group: int = 0, split_k: int = 0, out=None):
    """The GEMM with the step that follows it fused into its epilogue: ``act(a @ b.T + bias)``.

    ``nvfp4_out=False`` writes fp16 into ``data[6]`` and returns it.  ``nvfp4_out=True`` returns
    the result re-quantised to NVFP4 as ``(packed, sf, sf_permuted)`` -- [M, N/2, L] packed e2m1,
    [M, N/16, L] e4m3 scales and the same scales in the permuted atom layout -- i.e. the ``a``,
    ``sfa`` and ``sfa_permuted`` of a following ``custom_kernel`` call whose K is this N; ``data[6]``
    may then be None; ``out`` may pass the triple a previous call returned, to be overwritten
    instead of allocating a new one.  The reference writes fp16 only (sub_cub.py:98-104); no
    counterpart."""
    from .inputs import FP4_DTYPE, SF_DTYPE
    lib = _lib.load()
    a, b = data[0], data[1]
    _require_cuda(data)
    m, _, l = a.shape
    n = b.shape[0]
    dev = a.device
    if data[6] is None and not nvfp4_out:
        raise ValueError("an fp16 output needs data[6]")
    problem = make_problem(data)
    epi = _lib.Epilogue()
    if bias is not None:
        if bias.dtype != torch.float16 or bias.numel() != n or not bias.is_contiguous():
            raise ValueError("bias must be a contiguous fp16 vector of length n")
        epi.bias = bias.data_ptr()
    epi.activation = _ACTIVATIONS[activation]
    if not nvfp4_out:
        out = data[6]
    if nvfp4_out:
        rest_m, rest_k = (m + 127) // 128, n // 64
        if out is None:
            packed = torch.empty((l, m, n // 2), dtype=torch.uint8, device=dev)
            sf = torch.empty((l, m, n // 16), dtype=torch.uint8, device=dev)
            sf_perm = torch.empty((l, rest_m, rest_k, 32, 4, 4), dtype=torch.uint8, device=dev)
            out = (packed.permute(1, 2, 0).view(FP4_DTYPE), sf.permute(1, 2, 0).view(SF_DTYPE),
                   sf_perm.permute(3, 4, 1, 5, 2, 0).view(SF_DTYPE))
        epi.output = _lib.OUT_NVFP4
        epi.out_packed, epi.out_sf, epi.out_sf_perm = out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr()
        epi.out_packed_row_stride, epi.out_packed_batch_stride = n // 2, m * (n // 2)
        epi.out_sf_row_stride, epi.out_sf_batch_stride = n // 16, m * (n // 16)
        epi.out_sf_perm_batch_stride = rest_m * rest_k * 512
    cfg = GemmConfig(tile_n, 0, grid, cta_group, split_k, 0)
    stream = torch.cuda.current_stream(dev).cuda_stream
    with torch.cuda.device(dev):
        _lib.check(lib.nvfp4_gemm_epilogue(problem, cfg, epi, stream))
    return out


def check_scale_layouts(data: input_t) -> None:
    """Validate that the plain and the permuted scale tensors of one operator call say the same
    (the harness passes both, template.py:11-14; the GEMM reads the permuted ones, the GEMV the
    plain ones).  Compared on the device by ``nvfp4_compare_scale_layouts``; synchronises the
    current stream and raises ValueError naming the first differing scale."""
    a, b, sfa, sfb, sfa_perm, sfb_perm, _ = data
    _require_cuda(data)
    lib = _lib.load()
    k = 2 * a.shape[1]
    stream = torch.cuda.current_stream(a.device).cuda_stream
    result = torch.empty((2, 2), dtype=torch.int64, device=a.device)
    for i, (name, plain, perm, rows) in enumerate((("sfa", sfa, sfa_perm, a.shape[0]), ("sfb", sfb, sfb_perm, b.shape[0]))):
        if perm is None:
            raise ValueError(f"{name}_permuted is missing")
        _lib.check(lib.nvfp4_compare_scale_layouts(plain.data_ptr(), perm.data_ptr(), rows, k, a.shape[2],
                                                   plain.stride(0) if rows > 1 else k // 16, _batch_stride(plain),
                                                   _batch_stride(perm, 5), result[i].data_ptr(), stream))
    counts = result.cpu()
    for i, (name, rows) in enumerate((("sfa", a.shape[0]), ("sfb", b.shape[0]))):
        bad, first = int(counts[i, 0]), int(counts[i, 1])
        if bad:
            col = first % (k // 16)
            row = (first // (k // 16)) % rows
            batch = first // (k // 16) // rows
            raise ValueError(f"{name} and {name}_permuted differ in {bad} scale(s); first at row {row}, scale column {col}, batch {batch}")


def release_stream(stream=None) -> None:
    """Give back the scratch set the GEMM keeps for ``stream`` (default: the current stream), once
    none of its GEMMs is in flight and no graph captured on it will be replayed again."""
    lib = _lib.load()
    stream = stream if stream is not None else torch.cuda.current_stream()
    _lib.check(lib.nvfp4_release_stream(stream.cuda_stream))


def check_status() -> None:
    """Synchronise the current stream and raise if a kernel reported a timed-out wait."""
    lib = _lib.load()
    _lib.check(lib.nvfp4_check_status(torch.cuda.current_stream().cuda_stream))


def last_kernel() -> str:
    return _lib.load().nvfp4_last_kernel().decode()


def launch_count() -> int:
    return int(_lib.load().nvfp4_launch_count())


__all__ = ["custom_kernel", "gemm", "check_status", "last_kernel", "launch_count", "make_problem", "Nvfp4Error"]
