"""CPU oracle for the NVFP4 block-scaled matmul path.  TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the bench's CPU-baseline leg may import
this module; the product path (``nvfp4_gemm_b200``) never does and fails loudly
when its CUDA library is missing.

PARITY PINNED by outputs of the reference's own code: its cuBLASLt submission
(sub_cub.py:48-143, bound by custom_kernel at sub_cub.py:165-169) is compiled from the
reference's source by ``oracle/build_ref.py`` and run on a B200 on this repository's
seeded inputs -- live in ``tests/test_reference_pin_gpu.py`` and as committed fixtures
``tests/golden/ref_cublaslt.json`` (config 0, the test shapes of task.yml:41-51 and the
benchmark shapes of task.yml:53-56), which ``tests/test_oracle_cpu.py`` holds this oracle
to bit for bit.  The reference holds no golden vectors, no CPU implementation and no tests
of its own for this path, and the harness file that defines ``ref_kernel`` (named at
task.yml:5 as ``reference.py``) is not part of it, so the arithmetic below restates the
published definition of the operator -- dequantise to fp32, accumulate in fp32, cast to
fp16 -- using the layout facts the reference does pin:

* tensor shapes / dtypes / packing: template.py:9-22, task.yml:18-22
  (``a`` is [M, K/2, L] bytes, two e2m1 nibbles per byte, K-major);
* one scale factor per 16 consecutive K elements: submission.py:29
  (``sf_vec_size = 16``), sub_cub.py:77-88 (VEC16_UE4M3);
* scale bytes are e4m3 with bias 7 (hardware "UE4M3"): s_128t.py:88 (idesc bit
  23 = 0), sub_cub.py:77;
* permuted scale layout [32, 4, rest_m, 4, rest_k, L] with strides
  (16, 4, rest_k*512, 1, 512, rest_m*rest_k*512): ref.txt:31, s_128t.py:554-562;
* per-16-block semantics (exact block dot product, times sfa*sfb, fp32
  accumulate): old_files/sub_gemm.py:170-174,211-218.

Further pins used by the tests: torch's own ``float8_e4m3fn -> float32``
conversion for the scale decode, hand-computable known-answer cases, fp64
re-computation, and (on a GPU) cuBLASLt's block-scaled FP4 matmul, which is the
library call the reference configures in sub_cub.py:67-133.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent

# e2m1 code -> value (submission.py:23-29 names the format; the table is the
# OCP FP4 E2M1 definition: sign, 2-bit exponent bias 1, 1-bit mantissa).
E2M1_LUT = np.array(
    [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
     -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], dtype=np.float32)


def e4m3fn_to_f32(byte_values: np.ndarray) -> np.ndarray:
    """Decode e4m3 "fn" bytes (bias 7, no inf, 0x7f/0xff = NaN) to float32."""
    b = np.asarray(byte_values, dtype=np.uint8).astype(np.int32)
    sign = np.where(b & 0x80, -1.0, 1.0)
    exp = (b >> 3) & 0xF
    man = b & 0x7
    normal = (1.0 + man / 8.0) * np.exp2(exp.astype(np.float64) - 7.0)
    subnormal = (man / 8.0) * 2.0 ** -6
    val = np.where(exp == 0, subnormal, normal)
    val = np.where((exp == 15) & (man == 7), np.nan, val)
    return (sign * val).astype(np.float32)


E4M3_LUT = e4m3fn_to_f32(np.arange(256, dtype=np.uint8))


def unpack_e2m1(packed: np.ndarray) -> np.ndarray:
    """[rows, K/2] bytes -> [rows, K] float32; low nibble is the lower k
    (template.py:22: the k extent of ``a``/``b`` is really k/2 bytes)."""
    p = np.asarray(packed, dtype=np.uint8)
    out = np.empty(p.shape[:-1] + (p.shape[-1] * 2,), dtype=np.float32)
    out[..., 0::2] = E2M1_LUT[p & 0xF]
    out[..., 1::2] = E2M1_LUT[p >> 4]
    return out


def dequantize(packed: np.ndarray, sf: np.ndarray) -> np.ndarray:
    """e2m1 value times its block's e4m3 scale, in fp32 (exact: <= 6 significant bits)."""
    vals = unpack_e2m1(packed)
    scale = E4M3_LUT[np.asarray(sf, dtype=np.uint8)]
    return vals * np.repeat(scale, 16, axis=-1)


def ref_gemm(a, b, sfa, sfb, accumulate="f32") -> np.ndarray:
    """C[M,N,L] fp16 = dequant(A) . dequant(B)^T for every batch l.

    a: [M, K/2, L] uint8, b: [N, K/2, L] uint8, sfa: [M, K/16, L], sfb: [N, K/16, L]
    (plain scale layout).  ``accumulate='f64'`` recomputes in double as a check on
    the fp32 accumulation.  A GEMV is the N == 1 case (task_gemv.yml:18-22).
    """
    a, b, sfa, sfb = (np.asarray(x, dtype=np.uint8) for x in (a, b, sfa, sfb))
    M, _, L = a.shape
    N = b.shape[0]
    c = np.empty((M, N, L), dtype=np.float16)
    dt = np.float64 if accumulate == "f64" else np.float32
    for l in range(L):
        aq = dequantize(a[:, :, l], sfa[:, :, l]).astype(dt)
        bq = dequantize(b[:, :, l], sfb[:, :, l]).astype(dt)
        with np.errstate(over="ignore"):
            c[:, :, l] = (aq @ bq.T).astype(np.float32).astype(np.float16)
    return c


def ref_gemm_f32(a, b, sfa, sfb) -> np.ndarray:
    """The accumulator before the fp16 cast: [M, N, L] fp32 (numpy path; small shapes)."""
    a, b, sfa, sfb = (np.asarray(x, dtype=np.uint8) for x in (a, b, sfa, sfb))
    M, _, L = a.shape
    N = b.shape[0]
    c = np.empty((M, N, L), dtype=np.float32)
    for l in range(L):
        c[:, :, l] = dequantize(a[:, :, l], sfa[:, :, l]) @ dequantize(b[:, :, l], sfb[:, :, l]).T
    return c


def ref_epilogue(acc: np.ndarray, bias=None, activation: str = "none") -> np.ndarray:
    """What the GEMM's extended epilogue computes from the fp32 accumulator [M, N, L]:
    fp16(act(acc + bias[column])), the bias added in fp32.  No counterpart in the reference
    (it writes the plain fp16 cast, sub_cub.py:98-104); the definition is this library's."""
    x = np.asarray(acc, dtype=np.float32)
    if bias is not None:
        x = x + np.asarray(bias, dtype=np.float16).astype(np.float32)[None, :, None]
    if activation == "relu":
        x = np.maximum(x, np.float32(0))
    elif activation == "silu":
        with np.errstate(over="ignore"):
            x = (x.astype(np.float64) / (1.0 + np.exp(-x.astype(np.float64)))).astype(np.float32)
    elif activation != "none":
        raise ValueError(activation)
    with np.errstate(over="ignore"):
        return x.astype(np.float16)


def ref_requantize(c16: np.ndarray):
    """NVFP4 form of an fp16 result [M, N, L]: (packed [M, N/2, L], sf [M, N/16, L]), the
    quantiser's rule (:func:`quantize_rows`) applied to every batch."""
    M, N, L = c16.shape
    packed = np.empty((M, N // 2, L), dtype=np.uint8)
    sf = np.empty((M, N // 16, L), dtype=np.uint8)
    for l in range(L):
        packed[:, :, l], sf[:, :, l] = quantize_rows(c16[:, :, l].astype(np.float32))
    return packed, sf


def permuted_sf_offset(row, col, n_kblk):
    """Byte offset of scale (row, col = k/16) inside one batch of the permuted
    layout (ref.txt:31; s_128t.py:42-45,554-562): 512-byte atoms of 128 rows x 4
    scales, atoms K-major inside a 128-row block."""
    return ((row // 128) * n_kblk + (col // 4)) * 512 + (row % 32) * 16 + ((row // 32) % 4) * 4 + (col % 4)


def permute_sf(sf: np.ndarray) -> np.ndarray:
    """Plain [rows, K/16, L] bytes -> flat permuted bytes [L * ceil(rows/128) * K/64 * 512],
    rows padded to a multiple of 128 with zero bytes."""
    sf = np.asarray(sf, dtype=np.uint8)
    rows, cols, L = sf.shape
    assert cols % 4 == 0
    n_kblk = cols // 4
    n_rblk = (rows + 127) // 128
    out = np.zeros((L, n_rblk * n_kblk * 512), dtype=np.uint8)
    r = np.arange(rows)[:, None]
    c = np.arange(cols)[None, :]
    off = permuted_sf_offset(r, c, n_kblk)
    for l in range(L):
        out[l, off] = sf[:, :, l]
    return out.reshape(-1)


def unpermute_sf(flat: np.ndarray, rows: int, cols: int, L: int) -> np.ndarray:
    """Inverse of :func:`permute_sf` (drops the row padding)."""
    flat = np.asarray(flat, dtype=np.uint8).reshape(L, -1)
    r = np.arange(rows)[:, None]
    c = np.arange(cols)[None, :]
    off = permuted_sf_offset(r, c, cols // 4)
    out = np.empty((rows, cols, L), dtype=np.uint8)
    for l in range(L):
        out[:, :, l] = flat[l, off]
    return out


def ref_gemm_from_permuted(a, b, sfa_perm_flat, sfb_perm_flat) -> np.ndarray:
    """Same result as :func:`ref_gemm`, but reading the permuted scale tensors
    (what the tensor-core kernels of the reference consume, s_128t.py:556-577)."""
    M, kb, L = a.shape
    N = b.shape[0]
    sfa = unpermute_sf(sfa_perm_flat, M, kb // 8, L)
    sfb = unpermute_sf(sfb_perm_flat, N, kb // 8, L)
    return ref_gemm(a, b, sfa, sfb)


def quantize_rows(x: np.ndarray):
    """Reference statement of the NVFP4 quantiser that precedes the path
    (contract rows for the element formats: submission.py:23-29): per 16
    consecutive K elements, scale = e4m3(max|x| / 6) rounded to nearest-even,
    elements = round-to-nearest-even onto the e2m1 grid of x / scale.
    Returns (packed [rows, K/2] uint8, sf [rows, K/16] uint8)."""
    x = np.asarray(x, dtype=np.float32)
    rows, K = x.shape
    blocks = x.reshape(rows, K // 16, 16)
    amax = np.abs(blocks).max(axis=-1)
    sf_bytes = f32_to_e4m3fn(amax / np.float32(6.0))
    scale = E4M3_LUT[sf_bytes]
    with np.errstate(divide="ignore", invalid="ignore"):
        y = np.where(scale[..., None] > 0, blocks / scale[..., None], 0.0).astype(np.float32)
    codes = f32_to_e2m1(y).reshape(rows, K)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    return packed, sf_bytes


def f32_to_e4m3fn(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even, saturating (to 448) conversion of non-negative fp32 to e4m3fn bytes."""
    x = np.asarray(x, dtype=np.float32)
    grid = E4M3_LUT[:0x7F].astype(np.float64)        # 0 .. 448, ascending
    xv = np.clip(x.astype(np.float64), 0.0, 448.0)
    idx = np.searchsorted(grid, xv, side="left")
    idx = np.clip(idx, 1, len(grid) - 1)
    lo, hi = grid[idx - 1], grid[idx]
    pick_hi = (xv - lo) > (hi - xv)
    tie = (xv - lo) == (hi - xv)
    res = np.where(pick_hi, idx, idx - 1)
    res = np.where(tie, np.where((idx % 2) == 0, idx, idx - 1), res)   # even code wins ties
    res = np.where(xv <= 0, 0, res)
    return res.astype(np.uint8)


def f32_to_e2m1(y: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even (ties to the even mantissa code), saturating to +-6."""
    y = np.asarray(y, dtype=np.float32)
    mag = np.minimum(np.abs(y).astype(np.float64), 6.0)
    grid = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
    idx = np.clip(np.searchsorted(grid, mag, side="left"), 1, 7)
    lo, hi = grid[idx - 1], grid[idx]
    pick_hi = (mag - lo) > (hi - mag)
    tie = (mag - lo) == (hi - mag)
    res = np.where(pick_hi, idx, idx - 1)
    res = np.where(tie, np.where((idx % 2) == 0, idx, idx - 1), res)
    res = np.where(mag == 0, 0, res)
    sign = (np.signbit(y)).astype(np.int64) << 3
    return (res | sign).astype(np.uint8)


# --------------------------------------------------------------------------
# C restatement (oracle/nvfp4_oracle.c), used where numpy is too slow and as
# the timed CPU baseline.
# --------------------------------------------------------------------------
_LIB = None


def c_lib_path() -> Path:
    return _HERE / "libnvfp4_oracle.so"


def build_c(force: bool = False) -> Path:
    so = c_lib_path()
    src = _HERE / "nvfp4_oracle.c"
    if force or not so.exists() or so.stat().st_mtime < src.stat().st_mtime:
        subprocess.check_call(["make", "-C", str(_HERE), "-s", "libnvfp4_oracle.so"])
    return so


def _lib():
    global _LIB
    if _LIB is None:
        so = c_lib_path()
        if not so.exists():
            build_c()
        lib = ctypes.CDLL(str(so))
        lib.nvfp4_oracle_gemm.restype = ctypes.c_int
        lib.nvfp4_oracle_gemm.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int] * 5
        lib.nvfp4_oracle_max_threads.restype = ctypes.c_int
        _LIB = lib
    return _LIB


def c_max_threads() -> int:
    return int(_lib().nvfp4_oracle_max_threads())


def ref_gemm_c(a, b, sfa, sfb, permuted_sf: bool = False, threads: int = 0) -> np.ndarray:
    """C oracle, one batch at a time.  With ``permuted_sf`` the scale arguments are the
    flat permuted byte arrays (all batches), otherwise plain [rows, K/16, L]."""
    a = np.asarray(a, dtype=np.uint8)
    b = np.asarray(b, dtype=np.uint8)
    M, kb, L = a.shape
    N = b.shape[0]
    K = kb * 2
    c = np.empty((M, N, L), dtype=np.float16)
    lib = _lib()
    if permuted_sf:
        sfa_f = np.ascontiguousarray(np.asarray(sfa, dtype=np.uint8).reshape(L, -1))
        sfb_f = np.ascontiguousarray(np.asarray(sfb, dtype=np.uint8).reshape(L, -1))
    for l in range(L):
        al = np.ascontiguousarray(a[:, :, l])
        bl = np.ascontiguousarray(b[:, :, l])
        if permuted_sf:
            sa, sb = sfa_f[l], sfb_f[l]
        else:
            sa = np.ascontiguousarray(np.asarray(sfa, dtype=np.uint8)[:, :, l])
            sb = np.ascontiguousarray(np.asarray(sfb, dtype=np.uint8)[:, :, l])
        cl = np.empty((M, N), dtype=np.float16)
        rc = lib.nvfp4_oracle_gemm(al.ctypes.data, bl.ctypes.data, sa.ctypes.data, sb.ctypes.data,
                                   cl.ctypes.data, M, N, K, 1 if permuted_sf else 0, threads)
        if rc != 0:
            raise RuntimeError(f"nvfp4_oracle_gemm failed with code {rc}")
        c[:, :, l] = cl
    return c


def tensors_to_numpy(data):
    """(a, b, sfa, sfb, sfa_permuted, sfb_permuted, c) torch tensors -> numpy byte views
    (a, b, sfa, sfb) in their logical [rows, cols, L] shape."""
    import torch

    def as_u8(t):
        return t.detach().cpu().view(torch.uint8).numpy()

    a, b, sfa, sfb = data[0], data[1], data[2], data[3]
    return as_u8(a), as_u8(b), as_u8(sfa), as_u8(sfb)


if __name__ == "__main__":
    print(build_c(force=True))
