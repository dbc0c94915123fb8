"""Shared helpers for the parity tests (oracle = checker, never the thing under test)."""
import numpy as np
import torch


def expected_fp16(oracle, data, use_c=True):
    a, b, sfa, sfb = oracle.tensors_to_numpy(data)
    return oracle.ref_gemm_c(a, b, sfa, sfb) if use_c else oracle.ref_gemm(a, b, sfa, sfb)


def assert_bit_exact(got: torch.Tensor, exp: np.ndarray, what=""):
    """fp16 bit patterns equal (so +-inf from overflow must match too)."""
    g = got.detach().cpu().numpy()
    assert g.shape == exp.shape, (g.shape, exp.shape)
    neq = g.view(np.uint16) != exp.view(np.uint16)
    # +0 / -0 compare equal numerically; accept either sign of zero
    neq &= ~((g == 0) & (exp == 0))
    if neq.any():
        idx = np.argwhere(neq)
        i = tuple(idx[0])
        raise AssertionError(f"{what}: {int(neq.sum())} of {neq.size} fp16 values differ; first at {i}: "
                             f"got {g[i]} expected {exp[i]}")


def assert_close(got: torch.Tensor, exp: np.ndarray, rtol=1e-3, atol=1e-3, what=""):
    """The operator's stated tolerance (rtol = atol = 1e-3 on the fp16 output), infs must agree."""
    g = got.detach().cpu().numpy().astype(np.float32)
    e = exp.astype(np.float32)
    assert np.array_equal(np.isinf(g), np.isinf(e)), f"{what}: overflow pattern differs"
    fin = np.isfinite(e)
    np.testing.assert_allclose(g[fin], e[fin], rtol=rtol, atol=atol, err_msg=what)
