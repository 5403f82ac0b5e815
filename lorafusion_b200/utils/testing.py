"""Numerical comparison helpers for kernel tests.

``assert_close_two_rounds`` mirrors the acceptance rule the reference uses for its Triton
kernels (``lorafusion/utils/testing.py:98-188``): a strict ``allclose`` first; if that
fails, the result is still accepted when almost no element is off *and* the error stays
within a small multiple of the rounding error that the low-precision output format itself
introduces.  Unlike the reference's scripts, a failure here raises.
"""

from __future__ import annotations

import torch

DEFAULT_TOL = {
    torch.float32: dict(rtol=1e-5, atol=1e-6),
    torch.float16: dict(rtol=1e-3, atol=1e-4),
    torch.bfloat16: dict(rtol=1.6e-2, atol=1e-4),
}


def mismatch_report(actual: torch.Tensor, expected: torch.Tensor, rtol: float, atol: float,
                    max_print: int = 5) -> tuple[bool, str, float]:
    a = actual.detach().float().cpu()
    e = expected.detach().float().cpu()
    if a.shape != e.shape:
        return False, f"shape mismatch {tuple(a.shape)} vs {tuple(e.shape)}", 1.0
    diff = (a - e).abs()
    tol = atol + rtol * e.abs()
    bad = (diff > tol) | ~torch.isfinite(a)
    nbad = int(bad.sum())
    if nbad == 0:
        return True, "", 0.0
    ratio = nbad / max(a.numel(), 1)
    idx = torch.nonzero(bad)[:max_print]
    lines = [f"{nbad}/{a.numel()} mismatched ({100 * ratio:.4f}%), max abs diff "
             f"{float(diff[torch.isfinite(diff)].max()) if torch.isfinite(diff).any() else float('nan'):.5g}"]
    for i in idx:
        t = tuple(int(v) for v in i)
        lines.append(f"  at {t}: actual {float(a[t]):.6g} expected {float(e[t]):.6g}")
    return False, "\n".join(lines), ratio


def verbose_allclose(actual: torch.Tensor, expected: torch.Tensor, rtol: float | None = None,
                     atol: float | None = None, msg: str = "", print_fn=print) -> bool:
    """``allclose`` that says what differs: prints the count, the share and the first few
    positions of the mismatches and returns whether the tensors are close (it never raises).
    Counterpart of ``verbose_allclose`` in ``lorafusion/utils/testing.py:18-95``."""
    tol = DEFAULT_TOL.get(actual.dtype, DEFAULT_TOL[torch.float32])
    ok, text, _ = mismatch_report(actual, expected, tol["rtol"] if rtol is None else rtol,
                                  tol["atol"] if atol is None else atol)
    if not ok:
        print_fn(f"{msg}: {text}" if msg else text)
    return ok


def assert_close(actual: torch.Tensor, expected: torch.Tensor, rtol: float | None = None,
                 atol: float | None = None, msg: str = "") -> None:
    tol = DEFAULT_TOL.get(actual.dtype, DEFAULT_TOL[torch.float32])
    rtol = tol["rtol"] if rtol is None else rtol
    atol = tol["atol"] if atol is None else atol
    ok, text, _ = mismatch_report(actual, expected, rtol, atol)
    if not ok:
        raise AssertionError(f"{msg}: {text}")


def assert_close_two_rounds(actual: torch.Tensor, expected_fp32: torch.Tensor, *,
                            rtol: float | None = None, atol: float = 5e-3,
                            max_mismatch_ratio: float = 1e-3, rounding_factor: float = 2.5,
                            scale_atol_by_rms: bool = False, msg: str = "") -> None:
    """Compare a low-precision kernel output with an fp32 oracle.

    Strict pass: ``|a - e| <= atol + rtol * |e|`` everywhere.  Relaxed pass (only if that fails):
    fewer than ``max_mismatch_ratio`` of the elements may be off, and they must be within
    ``rounding_factor`` times the largest rounding error that casting the oracle to the
    kernel's output dtype produces.

    ``scale_atol_by_rms`` multiplies ``atol`` by ``max(1, rms(expected))``: long reductions
    with cancelling terms (weight gradients summed over thousands of tokens) carry an
    absolute error proportional to the typical magnitude of the result, not to each element.
    """
    tol = DEFAULT_TOL.get(actual.dtype, DEFAULT_TOL[torch.float32])
    rtol = tol["rtol"] if rtol is None else rtol
    if scale_atol_by_rms:
        atol = atol * max(1.0, float(expected_fp32.detach().float().pow(2).mean().sqrt()))
    ok, text, ratio = mismatch_report(actual, expected_fp32, rtol, atol)
    if ok:
        return
    e = expected_fp32.detach().float().cpu()
    round_err = float((e.to(actual.dtype).float() - e).abs().max()) if actual.dtype != torch.float32 else 0.0
    atol2 = max(atol, rounding_factor * round_err)
    ok2, text2, _ = mismatch_report(actual, expected_fp32, rtol, atol2)
    if ok2 and ratio < max_mismatch_ratio:
        return
    raise AssertionError(f"{msg}: strict pass: {text}\nrelaxed pass (atol {atol2:.4g}): {text2}")
