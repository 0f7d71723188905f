"""Shared numeric checks for the GPU tests."""

import torch


def rel_fro(got: torch.Tensor, want: torch.Tensor) -> float:
    """||got - want||_F / ||want||_F in fp32: catches a systematic error of a few percent that a
    max-abs bound on unit-variance data lets through."""
    got, want = got.detach().float(), want.detach().float()
    return ((got - want).norm() / want.norm().clamp_min(1e-20)).item()


def assert_rel_fro(got: torch.Tensor, want: torch.Tensor, tol: float, what: str = "") -> None:
    r = rel_fro(got, want)
    assert r <= tol, f"{what} relative Frobenius error {r:.3e} > {tol:.1e}"
