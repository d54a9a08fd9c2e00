"""Eigenvalue maps that turn a (damped) spectrum into an inverse multiplier.

With ``c`` the damping factor, ``l`` an eigenvalue and ``mean`` the mean of the whole
spectrum (reference ``bergson/hessians/inversion.py:43-218``):

* ``damped_inverse``     ``1 / (l + c*mean)``
* ``tikhonov_filtered``  ``l / (l^2 + (c*mean)^2)``
* ``pseudoinverse``      ``1/l`` if ``l > c*mean`` else ``0``
* ``factored_tikhonov``  ``1 / (l + pi*sqrt(g)*l_G + sqrt(g)/pi*l_A + g)`` with
  ``g = c*mean`` and ``pi = sqrt(mean(l_A) / mean(l_G))`` (Kronecker-factored only)

``power = -0.5`` takes the square root of the multiplier so that applying it twice
gives the full inverse.
"""

from __future__ import annotations

from typing import Callable, Literal

import torch
from torch import Tensor

Inversion = Literal["damped_inverse", "factored_tikhonov", "pseudoinverse", "tikhonov_filtered"]
INVERSIONS: tuple[str, ...] = ("damped_inverse", "factored_tikhonov", "pseudoinverse", "tikhonov_filtered")


def damped_inverse_eigfn(eigvals: Tensor, mean: Tensor, damping_factor: float) -> Tensor:
    return 1.0 / (eigvals + damping_factor * mean)


def tikhonov_filtered_eigfn(eigvals: Tensor, mean: Tensor, damping_factor: float) -> Tensor:
    alpha = damping_factor * mean
    return eigvals / (eigvals.square() + alpha * alpha)


def pseudoinverse_eigfn(eigvals: Tensor, mean: Tensor, damping_factor: float) -> Tensor:
    keep = eigvals > damping_factor * mean
    return torch.where(keep, 1.0 / eigvals, torch.zeros_like(eigvals))


EIGENFNS: dict[str, Callable[[Tensor, Tensor, float], Tensor]] = {
    "damped_inverse": damped_inverse_eigfn,
    "tikhonov_filtered": tikhonov_filtered_eigfn,
    "pseudoinverse": pseudoinverse_eigfn,
}


def factored_tikhonov_damped(eigvals, factor_a, factor_g, mean, mean_a, mean_g, damping_factor: float) -> Tensor:
    """Damped eigenvalue grid ``[O, I]`` before inversion; ``factor_a`` [I] and
    ``factor_g`` [O] are the per-factor eigenvalues.  Means are passed in so that a
    sharded caller can supply global values."""
    tiny = torch.finfo(eigvals.dtype).tiny
    gamma = damping_factor * mean
    root = gamma.clamp_min(0).sqrt()
    pi = (mean_a / mean_g.clamp_min(tiny)).clamp_min(tiny).sqrt()
    return eigvals + (pi * root) * factor_g[:, None] + (root / pi) * factor_a[None, :] + gamma


def eigenvalue_multiplier(
    inversion: str,
    eigvals: Tensor,
    mean: Tensor,
    damping_factor: float,
    *,
    factor_a: Tensor | None = None,
    factor_g: Tensor | None = None,
    mean_a: Tensor | None = None,
    mean_g: Tensor | None = None,
    power: float = -1.0,
) -> Tensor:
    """Elementwise multiplier ``m(l)`` for ``inversion`` at matrix power ``power``."""
    if inversion == "factored_tikhonov":
        assert None not in (factor_a, factor_g, mean_a, mean_g), (
            "factored_tikhonov needs the per-factor eigenvalues and their means"
        )
        m = 1.0 / factored_tikhonov_damped(eigvals, factor_a, factor_g, mean, mean_a, mean_g, damping_factor)
    else:
        m = EIGENFNS[inversion](eigvals, mean, damping_factor)
    if -power != 1.0:
        m = m.clamp_min(0).pow(-power)
    return m


def invert_psd_matrix(
    H: Tensor,
    inversion: str = "damped_inverse",
    damping_factor: float = 0.1,
    power: float = -1.0,
    dtype: torch.dtype = torch.float64,
) -> Tensor:
    """``Q m(L) Q^T`` of a p.s.d. matrix through an fp64 ``eigh`` (negative round-off
    eigenvalues clamped to zero).  ``factored_tikhonov`` has no dense form and falls
    back to ``damped_inverse``."""
    out_dtype = H.dtype
    vals, vecs = torch.linalg.eigh(H.to(dtype))
    vals = vals.clamp_min(0)
    mode = "damped_inverse" if inversion == "factored_tikhonov" else inversion
    m = eigenvalue_multiplier(mode, vals, vals.mean(), damping_factor, power=power)
    return ((vecs * m) @ vecs.mH).to(out_dtype)
