"""Optimizers assembled from the transformations."""

from __future__ import annotations

from ..transform import add_decayed_weights, chain, scale_by_adam, scale_by_neg_lr, trace
from ..typing import GradientTransformation


def adamw(lr=1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 1e-2, *, eps_root: float = 0.0,
          moment_requires_grad: bool = False, maximize: bool = False,
          use_accelerated_op: bool = False) -> GradientTransformation:
    if maximize or use_accelerated_op:
        raise NotImplementedError("stand-in: maximize / use_accelerated_op are not provided")
    b1, b2 = betas
    return chain(scale_by_adam(b1, b2, eps, eps_root, moment_requires_grad), add_decayed_weights(weight_decay),
                 scale_by_neg_lr(lr))


def sgd(lr, momentum: float = 0.0, dampening: float = 0.0, weight_decay: float = 0.0, nesterov: bool = False, *,
        moment_requires_grad: bool = False, maximize: bool = False) -> GradientTransformation:
    if maximize:
        raise NotImplementedError("stand-in: maximize is not provided")
    # Coupled weight decay (added to the gradient before the momentum), as in torch.optim.SGD.
    return chain(add_decayed_weights(weight_decay), trace(momentum, dampening, nesterov, moment_requires_grad),
                 scale_by_neg_lr(lr))
