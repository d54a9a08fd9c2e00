"""Stand-in for the ``torchopt`` package (functional, differentiable optimizers), limited to
what the reference's MAGIC trainer imports: ``adamw``, ``sgd``, ``apply_updates``,
``pytree``, ``typing``, ``combine.chain`` and ``alias.utils``.  Written from the documented
behaviour of those functions with plain tensor operations; no accelerated kernels."""

from . import alias, combine, pytree, transform, typing  # noqa: F401
from .alias import adamw, sgd
from .combine import chain
from .pytree import tree_map as _tree_map

__version__ = "0.0.stand-in"


def apply_updates(params, updates, *, inplace: bool = True):
    """``p + u`` per leaf (in place when asked); leaves without an update pass through."""
    def add_(p, u):
        if u is not None:
            p.data.add_(u)
        return p

    if inplace:
        return _tree_map(add_, params, updates)
    return _tree_map(lambda p, u: p if u is None else p.add(u), params, updates)


__all__ = ["adamw", "sgd", "apply_updates", "chain", "pytree", "typing", "alias", "combine"]
