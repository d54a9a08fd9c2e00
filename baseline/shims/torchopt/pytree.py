"""Nested-container utilities with the call shapes the reference uses from
``torchopt.pytree``: dicts (visited in sorted key order), lists, tuples and named tuples are
containers, ``None`` holds no leaves, everything else is a leaf."""

from __future__ import annotations

from typing import Any, Callable, Iterator


def _is_namedtuple(x) -> bool:
    return isinstance(x, tuple) and hasattr(x, "_fields")


def _children(node) -> list[tuple[Any, Any]] | None:
    if node is None:
        return []
    if isinstance(node, dict):
        return [(k, node[k]) for k in sorted(node)]
    if isinstance(node, (list, tuple)):
        return list(enumerate(node))
    return None


def _rebuild(node, values: list):
    if node is None:
        return None
    if isinstance(node, dict):
        by_key = dict(zip(sorted(node), values))  # leaves are visited in sorted order ...
        return {k: by_key[k] for k in node}  # ... the rebuilt dict keeps the original order
    if _is_namedtuple(node):
        return type(node)(*values)
    return type(node)(values)


def tree_flatten_with_path(tree) -> tuple[list[tuple], list, Any]:
    paths, leaves = [], []

    def walk(node, path):
        kids = _children(node)
        if kids is None:
            paths.append(path)
            leaves.append(node)
            return
        for key, child in kids:
            walk(child, path + (key,))

    walk(tree, ())
    return paths, leaves, tree


def tree_flatten(tree) -> tuple[list, Any]:
    _, leaves, spec = tree_flatten_with_path(tree)
    return leaves, spec


def tree_leaves(tree) -> list:
    return tree_flatten(tree)[0]


def tree_iter(tree) -> Iterator:
    return iter(tree_leaves(tree))


def tree_unflatten(spec, leaves):
    it = iter(leaves)

    def build(node):
        kids = _children(node)
        if kids is None:
            return next(it)
        return _rebuild(node, [build(child) for _, child in kids])

    return build(spec)


def tree_map(fn: Callable, tree, *rests):
    """Apply ``fn`` to corresponding leaves; ``rests`` must contain ``tree``'s structure as a
    prefix (a ``None`` in ``tree`` skips the matching subtree)."""

    def walk(node, others):
        kids = _children(node)
        if kids is None:
            return fn(node, *others)
        if node is None:
            return None
        out = []
        for key, child in kids:
            out.append(walk(child, [o[key] for o in others]))
        return _rebuild(node, out)

    return walk(tree, list(rests))


def tree_map_(fn: Callable, tree, *rests):
    tree_map(fn, tree, *rests)
    return tree
