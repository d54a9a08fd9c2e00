"""Dataclass <-> argparse <-> YAML layer used by every command.

The reference builds its CLI on the third-party ``simple_parsing`` package
(``bergson/__main__.py:81-115``, ``bergson/config/config.py:9``).  That package is
not a dependency here; this module provides the subset of its behaviour the
command surface relies on:

* ``field(positional=True)`` for the positional ``run_path``;
* ``Serializable.to_dict`` / ``from_dict(drop_extra_fields=...)`` for the
  replayable ``config.yaml``;
* nested dataclasses addressable both flat (``--projection_dim``) and dotted
  (``--data.dataset``, ``--index_cfg.data.dataset``): every *unique* suffix of a
  leaf's dotted path becomes an option string;
* ``Literal`` -> ``choices``, ``Optional[X]``, ``list[X]``, bool flags that take
  an optional explicit value, attribute docstrings used as ``--help`` text.
"""

from __future__ import annotations

import argparse
import ast
import dataclasses
import inspect
import textwrap
import types
import typing
from dataclasses import MISSING, fields, is_dataclass
from typing import Any, Literal, Union, get_args, get_origin, get_type_hints

__all__ = [
    "field",
    "Serializable",
    "DataclassArgumentParser",
    "parse_command",
    "to_dict",
    "from_dict",
]


def field(*, positional: bool = False, **kwargs) -> Any:
    """``dataclasses.field`` with a ``positional`` marker in the metadata."""
    metadata = dict(kwargs.pop("metadata", None) or {})
    if positional:
        metadata["positional"] = True
    return dataclasses.field(metadata=metadata, **kwargs)


# --------------------------------------------------------------------------- #
# (de)serialisation
# --------------------------------------------------------------------------- #


def to_dict(obj: Any) -> Any:
    """Recursively convert a dataclass tree to plain YAML-safe containers."""
    if is_dataclass(obj) and not isinstance(obj, type):
        return {f.name: to_dict(getattr(obj, f.name)) for f in fields(obj) if f.init}
    if isinstance(obj, dict):
        return {str(k): to_dict(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple, set)):
        return [to_dict(v) for v in obj]
    if hasattr(obj, "__fspath__"):
        return str(obj)
    return obj


def _strip_optional(tp: Any) -> tuple[Any, bool]:
    origin = get_origin(tp)
    if origin in (Union, types.UnionType):
        args = [a for a in get_args(tp) if a is not type(None)]
        optional = len(args) != len(get_args(tp))
        if len(args) == 1:
            return args[0], optional
        return Union[tuple(args)], optional  # type: ignore[return-value]
    return tp, False


def _hints(cls: type) -> dict[str, Any]:
    try:
        return get_type_hints(cls)
    except Exception:  # pragma: no cover - forward refs that cannot resolve
        return {f.name: f.type for f in fields(cls)}


def _coerce(value: Any, tp: Any, drop_extra: bool | None) -> Any:
    tp, optional = _strip_optional(tp)
    if value is None:
        return None
    if is_dataclass(tp) and isinstance(value, dict):
        return from_dict(tp, value, drop_extra_fields=drop_extra)
    origin = get_origin(tp)
    if origin in (list, typing.List) and isinstance(value, (list, tuple)):
        (inner,) = get_args(tp) or (Any,)
        return [_coerce(v, inner, drop_extra) for v in value]
    if origin in (Union, types.UnionType):
        for cand in get_args(tp):
            try:
                return _coerce(value, cand, drop_extra)
            except (TypeError, ValueError):
                continue
        return value
    if tp is float and isinstance(value, (int, str)) and not isinstance(value, bool):
        return float(value)
    if tp is int and isinstance(value, str):
        return int(value)
    if tp is int and isinstance(value, float) and value.is_integer():
        return int(value)
    return value


def from_dict(cls: type, obj: dict[str, Any], drop_extra_fields: bool | None = None):
    """Build ``cls`` from a mapping; nested dataclasses are hydrated recursively.

    ``drop_extra_fields=False`` raises on unknown keys, ``True``/``None`` ignores
    them (``None`` mirrors the lenient default used when re-reading old configs).
    """
    if not isinstance(obj, dict):
        raise TypeError(f"Expected a mapping for {cls.__name__}, got {type(obj)}")
    hints = _hints(cls)
    known = {f.name: f for f in fields(cls) if f.init}
    extra = set(obj) - set(known)
    if extra and drop_extra_fields is False:
        raise ValueError(
            f"Unknown field(s) {sorted(extra)} for {cls.__name__}; "
            f"valid fields: {sorted(known)}"
        )
    kwargs = {}
    for name, f in known.items():
        if name in obj:
            kwargs[name] = _coerce(obj[name], hints.get(name, Any), drop_extra_fields)
        elif f.default is MISSING and f.default_factory is MISSING:  # type: ignore
            tp, _ = _strip_optional(hints.get(name, Any))
            if is_dataclass(tp):
                kwargs[name] = from_dict(tp, {}, drop_extra_fields)
    return cls(**kwargs)


class Serializable:
    """Mixin giving dataclasses ``to_dict`` / ``from_dict`` / YAML round trips."""

    def to_dict(self) -> dict[str, Any]:
        return to_dict(self)

    @classmethod
    def from_dict(cls, obj: dict[str, Any], drop_extra_fields: bool | None = None):
        return from_dict(cls, obj, drop_extra_fields)

    def save_yaml(self, path) -> None:
        import yaml

        with open(path, "w") as f:
            yaml.safe_dump(self.to_dict(), f, sort_keys=False)

    @classmethod
    def load_yaml(cls, path):
        import yaml

        with open(path) as f:
            return cls.from_dict(yaml.safe_load(f) or {})


# --------------------------------------------------------------------------- #
# argparse construction
# --------------------------------------------------------------------------- #


def _attribute_docstrings(cls: type) -> dict[str, str]:
    """Collect ``name: type = default`` + following string literal pairs."""
    docs: dict[str, str] = {}
    for klass in reversed(cls.__mro__):
        if klass is object or not is_dataclass(klass):
            continue
        try:
            src = textwrap.dedent(inspect.getsource(klass))
            tree = ast.parse(src)
        except (OSError, TypeError, SyntaxError):
            continue
        body = tree.body[0].body if tree.body else []  # type: ignore[attr-defined]
        for node, nxt in zip(body, body[1:]):
            if (
                isinstance(node, ast.AnnAssign)
                and isinstance(node.target, ast.Name)
                and isinstance(nxt, ast.Expr)
                and isinstance(nxt.value, ast.Constant)
                and isinstance(nxt.value.value, str)
            ):
                docs[node.target.id] = " ".join(nxt.value.value.split())
    return docs


def _str2bool(v: str) -> bool:
    s = str(v).strip().lower()
    if s in {"1", "true", "t", "yes", "y", "on"}:
        return True
    if s in {"0", "false", "f", "no", "n", "off"}:
        return False
    raise argparse.ArgumentTypeError(f"expected a boolean, got {v!r}")


def _none_or(fn):
    def parse(v: str):
        if v.lower() in {"none", "null"}:
            return None
        return fn(v)

    parse.__name__ = getattr(fn, "__name__", "value")
    return parse


@dataclasses.dataclass
class _Leaf:
    path: tuple[str, ...]
    tp: Any
    default: Any
    required: bool
    positional: bool
    help: str

    @property
    def dest(self) -> str:
        return ".".join(self.path)


def _default_of(f: dataclasses.Field) -> tuple[Any, bool]:
    if f.default is not MISSING:
        return f.default, False
    if f.default_factory is not MISSING:  # type: ignore[misc]
        return f.default_factory(), False  # type: ignore[misc]
    return None, True


def _collect(cls: type, prefix: tuple[str, ...], out: list[_Leaf]) -> None:
    hints = _hints(cls)
    docs = _attribute_docstrings(cls)
    for f in fields(cls):
        if not f.init:
            continue
        tp = hints.get(f.name, f.type)
        base, _ = _strip_optional(tp)
        path = prefix + (f.name,)
        if is_dataclass(base):
            _collect(base, path, out)
            continue
        default, required = _default_of(f)
        out.append(
            _Leaf(
                path=path,
                tp=tp,
                default=default,
                required=required,
                positional=bool(f.metadata.get("positional")),
                help=docs.get(f.name, ""),
            )
        )


def _add_leaf(parser: argparse.ArgumentParser, leaf: _Leaf, names: list[str]) -> None:
    base, optional = _strip_optional(leaf.tp)
    kw: dict[str, Any] = {"dest": leaf.dest, "help": leaf.help or None}
    origin = get_origin(base)
    if origin is Literal:
        choices = list(get_args(base))
        kw["choices"] = choices + ([None] if optional else [])
        elem = type(choices[0])
        kw["type"] = _none_or(elem) if optional else elem
    elif base is bool:
        kw.update(type=_str2bool, nargs="?", const=True)
    elif origin in (list, typing.List):
        (inner,) = get_args(base) or (str,)
        inner, _ = _strip_optional(inner)
        kw.update(type=inner if inner in (int, float, str) else str, nargs="*")
    elif origin in (Union, types.UnionType):
        # e.g. ``str | list[str]``: accept one or many strings.
        kw.update(type=str, nargs="+")
    elif base in (int, float, str):
        kw["type"] = _none_or(base) if optional else base
    else:
        kw["type"] = str

    if leaf.positional:
        # A positional may also be given by name (YAML replays do that).
        parser.add_argument(
            leaf.dest,
            nargs="?" if not leaf.required else None,
            default=argparse.SUPPRESS,
            type=kw.get("type", str),
            help=kw["help"],
        )
        return
    kw["default"] = argparse.SUPPRESS
    if leaf.required:
        kw["required"] = True
    if leaf.default is not None and not leaf.required and kw.get("help"):
        kw["help"] = f"{kw['help']} (default: {leaf.default!r})"
    parser.add_argument(*names, **kw)


class DataclassArgumentParser:
    """Build an ``argparse`` parser from a (nested) dataclass and parse into it."""

    def __init__(self, cls: type, prog: str | None = None, description: str | None = None):
        self.cls = cls
        self.leaves: list[_Leaf] = []
        _collect(cls, (), self.leaves)
        self.parser = argparse.ArgumentParser(
            prog=prog,
            description=description or inspect.getdoc(cls),
            formatter_class=argparse.RawDescriptionHelpFormatter,
        )
        # Every suffix of the dotted path that identifies exactly one leaf is an
        # accepted spelling of that option.
        suffix_owner: dict[str, list[_Leaf]] = {}
        for leaf in self.leaves:
            for i in range(len(leaf.path)):
                suffix_owner.setdefault(".".join(leaf.path[i:]), []).append(leaf)
        for leaf in self.leaves:
            names = []
            for i in range(len(leaf.path)):
                s = ".".join(leaf.path[i:])
                if len(suffix_owner[s]) == 1:
                    names.append("--" + s)
            if not names:
                names = ["--" + leaf.dest]
            # Shortest spelling first so ``--help`` shows the convenient name.
            names.sort(key=len)
            _add_leaf(self.parser, leaf, names)

    def parse(self, argv: list[str] | None = None):
        ns = self.parser.parse_args(argv)
        tree: dict[str, Any] = {}
        for leaf in self.leaves:
            if not hasattr(ns, leaf.dest):
                if leaf.required:
                    self.parser.error(f"missing required argument: {leaf.dest}")
                continue
            value = getattr(ns, leaf.dest)
            base, _ = _strip_optional(leaf.tp)
            if get_origin(base) in (Union, types.UnionType) and isinstance(value, list):
                value = value[0] if len(value) == 1 else value
            node = tree
            for key in leaf.path[:-1]:
                node = node.setdefault(key, {})
            node[leaf.path[-1]] = value
        return from_dict(self.cls, tree, drop_extra_fields=False)


def parse_command(registry: dict[str, type], argv: list[str], prog: str = "bergson"):
    """Dispatch ``argv[0]`` to a command dataclass and parse the rest into it."""
    top = argparse.ArgumentParser(
        prog=prog,
        description="Data attribution for language models on Blackwell GPUs.",
    )
    top.add_argument("command", choices=sorted(registry), help="sub-command to run")
    if not argv or argv[0] in {"-h", "--help"}:
        top.parse_args(argv or ["--help"])
    name = argv[0].lower()
    if name not in registry:
        top.parse_args(argv[:1])
    cls = registry[name]
    return DataclassArgumentParser(cls, prog=f"{prog} {name}").parse(argv[1:])
