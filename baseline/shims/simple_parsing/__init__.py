"""Minimal stand-in for the parts of ``simple_parsing`` that the reference imports at
module import time (dataclass field helper, ``Serializable`` mixin, parser names)."""

import argparse
import dataclasses
import enum
import typing


def field(*args, positional=False, **kwargs):
    kwargs.pop("alias", None)
    kwargs.pop("choices", None)
    meta = dict(kwargs.pop("metadata", None) or {})
    if positional:
        meta["positional"] = True
    return dataclasses.field(*args, metadata=meta, **kwargs)


def _to_dict(obj):
    if dataclasses.is_dataclass(obj) and not isinstance(obj, type):
        return {f.name: _to_dict(getattr(obj, f.name)) for f in dataclasses.fields(obj)}
    if isinstance(obj, dict):
        return {k: _to_dict(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [_to_dict(v) for v in obj]
    return obj


class Serializable:
    def to_dict(self):
        return _to_dict(self)

    @classmethod
    def from_dict(cls, obj, drop_extra_fields=None):
        hints = typing.get_type_hints(cls)
        kwargs = {}
        for f in dataclasses.fields(cls):
            if f.name not in obj:
                continue
            tp = hints.get(f.name)
            val = obj[f.name]
            if dataclasses.is_dataclass(tp) and isinstance(val, dict):
                val = tp.from_dict(val) if hasattr(tp, "from_dict") else tp(**val)
            kwargs[f.name] = val
        return cls(**kwargs)


class ConflictResolution(enum.Enum):
    EXPLICIT = "explicit"


class ArgumentParser(argparse.ArgumentParser):
    def __init__(self, *args, conflict_resolution=None, **kwargs):
        super().__init__(*args, **kwargs)

    def add_arguments(self, cls, dest):
        raise NotImplementedError("the CLI of the reference is not used by the benchmark harness")
