"""Jinja2 dataset formatting (reference ``bergson/format.py:27-58``).  The YAML holds
``doc_to_text`` (prompt template), optional ``doc_to_target`` (column name or template)
and optional ``doc_to_choice`` (labels; the target is then an index into them)."""

from __future__ import annotations

from pathlib import Path

import yaml
from datasets import Dataset


def apply_format(ds: Dataset, format_path: str) -> Dataset:
    """Adds ``text`` (prompt only) or ``prompt`` + ``completion`` columns."""
    from jinja2 import BaseLoader, Environment

    spec = yaml.safe_load(Path(format_path).read_text())
    env = Environment(loader=BaseLoader())
    text_t = env.from_string(spec["doc_to_text"])
    target, choices = spec.get("doc_to_target"), spec.get("doc_to_choice")
    target_t = env.from_string(target) if target and ("{{" in target or "{%" in target) else None

    def fmt(row: dict) -> dict:
        prompt = text_t.render(**row)
        if target is None:
            return {"text": prompt}
        val = target_t.render(**row) if target_t is not None else row[target]
        if choices is not None:
            val = choices[int(val)]
        return {"prompt": prompt, "completion": str(val)}

    return ds.map(fmt)
