"""Reading and writing the replayable ``config.yaml`` of a run.

Document shape (reference ``bergson/config/config_io.py:54-70``)::

    run_path: <dir>            # pipelines only
    steps:
      - <command>: {<config tree>, matrix?: {key: [v, ...]}}
    metadata: {bergson_version, created, git_sha?}
"""

from __future__ import annotations

import itertools
import random
import subprocess
from datetime import datetime, timezone
from pathlib import Path
from typing import Any, TypeVar

import yaml

CONFIG_FILENAME = "config.yaml"
T = TypeVar("T")

_ADJ = "amber brisk calm deft eager fond glad hardy keen lucid merry noble proud quick rapid sunny tidy vivid warm zesty".split()
_NOUN = "auk bison crane dingo egret finch gecko heron ibis jay koala lemur mole newt otter puffin quail raven stoat tern".split()


def _config_file(path: str | Path) -> Path:
    path = Path(path)
    return path / CONFIG_FILENAME if path.is_dir() else path


def _git_sha() -> str | None:
    try:
        out = subprocess.run(
            ["git", "rev-parse", "--short", "HEAD"],
            cwd=Path(__file__).resolve().parent,
            capture_output=True,
            text=True,
            check=True,
            timeout=5,
        ).stdout.strip()
    except (subprocess.SubprocessError, OSError):
        return None
    return out or None


def make_metadata() -> dict[str, Any]:
    """Version, UTC creation time and (when available) the source git sha."""
    from .. import __version__

    meta: dict[str, Any] = {
        "bergson_version": __version__,
        "created": datetime.now(timezone.utc).isoformat(timespec="seconds"),
    }
    if (sha := _git_sha()) is not None:
        meta["git_sha"] = sha
    return meta


def _dump(steps: list[dict], target: Path, run_path: str | Path | None = None) -> None:
    doc: dict[str, Any] = {}
    if run_path is not None:
        doc["run_path"] = str(run_path)
    doc["steps"] = steps
    doc["metadata"] = make_metadata()
    target.parent.mkdir(parents=True, exist_ok=True)
    with target.open("w") as f:
        yaml.safe_dump(doc, f, sort_keys=False)


def save_run_config(command: Any, run_path: str | Path) -> None:
    """Write a one-step ``config.yaml`` for ``command`` into ``run_path``."""
    _dump(
        [{type(command).__name__.lower(): command.to_dict()}],
        Path(run_path) / CONFIG_FILENAME,
    )


def generate_run_name(rng: random.Random | None = None) -> str:
    """Two-word run name, e.g. ``lucid_heron``."""
    rng = rng or random.Random()
    return f"{rng.choice(_ADJ)}_{rng.choice(_NOUN)}"


def save_pipeline_config(steps: list[tuple[str, Any]], run_path: str | Path | None):
    """Write the resolved multi-step document; auto-name under ``runs/`` if needed."""
    if not run_path:
        run_path = f"runs/{generate_run_name()}"
        print(f"No top-level run_path in the pipeline YAML; writing config to {run_path}")
    run_path = Path(run_path)
    _dump(
        [{name: cmd.to_dict()} for name, cmd in steps],
        run_path / CONFIG_FILENAME,
        run_path=run_path,
    )
    return run_path


def read_config(path: str | Path) -> dict[str, Any]:
    """Load a ``config.yaml`` (file or run directory)."""
    path = _config_file(path)
    with path.open() as f:
        doc = yaml.safe_load(f)
    if not isinstance(doc, dict) or not isinstance(doc.get("steps"), list):
        raise ValueError(
            f"{path} must be a mapping with a `steps:` list of "
            f"`- command: {{...}}` entries; got a top-level {type(doc).__name__}."
        )
    return doc


def load_subconfig(path: str | Path, field: str, config_cls: type[T]) -> T | None:
    """First occurrence of sub-tree ``field`` in any step, hydrated as ``config_cls``."""
    if not _config_file(path).exists():
        return None
    for step in read_config(path)["steps"]:
        for body in step.values():
            sub = (body or {}).get(field)
            if sub is not None:
                return config_cls.from_dict(sub)  # type: ignore[attr-defined]
    return None


def _substitute(value: Any, cell: dict[str, Any]) -> Any:
    if isinstance(value, dict):
        return {k: _substitute(v, cell) for k, v in value.items()}
    if isinstance(value, list):
        return [_substitute(v, cell) for v in value]
    if isinstance(value, str):
        for key, cell_value in cell.items():
            token = "{" + key + "}"
            if value == token:
                return cell_value  # keep the grid value's type
            value = value.replace(token, str(cell_value))
    return value


def _iter_run_paths(value: Any):
    if isinstance(value, dict):
        for k, v in value.items():
            if k == "run_path":
                yield v
            else:
                yield from _iter_run_paths(v)


def expand_matrix(cmd_dict: dict) -> list[dict]:
    """Expand a ``matrix: {k: [..]}`` grid into one config per cell."""
    matrix = cmd_dict.pop("matrix", None)
    if matrix is None:
        return [cmd_dict]
    if not isinstance(matrix, dict) or not all(
        isinstance(v, list) and v for v in matrix.values()
    ):
        raise ValueError(f"matrix must map keys to non-empty lists; got {matrix!r}.")
    keys = list(matrix)
    cells = [dict(zip(keys, combo)) for combo in itertools.product(*matrix.values())]
    expanded = [_substitute(cmd_dict, cell) for cell in cells]
    owner: dict[Any, dict] = {}
    for cfg, cell in zip(expanded, cells):
        for rp in _iter_run_paths(cfg):
            if rp in owner:
                raise ValueError(
                    f"matrix cells {owner[rp]} and {cell} both write {rp}; "
                    "vary run_path with a {key} substitution."
                )
            owner[rp] = cell
    if len(cells) > 1 and not owner:
        raise ValueError("matrix step has no run_path; cells would collide.")
    return expanded


def parse_steps(steps: list, registry: dict[str, type]) -> list[tuple[str, Any]]:
    """Instantiate ``(command_name, command)`` pairs from raw step mappings."""
    out: list[tuple[str, Any]] = []
    for step in steps:
        if not isinstance(step, dict) or len(step) != 1:
            raise ValueError(
                "Each step must be a single command-key mapping "
                f"(e.g. `- build: {{...}}`); got {step!r}."
            )
        ((name, body),) = step.items()
        cls = registry.get(str(name).lower())
        if cls is None:
            raise ValueError(
                f"Unknown command '{name}'. Valid commands: {sorted(registry)}."
            )
        for cell in expand_matrix(dict(body or {})):
            out.append((name, cls.from_dict(cell, drop_extra_fields=False)))
    return out
