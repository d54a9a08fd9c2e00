"""Export trainer checkpoints (``step_i.ckpt``) to HF-style ``checkpoint-i/`` directories
(reference ``bergson/utils/trainer_export.py:26-143``)."""

from __future__ import annotations

import os
import shutil
from pathlib import Path

import torch

EXPORT_DIRNAME = "exported"  # where export_checkpoints puts checkpoint-<i> by default


def save_state_as_pretrained(trainer, state, out_dir: str, cfg=None) -> str:
    """Write the model with ``state``'s parameters to ``out_dir`` (``save_pretrained``
    layout) plus the tokenizer when one can be loaded."""
    from ..magic.fsdp import gather_params

    os.makedirs(out_dir, exist_ok=True)
    params = state.params
    if trainer.param_shapes is not None:
        with torch.no_grad():
            params = gather_params(params, trainer.param_shapes)
    model = trainer.model
    saved = {}
    with torch.no_grad():
        for name, p in model.named_parameters():
            if name in params:
                saved[name] = p.data
                p.data = params[name].detach().to(p.dtype)
        try:
            if hasattr(model, "save_pretrained"):
                model.save_pretrained(out_dir, safe_serialization=True)
            else:
                torch.save(model.state_dict(), os.path.join(out_dir, "pytorch_model.bin"))
        finally:
            for name, p in model.named_parameters():
                if name in saved:
                    p.data = saved[name]
    if cfg is not None and not str(cfg.model).startswith("native:"):
        try:
            from transformers import AutoTokenizer

            AutoTokenizer.from_pretrained(cfg.tokenizer or cfg.model).save_pretrained(out_dir)
        except Exception as e:  # noqa: BLE001
            print(f"Tokenizer not exported ({e})")
    return out_dir


def export_checkpoint(trainer, state, ckpt_path: str, out_dir: str, cfg=None) -> str:
    """Load ``ckpt_path`` into ``state`` and export it; ``optimizer.pt`` is copied along."""
    state.load(ckpt_path)
    save_state_as_pretrained(trainer, state, out_dir, cfg)
    opt = Path(ckpt_path) / "optimizer.pt"
    if opt.exists():
        shutil.copy2(opt, Path(out_dir) / "optimizer.pt")
    return out_dir


def sorted_dcp_checkpoints(checkpoints_dir: str | Path) -> list[tuple[int, Path]]:
    """``(step, path)`` of every ``step_<i>[.ckpt]`` directory, ascending
    (reference ``bergson/utils/trainer_export.py:26-39``)."""
    checkpoints_dir = Path(checkpoints_dir)
    if not checkpoints_dir.is_dir():
        raise NotADirectoryError(f"{checkpoints_dir} is not a directory")
    found = []
    for entry in checkpoints_dir.iterdir():
        stem = entry.name.removesuffix(".ckpt").removeprefix("step_")
        if entry.is_dir() and entry.name.startswith("step_") and stem.isdigit():
            found.append((int(stem), entry))
    return sorted(found, key=lambda pair: pair[0])


def export_checkpoints(run_path: str | Path, out_dir: str | Path | None = None, *, training_cfg=None,
                       steps: list[int] | None = None, overwrite: bool = False) -> list[Path]:
    """Export the trainer checkpoints of a finished run to ``checkpoint-<i>/`` directories (model
    in ``save_pretrained`` layout, ``optimizer.pt`` copied along), in step order, without a
    trainer in hand: model and state are rebuilt from the run's recorded config
    (reference ``bergson/utils/trainer_export.py:42-113``).  ``out_dir`` defaults to
    ``<run>/exported``, where ``ensure_exported`` and the SOURCE pipeline look."""
    from ..approx_unrolling.train_cfg_io import load_training_config
    from ..magic.trainer import prepare_trainer

    run_path = Path(run_path)
    out_dir = Path(out_dir) if out_dir is not None else run_path / EXPORT_DIRNAME
    cfg = training_cfg if training_cfg is not None else load_training_config(run_path)
    available = [(s, p) for s, p in sorted_dcp_checkpoints(run_path / "checkpoints") if (p / ".metadata").exists()]
    if not available:
        raise FileNotFoundError(f"No complete step_<i>.ckpt directories under {run_path / 'checkpoints'}; "
                                "train with a save_mode that writes checkpoints.")
    if steps is not None:
        by_step = dict(available)
        missing = [s for s in steps if s not in by_step]
        if missing:
            raise FileNotFoundError(f"Requested steps {missing} were not saved; available: {[s for s, _ in available]}")
        available = [(s, by_step[s]) for s in sorted(steps)]
    clashes = [out_dir / f"checkpoint-{s}" for s, _ in available if (out_dir / f"checkpoint-{s}").exists()]
    if clashes and not overwrite:
        raise FileExistsError(f"{[str(c) for c in clashes]} already exist; pass overwrite=True.")
    trainer, state, _ = prepare_trainer(cfg, rank=0, schedule=lambda step: 0.0)
    exported = []
    for step, ckpt in available:
        dst = out_dir / f"checkpoint-{step}"
        if dst.exists():
            shutil.rmtree(dst)
        export_checkpoint(trainer, state, str(ckpt), str(dst), cfg)
        exported.append(dst)
    return exported


def ensure_exported(checkpoints: list[str]) -> list[str]:
    """Checkpoint paths as model directories: a raw trainer checkpoint
    ``<run>/checkpoints/step_<n>.ckpt`` becomes ``<run>/exported/checkpoint-<n>``, exported now
    unless it already exists (one ``export_checkpoints`` call per run, so the model is rebuilt
    once); every other path passes through (reference ``bergson/utils/trainer_export.py:116-143``)."""
    resolved = [str(c) for c in checkpoints]
    todo: dict[Path, set[int]] = {}
    for i, c in enumerate(resolved):
        p = Path(c)
        stem = p.name.removesuffix(".ckpt").removeprefix("step_")
        if not (p.name.endswith(".ckpt") and p.name.startswith("step_") and stem.isdigit()):
            continue
        run = p.parent.parent
        dst = run / EXPORT_DIRNAME / f"checkpoint-{int(stem)}"
        resolved[i] = str(dst)
        if not dst.exists():
            todo.setdefault(run, set()).add(int(stem))
    for run, steps in todo.items():
        print(f"Exporting trainer checkpoints {sorted(steps)} of {run}")
        export_checkpoints(run, steps=sorted(steps), overwrite=False)
    return resolved
