"""Export trainer checkpoints (``step_i.ckpt``) to HF-style ``checkpoint-i/`` directories
(reference ``bergson/utils/trainer_export.py:26-143``)."""

from __future__ import annotations

import os
import shutil
from pathlib import Path

import torch

from ..data import sorted_checkpoints


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


def ensure_exported(trainer, state, run_path: str, cfg=None) -> list[tuple[int, str]]:
    """Export every ``checkpoints/step_i.ckpt`` of a run to ``checkpoint-i/`` once."""
    out = []
    for step, path in sorted_checkpoints(os.path.join(run_path, "checkpoints")):
        if not os.path.exists(os.path.join(path, ".metadata")):
            continue
        dst = os.path.join(run_path, f"checkpoint-{step}")
        if not os.path.exists(os.path.join(dst, "config.json")):
            export_checkpoint(trainer, state, path, dst, cfg)
        out.append((step, dst))
    return out
