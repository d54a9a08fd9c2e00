"""Empirical metasmoothness of a training configuration: train three times with data
weights ``1``, ``1 + h v`` and ``1 + 2 h v`` (``v ~ N(0, I)`` over documents) and measure
how consistently the parameters keep moving in the same direction
(reference ``bergson/magic/metasmoothness.py:32-170``)."""

from __future__ import annotations

import json
import os

import torch

from ..config.config import MetasmoothnessConfig
from ..distributed import init_dist, launch_distributed_run
from ..utils.utils import get_device
from ..utils.worker_utils import setup_data_pipeline
from .cli import attach_doc_ids_if_missing, shuffled_epochs
from .data_stream import DataStream, pad_dataset_to_batch_size
from .trainer import prepare_trainer


def metasmoothness_score(theta0: torch.Tensor, theta_h: torch.Tensor, theta_2h: torch.Tensor) -> float:
    """``sum_j (d_j / |d|_1) sign(theta_h - theta_0)_j sign(theta_2h - theta_h)_j`` with
    ``d = |theta_2h - theta_0|``; 1.0 when nothing moved."""
    d = (theta_2h - theta0).abs()
    total = d.sum()
    if total == 0:
        return 1.0
    return float((d / total * torch.sign(theta_h - theta0) * torch.sign(theta_2h - theta_h)).sum())


def metasmoothness_worker(global_rank: int, rank: int, world_size: int, train_dataset, num_train_docs: int,
                          run_cfg: MetasmoothnessConfig):
    init_dist(global_rank, rank, world_size, mixed=True)
    assert not run_cfg.fsdp, "metasmoothness does not support sharded parameters"
    assert run_cfg.batch_size % world_size == 0
    train_dataset, num_train_docs, pad_count, weight_pad = pad_dataset_to_batch_size(
        train_dataset, run_cfg.batch_size, num_train_docs, "Train", global_rank)
    stream = DataStream(train_dataset, run_cfg.batch_size, device=get_device(rank),
                        input_key=run_cfg.data.prompt_column, weight_shape=(num_train_docs,))
    schedule = run_cfg.lr_schedule.get_schedule(len(stream))
    v = torch.randn(num_train_docs, generator=torch.Generator().manual_seed(run_cfg.direction_seed))
    if pad_count:
        v[-weight_pad:] = 0.0
    thetas = []
    for k in range(3):
        w = 1.0 + run_cfg.fd_step * k * v
        if pad_count:
            w[-weight_pad:] = 0.0
        stream.weights.data.copy_(w.to(stream.weights))
        torch.manual_seed(run_cfg.seed)
        if torch.cuda.is_available():
            torch.cuda.manual_seed_all(run_cfg.seed)
        trainer, state, _ = prepare_trainer(run_cfg, rank, schedule)
        state.detach_()
        state = trainer.train(state, stream, inplace=True, max_grad_norm=run_cfg.max_grad_norm,
                              grad_accum_steps=run_cfg.grad_accum_steps)
        if global_rank == 0:
            thetas.append(torch.cat([p.detach().float().cpu().flatten() for p in state.params.values()]))
            print(f"[metasmoothness] finished training {k + 1}/3 (w = 1 + {k}*h*v)")
            if k == 0 and run_cfg.save_models:
                from ..utils.trainer_export import save_state_as_pretrained

                save_state_as_pretrained(trainer, state, os.path.join(run_cfg.run_path, "model"), run_cfg)
    if global_rank == 0:
        result = {"score": metasmoothness_score(*thetas), "fd_step": run_cfg.fd_step,
                  "direction_seed": run_cfg.direction_seed,
                  "total_movement_l1": float((thetas[2] - thetas[0]).abs().sum())}
        print(f"[metasmoothness] score = {result['score']:.4f} (h={run_cfg.fd_step})")
        os.makedirs(run_cfg.run_path, exist_ok=True)
        with open(os.path.join(run_cfg.run_path, "metasmoothness.json"), "w") as f:
            json.dump(result, f, indent=2)


def run_metasmoothness(run_cfg: MetasmoothnessConfig):
    os.makedirs(run_cfg.run_path, exist_ok=True)
    ds, n = setup_data_pipeline(run_cfg)
    ds = shuffled_epochs(attach_doc_ids_if_missing(ds), run_cfg.seed, max(1, run_cfg.num_epochs))
    launch_distributed_run("metasmoothness", metasmoothness_worker, [ds, n, run_cfg], run_cfg.distributed)
