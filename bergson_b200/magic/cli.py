"""``magic`` / ``train`` / ``validate`` driver: train with checkpoints, take the query
gradient at the final parameters, sweep backward through training to get
``dL_query / dw`` for every training document (or token), save the scores, optionally
validate them by retraining (reference ``bergson/magic/cli.py:55-676``).
"""

from __future__ import annotations

import json
import os
import shutil
import time
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
from datasets import Dataset, concatenate_datasets
from tqdm.auto import tqdm

from ..config.config import MagicConfig, TrainingConfig, ValidationConfig
from ..config.config_io import save_run_config
from ..data import compute_num_token_grads, load_scores_loss_signed
from ..distributed import init_dist, launch_distributed_run
from ..score.score_writer import save_sequence_scores, save_token_scores
from ..utils.utils import current_device, get_device
from ..utils.worker_utils import setup_data_pipeline
from .data_stream import DataStream, pad_dataset_to_batch_size
from .grad_accum import accumulate_grads
from .optim import tree_iter
from .trainer import BackwardState, Trainer, TrainerState, prepare_trainer, write_lr_history


def compute_query_gradients(trainer: Trainer, fwd_state: TrainerState, query_stream: DataStream, method: str = "mean",
                            fsdp: bool = False, grad_accum_steps: int = 1):
    """Parameter gradient of the query loss summed (or averaged) over the query batches
    and ranks.  Returns ``(grads, loss)``."""
    world = dist.get_world_size() if dist.is_initialized() else 1
    main = not dist.is_initialized() or dist.get_rank() == 0
    # Sharded parameters: the gather's backward sums gradients over ranks; replicated
    # parameters: the all-reduce below sums them.  Either way the mean divides by world.
    denom = len(query_stream) * world
    params = {k: v.detach().requires_grad_(True) for k, v in fwd_state.params.items()}
    call = lambda p, mb: trainer.call_model(p, mb, fwd_state.buffers)  # noqa: E731
    total: dict[str, torch.Tensor] | None = None
    loss_sum = 0.0
    for batch in tqdm(query_stream, desc="Query", disable=not main):
        batch = {k: v for k, v in batch.items() if k != "example_weight"}
        grads, loss = accumulate_grads(call, params, batch, grad_accum_steps, create_graph=False)
        if total is None:
            total = {k: g.detach().clone() for k, g in grads.items() if g is not None}
        else:
            for k, g in grads.items():
                if g is not None:
                    total[k] += g.detach()
        loss_sum += loss
    assert total is not None, "Query stream was empty"
    if method == "mean":
        total = {k: g / denom for k, g in total.items()}
        loss_sum /= denom
    if dist.is_initialized():
        if not fsdp:  # sharded gradients were already reduced by the parameter gather's backward
            for g in total.values():
                dist.all_reduce(g, op=dist.ReduceOp.SUM)
        t = torch.tensor(loss_sum, device=current_device())
        dist.all_reduce(t)
        loss_sum = float(t)
    return total, float(loss_sum)


def scores_are_per_token(score_path: str) -> bool:
    info = os.path.join(score_path, "info.json")
    if not os.path.isfile(info):
        return False
    with open(info) as f:
        return bool(json.load(f).get("attribute_tokens", False))


def attach_doc_ids_if_missing(dataset: Dataset) -> Dataset:
    """Add ``doc_ids`` = ``[row] * max_len`` for one-document-per-row data."""
    if "doc_ids" in dataset.column_names:
        return dataset
    if "length" in dataset.column_names:
        seq_len = max(dataset["length"])
    else:
        seq_len = max(len(r) for r in dataset["input_ids"])
    return dataset.map(lambda _, i: {"doc_ids": [i] * seq_len}, with_indices=True, desc="Attaching doc_ids")


def save_magic_scores(run_path: str, scores: torch.Tensor, train_dataset: Dataset, pad_count: int, per_token: bool) -> str:
    """Write ``<run>/scores`` (sequence store, or ragged token store + ``doc_ids.npy``)."""
    path = Path(run_path) / "scores"
    if not per_token:
        arr = scores.float().numpy()
        save_sequence_scores(path, arr if arr.ndim > 1 else arr[:, None])
        print(f"Saved attribution scores to {path}")
        return str(path)
    counts = compute_num_token_grads(train_dataset)
    doc_ids = np.asarray(train_dataset["doc_ids"], dtype=np.int64)
    if pad_count:
        counts, doc_ids = counts[:-pad_count], doc_ids[:-pad_count]
    offsets = np.zeros(len(counts) + 1, dtype=np.int64)
    np.cumsum(counts, out=offsets[1:])
    grid = scores.float().numpy()
    grid = grid[:, :, None] if grid.ndim == 2 else grid
    flat = np.concatenate([grid[r, : counts[r]] for r in range(len(counts))])
    save_token_scores(path, flat, offsets)
    np.save(path / "doc_ids.npy", doc_ids)
    print(f"Saved attribution scores to {path}")
    return str(path)


def shuffled_epochs(dataset: Dataset, seed: int, num_epochs: int) -> Dataset:
    """``num_epochs`` shuffled copies (epoch e seeded ``seed + e``), concatenated."""
    assert num_epochs >= 1, f"num_epochs must be >= 1, got {num_epochs}"
    return concatenate_datasets([dataset.shuffle(seed=seed + e) for e in range(num_epochs)])


def _zero_opt_cotangents(state: TrainerState) -> list[torch.Tensor]:
    return [torch.zeros_like(t) for t in tree_iter(state.opt_state) if isinstance(t, torch.Tensor) and t.is_floating_point()]


def _backward_kwargs(cfg: MagicConfig) -> dict:
    return dict(cleanup=cfg.cleanup_ckpts, debug=cfg.debug, inplace=True, fsdp=cfg.fsdp, resume=cfg.resume,
                save_every=cfg.backward_save_every, save_mode=cfg.save_mode, max_grad_norm=cfg.max_grad_norm,
                grad_accum_steps=cfg.grad_accum_steps, double_backward_batch_size=cfg.double_backward_batch_size)


def compute_per_query_magic_scores(trainer, ckpts_path, stream, fwd_state, query_dataset, num_real_queries, cfg,
                                   world_size, global_rank, pad_count, weight_pad_count) -> torch.Tensor:
    """One backward sweep per query document, sharing the forward checkpoints; results are
    saved incrementally under ``<run>/per_query`` so an interrupted run resumes."""
    out_dir = Path(cfg.run_path) / "per_query"
    out_dir.mkdir(parents=True, exist_ok=True)
    cols = []
    for q in range(num_real_queries):
        cache = out_dir / f"q{q}.pt"
        if cache.exists():
            cols.append(torch.load(cache, map_location="cpu", weights_only=True))
            continue
        row = query_dataset.select([q])
        x = torch.tensor(row["input_ids"], device=stream.device)
        y = torch.tensor(row["labels"], device=stream.device) if "labels" in row.column_names else x
        params = {k: v.detach().requires_grad_(True) for k, v in fwd_state.params.items()}
        loss = trainer.call_model(params, {"input_ids": x, "labels": y}, fwd_state.buffers).loss
        grads = torch.autograd.grad(loss, list(params.values()), allow_unused=True)
        qg = {k: (g if g is not None else torch.zeros_like(p)) for (k, p), g in zip(params.items(), grads)}
        stream.requires_grad = True
        bwd = BackwardState(qg, _zero_opt_cotangents(fwd_state), torch.zeros_like(stream.weights))
        kw = _backward_kwargs(cfg)
        kw["cleanup"] = False  # later queries replay the same checkpoints
        bwd = trainer.backward(ckpts_path, stream, bwd, fwd_state.to(stream.device), **kw)
        if world_size > 1:
            dist.all_reduce(bwd.weight_grads, op=dist.ReduceOp.SUM)
        col = bwd.weight_grads.detach().cpu()
        if pad_count:
            col = col[:-weight_pad_count] if col.ndim == 1 else col[:-pad_count]
        if global_rank == 0:
            torch.save(col, cache)
        cols.append(col)
    return torch.stack(cols, dim=-1)


def worker(global_rank: int, rank: int, world_size: int, train_dataset: Dataset, query_dataset: Dataset | None,
           num_train_docs: int, num_query_docs: int, run_cfg: TrainingConfig, score_path: str = ""):
    init_dist(global_rank, rank, world_size, mixed=True)
    assert run_cfg.batch_size % world_size == 0, "batch_size must be divisible by the world size"
    train_dataset, num_train_docs, pad_count, weight_pad = pad_dataset_to_batch_size(
        train_dataset, run_cfg.batch_size, num_train_docs, "Train", global_rank)
    per_token = (isinstance(run_cfg, MagicConfig) and run_cfg.attribute_tokens) or (
        bool(score_path) and scores_are_per_token(score_path))
    if per_token:
        seq_len = run_cfg.data.chunk_length if run_cfg.data.chunk_length > 0 else max(train_dataset["length"])
        w_shape: tuple[int, ...] = (len(train_dataset), seq_len)
    else:
        w_shape = (num_train_docs,)
    device = get_device(rank)
    stream = DataStream(train_dataset, run_cfg.batch_size, device=device, input_key=run_cfg.data.prompt_column,
                        weight_shape=w_shape)
    if pad_count:
        if stream.weights.ndim == 1:
            stream.weights.data[-weight_pad:] = 0.0
        else:
            stream.weights.data[-pad_count:] = 0.0
    log_fn = None
    if run_cfg.wandb_project and global_rank == 0:
        from ..utils.logging import wandb_log_fn

        log_fn = wandb_log_fn(run_cfg.wandb_project, config=run_cfg.to_dict())
    if dist.is_initialized():
        dist.barrier()
    schedule = run_cfg.lr_schedule.get_schedule(len(stream))
    torch.manual_seed(run_cfg.seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(run_cfg.seed)
    trainer, fwd_state, model = prepare_trainer(run_cfg, rank, schedule)
    ckpts = os.path.join(run_cfg.run_path, "checkpoints")
    if global_rank == 0:
        write_lr_history(ckpts, schedule, len(stream))
    opt_cfg = dict(betas=(run_cfg.adam_beta1, run_cfg.adam_beta2), eps=run_cfg.adam_eps, eps_root=run_cfg.eps_root)
    fwd_state = trainer.train(
        fwd_state, stream, debug=run_cfg.debug, inplace=True, save_dir=ckpts, save_mode=run_cfg.save_mode,
        log_fn=log_fn, resume=run_cfg.resume, fsdp=run_cfg.fsdp, max_grad_norm=run_cfg.max_grad_norm,
        grad_accum_steps=run_cfg.grad_accum_steps,
        optimizer_cfg=opt_cfg if run_cfg.save_optimizer_state == "all" else None, save_interval=run_cfg.save_interval)
    if run_cfg.save_optimizer_state != "none":
        from ..utils.load_from_optimizer import save_second_moments_as_optimizer_pt

        save_second_moments_as_optimizer_pt(model, fwd_state.opt_state, os.path.join(run_cfg.run_path, "optimizer.pt"))
    trails = isinstance(run_cfg, ValidationConfig) and run_cfg.subset_start != 0
    if run_cfg.save_models and global_rank == 0 and not trails:
        from ..utils.trainer_export import save_state_as_pretrained

        sub = ("retrained", "base") if isinstance(run_cfg, ValidationConfig) else ("model",)
        save_state_as_pretrained(trainer, fwd_state, os.path.join(run_cfg.run_path, *sub), run_cfg)
    if query_dataset is None:
        return
    if not isinstance(run_cfg, ValidationConfig):
        raise RuntimeError("run_cfg must be a ValidationConfig if query_dataset is provided")

    real_queries = num_query_docs
    query_dataset, num_query_docs, q_pad, q_weight_pad = pad_dataset_to_batch_size(
        query_dataset, run_cfg.batch_size, num_query_docs, "Query", global_rank)
    if len(query_dataset) < run_cfg.batch_size:
        raise ValueError(f"Query dataset has {len(query_dataset)} examples, fewer than batch_size={run_cfg.batch_size}.")
    query_stream = DataStream(query_dataset, run_cfg.batch_size, device=device, input_key=run_cfg.query.prompt_column,
                              weight_shape=(num_query_docs,))
    if q_pad:
        query_stream.weights.data[-q_weight_pad:] = 0.0
    query_grads, baseline = compute_query_gradients(trainer, fwd_state, query_stream, run_cfg.query_method,
                                                    run_cfg.fsdp, run_cfg.grad_accum_steps)
    multi_query = False
    if not score_path:
        if not isinstance(run_cfg, MagicConfig):
            raise RuntimeError("run_cfg must be a MagicConfig to compute scores")
        if run_cfg.save_mode == "interval":
            raise ValueError("save_mode='interval' not supported for MAGIC attribution")
        if run_cfg.query_method == "none":
            scores = compute_per_query_magic_scores(trainer, ckpts, stream, fwd_state, query_dataset, real_queries,
                                                    run_cfg, world_size, global_rank, pad_count, weight_pad)
            multi_query = True
        else:
            stream.requires_grad = True
            bwd = BackwardState(query_grads, _zero_opt_cotangents(fwd_state), torch.zeros_like(stream.weights))
            bwd = trainer.backward(ckpts, stream, bwd, fwd_state, **_backward_kwargs(run_cfg))
            if world_size > 1:
                dist.all_reduce(bwd.weight_grads, op=dist.ReduceOp.SUM)
            scores = bwd.weight_grads.detach().cpu()
            if pad_count:
                scores = scores[:-weight_pad] if scores.ndim == 1 else scores[:-pad_count]
        if global_rank == 0:
            print(f"Baseline loss: {baseline}")
            flat = scores.flatten().float()
            print(f"Score summary: n={flat.numel()} min={flat.min():.4g} max={flat.max():.4g} "
                  f"mean={flat.mean():.4g} std={flat.std():.4g}")
            score_path = save_magic_scores(run_cfg.run_path, scores, train_dataset, pad_count, bool(per_token))
    else:
        scores, multi_query = load_scores_loss_signed(score_path)
    stream.requires_grad = False
    if isinstance(run_cfg, MagicConfig) and run_cfg.skip_validation:
        return
    from ..validate import validate_scores

    validate_scores(run_cfg, scores, multi_query, global_rank=global_rank, rank=rank, world_size=world_size,
                    schedule=schedule, stream=stream, query_stream=query_stream, fwd_state=fwd_state, model=model,
                    trainer=trainer, baseline=baseline, num_query_docs=num_query_docs,
                    query_weight_pad_count=q_weight_pad, pad_count=pad_count, weight_pad_count=weight_pad)


def run_magic(run_cfg: TrainingConfig, *, score_path: str = ""):
    run_path = Path(run_cfg.run_path)
    main_node = int(os.environ.get("SLURM_PROCID", 0)) == 0
    multi_node = run_cfg.distributed.nnode > 1
    if main_node:
        if run_path.exists() and not run_cfg.resume:
            if not run_cfg.overwrite:
                raise FileExistsError(f"Run path {run_path} already exists. Use --overwrite to overwrite it.")
            shutil.rmtree(run_path)
        run_path.mkdir(parents=True, exist_ok=True)
        save_run_config(run_cfg, run_path)
    # Other nodes wait until the main node has finished preprocessing (dataset caches are
    # not safe for concurrent writers).
    flag = run_path / ".preprocess_done" if multi_node else None
    if flag is not None and not main_node:
        run_path.mkdir(parents=True, exist_ok=True)
        while not flag.exists():
            time.sleep(0.5)
    train_ds, train_n = setup_data_pipeline(run_cfg)
    train_ds = shuffled_epochs(attach_doc_ids_if_missing(train_ds), run_cfg.seed, max(1, run_cfg.num_epochs))
    if isinstance(run_cfg, ValidationConfig):
        query_ds, query_n = setup_data_pipeline(run_cfg, run_cfg.query)
    else:
        query_ds, query_n = None, 0
    if flag is not None and main_node:
        flag.touch()
    launch_distributed_run("run_magic", worker, [train_ds, query_ds, train_n, query_n, run_cfg, score_path],
                           run_cfg.distributed)


def main(argv: list[str] | None = None) -> None:
    """``python -m bergson_b200.magic.cli <run_path> --flags``: the ``magic`` command on its own
    (reference ``bergson/magic/cli.py:679-685``)."""
    import sys

    from ..__main__ import main as run_command

    run_command(["magic", *(sys.argv[1:] if argv is None else argv)])


if __name__ == "__main__":
    main()
