"""``hessian``: fit an autocorrelation Hessian or Kronecker factors (+ eigenvectors,
eigenvalue grids, optional EK-FAC correction) (reference
``bergson/hessians/hessian_approximations.py``)."""

from __future__ import annotations

import os
import shutil
import warnings

import torch
import torch.distributed as dist
from datasets import Dataset

from ..collector.collector import CollectorComputer, fwd_bwd_hessian_factory
from ..config.config import AttentionConfig, HessianConfig, IndexConfig
from ..data import allocate_batches
from ..distributed import init_dist, launch_distributed_run
from ..gradients import GradientProcessor
from ..utils.utils import convert_precision_to_torch, setup_reproducibility
from ..utils.worker_utils import create_processor, setup_data_pipeline, setup_model_and_peft
from .autocorrelation import AutocorrelationCollector
from .eigenvectors import LambdaCollector, compute_eigendecomposition, save_uncorrected_eigenvalues
from .kfac import CovarianceCollector
from .shampoo import ShampooCollector
from .tkfac import TraceCovarianceCollector

HESSIAN_APPROXIMATIONS = {
    "kfac": CovarianceCollector,
    "tkfac": TraceCovarianceCollector,
    "shampoo": ShampooCollector,
}


def approximate_hessians(index_cfg: IndexConfig, hessian_cfg: HessianConfig, *, do_eigendecomposition: bool = True) -> str:
    if hessian_cfg.ev_correction and index_cfg.projection_dim != 0:
        raise ValueError(
            "EK-FAC (ev_correction=True) does not support gradient projection; got "
            f"index_cfg.projection_dim={index_cfg.projection_dim}. Set projection_dim=0."
        )
    if hessian_cfg.method == "autocorrelation" and index_cfg.projection_dim == 0:
        warnings.warn(
            "Computing an autocorrelation (dense) Hessian with index_cfg.projection_dim=0 (uncompressed "
            "gradients); this scales quadratically with the uncompressed gradient dimension."
        )
    if index_cfg.debug:
        setup_reproducibility()
    index_cfg.partial_run_path.mkdir(parents=True, exist_ok=True)
    ds, _ = setup_data_pipeline(index_cfg)
    launch_distributed_run("hessian", hessian_worker, [index_cfg, hessian_cfg, ds, do_eigendecomposition],
                           index_cfg.distributed)
    if index_cfg.distributed.rank == 0:
        shutil.move(index_cfg.partial_run_path, index_cfg.run_path)
    return index_cfg.run_path


def hessian_worker(rank: int, local_rank: int, world_size: int, index_cfg: IndexConfig, hessian_cfg: HessianConfig,
                   ds: Dataset, do_eigendecomposition: bool = True, target_modules: set[str] | None = None):
    init_dist(rank, local_rank, world_size)
    model, peft_targets = setup_model_and_peft(index_cfg)
    target_modules = peft_targets if target_modules is None else target_modules
    attention_cfgs = {m: index_cfg.attention for m in index_cfg.split_attention_modules}
    batches = allocate_batches(ds["length"][:], index_cfg.token_batch_size)

    if hessian_cfg.method == "autocorrelation":
        processor = create_processor(model, index_cfg, target_modules)
        collector = AutocorrelationCollector(
            model=model.base_model, data=ds, path=str(index_cfg.partial_run_path), processor=processor,
            target_modules=target_modules, attention_cfgs=attention_cfgs, filter_modules=index_cfg.filter_modules,
        )
        collector.attribute_tokens = index_cfg.attribute_tokens
        CollectorComputer(model=model, data=ds, collector=collector, batches=batches, cfg=index_cfg
                          ).run_with_collector_hooks(desc="Approximating autocorrelation Hessian")
        return

    kwargs = dict(model=model, data=ds, index_cfg=index_cfg, hessian_cfg=hessian_cfg, target_modules=target_modules,
                  attention_cfgs=attention_cfgs, batches=batches)
    collect_hessians(**kwargs)
    if dist.is_initialized():
        dist.barrier()
    if not do_eigendecomposition:
        return
    total = torch.load(f"{index_cfg.partial_run_path}/total_processed.pt", map_location="cpu", weights_only=False)
    vals_a = compute_eigendecomposition(os.path.join(index_cfg.partial_run_path, "activation_sharded"), total)
    vals_g = compute_eigendecomposition(os.path.join(index_cfg.partial_run_path, "gradient_sharded"), total)
    if dist.is_initialized():
        dist.barrier()
    save_uncorrected_eigenvalues(index_cfg.partial_run_path, vals_a, vals_g, total,
                                 dist.get_rank() if dist.is_initialized() else 0,
                                 dist.get_world_size() if dist.is_initialized() else 1)
    if hessian_cfg.ev_correction:
        if dist.is_initialized():
            dist.barrier()
        collect_hessians(**kwargs, ev_correction=True)


def collect_hessians(model, data: Dataset, index_cfg: IndexConfig, *, batches=None, target_modules=None,
                     attention_cfgs: dict[str, AttentionConfig] | None = None, hessian_cfg: HessianConfig,
                     ev_correction: bool = False, eigen_path: str | None = None,
                     output_subdir: str = "eigenvalue_correction_sharded"):
    """One data pass with a factor collector (or the eigenvalue-correction collector)."""
    args = dict(
        model=model.base_model, target_modules=target_modules, attention_cfgs=attention_cfgs or {},
        path=str(index_cfg.partial_run_path), filter_modules=index_cfg.filter_modules,
        processor=GradientProcessor(include_bias=index_cfg.include_bias),
        dtype=convert_precision_to_torch(hessian_cfg.hessian_dtype),
    )
    desc = f"Approximating Hessians with {hessian_cfg.method}"
    if ev_correction:
        collector = LambdaCollector(**args, eigen_path=eigen_path, output_subdir=output_subdir)
        desc += " (eigenvalue correction)"
    else:
        collector = HESSIAN_APPROXIMATIONS[hessian_cfg.method](**args)
    computer = CollectorComputer(model=model, data=data, collector=collector, batches=batches, cfg=index_cfg)
    computer.forward_backward = fwd_bwd_hessian_factory(index_cfg, hessian_cfg)
    computer.run_with_collector_hooks(desc=desc)
