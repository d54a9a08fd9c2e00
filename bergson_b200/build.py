"""``build``: dataset -> on-disk gradient store (reference ``bergson/build.py``)."""

from __future__ import annotations

import shutil
from datetime import timedelta

from datasets import Dataset

from .collection import collect_gradients
from .config.config import IndexConfig, PreprocessConfig
from .data import allocate_batches
from .distributed import cap_world_size_to_dataset, init_dist, launch_distributed_run, parent_barrier
from .utils.utils import setup_reproducibility
from .utils.worker_utils import create_processor, setup_data_pipeline, setup_model_and_peft


def build_worker(rank: int, local_rank: int, world_size: int, index_cfg: IndexConfig,
                 preprocess_cfg: PreprocessConfig, ds: Dataset):
    """One rank of a build: load the model, take this rank's batches, collect."""
    init_dist(rank, local_rank, world_size, timeout=timedelta(minutes=30))
    model, target_modules = setup_model_and_peft(index_cfg)
    processor = create_processor(model, index_cfg, target_modules)
    if index_cfg.auto_batch_size:
        from .utils.batch_size import maybe_auto_batch_size

        maybe_auto_batch_size(index_cfg, model, ds, processor, target_modules, rank)
    attention_cfgs = {m: index_cfg.attention for m in index_cfg.split_attention_modules}
    batches = allocate_batches(ds["length"][:], index_cfg.token_batch_size, max_batch_size=index_cfg.max_batch_size)
    collect_gradients(
        model=model, data=ds, processor=processor, cfg=index_cfg, target_modules=target_modules,
        attention_cfgs=attention_cfgs, preprocess_cfg=preprocess_cfg, batches=batches,
    )


def build(index_cfg: IndexConfig, preprocess_cfg: PreprocessConfig):
    """Preprocess the data in the parent, run the workers, promote ``<run>.part``."""
    if index_cfg.debug:
        setup_reproducibility()
    index_cfg.partial_run_path.mkdir(parents=True, exist_ok=True)
    ds, _ = setup_data_pipeline(index_cfg)
    dist_cfg = index_cfg.distributed
    if isinstance(ds, Dataset) and len(ds) < dist_cfg.world_size:
        dist_cfg = cap_world_size_to_dataset(index_cfg.distributed, len(ds))
        print(f"reducing to nnode=1 and nproc_per_node={dist_cfg.nproc_per_node} for step")
    launch_distributed_run("build", build_worker, [index_cfg, preprocess_cfg, ds], dist_cfg)
    if dist_cfg.rank == 0:
        shutil.move(index_cfg.partial_run_path, index_cfg.run_path)
    if dist_cfg.world_size < index_cfg.distributed.world_size:
        parent_barrier(index_cfg.distributed)
