"""``score``: stream a dataset's gradients against a stored query set
(reference ``bergson/score/score.py``)."""

from __future__ import annotations

import json
import shutil
from pathlib import Path

import numpy as np
import torch
from datasets import Dataset

from ..collection import collect_gradients
from ..config.config import IndexConfig, PreprocessConfig, ScoreConfig
from ..config.config_io import load_subconfig
from ..data import allocate_batches, column_offsets, load_gradients
from ..distributed import cap_world_size_to_dataset, init_dist, launch_distributed_run, parent_barrier
from ..hessians.preconditioner import DensePreconditioner, is_factored_hessian, load_preconditioner
from ..process_grads import normalize_and_aggregate_grads
from ..utils.utils import convert_precision_to_torch, get_device, get_gradient_dtype, numpy_to_tensor
from ..utils.worker_utils import create_processor, setup_data_pipeline, setup_model_and_peft
from .score_writer import MemmapSequenceScoreWriter, MemmapTokenScoreWriter
from .scorer import Scorer


def get_query_grads(score_cfg: ScoreConfig, query_range: tuple[int, int] | None = None):
    """Per-module query tensors from the query store (+ the preprocessing recorded when
    that store was built)."""
    qpath = Path(score_cfg.query_path)
    if not qpath.exists():
        raise FileNotFoundError(
            f"Query dataset not found at {score_cfg.query_path}. Please build a query dataset index first."
        )
    with open(qpath / "info.json") as f:
        sizes = json.load(f)["grad_sizes"]
    recorded = load_subconfig(qpath, "preprocess_cfg", PreprocessConfig) or PreprocessConfig()
    if not score_cfg.modules:
        score_cfg.modules = list(sizes)
    mm = load_gradients(qpath)
    if query_range is not None:
        mm = mm[query_range[0] : query_range[1]]
    grads = {}
    for name, (lo, hi) in column_offsets(sizes).items():
        block = np.ascontiguousarray(mm[:, lo:hi])
        grads[name] = numpy_to_tensor(block).float() if not np.issubdtype(block.dtype, np.floating) else torch.from_numpy(block)
    return grads, recorded


def _make_split_hessian(hessians: dict[str, torch.Tensor], modules: list[str], device, dtype):
    """Index transform ``g_m -> g_m @ H_m^-1/2`` for all modules in one batched GEMM."""
    stacked = torch.stack([hessians[m] for m in modules]).to(device=device, dtype=dtype)

    def transform(grads: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
        g = torch.stack([grads[m].to(device, dtype, non_blocking=True) for m in modules], dim=0)
        out = torch.bmm(g, stacked)
        return {m: out[i] for i, m in enumerate(modules)}

    return transform


def _gather_queries_obstacle(score_cfg: ScoreConfig, preprocess_cfg: PreprocessConfig, device, dtype,
                             attribute_tokens) -> str | None:
    """None when the queries can stay sharded over the ranks and be read through the fused
    all-gather + score GEMM, else the reason why not: it takes CUDA ranks of one NVLink domain,
    16-bit scoring and row-wise query preprocessing only (no aggregation over queries, no
    index-side transform).  Every input is the same on all ranks, so all ranks take the same
    branch."""
    import os

    import torch.distributed as dist

    from ..parallel.peer import symmetric_memory_available

    if not (dist.is_initialized() and dist.get_world_size() > 1):
        return "single rank"
    if torch.device(device).type != "cuda":
        return "not on GPUs"
    if os.environ.get("BERGSON_B200_DISABLE_PEER") == "1":
        return "BERGSON_B200_DISABLE_PEER=1"
    if not symmetric_memory_available():
        return "peer memory is not available to these ranks"
    if dtype not in (torch.bfloat16, torch.float16):
        return f"scoring in {dtype}"
    if attribute_tokens:
        return "per-token rows"
    if preprocess_cfg.aggregation != "none" or preprocess_cfg.normalize_aggregated_grad:
        return "queries are aggregated"
    if preprocess_cfg.hessian_path and preprocess_cfg.unit_normalize:
        return "index-side preconditioning"
    return None


def _gather_queries_ok(score_cfg: ScoreConfig, preprocess_cfg: PreprocessConfig, device, dtype, attribute_tokens) -> bool:
    return _gather_queries_obstacle(score_cfg, preprocess_cfg, device, dtype, attribute_tokens) is None


def create_scorer(path: Path, data: Dataset, score_cfg: ScoreConfig, preprocess_cfg: PreprocessConfig, device,
                  dtype, *, attribute_tokens: bool = False, query_range=None, num_queries_total=None,
                  shard_queries: bool = False) -> Scorer:
    """Load and preprocess the queries (precondition once unless the query store already
    was, unit-normalise / aggregate unless already done) and set up the writer.

    ``shard_queries`` (collective: all ranks pass the same value): each rank loads and
    preprocesses only its slice of the query rows and the scorer reads the other ranks' slices
    through peer memory inside the score GEMM."""
    gather_info = None
    if shard_queries:
        import torch.distributed as dist

        from ..hessians.sharded_computation import shard_bounds

        with open(Path(score_cfg.query_path) / "info.json") as f:
            n_all = json.load(f)["num_grads"]
        base_lo, base_hi = query_range if query_range is not None else (0, n_all)
        lo, hi = shard_bounds(base_hi - base_lo, dist.get_rank(), dist.get_world_size())
        gather_info = (base_hi - base_lo, base_lo)
        query_grads, recorded = get_query_grads(score_cfg, (base_lo + lo, base_lo + hi))
        if recorded.aggregation != "none":
            raise ValueError("sharded queries need a query store with one row per query (aggregation='none')")
    else:
        query_grads, recorded = get_query_grads(score_cfg, query_range)
    pre = load_preconditioner(
        preprocess_cfg.hessian_path, inversion_cfg=preprocess_cfg.inversion_cfg,
        power=-0.5 if preprocess_cfg.unit_normalize else -1.0, ev_correction=preprocess_cfg.ev_correction,
        device=device,
    )
    if pre is not None and not recorded.hessian_path:
        query_grads = pre.apply(query_grads)
    if pre is None or not preprocess_cfg.unit_normalize:
        index_transform = None
    elif isinstance(pre, DensePreconditioner):
        index_transform = _make_split_hessian(pre.h_inv, score_cfg.modules, device, dtype)
    else:
        index_transform = pre.apply

    aggregation = "none" if recorded.aggregation != "none" else preprocess_cfg.aggregation
    query_grads = normalize_and_aggregate_grads(
        query_grads, score_cfg.modules,
        unit_normalize=False if recorded.unit_normalize else preprocess_cfg.unit_normalize,
        device=device, aggregate_grads=aggregation,
        normalize_aggregated_grad=False if recorded.normalize_aggregated_grad else preprocess_cfg.normalize_aggregated_grad,
    )
    if query_range is not None and aggregation != "none":
        raise ValueError("query_batch_size requires aggregation='none': aggregation mixes gradients across "
                         "queries, which a row slice would corrupt.")
    if query_range is not None and score_cfg.score != "individual":
        raise ValueError("query_batch_size requires score='individual': 'nearest' reduces over all queries, "
                         "which per-chunk passes would compute wrongly.")
    n_q = len(query_grads[score_cfg.modules[0]]) if gather_info is None else gather_info[0]
    num_scores = 1 if score_cfg.score == "nearest" else (num_queries_total if num_queries_total is not None else n_q)
    if attribute_tokens:
        writer = MemmapTokenScoreWriter.from_dataset(path, data, num_scores, dtype=dtype)
    else:
        writer = MemmapSequenceScoreWriter(path, len(data), num_scores, dtype=dtype)
    gathered = None
    if gather_info is not None:
        from .scorer import GatheredQueries

        local = torch.cat([query_grads[m].to(device=device, dtype=torch.float32) for m in score_cfg.modules], dim=1)
        gathered = GatheredQueries(local, gather_info[0], dtype)
    return Scorer(
        query_grads=query_grads, modules=score_cfg.modules, writer=writer, device=device, dtype=dtype,
        unit_normalize=preprocess_cfg.unit_normalize, score_mode=score_cfg.score, attribute_tokens=attribute_tokens,
        index_transform=index_transform, query_offset=query_range[0] if query_range is not None else 0,
        gathered=gathered,
    )


def score_worker(rank: int, local_rank: int, world_size: int, index_cfg: IndexConfig, score_cfg: ScoreConfig,
                 preprocess_cfg: PreprocessConfig, ds: Dataset):
    init_dist(rank, local_rank, world_size)
    model, target_modules = setup_model_and_peft(index_cfg)
    processor = create_processor(model, index_cfg, target_modules)
    attention_cfgs = {m: index_cfg.attention for m in index_cfg.split_attention_modules}
    dtype = convert_precision_to_torch(score_cfg.precision) if score_cfg.precision != "auto" else get_gradient_dtype(model)
    device = torch.device(get_device(local_rank))
    batches = allocate_batches(ds["length"][:], index_cfg.token_batch_size, max_batch_size=index_cfg.max_batch_size)
    with open(Path(score_cfg.query_path) / "info.json") as f:
        num_queries = json.load(f)["num_grads"]
    qbs = score_cfg.query_batch_size
    # Every rank walks the same slices so that collectives inside the passes line up.
    ranges = [None] if qbs is None or qbs >= num_queries else [
        (lo, min(lo + qbs, num_queries)) for lo in range(0, num_queries, qbs)
    ]
    obstacle = _gather_queries_obstacle(score_cfg, preprocess_cfg, device, dtype, index_cfg.attribute_tokens)
    shard_queries = obstacle is None
    if rank == 0 and world_size > 1:
        print(f"score: query rows sharded over {world_size} ranks in peer memory (all-gather fused into the score GEMM)"
              if shard_queries else f"score: query rows replicated on every rank ({obstacle})", flush=True)
    for qr in ranges:
        scorer = create_scorer(index_cfg.partial_run_path, ds, score_cfg, preprocess_cfg, device=device, dtype=dtype,
                               attribute_tokens=index_cfg.attribute_tokens, query_range=qr,
                               num_queries_total=num_queries, shard_queries=shard_queries)
        collect_gradients(model=model, data=ds, processor=processor, cfg=index_cfg, target_modules=target_modules,
                          attention_cfgs=attention_cfgs, batches=batches, scorer=scorer)
        scorer.writer.flush()


def score_dataset(index_cfg: IndexConfig, score_cfg: ScoreConfig, preprocess_cfg: PreprocessConfig):
    if preprocess_cfg.hessian_path and index_cfg.projection_dim != 0 and is_factored_hessian(preprocess_cfg.hessian_path):
        extra = ("and unit_normalize=True (cosine similarity) requires projection_dim=0: split (two-sided H^-1/2) "
                 "scoring needs full, unprojected index gradients, but"
                 if preprocess_cfg.unit_normalize else "requires projection_dim=0, but")
        raise ValueError(
            f"Scoring with a factored (EKFAC) hessian at {preprocess_cfg.hessian_path} {extra} "
            f"index_cfg.projection_dim={index_cfg.projection_dim}. Rebuild the index and query with "
            "projection_dim=0, or use a dense (autocorrelation) hessian."
        )
    index_cfg.partial_run_path.mkdir(parents=True, exist_ok=True)
    ds, _ = setup_data_pipeline(index_cfg)
    dist_cfg = index_cfg.distributed
    if isinstance(ds, Dataset) and len(ds) < dist_cfg.world_size:
        dist_cfg = cap_world_size_to_dataset(dist_cfg, len(ds))
        print(f"reducing to nnode=1 and nproc_per_node={dist_cfg.nproc_per_node} for step")
    launch_distributed_run("score", score_worker, [index_cfg, score_cfg, preprocess_cfg, ds], dist_cfg)
    if dist_cfg.rank == 0:
        shutil.move(index_cfg.partial_run_path, index_cfg.run_path)
    if dist_cfg.world_size < index_cfg.distributed.world_size:
        parent_barrier(index_cfg.distributed)
