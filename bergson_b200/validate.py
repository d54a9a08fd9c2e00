"""Leave-k-out validation (LDS) of attribution scores
(reference ``bergson/validate.py:42-739``).

For each random subset S of training documents the model is retrained with the subset's
weights set to ``subset_weight``; the change of the query loss, ``L_base - L_S``, is
correlated (Spearman / Pearson) with the summed scores of S.  ``weight_lrs`` instead
retrains with ``w = 1 - lr * score`` and compares with the first-order prediction.
Scores follow the loss-signed convention: ``s_i = dL_query / dw_i``.
"""

from __future__ import annotations

import hashlib
import json
import os
import random
from collections.abc import Callable

import numpy as np
import torch
import torch.distributed as dist
import torch.nn.functional as F
from scipy.stats import pearsonr, spearmanr
from tqdm.auto import tqdm

from .config.config import ValidationConfig
from .data import load_scores_loss_signed, pad_and_tensor
from .magic.data_stream import DataStream
from .utils.csv_writer import CSVWriter


def bank_loss_cache_key(run_cfg: ValidationConfig, multi_query: bool, num_subsets: int) -> str:
    """File name of the cached per-subset query losses of a bank of retrained models; the
    key covers everything the losses depend on."""
    q = run_cfg.query
    ident = {
        "model": run_cfg.model, "model_kwargs": run_cfg.model_kwargs, "query_dataset": q.dataset,
        "query_split": q.split, "query_subset": q.subset, "query_prompt_column": q.prompt_column,
        "query_completion_column": q.completion_column, "query_truncation": q.truncation,
        "query_format_template": q.format_template, "query_data_kwargs": q.data_kwargs,
        "query_chunk_length": q.chunk_length, "batch_size": run_cfg.batch_size, "multi_query": multi_query,
        "num_subsets": num_subsets,
    }
    return f"losses_{hashlib.sha256(json.dumps(ident, sort_keys=True, default=str).encode()).hexdigest()[:16]}.pt"


def _load_banked_model(run_cfg: ValidationConfig, out_dir: str, device) -> torch.nn.Module:
    """A model banked by ``save_models``: a full checkpoint, or -- when the run trained an
    adapter -- a directory holding only the adapter, which has to be applied to the run's base
    model (pointing a checkpoint loader at such a directory would give the bare base model)
    (reference ``bergson/validate.py:74-85``)."""
    from .models import load_model

    if os.path.isfile(os.path.join(out_dir, "adapter_config.json")):
        try:
            from peft import PeftModel
        except ImportError as e:
            raise ImportError(f"{out_dir} holds an adapter only; loading it needs the peft package") from e
        base = load_model(run_cfg.model, dtype=torch.float32, device=device)
        return PeftModel.from_pretrained(base, out_dir).to(device)
    if not os.path.isdir(out_dir):
        raise FileNotFoundError(f"no banked model at {out_dir} (was the run made with save_models?)")
    return load_model(out_dir, dtype=torch.float32, device=device)


def per_doc_query_losses(forward: Callable, query_stream: DataStream, num_docs: int) -> torch.Tensor:
    """Mean CE of each query document.  ``forward(input_ids)`` returns logits; a model (an
    ``nn.Module`` whose output has ``.logits``) may be passed instead.  Token losses are
    scattered by the document id of the *label* token and reduced over ranks."""
    if isinstance(forward, torch.nn.Module):
        module = forward
        forward = lambda x: module(input_ids=x).logits  # noqa: E731
    device = query_stream.device
    sums = torch.zeros(num_docs, device=device)
    counts = torch.zeros(num_docs, device=device)
    ds = query_stream.dataset
    with torch.no_grad():
        for i in range(len(query_stream)):
            rows = query_stream.batch_rows(i)
            batch = ds[rows]
            x, y, _, _ = pad_and_tensor(batch["input_ids"], labels=batch.get("labels"), device=device)
            if "doc_ids" in batch:
                ids = torch.tensor(batch["doc_ids"], device=device)[:, : x.shape[1]]
            else:
                ids = torch.tensor(rows, device=device)[:, None].expand(-1, x.shape[1])
            logits = forward(x)
            tgt = y[:, 1:]
            tok = F.cross_entropy(logits[:, :-1].flatten(0, 1).float(), tgt.flatten(), reduction="none",
                                  ignore_index=-100).view_as(tgt)
            m = tgt != -100
            sel = ids[:, 1:][m]
            sums.scatter_add_(0, sel, tok[m])
            counts.scatter_add_(0, sel, torch.ones_like(sel, dtype=counts.dtype))
    if dist.is_initialized():
        dist.all_reduce(sums)
        dist.all_reduce(counts)
    return sums / counts.clamp_min(1.0)


def report_multi_query_validation(run_path: str, diffs, score_sums, baselines, num_subsets: int,
                                  summary_name: str = "summary.csv"):
    n_q = len(diffs[0])
    w = CSVWriter(os.path.join(run_path, summary_name),
                  ["query", "spearman_corr", "spearman_p", "pearson_corr", "pearson_p", "N", "baseline_loss"])
    rhos = []
    for q in range(n_q):
        d, s = [r[q] for r in diffs], [r[q] for r in score_sums]
        sp, pe = spearmanr(d, s), pearsonr(d, s)
        rhos.append(sp.statistic)
        print(f"Query {q}: Spearman {sp.statistic:.4f} (p={sp.pvalue:.2e})  Pearson {pe.statistic:.4f} (p={pe.pvalue:.2e})")
        w.writerow(q, sp.statistic, sp.pvalue, pe.statistic, pe.pvalue, num_subsets, float(baselines[q]))
    w.close()
    print(f"Mean Spearman across {n_q} queries: {np.mean(rhos):.4f}")


def draw_subsets(run_cfg: ValidationConfig, valid: torch.Tensor) -> list[torch.Tensor]:
    """Subsets of the validation pool: independent draws of ``subset_fraction`` of the pool,
    or a partition of a random permutation into ``num_subsets`` chunks (then shuffled)."""
    gen = torch.Generator().manual_seed(run_cfg.seed)
    if run_cfg.subset_fraction > 0:
        size = max(1, round(run_cfg.subset_fraction * len(valid)))
        return [valid[torch.randperm(len(valid), generator=gen)[:size]] for _ in range(run_cfg.num_subsets)]
    subsets = list(valid[torch.randperm(len(valid), generator=gen)].chunk(run_cfg.num_subsets))
    random.Random(run_cfg.seed).shuffle(subsets)
    return subsets


def _reset_weights(stream: DataStream, pad_count: int, weight_pad_count: int) -> None:
    stream.weights.data.fill_(1.0)
    if pad_count:
        if stream.weights.ndim == 1:
            stream.weights.data[-weight_pad_count:] = 0.0
        else:
            stream.weights.data[-pad_count:] = 0.0


def _retrain(run_cfg, rank, schedule, stream):
    from .magic.trainer import prepare_trainer

    torch.manual_seed(run_cfg.seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(run_cfg.seed)
    trainer, state, model = prepare_trainer(run_cfg, rank, schedule)
    state.detach_()
    for batch in stream:
        state = trainer.step(state, batch, inplace=True, fsdp=run_cfg.fsdp, max_grad_norm=run_cfg.max_grad_norm,
                             grad_accum_steps=run_cfg.grad_accum_steps)
    return trainer, state


def _mean_query_loss(trainer, state, query_stream, world_size) -> float:
    loss = torch.zeros((), device=query_stream.device)
    with torch.no_grad():
        for batch in query_stream:
            batch = {k: v for k, v in batch.items() if k != "example_weight"}
            loss += trainer.call_model(state.params, batch, state.buffers).loss.detach() / len(query_stream)
    if world_size > 1:
        dist.all_reduce(loss, op=dist.ReduceOp.AVG)
    return float(loss)


def validate_scores(run_cfg: ValidationConfig, scores: torch.Tensor, multi_query: bool, *, global_rank: int,
                    rank: int, world_size: int, schedule: Callable, stream: DataStream, query_stream: DataStream,
                    fwd_state, model, trainer, baseline: float, num_query_docs: int, query_weight_pad_count: int,
                    pad_count: int, weight_pad_count: int):
    real_q = num_query_docs - query_weight_pad_count
    base_per_doc = torch.zeros(real_q)
    fwd = lambda tr, st: (lambda x: tr.call_model(st.params, {"input_ids": x}, st.buffers).logits)  # noqa: E731
    if multi_query:
        if scores.shape[-1] != real_q:
            raise ValueError(f"scores has {scores.shape[-1]} query columns but the query dataset has {real_q} "
                             "documents; multi-query validation requires one score column per query document")
        base_per_doc = per_doc_query_losses(fwd(trainer, fwd_state), query_stream, num_query_docs)[:real_q].cpu()
    elif not (scores.ndim == 2 and scores.shape[1] > 1):
        scores = scores.flatten()
    n_q = scores.shape[-1] if multi_query else 1
    flat = scores.reshape(-1, n_q).float()
    main = global_rank == 0

    if run_cfg.weight_lrs:
        step = flat.mean(dim=1)
        predicted = (flat * step[:, None]).sum(dim=0)
        path = os.path.join(run_cfg.run_path, "weight_step.csv")
        cols = ["lr", "query", "diff", "predicted_diff"] if multi_query else ["lr", "diff", "predicted_diff"]
        w = CSVWriter(path, cols, enabled=main)
        for lr in run_cfg.weight_lrs:
            _reset_weights(stream, pad_count, weight_pad_count)
            stream.weights.data.view(-1)[: len(step)] -= lr * step.to(stream.weights)
            tr, st = _retrain(run_cfg, rank, schedule, stream)
            if multi_query:
                per = per_doc_query_losses(fwd(tr, st), query_stream, num_query_docs)[:real_q].cpu()
                d = base_per_doc - per
                for q in range(real_q):
                    w.writerow(lr, q, d[q].item(), lr * predicted[q].item())
            else:
                diff = baseline - _mean_query_loss(tr, st, query_stream, world_size)
                w.writerow(lr, diff, lr * predicted.mean().item())
                if main:
                    print(f"lr {lr:g}: diff {diff:.6f} (predicted {lr * predicted.mean().item():.6f})")
        w.close()
        return

    valid = torch.nonzero((flat != 0).any(dim=1), as_tuple=True)[0] if run_cfg.exclude_zero_scores else torch.arange(flat.shape[0])
    subsets_path = run_cfg.subsets or os.path.join(run_cfg.run_path, "subsets.json")
    if os.path.exists(subsets_path):
        with open(subsets_path) as f:
            subsets = [torch.tensor(s, dtype=torch.long) for s in json.load(f)]
    else:
        subsets = draw_subsets(run_cfg, valid)
    start = run_cfg.subset_start
    stop = len(subsets) if run_cfg.subset_stop is None else run_cfg.subset_stop
    sliced = (start, stop) != (0, len(subsets))
    csv_path = os.path.join(run_cfg.run_path, f"validation_{start}_{stop}.csv" if sliced else "validation.csv")
    cols = ["subset", "query", "diff", "score_sum"] if multi_query else ["subset", "diff", "score_sum"]
    w = CSVWriter(csv_path, cols, enabled=main)
    if run_cfg.save_models and main and start == 0:
        with open(os.path.join(run_cfg.run_path, "subsets.json"), "w") as f:
            json.dump([s.tolist() for s in subsets], f)
    diffs, sums = [], []
    bar = tqdm(subsets[start:stop], desc="Validating", disable=not main)
    for i, subset in enumerate(bar, start=start):
        _reset_weights(stream, pad_count, weight_pad_count)
        stream.weights.data.view(-1)[subset] = run_cfg.subset_weight
        tr, st = _retrain(run_cfg, rank, schedule, stream)
        if run_cfg.save_models and main:
            from .utils.trainer_export import save_state_as_pretrained

            save_state_as_pretrained(tr, st, os.path.join(run_cfg.run_path, "retrained", f"subset_{i}"), run_cfg)
        if multi_query:
            per = per_doc_query_losses(fwd(tr, st), query_stream, num_query_docs)[:real_q].cpu()
            d, s = base_per_doc - per, flat[subset].sum(dim=0)
            for q in range(real_q):
                w.writerow(i, q, d[q].item(), s[q].item())
            diffs.append(d.tolist())
            sums.append(s.tolist())
            continue
        diff = baseline - _mean_query_loss(tr, st, query_stream, world_size)
        s = flat[subset].sum().item()
        w.writerow(i, diff, s)
        diffs.append(diff)
        sums.append(s)
        if main and len(diffs) >= 2:
            bar.set_postfix({"rho": spearmanr(diffs, sums).statistic})
    w.close()
    _reset_weights(stream, pad_count, weight_pad_count)
    if not main:
        return
    if multi_query:
        report_multi_query_validation(run_cfg.run_path, diffs, sums, base_per_doc, stop - start,
                                      f"summary_{start}_{stop}.csv" if sliced else "summary.csv")
        return
    sp, pe = spearmanr(diffs, sums), pearsonr(diffs, sums)
    print(f"Final Spearman correlation: {sp.statistic:.4f} (p={sp.pvalue:.2e})")
    print(f"Final Pearson correlation:  {pe.statistic:.4f} (p={pe.pvalue:.2e})")
    sw = CSVWriter(os.path.join(run_cfg.run_path, "summary.csv"),
                   ["spearman_corr", "spearman_p", "pearson_corr", "pearson_p", "N", "baseline_loss"])
    sw.writerow(sp.statistic, sp.pvalue, pe.statistic, pe.pvalue, len(subsets), baseline)
    sw.close()


def evaluate_retrained(run_cfg: ValidationConfig, retrained_dir, *, score_path: str):
    """Validation against banks of already retrained models (``retrained/base`` and
    ``retrained/subset_i`` written with ``save_models``); several banks average the query
    losses.  Per-bank losses are cached under a key of the query identity."""
    from .distributed import init_dist  # noqa: F401  (single process evaluation)
    from .models import load_model
    from .utils.utils import get_device
    from .utils.worker_utils import setup_data_pipeline

    dirs = [retrained_dir] if isinstance(retrained_dir, str) else list(retrained_dir)
    scores, multi_query = load_scores_loss_signed(score_path)
    query_ds, n_q = setup_data_pipeline(run_cfg, run_cfg.query)
    device = get_device(0)
    qstream = DataStream(query_ds, min(run_cfg.batch_size, len(query_ds)), device=device)
    with open(run_cfg.subsets or os.path.join(dirs[0], "subsets.json")) as f:
        subsets = [torch.tensor(s, dtype=torch.long) for s in json.load(f)]

    def losses_of(model_dir: str) -> torch.Tensor:
        m = _load_banked_model(run_cfg, model_dir, device)
        m.eval()
        return per_doc_query_losses(lambda x: m(x).logits, qstream, len(query_ds)).cpu()

    bank_losses = []
    for d in dirs:
        cache = os.path.join(d, bank_loss_cache_key(run_cfg, multi_query, len(subsets)))
        if os.path.exists(cache):
            bank_losses.append(torch.load(cache, weights_only=True))
            continue
        rows = [losses_of(os.path.join(d, "retrained", "base"))]
        rows += [losses_of(os.path.join(d, "retrained", f"subset_{i}")) for i in range(len(subsets))]
        t = torch.stack(rows)
        torch.save(t, cache)
        bank_losses.append(t)
    losses = torch.stack(bank_losses).mean(0)  # [1 + subsets, queries]
    base, per_subset = losses[0], losses[1:]
    flat = scores.reshape(scores.shape[0], -1).float()
    os.makedirs(run_cfg.run_path, exist_ok=True)
    if multi_query:
        diffs = [(base - per_subset[i]).tolist() for i in range(len(subsets))]
        sums = [flat[s].sum(0).tolist() for s in subsets]
        report_multi_query_validation(run_cfg.run_path, diffs, sums, base, len(subsets))
        return
    diffs = [(base.mean() - per_subset[i].mean()).item() for i in range(len(subsets))]
    sums = [flat[s].sum().item() for s in subsets]
    sp, pe = spearmanr(diffs, sums), pearsonr(diffs, sums)
    print(f"Final Spearman correlation: {sp.statistic:.4f} (p={sp.pvalue:.2e})")
    sw = CSVWriter(os.path.join(run_cfg.run_path, "summary.csv"),
                   ["spearman_corr", "spearman_p", "pearson_corr", "pearson_p", "N", "baseline_loss"])
    sw.writerow(sp.statistic, sp.pvalue, pe.statistic, pe.pvalue, len(subsets), base.mean().item())
    sw.close()
