"""MRR / Recall@k of attribution scores on the synthetic-facts benchmark: for every
question, rank all training statements by score and find the statements that state the
asked fact (reference ``bergson/recall/recall.py:60-189``)."""

from __future__ import annotations

import os
from collections import defaultdict
from pathlib import Path

import numpy as np
from datasets import load_from_disk

from ..config.config import RecallConfig, ScoreConfig
from ..config.config_io import load_subconfig
from ..data import load_scores
from ..utils.csv_writer import CSVWriter
from .generate import ensure_recall_datasets


def gold_ranks(scores_col: np.ndarray, gold_idx: np.ndarray) -> np.ndarray:
    """1-based ranks under a descending, stable sort (ties keep row order)."""
    out = np.empty(len(gold_idx), dtype=np.int64)
    for j, i in enumerate(gold_idx):
        out[j] = int((scores_col > scores_col[i]).sum()) + int((scores_col[:i] == scores_col[i]).sum()) + 1
    return out


def resolve_higher_is_better(scores_path: str, explicit: bool | None) -> bool:
    if explicit is not None:
        return explicit
    cfg = load_subconfig(scores_path, "score_cfg", ScoreConfig) if scores_path and os.path.isdir(scores_path) else None
    if cfg is None:
        return True
    print(f"Using higher_is_better={cfg.higher_is_better} recorded in {scores_path}")
    return cfg.higher_is_better


def run_recall(cfg: RecallConfig) -> dict[str, float]:
    s_path, q_path = ensure_recall_datasets(cfg.data)
    statements, questions = load_from_disk(str(s_path)), load_from_disk(str(q_path))
    scores = load_scores(Path(cfg.scores))
    if len(scores) != len(statements):
        raise ValueError(f"Scores at {cfg.scores} cover {len(scores)} items but {s_path} has {len(statements)} statements.")
    if scores.num_scores != len(questions):
        raise ValueError(f"Scores at {cfg.scores} have {scores.num_scores} queries but {q_path} has {len(questions)} questions.")
    if not scores.is_written():
        print("Warning: not all score entries have been written; results may be incomplete.")
    gold: dict[tuple, list[int]] = defaultdict(list)
    for i, key in enumerate(zip(statements["identifier"], statements["field"])):
        gold[key].append(i)
    hib = resolve_higher_is_better(cfg.scores, cfg.higher_is_better)
    k = cfg.k
    os.makedirs(cfg.run_path, exist_ok=True)
    w = CSVWriter(os.path.join(cfg.run_path, "recall.csv"),
                  ["question_idx", "identifier", "field", "answer", "first_gold_rank", "reciprocal_rank", f"hit_at_{k}",
                   f"strict_recall_at_{k}", "num_gold"])
    ids, fields, answers = questions["identifier"], questions["field"], questions["answer"]
    rr, hits, strict = [], [], []
    for q in range(len(questions)):
        col = np.asarray(scores.get(slice(None), q), dtype=np.float64)
        col = col if hib else -col
        g = np.asarray(gold[(ids[q], fields[q])])
        ranks = gold_ranks(col, g)
        first = int(ranks.min())
        rr.append(1.0 / first)
        hits.append(int(first <= k))
        strict.append(float((ranks <= k).mean()))
        w.writerow(q, ids[q], fields[q], answers[q], first, rr[-1], hits[-1], strict[-1], len(g))
    w.close()
    out = {"mrr": float(np.mean(rr)), f"recall_at_{k}": float(np.mean(hits)), f"strict_recall_at_{k}": float(np.mean(strict))}
    sw = CSVWriter(os.path.join(cfg.run_path, "summary.csv"), ["MRR", f"recall_at_{k}", f"strict_recall_at_{k}", "N", "num_people"])
    sw.writerow(out["mrr"], out[f"recall_at_{k}"], out[f"strict_recall_at_{k}"], len(questions), cfg.data.num_people)
    sw.close()
    print(f"MRR: {out['mrr']:.4f}  Recall@{k}: {out[f'recall_at_{k}']:.4f}  (N={len(questions)} questions, {len(statements)} statements)")
    return out
