"""``query``: interactive prompt loop over a store, or (with ``query_dataset``) a
non-interactive run over pre-tokenised queries that writes ``query_results.json``
(reference ``bergson/query/query_index.py:48-156``)."""

from __future__ import annotations

import csv
import json
from contextlib import contextmanager
from dataclasses import asdict
from pathlib import Path

import torch

from ..config.config import IndexConfig, QueryConfig
from ..config.config_io import CONFIG_FILENAME, load_subconfig
from ..data import load_data_string, pad_and_tensor
from ..utils.utils import get_device, setup_reproducibility
from ..utils.worker_utils import setup_model_and_peft
from .attributor import Attributor


@contextmanager
def csv_recorder(path: str):
    """Yield ``record(row)`` appending to ``path`` (header written once), or None."""
    if not path:
        yield None
        return
    p = Path(path)
    p.parent.mkdir(parents=True, exist_ok=True)
    new = not p.exists()
    with p.open("a", newline="") as f:
        w = csv.writer(f)
        if new:
            w.writerow(["query", "direction", "result", "result_index", "score"])

        def record(row):
            w.writerow(row)
            f.flush()

        yield record


def _trace_both(attr: Attributor, model, x: torch.Tensor, k: int, modules):
    out = []
    for reverse in (False, True):
        with attr.trace(model.base_model, k, modules=modules, reverse=reverse) as res:
            model(x, labels=x).loss.backward()
            model.zero_grad()
        out.append(res)
    return out


def query(query_cfg: QueryConfig):
    index_cfg = load_subconfig(query_cfg.index, "index_cfg", IndexConfig)
    if index_cfg is None:
        raise FileNotFoundError(f"Could not load an index config from '{query_cfg.index}'. Expected a '{CONFIG_FILENAME}'.")
    if index_cfg.debug:
        setup_reproducibility()
    model_cfg = index_cfg
    if query_cfg.model:
        model_cfg = IndexConfig.from_dict({**index_cfg.to_dict(), "model": query_cfg.model})
    model, target_modules = setup_model_and_peft(model_cfg, device_map_auto=query_cfg.device_map_auto)
    attr = Attributor(
        Path(query_cfg.index), device=get_device(), unit_norm=query_cfg.unit_norm,
        faiss_cfg=query_cfg.faiss_cfg if query_cfg.faiss else None, inversion_cfg=query_cfg.inversion_cfg,
        hessian_path=query_cfg.hessian_path, ev_correction=query_cfg.ev_correction,
    )
    device = next(model.parameters()).device

    if query_cfg.query_dataset:
        qds = load_data_string(query_cfg.query_dataset)
        results = []
        for row in qds:
            x, _, _, _ = pad_and_tensor([row["input_ids"]], device=device, sync_max_len=False)
            top, bottom = _trace_both(attr, model, x, query_cfg.top_k, target_modules)
            results.append({
                "top_indices": top.indices.squeeze(0).tolist(), "top_scores": top.scores.squeeze(0).tolist(),
                "bottom_indices": bottom.indices.squeeze(0).tolist(), "bottom_scores": bottom.scores.squeeze(0).tolist(),
            })
        out = Path(query_cfg.index) / "query_results.json"
        with out.open("w") as f:
            json.dump(results, f)
        print(f"Wrote {len(results)} query results to {out}")
        return results

    from transformers import AutoTokenizer

    tokenizer = AutoTokenizer.from_pretrained(query_cfg.model or index_cfg.model)
    ds = load_data_string(index_cfg.data.dataset, index_cfg.data.split, index_cfg.data.subset, index_cfg.data.data_kwargs)
    with csv_recorder(query_cfg.record) as record:
        while True:
            text = input("Enter your query: ")
            if text.lower() == "exit":
                break
            x = tokenizer(text, return_tensors="pt").to(device)["input_ids"]
            for direction, res in zip(("Top", "Bottom"), _trace_both(attr, model, x, query_cfg.top_k, target_modules)):
                print(f"\n{direction} {query_cfg.top_k} results for '{text}':")
                for i, (score, idx) in enumerate(zip(res.scores.reshape(-1), res.indices.reshape(-1))):
                    if idx.item() == -1:
                        print("Found invalid result, skipping")
                        continue
                    doc = str(ds[int(idx)][query_cfg.text_field])
                    print(doc[:2000] + ("\n. . ." if len(doc) > 2000 else ""))
                    print(f"{i + 1}: (distance: {score.item():.4f})")
                    if record is not None:
                        record([text, direction, doc, int(idx), score.item()])
