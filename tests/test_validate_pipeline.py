"""Leave-subsets-out validation end to end on CPU: retraining in process, banking the
retrained models, and re-evaluating the bank give the same numbers."""

import csv
import json

import pytest
import torch

from bergson_b200.__main__ import main
from bergson_b200.config import ValidationConfig
from bergson_b200.models import load_model
from bergson_b200.validate import _load_banked_model

MODEL = "native:llama-tiny?vocab_size=256&num_hidden_layers=1"
TRAIN = "synthetic:zipf?n=8&len=12&vocab=256&seed=0&min_len=12"
QUERY = "synthetic:zipf?n=4&len=12&vocab=256&seed=1&min_len=12"
BASE = ["--model", MODEL, "--data.dataset", TRAIN, "--query.dataset", QUERY, "--batch_size", "4", "--lr", "1e-2",
        "--nproc_per_node", "1"]


def _rows(path):
    with open(path) as f:
        return list(csv.DictReader(f))


def test_validation_banks_models_and_the_bank_reproduces_it(tmp_path):
    run = tmp_path / "run"
    main(["magic", str(run), *BASE, "--query_method", "mean", "--skip_validation", "false", "--num_subsets", "4",
          "--subset_fraction", "0.25", "--save_models", "true"])
    rows = _rows(run / "validation.csv")
    subsets = json.load(open(run / "subsets.json"))
    assert len(rows) == 4 and len(subsets) == 4 and all(len(s) == 2 for s in subsets)  # a quarter of 8 documents
    assert all((run / "retrained" / d / "model.safetensors").exists() for d in ["base"] + [f"subset_{i}" for i in range(4)])
    live = _rows(run / "summary.csv")[0]

    # the banked base model is the trained model; a subset model differs from it
    base = load_model(str(run / "retrained" / "base"))
    sub0 = load_model(str(run / "retrained" / "subset_0"))
    assert any(not torch.equal(a, b) for a, b in zip(base.parameters(), sub0.parameters()))

    ev = tmp_path / "eval"
    main(["validate", str(ev), *BASE, "--query_method", "mean", "--scores", str(run / "scores"), "--retrained_dir", str(run),
          "--num_subsets", "4"])
    banked = _rows(ev / "summary.csv")[0]
    assert float(banked["baseline_loss"]) == pytest.approx(float(live["baseline_loss"]), rel=1e-5)
    assert float(banked["spearman_corr"]) == pytest.approx(float(live["spearman_corr"]), abs=1e-9)
    assert float(banked["pearson_corr"]) == pytest.approx(float(live["pearson_corr"]), abs=1e-3)
    # the per-bank query losses are cached beside the bank and reused
    caches = list(run.glob("losses_*.pt"))
    assert len(caches) == 1 and torch.load(caches[0], weights_only=True).shape == (5, 4)  # base + 4 subsets, 4 queries
    stamp = caches[0].stat().st_mtime_ns
    main(["validate", str(tmp_path / "eval2"), *BASE, "--query_method", "mean", "--scores", str(run / "scores"),
          "--retrained_dir", str(run), "--num_subsets", "4"])
    assert caches[0].stat().st_mtime_ns == stamp


def test_banked_model_loading(tmp_path):
    cfg = ValidationConfig(run_path=str(tmp_path), model=MODEL)
    model = load_model(MODEL)
    with torch.no_grad():
        next(model.parameters()).add_(1.0)  # neither the seeded init nor a fresh one can pass by accident
    model.save_pretrained(tmp_path / "subset_0")
    back = _load_banked_model(cfg, str(tmp_path / "subset_0"), "cpu")
    x = torch.arange(8)[None]
    with torch.no_grad():
        torch.testing.assert_close(back(x).logits, model(x).logits)
    with pytest.raises(FileNotFoundError, match="save_models"):
        _load_banked_model(cfg, str(tmp_path / "subset_9"), "cpu")
    adapter = tmp_path / "adapter_only"
    adapter.mkdir()
    (adapter / "adapter_config.json").write_text("{}")
    try:
        import peft  # noqa: F401
    except ImportError:
        with pytest.raises(ImportError, match="adapter only"):
            _load_banked_model(cfg, str(adapter), "cpu")


@pytest.mark.parametrize("optimizer,lr,extra", [("sgd", "5e-2", ["--adam_beta1", "0.0"]), ("adamw", "1e-3", ["--eps_root", "1e-2"])])
def test_scores_predict_leave_subset_out_retraining(tmp_path, optimizer, lr, extra):
    """Linear datamodelling score: the summed scores of a removed subset must rank the loss changes
    of actually retraining without it.  Four steps of plain SGD, or of Adam with a regularised
    denominator, respond smoothly to the data weights and the correlation is close to one.  (With
    Adam's default tiny `eps_root` the first updates are nearly sign(g), whose derivative with respect
    to the weights vanishes: a four-step toy then has nothing linear to predict, which says nothing
    about the scores.)"""
    run = tmp_path / "run"
    main(["magic", str(run), "--model", MODEL, "--data.dataset", "synthetic:zipf?n=32&len=16&vocab=256&seed=0&min_len=16",
          "--query.dataset", "synthetic:zipf?n=8&len=16&vocab=256&seed=1&min_len=16", "--batch_size", "8", "--lr", lr,
          "--optimizer", optimizer, *extra, "--nproc_per_node", "1", "--query_method", "mean", "--skip_validation", "false",
          "--num_subsets", "16", "--subset_fraction", "0.25", "--precision", "fp32"])
    summary = _rows(run / "summary.csv")[0]
    assert float(summary["spearman_corr"]) > 0.9 and float(summary["pearson_corr"]) > 0.9, summary
    rows = _rows(run / "validation.csv")
    same_sign = sum((float(r["diff"]) > 0) == (float(r["score_sum"]) > 0) for r in rows)
    assert same_sign >= 14  # removing helpful documents raises the query loss, and the scores say so
