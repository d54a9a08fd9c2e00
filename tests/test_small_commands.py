"""The small commands end to end on CPU: mixing two curvature estimates, the padding /
batching diagnosis of a model configuration, and the recall benchmark through the CLI."""

import csv

import numpy as np
import pytest
import torch

from bergson_b200.__main__ import main
from bergson_b200.gradients import GradientProcessor
from bergson_b200.utils.math import compute_lambda

MODEL = "native:llama-tiny?vocab_size=256"


def _hessian(path, data):
    main(["hessian", str(path), "--model", MODEL, "--index_cfg.data.dataset", data, "--method", "autocorrelation",
          "--projection_dim", "4", "--token_batch_size", "64", "--nproc_per_node", "1"])
    return GradientProcessor.load(path)


def test_mix_blends_two_autocorrelation_hessians(tmp_path):
    q = _hessian(tmp_path / "q", "synthetic:zipf?n=6&len=14&vocab=256&seed=1&min_len=8")
    i = _hessian(tmp_path / "i", "synthetic:zipf?n=12&len=14&vocab=256&seed=0&min_len=6")
    assert q.hessians and set(q.hessians) == set(i.hessians)
    main(["mix", "--query_path", str(tmp_path / "q"), "--index_path", str(tmp_path / "i"), "--output_path", str(tmp_path / "m"),
          "--target_downweight_components", "5"])
    mixed = GradientProcessor.load(tmp_path / "m")
    lam = compute_lambda(q.hessians_eigen, i.hessians_eigen, 5)
    assert 0.0 < lam < 1.0
    for k in q.hessians:
        torch.testing.assert_close(mixed.hessians[k], lam * q.hessians[k] + (1 - lam) * i.hessians[k], rtol=1e-5, atol=1e-8)
    assert mixed.projection_dim == 4 and (tmp_path / "m" / "config.yaml").exists()
    # only autocorrelation estimates can be mixed
    main(["hessian", str(tmp_path / "k"), "--model", MODEL, "--index_cfg.data.dataset", "synthetic:zipf?n=6&len=14&vocab=256&seed=1&min_len=8",
          "--method", "kfac", "--token_batch_size", "64", "--nproc_per_node", "1", "--use_dataset_labels"])
    with pytest.raises(AssertionError, match="autocorrelation"):
        main(["mix", "--query_path", str(tmp_path / "k"), "--index_path", str(tmp_path / "i"), "--output_path", str(tmp_path / "m2")])
    with pytest.raises(ValueError, match="requires"):
        main(["mix", "--query_path", str(tmp_path / "q")])


def test_model_configuration_diagnosis_passes_in_fp32(tmp_path, capsys):
    """Gradients of a document must not depend on what it is batched and padded with; in fp32
    on CPU the in-tree model passes every trial."""
    main(["test_model_configuration", "--model", MODEL, "--dataset", "synthetic:zipf?n=12&len=20&vocab=256&seed=3&min_len=5",
          "--precision", "fp32", "--n_trials", "4", "--device", "cpu"])
    out = capsys.readouterr().out
    assert "PASS  Special token check" in out and "PASS  Equal-length batching" in out
    assert "PASS  precision=fp32" in out and "FAIL" not in out
    assert "Flagged:  0/4" in out


def test_recall_command(tmp_path):
    from datasets import load_from_disk

    from bergson_b200.config import RecallDataConfig
    from bergson_b200.recall import ensure_recall_datasets
    from bergson_b200.score.score_writer import save_sequence_scores

    data = RecallDataConfig(num_people=4, seed=0, data_dir=str(tmp_path / "data"))
    s_path, q_path = ensure_recall_datasets(data)
    st, qs = load_from_disk(str(s_path)), load_from_disk(str(q_path))
    scores = np.zeros((len(st), len(qs)), dtype=np.float32)
    for q, key in enumerate(zip(qs["identifier"], qs["field"])):
        for i, skey in enumerate(zip(st["identifier"], st["field"])):
            scores[i, q] = 1.0 if skey == key else 0.0
    save_sequence_scores(tmp_path / "scores", scores)
    main(["recall", str(tmp_path / "out"), "--scores", str(tmp_path / "scores"), "--k", "3", "--data.num_people", "4",
          "--data.seed", "0", "--data.data_dir", str(tmp_path / "data")])
    row = list(csv.DictReader(open(tmp_path / "out" / "summary.csv")))[0]
    assert float(row["MRR"]) == 1.0 and float(row["recall_at_3"]) == 1.0 and (tmp_path / "out" / "config.yaml").exists()


def test_eigenvalue_correction_refuses_projected_gradients(tmp_path):
    """The corrected eigenvalues live in the unprojected [O, I] basis of every layer."""
    with pytest.raises(ValueError, match="does not support gradient projection"):
        main(["hessian", str(tmp_path / "h"), "--model", MODEL, "--index_cfg.data.dataset",
              "synthetic:zipf?n=4&len=10&vocab=256&seed=0&min_len=6", "--method", "kfac", "--ev_correction", "true",
              "--projection_dim", "8", "--nproc_per_node", "1"])
    assert not (tmp_path / "h").exists() or not any((tmp_path / "h").glob("*_sharded"))
