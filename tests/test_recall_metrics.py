"""Recall benchmark metrics on hand-made score matrices: ranks under ties, misses, the sign
convention (explicit, or read from the scored run), size checks, dataset naming and caching."""

import csv

import numpy as np
import pytest
import yaml
from datasets import Dataset

from bergson_b200.config import RecallConfig, RecallDataConfig
from bergson_b200.recall import recall as recall_mod
from bergson_b200.recall.generate import NUM_FIELDS, ensure_recall_datasets, recall_dataset_paths
from bergson_b200.recall.recall import gold_ranks, resolve_higher_is_better, run_recall
from bergson_b200.score.score_writer import save_sequence_scores


def test_ranks_are_one_based_and_stable_under_ties():
    s = np.array([0.9, 0.1, 0.5, 0.7])
    assert gold_ranks(s, np.array([0])).tolist() == [1] and gold_ranks(s, np.array([3])).tolist() == [2]
    assert gold_ranks(s, np.array([1, 0])).tolist() == [4, 1]
    assert gold_ranks(np.full(4, 0.5), np.arange(4)).tolist() == [1, 2, 3, 4]  # ties keep row order
    t = np.array([0.5, 0.9, 0.5])
    assert gold_ranks(t, np.array([0])).tolist() == [2] and gold_ranks(t, np.array([2])).tolist() == [3]


def _setup(tmp_path, monkeypatch, matrix, hib_in_run=None):
    """Two people, one field, two paraphrases each: 4 statements, 2 questions."""
    st = Dataset.from_list([{"identifier": p, "field": "birthdate", "template": t} for p in (0, 1) for t in (0, 1)])
    qs = Dataset.from_list([{"identifier": p, "field": "birthdate", "answer": f"a{p}"} for p in (0, 1)])
    st.save_to_disk(str(tmp_path / "statements.hf"))
    qs.save_to_disk(str(tmp_path / "questions.hf"))
    monkeypatch.setattr(recall_mod, "ensure_recall_datasets", lambda _cfg: (tmp_path / "statements.hf", tmp_path / "questions.hf"))
    save_sequence_scores(tmp_path / "scores", np.asarray(matrix, dtype=np.float32))
    if hib_in_run is not None:
        (tmp_path / "scores" / "config.yaml").write_text(
            yaml.safe_dump({"steps": [{"score": {"score_cfg": {"higher_is_better": hib_in_run}}}]}))
    return RecallConfig(run_path=str(tmp_path / "out"), scores=str(tmp_path / "scores"), data=RecallDataConfig(num_people=2), k=2)


PERFECT = [[1.0, 0.0], [0.9, 0.1], [0.0, 1.0], [0.1, 0.9]]


def test_perfect_ranking(tmp_path, monkeypatch):
    out = run_recall(_setup(tmp_path, monkeypatch, PERFECT))
    assert out == {"mrr": 1.0, "recall_at_2": 1.0, "strict_recall_at_2": 1.0}
    rows = list(csv.DictReader(open(tmp_path / "out" / "recall.csv")))
    assert [r["first_gold_rank"] for r in rows] == ["1", "1"] and [r["num_gold"] for r in rows] == ["2", "2"]
    summary = list(csv.DictReader(open(tmp_path / "out" / "summary.csv")))[0]
    assert float(summary["MRR"]) == 1.0 and summary["N"] == "2"


def test_a_miss_pushes_the_rank_down(tmp_path, monkeypatch):
    # question 0: its statements (rows 0, 1) come 3rd and 4th; question 1 is perfect
    out = run_recall(_setup(tmp_path, monkeypatch, [[0.1, 0.0], [0.0, 0.1], [1.0, 1.0], [0.9, 0.9]]))
    assert out["mrr"] == pytest.approx((1 / 3 + 1.0) / 2)
    assert out["recall_at_2"] == 0.5 and out["strict_recall_at_2"] == 0.5


def test_sign_convention(tmp_path, monkeypatch):
    neg = (-np.asarray(PERFECT)).tolist()
    cfg = _setup(tmp_path, monkeypatch, neg)
    assert run_recall(cfg)["mrr"] < 1.0  # without information, higher is taken to be better
    cfg.higher_is_better = False
    assert run_recall(cfg)["mrr"] == 1.0


def test_sign_is_read_from_the_scored_run_unless_given(tmp_path, monkeypatch):
    neg = (-np.asarray(PERFECT)).tolist()
    cfg = _setup(tmp_path, monkeypatch, neg, hib_in_run=False)
    assert resolve_higher_is_better(cfg.scores, None) is False
    assert run_recall(cfg)["mrr"] == 1.0
    cfg.higher_is_better = True  # the explicit flag wins over the recorded one
    assert run_recall(cfg)["mrr"] < 1.0
    assert resolve_higher_is_better(str(tmp_path / "nowhere"), None) is True


def test_size_mismatches_are_errors(tmp_path, monkeypatch):
    with pytest.raises(ValueError, match="statements"):
        run_recall(_setup(tmp_path, monkeypatch, PERFECT[:3]))
    (tmp_path / "b").mkdir()
    with pytest.raises(ValueError, match="questions"):
        run_recall(_setup(tmp_path / "b", monkeypatch, [r + [0.0] for r in PERFECT]))


def test_dataset_naming_generation_and_cache(tmp_path):
    a = RecallDataConfig(num_people=5, seed=0, data_dir=str(tmp_path))
    b = RecallDataConfig(num_people=5, seed=1, data_dir=str(tmp_path))
    assert recall_dataset_paths(a) != recall_dataset_paths(b)
    s_path, q_path = ensure_recall_datasets(a)
    from datasets import load_from_disk

    st, qs = load_from_disk(str(s_path)), load_from_disk(str(q_path))
    assert len(qs) == 5 * NUM_FIELDS and len(st) % len(qs) == 0 and len(st) > len(qs)
    stamp = (s_path / "dataset_info.json").stat().st_mtime_ns
    assert ensure_recall_datasets(a) == (s_path, q_path)
    assert (s_path / "dataset_info.json").stat().st_mtime_ns == stamp  # reused, not regenerated
    single = RecallDataConfig(num_people=5, seed=0, data_dir=str(tmp_path), single_paraphrase=True)
    s1, _ = ensure_recall_datasets(single)
    assert len(load_from_disk(str(s1))) == 5 * NUM_FIELDS
    with pytest.raises(ValueError, match="requested"):
        ensure_recall_datasets(RecallDataConfig(num_people=10**7, seed=0, data_dir=str(tmp_path / "big")))
