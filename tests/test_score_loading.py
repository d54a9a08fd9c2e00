"""Loading scores in the "negative lowers the query loss" convention: score directories (one
or many query columns, per-token grids), the ``higher_is_better`` flip and tensors saved by
older runs."""

import numpy as np
import torch
import yaml

from bergson_b200.data import load_scores, load_scores_loss_signed
from bergson_b200.score.score_writer import MemmapSequenceScoreWriter, MemmapTokenScoreWriter


def test_directory_with_several_query_columns(tmp_path):
    w = MemmapSequenceScoreWriter(tmp_path, num_items=6, num_scores=3, distributed=False)
    values = torch.arange(18, dtype=torch.float32).reshape(6, 3)
    w(list(range(6)), values)
    w.flush()
    scores, multi = load_scores_loss_signed(str(tmp_path))
    assert multi and scores.shape == (6, 3)
    torch.testing.assert_close(scores, values)  # no saved score config: nothing is negated
    loaded = load_scores(tmp_path)
    assert loaded.num_scores == 3 and bool(np.asarray(loaded.mmap["written_2"]).all())


def test_single_column_directory_and_partial_writes(tmp_path):
    w = MemmapSequenceScoreWriter(tmp_path, num_items=4, num_scores=1, distributed=False)
    w([0, 2], torch.tensor([[1.0], [3.0]]))
    w.flush()
    scores, multi = load_scores_loss_signed(str(tmp_path))
    assert not multi and scores.shape == (4, 1)
    loaded = load_scores(tmp_path)
    assert np.asarray(loaded.mmap["written_0"]).tolist() == [True, False, True, False]
    # a second writer on the same path resumes instead of truncating
    w2 = MemmapSequenceScoreWriter(tmp_path, num_items=4, num_scores=1, distributed=False)
    w2([1, 3], torch.tensor([[2.0], [4.0]]))
    w2.flush()
    scores, _ = load_scores_loss_signed(str(tmp_path))
    assert scores[:, 0].tolist() == [1.0, 2.0, 3.0, 4.0]


def test_higher_is_better_stores_are_negated(tmp_path):
    w = MemmapSequenceScoreWriter(tmp_path, num_items=3, num_scores=1, distributed=False)
    w([0, 1, 2], torch.tensor([[1.0], [-2.0], [3.0]]))
    w.flush()
    (tmp_path / "config.yaml").write_text(yaml.safe_dump({"steps": [{"score": {"score_cfg": {"higher_is_better": True}}}]}))
    scores, _ = load_scores_loss_signed(str(tmp_path))
    assert scores[:, 0].tolist() == [-1.0, 2.0, -3.0]
    (tmp_path / "config.yaml").write_text(yaml.safe_dump({"steps": [{"score": {"score_cfg": {"higher_is_better": False}}}]}))
    assert load_scores_loss_signed(str(tmp_path))[0][:, 0].tolist() == [1.0, -2.0, 3.0]


def test_token_scores_come_back_as_a_padded_grid(tmp_path):
    counts = np.array([2, 0, 3])
    w = MemmapTokenScoreWriter(tmp_path, counts, num_scores=1, distributed=False)
    w([0, 2], torch.tensor([[1.0], [2.0], [3.0], [4.0], [5.0]]))
    w.flush()
    scores, multi = load_scores_loss_signed(str(tmp_path))
    assert not multi and scores.shape == (3, 4)  # sequence length = most gradient rows + 1 (the last position has none)
    assert scores[0].tolist() == [1.0, 2.0, 0.0, 0.0] and scores[2].tolist() == [3.0, 4.0, 5.0, 0.0]
    assert float(scores[1].abs().sum()) == 0.0


def test_tensors_saved_by_older_runs(tmp_path):
    per_token = torch.randn(6, 5)
    torch.save(per_token, tmp_path / "scores.pt")
    scores, multi = load_scores_loss_signed(str(tmp_path / "scores.pt"))
    assert not multi  # 2-D without a run config: per-token scores of one query
    torch.testing.assert_close(scores, per_token)
    (tmp_path / "config.yaml").write_text(yaml.safe_dump({"steps": [{"magic": {"query_method": "none"}}]}))
    assert load_scores_loss_signed(str(tmp_path / "scores.pt"))[1]  # the run was per-query
    torch.save(torch.randn(4, 6, 3), tmp_path / "tok.pt")
    scores, multi = load_scores_loss_signed(str(tmp_path / "tok.pt"))
    assert multi and scores.shape == (4, 6, 3)
