"""Per-token stores: row counts, ragged index layout (empty documents included), the builder's
out-of-order writes, the token score writer, and an end-to-end token build whose rows sum to
the per-document rows."""

import json

import numpy as np
import pytest
import torch
from datasets import Dataset

from bergson_b200.__main__ import main
from bergson_b200.builder import Builder
from bergson_b200.config import PreprocessConfig
from bergson_b200.data import (
    TokenGradients, compute_num_token_grads, create_token_index, load_gradients, load_scores, load_token_gradients)
from bergson_b200.score.score_writer import MemmapTokenScoreWriter


def test_rows_per_document_depend_on_length_only():
    ds = Dataset.from_dict({"input_ids": [[1, 2, 3], [4, 5, 6, 7]], "length": [3, 4]})
    np.testing.assert_array_equal(compute_num_token_grads(ds), [2, 3])
    # prompt positions carry gradient too (the completion's loss reaches them through attention):
    # the label mask does not change the row count
    masked = Dataset.from_dict({"input_ids": [[1, 2, 3, 4, 5]] * 2, "labels": [[-100, -100, 3, 4, 5], [-100] * 5], "length": [5, 5]})
    np.testing.assert_array_equal(compute_num_token_grads(masked), [4, 4])
    short = Dataset.from_dict({"input_ids": [[1] * 6, [], [1], [1] * 4], "length": [6, 0, 1, 4]})
    np.testing.assert_array_equal(compute_num_token_grads(short), [5, 0, 0, 3])
    no_len = Dataset.from_dict({"input_ids": [[1, 2, 3], [4, 5]]})
    np.testing.assert_array_equal(compute_num_token_grads(no_len), [2, 1])


def test_index_layout_with_an_empty_document(tmp_path):
    ds = Dataset.from_dict({"input_ids": [[1] * 6, [], [1] * 5, [1] * 4], "length": [6, 0, 5, 4]})
    mm, offsets = create_token_index(tmp_path, compute_num_token_grads(ds), {"m": 2}, np.float32)
    np.testing.assert_array_equal(offsets, [0, 5, 5, 9, 12])
    assert mm.shape == (12, 2) and json.load(open(tmp_path / "info.json"))["num_grads"] == 12
    for i in range(4):
        mm[offsets[i]:offsets[i + 1]] = i + 1
    mm.flush()
    tg = TokenGradients(tmp_path)
    np.testing.assert_array_equal(tg.num_token_grads, [5, 0, 4, 3])
    assert len(tg) == 4 and tg[1].shape == (0, 2)
    assert all((tg[i] == i + 1).all() for i in range(4))


def test_create_and_reload(tmp_path):
    counts = np.array([3, 5, 2], dtype=np.int64)
    mm, offsets = create_token_index(tmp_path, counts, {"mod_a": 4, "mod_b": 6}, np.float32)
    assert mm.shape == (10, 10)
    info = json.load(open(tmp_path / "info.json"))
    assert info["attribute_tokens"] is True and sum(info["grad_sizes"].values()) == 10
    mm[:] = np.arange(100, dtype=np.float32).reshape(10, 10)
    mm.flush()
    back, n, off = load_token_gradients(tmp_path)
    np.testing.assert_array_equal(n, counts)
    np.testing.assert_array_equal(off, [0, 3, 8, 10])
    np.testing.assert_array_equal(back[off[1]:off[2]], np.arange(30, 80, dtype=np.float32).reshape(5, 10))


def test_builder_writes_documents_out_of_order(tmp_path):
    ds = Dataset.from_dict({"input_ids": [[1, 2, 3], [4, 5, 6, 7], [8, 9]], "length": [3, 4, 2]})
    b = Builder(ds, {"m": 2}, torch.float32, PreprocessConfig(aggregation="none"), attribute_tokens=True, path=tmp_path)
    b([0, 2], {"m": torch.tensor([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]])})  # 2 rows of document 0, 1 row of document 2
    b([1], {"m": torch.tensor([[7.0, 8.0], [9.0, 10.0], [11.0, 12.0]])})
    b.flush()
    tg = TokenGradients(tmp_path)
    np.testing.assert_array_equal(tg[0], [[1.0, 2.0], [3.0, 4.0]])
    np.testing.assert_array_equal(tg[1], [[7.0, 8.0], [9.0, 10.0], [11.0, 12.0]])
    np.testing.assert_array_equal(tg[2], [[5.0, 6.0]])


def test_token_score_writer(tmp_path):
    ds = Dataset.from_dict({"input_ids": [[1, 2, 3, 4], [5, 6, 7]], "length": [4, 3]})
    w = MemmapTokenScoreWriter.from_dataset(tmp_path, ds, num_scores=2, dtype=torch.float32, distributed=False)
    w([1], torch.tensor([[10.0, 20.0], [30.0, 40.0]]))
    w.flush()
    assert not load_scores(tmp_path).is_written()  # document 0 is still missing
    w([0], torch.tensor([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]]))
    w.flush()
    info = json.load(open(tmp_path / "info.json"))
    assert info["attribute_tokens"] is True and info["num_rows"] == 5 and info["num_scores"] == 2
    s = load_scores(tmp_path)
    assert s.is_written()
    np.testing.assert_array_equal(s[s.offsets[0]:s.offsets[1]], [[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]])
    np.testing.assert_array_equal(s[s.offsets[1]:s.offsets[2]], [[10.0, 20.0], [30.0, 40.0]])
    grid = s.to_grid()
    assert grid.shape == (2, 4, 2) and grid[1, 2:].abs().sum() == 0


MODEL = "native:llama-tiny?vocab_size=256"


@pytest.mark.parametrize("labels", [False, True])
def test_token_build_rows_sum_to_document_rows(tmp_path, labels):
    """The per-document gradient is the sum of its positions' gradients -- also when a label
    mask confines the loss to a completion (prompt positions still get rows)."""
    from bergson_b200.data import zipf_token_ids

    ids = zipf_token_ids(6, 12, 256, seed=5, min_length=5) + [[7]]  # the last document is too short to have a label
    cols = {"input_ids": ids}
    if labels:
        cols["labels"] = [[-100] * (len(r) // 2) + r[len(r) // 2:] for r in ids]
    Dataset.from_dict(cols).save_to_disk(str(tmp_path / "data"))
    common = ["--model", MODEL, "--data.dataset", str(tmp_path / "data"), "--projection_dim", "4", "--token_batch_size", "64",
              "--nproc_per_node", "1"]
    main(["build", str(tmp_path / "doc"), *common])
    main(["build", str(tmp_path / "tok"), *common, "--attribute_tokens", "true"])
    doc = np.asarray(load_gradients(tmp_path / "doc")).astype(np.float64)
    tg = TokenGradients(tmp_path / "tok")
    np.testing.assert_array_equal(tg.num_token_grads, [max(len(r) - 1, 0) for r in ids])
    for i in range(len(ids)):
        np.testing.assert_allclose(tg[i].astype(np.float64).sum(0), doc[i], rtol=5e-3, atol=5e-4 * np.abs(doc).max())
    assert np.abs(doc[-1]).sum() == 0 and tg[len(ids) - 1].shape[0] == 0
    if labels:
        first = tg[0].astype(np.float64)
        assert np.abs(first[: len(ids[0]) // 2 - 1]).sum() > 0  # prompt positions are not empty rows
