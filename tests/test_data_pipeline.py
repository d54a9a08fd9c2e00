"""Dataset preparation: advantages, pre-tokenised inputs, token caps, per-epoch shuffling."""

import json
from collections import Counter

import pytest
from datasets import Dataset

from bergson_b200.config import DataConfig, IndexConfig
from bergson_b200.magic.cli import shuffled_epochs
from bergson_b200.utils.worker_utils import estimate_advantage, filter_by_max_tokens, setup_data_pipeline

MODEL = "native:llama-tiny?vocab_size=64&max_position_embeddings=32"


def _pretok(tmp_path, columns, **cfg_kwargs):
    path = tmp_path / "pretok"
    Dataset.from_dict(columns).save_to_disk(str(path))
    data_kwargs = {k: cfg_kwargs.pop(k) for k in list(cfg_kwargs) if k in ("truncation", "reward_column", "prompt_column", "skip_nan_rewards")}
    cfg = IndexConfig(run_path=str(tmp_path / "run"), model=MODEL, token_batch_size=32,
                      data=DataConfig(dataset=str(path), **data_kwargs), **cfg_kwargs)
    return setup_data_pipeline(cfg)


def test_advantage_is_reward_minus_group_mean():
    ds = Dataset.from_dict({"prompt": ["a", "a", "a", "b", "b"], "reward": [1.0, 3.0, 5.0, 10.0, 20.0]})
    adv = estimate_advantage(ds, DataConfig(dataset="", prompt_column="prompt", reward_column="reward"))
    assert adv == pytest.approx([-2.0, 0.0, 2.0, -5.0, 5.0])
    assert abs(sum(adv[:3])) < 1e-9 and abs(sum(adv[3:])) < 1e-9


def test_advantage_column_survives_drop_columns(tmp_path):
    ds, n = _pretok(tmp_path, {"input_ids": [[1, 2], [3, 4], [5, 6], [7, 8]], "prompt": ["p", "p", "q", "q"],
                               "reward": [1.0, 3.0, 10.0, 20.0]}, reward_column="reward", prompt_column="prompt",
                    drop_columns=True)
    assert n == 4 and "reward" not in ds.column_names and "prompt" not in ds.column_names
    assert ds["advantage"] == pytest.approx([-1.0, 1.0, -5.0, 5.0])
    assert {"input_ids", "length"} <= set(ds.column_names)


def test_nan_rewards_raise_or_are_skipped(tmp_path):
    cols = {"input_ids": [[1, 2], [3, 4], [5, 6]], "prompt": ["p", "p", "p"], "reward": [1.0, float("nan"), 3.0]}
    with pytest.raises(ValueError, match="NaN"):
        _pretok(tmp_path, cols, reward_column="reward", prompt_column="prompt")
    ds, n = _pretok(tmp_path / "b", cols, reward_column="reward", prompt_column="prompt", skip_nan_rewards=True)
    assert n == 2 and ds["advantage"] == pytest.approx([-1.0, 1.0])


@pytest.mark.parametrize("truncation", [True, False])
def test_pretokenised_rows_get_a_length_column(tmp_path, truncation):
    ids = [[1, 2, 3], [4, 5], [6, 7, 8, 9]]
    ds, _ = _pretok(tmp_path, {"input_ids": ids}, truncation=truncation)
    assert ds["length"] == [3, 2, 4] and ds["input_ids"] == ids


def test_existing_length_and_labels_are_kept(tmp_path):
    labels = [[-100, 2, 3], [-100, 5]]
    ds, _ = _pretok(tmp_path, {"input_ids": [[1, 2, 3], [4, 5]], "labels": labels, "length": [3, 2]}, drop_columns=True)
    assert ds["labels"] == labels and ds["length"] == [3, 2]


def test_token_batch_larger_than_the_context_is_refused(tmp_path):
    path = tmp_path / "d"
    Dataset.from_dict({"input_ids": [[1, 2]]}).save_to_disk(str(path))
    cfg = IndexConfig(run_path=str(tmp_path / "run"), model=MODEL, token_batch_size=64, data=DataConfig(dataset=str(path)))
    with pytest.raises(ValueError, match="exceeds model max length"):
        setup_data_pipeline(cfg)


def test_max_tokens_takes_a_prefix_or_tiles(tmp_path):
    ds = Dataset.from_dict({"input_ids": [[0] * n for n in (5, 7, 4, 6)], "length": [5, 7, 4, 6]})
    cfg = IndexConfig(run_path=str(tmp_path), model=MODEL, max_tokens=13)
    assert filter_by_max_tokens(ds, cfg)["length"] == [5, 7]  # the next row would pass the cap
    cfg.max_tokens = 50  # 22 tokens per pass: two whole passes and a prefix of the third
    out = filter_by_max_tokens(ds, cfg)["length"]
    assert out == [5, 7, 4, 6] * 2 + [5] and sum(out) <= 50
    cfg.max_tokens = None
    assert filter_by_max_tokens(ds, cfg) is ds


def test_json_lines_dataset_with_rewards(tmp_path):
    path = tmp_path / "rows.jsonl"
    rows = [{"input_ids": [1, 2, 3], "prompt": "x", "reward": 2.0}, {"input_ids": [4, 5], "prompt": "x", "reward": 4.0}]
    path.write_text("\n".join(json.dumps(r) for r in rows))
    cfg = IndexConfig(run_path=str(tmp_path / "run"), model=MODEL, token_batch_size=32,
                      data=DataConfig(dataset=str(path), reward_column="reward", prompt_column="prompt"))
    ds, n = setup_data_pipeline(cfg)
    assert n == 2 and ds["advantage"] == pytest.approx([-1.0, 1.0]) and ds["length"] == [3, 2]


N = 12


def _order(ds):
    return list(ds["doc_ids"])


def test_epochs_are_shuffled_independently_and_reproducibly():
    base = Dataset.from_dict({"doc_ids": list(range(N))})
    out = _order(shuffled_epochs(base, seed=0, num_epochs=3))
    epochs = [out[i * N:(i + 1) * N] for i in range(3)]
    assert all(sorted(e) == list(range(N)) for e in epochs)
    assert epochs[0] != epochs[1] and epochs[1] != epochs[2]
    assert out == _order(shuffled_epochs(base, seed=0, num_epochs=3))
    assert out != _order(shuffled_epochs(base, seed=1, num_epochs=3))
    assert Counter(_order(shuffled_epochs(base, seed=1, num_epochs=4))) == Counter({i: 4 for i in range(N)})
    single = _order(shuffled_epochs(base, seed=3, num_epochs=1))
    assert sorted(single) == list(range(N)) and single != list(range(N))
    with pytest.raises(AssertionError):
        shuffled_epochs(base, seed=0, num_epochs=0)


def test_over_long_documents_warn_and_then_fail_to_pack(tmp_path):
    import warnings

    from bergson_b200.data import allocate_batches

    with pytest.warns(UserWarning, match="longer than (the model can handle|token_batch_size)"):
        ds, _ = _pretok(tmp_path, {"input_ids": [[1] * 40, [2] * 5]}, truncation=False)
    with pytest.raises(RuntimeError, match="too long"):
        allocate_batches(ds["length"], 32)
    with warnings.catch_warnings():
        warnings.simplefilter("error")  # documents that fit do not warn
        _pretok(tmp_path / "ok", {"input_ids": [[1] * 30, [2] * 5]}, truncation=False)
