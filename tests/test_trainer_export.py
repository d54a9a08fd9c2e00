"""Trainer checkpoints of a finished run are exported to ``checkpoint-<i>`` model directories
from the run's recorded config alone."""

import pytest
import torch

from bergson_b200.__main__ import main
from bergson_b200.models import load_model
from bergson_b200.utils.trainer_export import export_checkpoints, sorted_dcp_checkpoints

MODEL = "native:llama-tiny?vocab_size=256&num_hidden_layers=1"
TRAIN = "synthetic:zipf?n=12&len=12&vocab=256&seed=0&min_len=12"


def test_export_of_a_train_run(tmp_path):
    run = tmp_path / "run"
    main(["train", str(run), "--model", MODEL, "--data.dataset", TRAIN, "--batch_size", "4", "--lr", "1e-2",
          "--nproc_per_node", "1", "--save_mode", "all", "--save_optimizer_state", "all"])
    found = sorted_dcp_checkpoints(run / "checkpoints")
    assert [s for s, _ in found] == sorted(s for s, _ in found) and len(found) >= 3
    (run / "checkpoints" / "step_x.ckpt").mkdir()  # not a step number: ignored
    (run / "checkpoints" / "notes.txt").write_text("")
    assert sorted_dcp_checkpoints(run / "checkpoints") == found
    with pytest.raises(NotADirectoryError):
        sorted_dcp_checkpoints(run / "nowhere")

    steps = [s for s, _ in found]
    out = export_checkpoints(run, tmp_path / "exported", steps=[steps[-1], steps[0]])
    assert [p.name for p in out] == [f"checkpoint-{steps[0]}", f"checkpoint-{steps[-1]}"]  # in step order
    first, last = (load_model(str(p)) for p in out)
    assert any(not torch.equal(a, b) for a, b in zip(first.parameters(), last.parameters()))  # training moved the weights
    assert (out[-1] / "optimizer.pt").exists()
    with pytest.raises(FileExistsError):
        export_checkpoints(run, tmp_path / "exported", steps=[steps[0]])
    again = export_checkpoints(run, tmp_path / "exported", steps=[steps[0]], overwrite=True)
    for a, b in zip(load_model(str(again[0])).parameters(), first.parameters()):
        assert torch.equal(a, b)
    with pytest.raises(FileNotFoundError, match="not saved"):
        export_checkpoints(run, tmp_path / "exported", steps=[10**6])
    empty = tmp_path / "empty"
    (empty / "checkpoints").mkdir(parents=True)
    (empty / "config.yaml").write_text((run / "config.yaml").read_text())
    with pytest.raises(FileNotFoundError, match="save_mode"):
        export_checkpoints(empty)


def test_raw_checkpoints_are_exported_on_demand_for_source(tmp_path):
    from bergson_b200.data import load_scores
    from bergson_b200.utils.trainer_export import ensure_exported

    run = tmp_path / "run"
    main(["train", str(run), "--model", MODEL, "--data.dataset", "synthetic:zipf?n=16&len=12&vocab=256&seed=0&min_len=12",
          "--batch_size", "4", "--lr", "1e-2", "--optimizer", "sgd", "--nproc_per_node", "1", "--save_mode", "all"])
    found = sorted_dcp_checkpoints(run / "checkpoints")
    raw = [str(p) for _, p in found[-4:]]
    other = str(tmp_path / "some" / "checkpoint-7")
    resolved = ensure_exported(raw[:2] + [other])
    assert resolved[2] == other  # not a trainer checkpoint: passed through
    assert all((run / "exported" / f"checkpoint-{s}" / "model.safetensors").exists() for s, _ in found[-4:-2])
    stamp = (run / "exported" / f"checkpoint-{found[-4][0]}" / "model.safetensors").stat().st_mtime_ns
    assert ensure_exported(raw[:2]) == resolved[:2]  # reused, not exported again
    assert (run / "exported" / f"checkpoint-{found[-4][0]}" / "model.safetensors").stat().st_mtime_ns == stamp

    out = tmp_path / "source"
    main(["approxunrolling", str(out), "--model", MODEL, "--index_cfg.data.dataset", TRAIN,
          "--approx_unrolling_cfg.query.dataset", "synthetic:zipf?n=3&len=12&vocab=256&seed=1&min_len=12",
          "--checkpoints", *raw, "--segments", "2", "--nproc_per_node", "1", "--token_batch_size", "64",
          "--ev_correction", "True", "--use_dataset_labels"])
    assert all((run / "exported" / f"checkpoint-{s}").is_dir() for s, _ in found[-4:])
    scores = load_scores(out / "scores") if (out / "scores").exists() else load_scores(out)
    import numpy as np

    s = np.asarray(scores[:], dtype=np.float64)
    assert s.shape[0] == 12 and np.isfinite(s).all() and np.abs(s).sum() > 0
