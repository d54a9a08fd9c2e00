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
