"""Loss logging that cannot break a run, and ``matrix:`` expansion of pipeline steps."""

from unittest.mock import MagicMock, patch

import pytest

from bergson_b200.config.config_io import expand_matrix
from bergson_b200.utils.logging import wandb_log_fn


def test_log_fn_starts_a_run_and_logs(monkeypatch):
    monkeypatch.delenv("WANDB_MODE", raising=False)
    fake = MagicMock()
    fake.run = None
    with patch.dict("sys.modules", {"wandb": fake}):
        log = wandb_log_fn("proj", config={"lr": 1e-4})
        fake.init.assert_called_once_with(project="proj", config={"lr": 1e-4})
        log(5, 0.25)
        fake.log.assert_called_once_with({"train/loss": 0.25}, step=5)


def test_log_fn_reuses_a_running_run(monkeypatch):
    monkeypatch.delenv("WANDB_MODE", raising=False)
    fake = MagicMock()
    fake.run = MagicMock()
    with patch.dict("sys.modules", {"wandb": fake}):
        log = wandb_log_fn("proj")
        fake.init.assert_not_called()
        log(0, 1.5)
        fake.log.assert_called_once_with({"train/loss": 1.5}, step=0)


def test_disabled_mode_never_imports_wandb(monkeypatch):
    monkeypatch.setenv("WANDB_MODE", "disabled")
    with patch.dict("sys.modules", {"wandb": None}):  # an import attempt would raise
        log = wandb_log_fn("proj", config={"a": 1})
        assert log(0, 1.0) is None and log(9, 0.1) is None


def test_missing_package_warns_and_does_nothing(monkeypatch):
    monkeypatch.delenv("WANDB_MODE", raising=False)
    with patch.dict("sys.modules", {"wandb": None}):
        with pytest.warns(UserWarning, match="wandb is not installed"):
            log = wandb_log_fn("proj")
        assert log(0, 1.0) is None


def test_failing_init_warns_and_does_nothing(monkeypatch):
    monkeypatch.delenv("WANDB_MODE", raising=False)
    fake = MagicMock()
    fake.run = None
    fake.init.side_effect = TimeoutError("service did not answer")
    with patch.dict("sys.modules", {"wandb": fake}):
        with pytest.warns(UserWarning, match="wandb.init failed"):
            log = wandb_log_fn("proj")
        log(0, 1.0)
        fake.log.assert_not_called()


def test_trainer_calls_log_fn_once_per_step():
    import torch

    from bergson_b200.magic.data_stream import DataStream
    from bergson_b200.magic.optim import adamw
    from bergson_b200.magic.trainer import Trainer
    from bergson_b200.models import build_model
    from bergson_b200.models.registry import parse_native_spec
    from datasets import Dataset

    args = parse_native_spec("native:llama-tiny?vocab_size=64&hidden_size=32&intermediate_size=64&num_hidden_layers=1")[0]
    model = build_model(args, dtype=torch.float32, device="cpu", seed=0)
    g = torch.Generator().manual_seed(0)
    rows = [torch.randint(0, 64, (12,), generator=g).tolist() for _ in range(6)]
    ds = Dataset.from_dict({"input_ids": rows, "labels": rows, "length": [12] * 6})
    trainer, state = Trainer.initialize(model, adamw(1e-3))
    stream = DataStream(ds, batch_size=2, device="cpu")
    calls = []
    trainer.train(state, stream, inplace=True, log_fn=lambda step, loss: calls.append((step, loss)))
    assert [c[0] for c in calls] == list(range(len(stream))) and all(isinstance(c[1], float) for c in calls)


def test_matrix_passthrough_and_typed_substitution():
    cfg = {"run_path": "runs/x", "seed": 1}
    assert expand_matrix(dict(cfg)) == [cfg]
    out = expand_matrix({"matrix": {"seed": [1, 2], "lr": [0.1]}, "run_path": "runs/s{seed}_lr{lr}", "seed": "{seed}",
                         "lr_schedule": {"lr": "{lr}"}})
    assert out[0] == {"run_path": "runs/s1_lr0.1", "seed": 1, "lr_schedule": {"lr": 0.1}}
    assert len(out) == 2 and out[1]["seed"] == 2 and out[1]["run_path"] == "runs/s2_lr0.1"


def test_matrix_cells_must_not_share_a_run_path():
    with pytest.raises(ValueError, match="both write"):
        expand_matrix({"matrix": {"seed": [1, 2]}, "run_path": "runs/same", "seed": "{seed}"})
    with pytest.raises(ValueError, match="both write"):
        expand_matrix({"matrix": {"d": [0.1, 0.2]}, "index_cfg": {"run_path": "runs/fixed"}, "damping": "{d}"})
    with pytest.raises(ValueError, match="no run_path"):
        expand_matrix({"matrix": {"seed": [1, 2]}, "seed": "{seed}"})
    with pytest.raises(ValueError, match="non-empty lists"):
        expand_matrix({"matrix": {"seed": 5}})
