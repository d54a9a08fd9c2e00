"""Units of the SOURCE (approximate unrolling) pipeline: segment step sizes under momentum,
the eigenvalue functions, per-document normalisation of segment eigenvalues, checkpoint step
parsing and the overwrite / resume polarity of the pipeline's steps."""

import json
from unittest.mock import patch

import pytest
import torch
from safetensors.torch import load_file, save_file

from bergson_b200.approx_unrolling import pipeline as pl
from bergson_b200.approx_unrolling.approx_unrolling_math import (
    _checkpoint_step, compute_lr_times_steps_per_segment, f_backward, f_one_minus_exp, f_segment)
from bergson_b200.approx_unrolling.segment_aggregation import (
    DOCUMENTS_PROCESSED_FILENAME, _sum_my_shard, lambda_denominator)
from bergson_b200.config import ApproxUnrollingConfig, HessianConfig, IndexConfig


def _cfg(**kw):
    base = dict(checkpoints=["a", "b"], segments=2, lr_list=[1e-3, 2e-3], step_size_list=[10, 20])
    base.update(kw)
    return ApproxUnrollingConfig(**base)


def test_momentum_scales_the_segment_step_sizes():
    base = compute_lr_times_steps_per_segment(_cfg())
    assert base == pytest.approx([1e-2, 4e-2])
    assert compute_lr_times_steps_per_segment(_cfg(momentum=0.9)) == pytest.approx([10 * b for b in base])
    for bad in (1.0, -0.1):
        with pytest.raises(ValueError, match="momentum"):
            compute_lr_times_steps_per_segment(_cfg(momentum=bad))


def test_step_sizes_from_the_logged_learning_rates(tmp_path):
    ckpts = [str(tmp_path / f"checkpoint-{s}") for s in (2, 4, 6, 8)]
    history = [{"step": s, "learning_rate": 0.1 * s} for s in range(1, 9)] + [{"step": 8, "eval_loss": 1.0}]
    (tmp_path / "log_history.json").write_text(json.dumps(history))
    got = compute_lr_times_steps_per_segment(ApproxUnrollingConfig(checkpoints=ckpts, segments=2))
    assert got == pytest.approx([0.1 * (1 + 2 + 3 + 4), 0.1 * (5 + 6 + 7 + 8)])  # boundaries at the segments' last checkpoints


def test_checkpoint_step_parsing():
    assert _checkpoint_step("runs/x/checkpoint-120") == 120
    assert _checkpoint_step("runs/x/step_7.ckpt") == 7 and _checkpoint_step("runs/x/step_7") == 7
    assert _checkpoint_step("runs/x/300") == 300
    with pytest.raises(ValueError, match="lr_list"):
        _checkpoint_step("runs/x/final")


def test_eigenvalue_functions():
    s = torch.tensor([0.0, 1e-12, 0.5, 3.0, 50.0], dtype=torch.float64)
    c = 0.7
    torch.testing.assert_close(f_backward(c)(s), torch.exp(-c * s))
    seg = f_segment(c)(s)
    assert float(seg[0]) == pytest.approx(c)  # the limit (1 - exp(-c s)) / s -> c as s -> 0
    assert float(seg[1]) == pytest.approx(c, rel=1e-9)
    torch.testing.assert_close(seg[2:], (1 - torch.exp(-c * s[2:])) / s[2:])
    torch.testing.assert_close(f_one_minus_exp(c)(s)[2:], seg[2:] * s[2:])
    # one segment followed by the next: exp(-c1 s) exp(-c2 s) = exp(-(c1 + c2) s)
    torch.testing.assert_close(f_backward(0.2)(s) * f_backward(0.5)(s), f_backward(0.7)(s))
    assert torch.isfinite(seg).all() and (seg > 0).all()


def test_segment_eigenvalues_are_divided_by_the_pooled_document_count(tmp_path):
    dirs = []
    for i in range(2):
        d = tmp_path / f"ckpt_{i}"
        d.mkdir()
        torch.save(torch.tensor(4599), d / DOCUMENTS_PROCESSED_FILENAME)
        dirs.append(d)
    assert lambda_denominator(dirs) == 2 * 4599
    (tmp_path / "ckpt_2").mkdir()
    with pytest.raises(FileNotFoundError, match="lambda step"):
        lambda_denominator(dirs + [tmp_path / "ckpt_2"])
    ins = []
    for i in range(2):
        p = tmp_path / f"in_{i}.safetensors"
        save_file({"w": torch.full((2, 3), float(i + 1)), "v": torch.arange(3.0) * (i + 1)}, str(p))
        ins.append(p)
    _sum_my_shard(ins, tmp_path / "out" / "shard_0.safetensors", device="cpu", divisor=6.0)
    got = load_file(str(tmp_path / "out" / "shard_0.safetensors"))
    torch.testing.assert_close(got["w"], torch.full((2, 3), 0.5))
    torch.testing.assert_close(got["v"], torch.arange(3.0) * 0.5)


class _Stop(Exception):
    pass


@pytest.mark.parametrize("overwrite", [True, False])
def test_overwrite_recomputes_every_step(overwrite, tmp_path):
    """``resume`` means "keep what is already there": every step must get the negation of
    ``overwrite``, whichever of the two flags it takes."""
    seen = {}

    def record(step, last=False):
        def stub(*args, **kwargs):
            if "resume" in kwargs:
                seen[step] = kwargs["resume"]
            elif "overwrite" in kwargs:
                seen[step] = not kwargs["overwrite"]
            if last:
                raise _Stop()
        return stub

    index_cfg = IndexConfig(run_path=str(tmp_path / "run"), model="native:llama-tiny", overwrite=overwrite)
    au = ApproxUnrollingConfig(checkpoints=[f"checkpoint-{i}" for i in (10, 20, 30, 40)], segments=2, lr_list=[1e-4, 1e-4],
                               step_size_list=[10, 10])
    with (patch.object(pl, "precompute_checkpoint_hessians", record("cov")),
          patch.object(pl, "aggregate_segment_covariances", record("cov_sum")),
          patch.object(pl, "precompute_checkpoint_averaged_lambdas", record("lambda")),
          patch.object(pl, "aggregate_segment_lambdas", record("lambda_sum", last=True))):
        with pytest.raises(_Stop):
            pl.approx_unrolling_pipeline(index_cfg, HessianConfig(method="ekfac", ev_correction=True), au)
    assert seen == {k: (not overwrite) for k in ("cov", "cov_sum", "lambda", "lambda_sum")}


def _trainer_run(tmp_path, **training):
    """A run directory as the trainer leaves it: config.yaml with one ``train`` step."""
    import yaml

    run = tmp_path / "trainer_run"
    run.mkdir(parents=True, exist_ok=True)
    body = dict(run_path=str(run), model=training.pop("model", "native:llama-tiny"), **training)
    (run / "config.yaml").write_text(yaml.safe_dump({"steps": [{"train": body}]}))
    return run


def test_momentum_is_derived_from_the_trainer_that_made_the_checkpoints(tmp_path):
    from bergson_b200.approx_unrolling.train_cfg_io import derive_momentum, resolve
    from bergson_b200.config import TrainingConfig

    # the trainer's SGD takes adam_beta1 as its heavy-ball momentum (0.95 unless set): 1 / (1 - 0.95) = 20 x lr * steps
    assert derive_momentum(TrainingConfig(run_path="x", optimizer="sgd", adam_beta1=0.9)) == 0.9
    assert 1.0 / (1.0 - derive_momentum(TrainingConfig(run_path="x", optimizer="sgd"))) == pytest.approx(20.0)
    assert derive_momentum(TrainingConfig(run_path="x", optimizer="adamw", adam_beta1=0.95)) == 0.0  # its own preconditioner covers it
    assert derive_momentum(TrainingConfig(run_path="x", optimizer="muon")) == 0.0

    # checkpoints that belong to no trainer run: nothing derived, the unset momentum becomes 0
    plain = resolve(ApproxUnrollingConfig(checkpoints=["a", "b"], model_path="gpt2"))
    assert plain.checkpoints == ["a", "b"] and plain.model_path == "gpt2" and plain.momentum == 0.0

    run = _trainer_run(tmp_path, optimizer="sgd", adam_beta1=0.9, model="native:llama-tiny?vocab_size=256")
    for sub in ("exported/checkpoint-0", "checkpoint-5"):
        (run / sub).mkdir(parents=True)
        got = resolve(ApproxUnrollingConfig(checkpoints=[str(run / sub)]))
        assert got.momentum == 0.9 and got.model_path == "native:llama-tiny?vocab_size=256"
    # what the user sets wins, zero included
    ck = str(run / "checkpoint-5")
    assert resolve(ApproxUnrollingConfig(checkpoints=[ck], momentum=0.5)).momentum == 0.5
    assert resolve(ApproxUnrollingConfig(checkpoints=[ck], momentum=0.0)).momentum == 0.0
    assert resolve(ApproxUnrollingConfig(checkpoints=[ck], model_path="mine")).model_path == "mine"
