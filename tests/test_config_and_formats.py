"""Config parsing, YAML round trips, store / score formats, batching, step state."""

import json

import numpy as np
import pytest
import torch

from bergson_b200.cli.commands import COMMANDS, Build, Trackstar
from bergson_b200.config import IndexConfig, LRScheduleConfig, PreprocessConfig
from bergson_b200.config.config_io import expand_matrix, load_subconfig, parse_steps, read_config, save_run_config
from bergson_b200.config.parsing import DataclassArgumentParser
from bergson_b200.data import (
    _allocate_batches_world,
    column_offsets,
    create_index,
    create_token_index,
    load_gradients,
    load_scores,
    pad_and_tensor,
    zipf_token_ids,
)
from bergson_b200.score.score_writer import (
    MemmapSequenceScoreWriter,
    _score_struct_dtype,
    save_sequence_scores,
    save_token_scores,
)
from bergson_b200.utils.step_state import partial_path, prepare_step, promote_step, step_state


def test_flat_and_dotted_flags():
    cmd = DataclassArgumentParser(Build).parse(
        ["runs/x", "--projection_dim", "16", "--data.dataset", "d", "--index_cfg.data.split", "train[:5]",
         "--unit_normalize", "--nproc_per_node", "2", "--filter_modules", "*.mlp.*", "--precision", "bf16"])
    assert cmd.index_cfg.run_path == "runs/x" and cmd.index_cfg.projection_dim == 16
    assert cmd.index_cfg.data.dataset == "d" and cmd.index_cfg.data.split == "train[:5]"
    assert cmd.preprocess_cfg.unit_normalize is True and cmd.index_cfg.distributed.nproc_per_node == 2
    assert cmd.index_cfg.precision == "bf16" and cmd.index_cfg.partial_run_path.name == "x.part"


def test_ambiguous_flag_needs_prefix_and_bad_choice_fails():
    p = DataclassArgumentParser(COMMANDS["ekfac"])
    with pytest.raises(SystemExit):
        p.parse(["r", "--ev_correction", "true"])
    cmd = p.parse(["r", "--hessian_cfg.ev_correction", "true", "--method", "shampoo"])
    assert cmd.hessian_cfg.ev_correction and cmd.hessian_cfg.method == "shampoo"
    with pytest.raises(SystemExit):
        p.parse(["r", "--method", "nope"])


def test_trackstar_default_projection_and_lists():
    cmd = DataclassArgumentParser(Trackstar).parse(["r", "--split_attention_modules", "a", "b", "--max_tokens", "none"])
    assert cmd.index_cfg.projection_dim == 16 and cmd.index_cfg.split_attention_modules == ["a", "b"]
    assert cmd.index_cfg.max_tokens is None


def test_config_yaml_round_trip_and_subconfig(tmp_path):
    cmd = Build(IndexConfig(run_path=str(tmp_path / "r"), projection_dim=8), PreprocessConfig(aggregation="mean"))
    save_run_config(cmd, tmp_path)
    doc = read_config(tmp_path)
    assert list(doc["steps"][0]) == ["build"] and "created" in doc["metadata"]
    sub = load_subconfig(tmp_path, "preprocess_cfg", PreprocessConfig)
    assert sub.aggregation == "mean"
    ((name, again),) = parse_steps(doc["steps"], COMMANDS)
    assert again.index_cfg.projection_dim == 8 and again.to_dict() == cmd.to_dict()
    with pytest.raises(ValueError):
        parse_steps([{"build": {"index_cfg": {"nonsense": 1}}}], COMMANDS)
    with pytest.raises(ValueError):
        parse_steps([{"nope": {}}], COMMANDS)


def test_matrix_expansion():
    cells = expand_matrix({"index_cfg": {"run_path": "runs/p{p}", "projection_dim": "{p}"}, "matrix": {"p": [4, 8]}})
    assert [c["index_cfg"]["run_path"] for c in cells] == ["runs/p4", "runs/p8"]
    assert [c["index_cfg"]["projection_dim"] for c in cells] == [4, 8]
    with pytest.raises(ValueError):
        expand_matrix({"index_cfg": {"run_path": "same"}, "matrix": {"p": [1, 2]}})


def test_lr_schedules():
    s = LRScheduleConfig(lr=1.0, lr_scheduler_type="linear", warmup_steps=2).get_schedule(10)
    assert s(0) == 0.0 and s(1) == 0.5 and s(2) == 1.0 and abs(s(6) - 0.5) < 1e-12
    c = LRScheduleConfig(lr=2.0, lr_scheduler_type="cosine").get_schedule(4)
    assert abs(c(0) - 2.0) < 1e-12 and abs(c(2) - 1.0) < 1e-12
    assert LRScheduleConfig(lr=3.0, lr_scheduler_type="constant").get_schedule(5)(4) == 3.0
    p = LRScheduleConfig(lr=1.0, lr_end=0.1, power=2.0, lr_scheduler_type="polynomial").get_schedule(10)
    assert abs(p(5) - (0.1 + 0.9 * 0.25)) < 1e-12


def test_gradient_store_layout(tmp_path):
    sizes = {"a": 3, "b": 2}
    mm = create_index(tmp_path / "s", 4, sizes, np.float16)
    mm[2] = np.arange(5, dtype=np.float16)
    mm.flush()
    info = json.load(open(tmp_path / "s" / "info.json"))
    assert info == {"attribute_tokens": False, "num_items": 4, "num_grads": 4, "grad_sizes": sizes, "base_dtype": "float16"}
    raw = np.fromfile(tmp_path / "s" / "gradients.bin", dtype=np.float16).reshape(4, 5)
    assert (raw[2] == np.arange(5)).all() and column_offsets(sizes) == {"a": (0, 3), "b": (3, 5)}
    tok, off = create_token_index(tmp_path / "t", np.array([2, 0, 3]), sizes, "bfloat16")
    assert tok.shape == (5, 5) and off.tolist() == [0, 2, 2, 5]
    assert load_gradients(tmp_path / "t").dtype == np.dtype("bfloat16")


def test_score_record_layout(tmp_path):
    spec, _ = _score_struct_dtype(3, np.dtype(np.float32))
    assert spec["offsets"] == [0, 4, 8, 12, 16, 20] and spec["itemsize"] == 24
    spec16, _ = _score_struct_dtype(3, np.dtype(np.float16))
    assert spec16["offsets"] == [0, 2, 4, 6, 8, 10] and spec16["itemsize"] == 16
    save_sequence_scores(tmp_path / "seq", np.arange(6, dtype=np.float32).reshape(3, 2))
    s = load_scores(tmp_path / "seq")
    assert s.is_written() and s[:].tolist() == [[0, 1], [2, 3], [4, 5]] and s.get(slice(None), 1).tolist() == [1, 3, 5]
    w = MemmapSequenceScoreWriter(tmp_path / "part", 4, 2, distributed=False)
    w([1, 3], torch.tensor([[1.0], [2.0]]), query_offset=1)
    w.flush()
    p = load_scores(tmp_path / "part")
    assert not p.is_written() and p.mmap["written_1"].tolist() == [False, True, False, True]
    save_token_scores(tmp_path / "tok", np.arange(5, dtype=np.float32), np.array([0, 2, 5]))
    t = load_scores(tmp_path / "tok")
    assert t.offsets.tolist() == [0, 2, 5] and t.to_grid().shape == (2, 4)


def test_batch_allocation_and_padding():
    lens = [9, 1, 4, 4, 7, 2, 3, 8, 5, 6]
    alloc = _allocate_batches_world(lens, 16, 2)
    seen = sorted(i for rank in alloc for b in rank for i in b)
    assert seen == [i for i, l in enumerate(lens) if l >= 2]
    assert len(alloc[0]) == len(alloc[1])
    for rank in alloc:
        for b in rank:
            assert max(lens[i] for i in b) * len(b) <= 16
    with pytest.raises(RuntimeError):
        _allocate_batches_world([40, 3], 16, 1)
    x, y, shift, collect = pad_and_tensor([[5, 6, 7], [8, 9]], labels=[[-100, 6, 7], [8, 9]], sync_max_len=False)
    assert x.tolist() == [[5, 6, 7], [8, 9, 0]] and y.tolist() == [[-100, 6, 7], [8, 9, -100]]
    assert shift.tolist() == [[True, True, False], [True, False, False]]
    assert collect.tolist() == [[True, True, False], [True, False, False]]


def test_zipf_data_is_seeded():
    a, b = zipf_token_ids(4, 16, 100, seed=3), zipf_token_ids(4, 16, 100, seed=3)
    assert a == b and a != zipf_token_ids(4, 16, 100, seed=4)
    flat = np.array(zipf_token_ids(200, 64, 1000, seed=0)).ravel()
    assert flat.min() >= 0 and flat.max() < 1000 and (flat == 0).mean() > (flat == 10).mean()


def test_step_state_protocol(tmp_path):
    out = tmp_path / "step"
    assert step_state(out) == "missing" and prepare_step(out, resume=True)
    partial_path(out).mkdir()
    (partial_path(out) / "f").write_text("1")
    assert step_state(out) == "partial"
    assert prepare_step(out, resume=True) and not partial_path(out).exists()  # interrupted output is cleared
    partial_path(out).mkdir()
    (partial_path(out) / "f").write_text("new")
    promote_step(out)
    assert step_state(out) == "complete" and not prepare_step(out, resume=True)
    assert prepare_step(out, resume=False) and out.exists()  # kept until the rerun is promoted
    partial_path(out).mkdir()
    (partial_path(out) / "f").write_text("newer")
    promote_step(out)
    assert (out / "f").read_text() == "newer" and not out.with_name("step.superseded").exists()
    with pytest.raises(FileNotFoundError):
        promote_step(out)


def test_interrupted_promotion_loses_nothing(tmp_path, monkeypatch):
    """A crash between parking the old output and renaming the new one into place leaves both
    on disk; the next run starts the step over from a clean slate."""
    import bergson_b200.utils.step_state as ss

    out = tmp_path / "step"
    partial_path(out).mkdir()
    (partial_path(out) / "old").write_text("1")
    promote_step(out)
    partial_path(out).mkdir()
    (partial_path(out) / "new").write_text("2")
    real = ss.Path.rename
    calls = {"n": 0}

    def crash_after_first(self, target):
        calls["n"] += 1
        result = real(self, target)
        if calls["n"] == 1:
            raise RuntimeError("crash in the middle of the swap")
        return result

    monkeypatch.setattr(ss.Path, "rename", crash_after_first)
    with pytest.raises(RuntimeError):
        promote_step(out)
    monkeypatch.setattr(ss.Path, "rename", real)
    assert (out.with_name("step.superseded") / "old").exists() and (partial_path(out) / "new").exists()
    assert step_state(out) == "partial"
    assert prepare_step(out, resume=True)
    assert not out.with_name("step.superseded").exists() and not partial_path(out).exists()
    # an unrelated neighbour's partial output is never touched
    other = partial_path(tmp_path / "other")
    other.mkdir()
    assert prepare_step(out, resume=False) and other.exists()
