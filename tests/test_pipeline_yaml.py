"""Pipelines described as a YAML ``steps:`` list: hydration in order, defaults, error messages,
the replayable manifest, sub-config lookup and an end-to-end two-step run with a matrix."""

import textwrap

import numpy as np
import pytest
import yaml

from bergson_b200.__main__ import main
from bergson_b200.cli.commands import COMMANDS
from bergson_b200.config import IndexConfig, PreprocessConfig, ScoreConfig
from bergson_b200.config.config_io import load_subconfig, parse_steps, read_config, save_pipeline_config
from bergson_b200.data import load_gradients, load_scores

MODEL = "native:llama-tiny?vocab_size=256"
TRAIN = "synthetic:zipf?n=10&len=14&vocab=256&seed=0&min_len=6"
QUERY = "synthetic:zipf?n=3&len=14&vocab=256&seed=1&min_len=8"


def _write(tmp_path, text):
    p = tmp_path / "pipeline.yaml"
    p.write_text(textwrap.dedent(text))
    return p


def test_steps_are_hydrated_in_order_with_defaults(tmp_path):
    p = _write(tmp_path, f"""\
        run_path: {tmp_path}/pipe
        steps:
          - Build:
              index_cfg: {{run_path: {tmp_path}/q, model: "{MODEL}", projection_dim: 4}}
          - score:
              index_cfg: {{run_path: {tmp_path}/s, model: "{MODEL}", projection_dim: 4}}
              score_cfg: {{query_path: {tmp_path}/q}}
        """)
    doc = read_config(p)
    assert doc["run_path"] == f"{tmp_path}/pipe"
    steps = parse_steps(doc["steps"], COMMANDS)
    assert [n.lower() for n, _ in steps] == ["build", "score"]  # command names are case-insensitive
    build, score = steps[0][1], steps[1][1]
    assert build.index_cfg.projection_dim == 4 and build.index_cfg.token_batch_size == IndexConfig(run_path="x").token_batch_size
    assert build.preprocess_cfg == PreprocessConfig()  # an omitted sub-tree is the dataclass default
    assert score.score_cfg.query_path == f"{tmp_path}/q" and not hasattr(build, "score_cfg")


@pytest.mark.parametrize("text,match", [
    ("run_path: x\n", "steps"),
    ("- build: {}\n", "steps"),
    ("steps:\n  - {build: {}, score: {}}\n", "single command-key"),
    ("steps:\n  - just_a_string\n", "single command-key"),
    ("steps:\n  - frobnicate: {}\n", "Unknown command"),
])
def test_malformed_documents_say_what_is_wrong(tmp_path, text, match):
    p = tmp_path / "bad.yaml"
    p.write_text(text)
    with pytest.raises(ValueError, match=match):
        parse_steps(read_config(p)["steps"], COMMANDS)


def test_manifest_is_replayable_and_named_when_no_run_path(tmp_path, monkeypatch):
    steps = parse_steps([{"build": {"index_cfg": {"run_path": "runs/a", "model": MODEL}}},
                         {"score": {"index_cfg": {"run_path": "runs/b", "model": MODEL}, "score_cfg": {"query_path": "runs/a"}}}],
                        COMMANDS)
    out = save_pipeline_config(steps, tmp_path / "pipe")
    doc = read_config(out)
    assert doc["run_path"] == str(tmp_path / "pipe") and "bergson_version" in doc["metadata"]
    again = parse_steps(doc["steps"], COMMANDS)
    assert [c.to_dict() for _, c in again] == [c.to_dict() for _, c in steps]
    monkeypatch.chdir(tmp_path)
    named = save_pipeline_config(steps, None)
    assert named.parent.name == "runs" and "_" in named.name and (named / "config.yaml").exists()
    # sub-configs are looked up in every step, the first match wins
    assert load_subconfig(out, "score_cfg", ScoreConfig).query_path == "runs/a"
    assert load_subconfig(out, "index_cfg", IndexConfig).run_path == "runs/a"
    assert load_subconfig(out, "no_such_cfg", ScoreConfig) is None
    assert load_subconfig(tmp_path / "nowhere", "score_cfg", ScoreConfig) is None


def test_two_step_pipeline_with_a_matrix_runs_end_to_end(tmp_path):
    p = _write(tmp_path, f"""\
        run_path: {tmp_path}/pipe
        steps:
          - build:
              index_cfg:
                run_path: {tmp_path}/q
                model: "{MODEL}"
                projection_dim: 4
                token_batch_size: 64
                data: {{dataset: "{QUERY}"}}
                distributed: {{nproc_per_node: 1}}
          - score:
              matrix: {{norm: [true, false]}}
              index_cfg:
                run_path: {tmp_path}/s_{{norm}}
                model: "{MODEL}"
                projection_dim: 4
                token_batch_size: 64
                data: {{dataset: "{TRAIN}"}}
                distributed: {{nproc_per_node: 1}}
              score_cfg: {{query_path: {tmp_path}/q}}
              preprocess_cfg: {{unit_normalize: "{{norm}}"}}
        """)
    main([str(p)])
    manifest = yaml.safe_load((tmp_path / "pipe" / "config.yaml").read_text())
    assert [list(s)[0] for s in manifest["steps"]] == ["build", "score", "score"]  # the matrix is written out resolved
    assert np.asarray(load_gradients(tmp_path / "q")).shape[0] == 3
    cos = np.asarray(load_scores(tmp_path / "s_True")[:], dtype=np.float64)
    raw = np.asarray(load_scores(tmp_path / "s_False")[:], dtype=np.float64)
    assert cos.shape == raw.shape == (10, 3) and np.abs(cos).max() <= 1.0 + 1e-3 and not np.allclose(cos, raw)
