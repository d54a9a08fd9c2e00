"""End-to-end CLI pipelines on CPU with tiny random-init models and synthetic data."""

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from bergson_b200.__main__ import main
from bergson_b200.data import load_gradients, load_scores

MODEL = "native:llama-tiny?vocab_size=256"
TRAIN = "synthetic:zipf?n=24&len=16&vocab=256&seed=0&min_len=6"
QUERY = "synthetic:zipf?n=5&len=16&vocab=256&seed=1&min_len=8"
COMMON = ["--model", MODEL, "--nproc_per_node", "1", "--token_batch_size", "64"]


def run(*args):
    main([str(a) for a in args])


def test_build_then_score_matches_direct_inner_products(tmp_path):
    run("build", tmp_path / "index", "--data.dataset", TRAIN, "--projection_dim", "4", *COMMON)
    run("build", tmp_path / "query", "--data.dataset", QUERY, "--projection_dim", "4", *COMMON)
    run("score", tmp_path / "scores", "--data.dataset", TRAIN, "--projection_dim", "4", "--query_path",
        tmp_path / "query", *COMMON)
    g = np.asarray(load_gradients(tmp_path / "index"), dtype=np.float64)
    q = np.asarray(load_gradients(tmp_path / "query"), dtype=np.float64)
    s = load_scores(tmp_path / "scores")
    assert s.is_written()
    np.testing.assert_allclose(s[:], g @ q.T, rtol=1e-4, atol=1e-5)
    info = json.load(open(tmp_path / "index" / "info.json"))
    assert info["num_grads"] == 24 and info["base_dtype"] == "float32"
    assert (tmp_path / "index" / "config.yaml").exists() and (tmp_path / "index" / "data.hf").exists()
    assert int(torch.load(tmp_path / "index" / "total_processed.pt")) > 0


def test_config_yaml_replays(tmp_path):
    run("build", tmp_path / "a", "--data.dataset", TRAIN, "--projection_dim", "4", *COMMON)
    cfg = (tmp_path / "a" / "config.yaml").read_text().replace(str(tmp_path / "a"), str(tmp_path / "b"))
    (tmp_path / "replay.yaml").write_text(cfg)
    run(tmp_path / "replay.yaml")
    np.testing.assert_array_equal(np.asarray(load_gradients(tmp_path / "a")), np.asarray(load_gradients(tmp_path / "b")))


def test_reduce_is_mean_of_rows(tmp_path):
    run("build", tmp_path / "index", "--data.dataset", TRAIN, "--projection_dim", "4", *COMMON)
    run("reduce", tmp_path / "mean", "--data.dataset", TRAIN, "--projection_dim", "4", "--aggregation", "mean", *COMMON)
    g = np.asarray(load_gradients(tmp_path / "index"), dtype=np.float64)
    m = np.asarray(load_gradients(tmp_path / "mean"), dtype=np.float64)
    assert m.shape[0] == 1
    np.testing.assert_allclose(m[0], g.mean(0), rtol=1e-4, atol=1e-6)


def test_unit_normalized_build_and_token_rows(tmp_path):
    run("build", tmp_path / "unit", "--data.dataset", TRAIN, "--projection_dim", "4", "--unit_normalize", *COMMON)
    g = np.asarray(load_gradients(tmp_path / "unit"), dtype=np.float64)
    np.testing.assert_allclose(np.linalg.norm(g, axis=1), 1.0, rtol=1e-4)
    run("build", tmp_path / "seq", "--data.dataset", TRAIN, "--projection_dim", "4", *COMMON)
    run("build", tmp_path / "tok", "--data.dataset", TRAIN, "--projection_dim", "4", "--attribute_tokens", *COMMON)
    from bergson_b200 import TokenGradients

    tok = TokenGradients(tmp_path / "tok")
    seq = np.asarray(load_gradients(tmp_path / "seq"))
    for i in (0, 7, 23):
        np.testing.assert_allclose(tok[i].sum(0), seq[i], rtol=1e-3, atol=1e-5)


def test_trackstar_pipeline(tmp_path):
    run("trackstar", tmp_path / "ts", "--index_cfg.data.dataset", TRAIN, "--trackstar_cfg.query.dataset", QUERY,
        "--projection_dim", "4", "--target_downweight_components", "10", "--unit_normalize", *COMMON)
    for d in ("value_hessian", "query_hessian", "mixed_hessian", "query", "scores"):
        assert (tmp_path / "ts" / d).exists(), d
    s = load_scores(tmp_path / "ts" / "scores")
    assert s[:].shape == (24, 5) and np.isfinite(s[:]).all() and np.abs(s[:]).max() <= 1.0 + 1e-4


@pytest.mark.parametrize("method", ["kfac", "shampoo", "tkfac"])
def test_ekfac_pipeline(tmp_path, method):
    run("ekfac", tmp_path / "ek", "--index_cfg.data.dataset", TRAIN, "--hessian_pipeline_cfg.query.dataset", QUERY,
        "--method", method, "--hessian_cfg.ev_correction", str(method == "kfac"), "--use_dataset_labels", *COMMON)
    root = tmp_path / "ek"
    for d in ("query", f"hessian/{method}/eigen_activation_sharded", f"hessian/{method}/eigenvalue_sharded",
              f"{method}_query", "scores"):
        assert (root / d).exists(), d
    if method == "kfac":
        assert (root / "hessian/kfac/eigenvalue_correction_sharded/shard_0.safetensors").exists()
    s = load_scores(root / "scores")
    assert s[:].shape == (24, 1) and np.isfinite(s[:]).all() and np.abs(s[:]).max() > 0


def test_query_noninteractive_finds_itself(tmp_path):
    run("build", tmp_path / "index", "--data.dataset", TRAIN, "--projection_dim", "8", *COMMON)
    res = None
    from bergson_b200.config import QueryConfig
    from bergson_b200.query.query_index import query

    from bergson_b200.data import load_data_string

    load_data_string(TRAIN).select(range(3)).save_to_disk(str(tmp_path / "q.hf"))
    res = query(QueryConfig(index=str(tmp_path / "index"), query_dataset=str(tmp_path / "q.hf"), top_k=3))
    assert [r["top_indices"][0] for r in res] == [0, 1, 2]
    assert all(r["top_scores"][0] > 0.99 for r in res)


def test_help_for_every_command():
    from bergson_b200.cli.commands import COMMANDS

    for name in COMMANDS:
        out = subprocess.run([sys.executable, "-m", "bergson_b200", name, "--help"], capture_output=True, text=True,
                             cwd=Path(__file__).resolve().parents[1])
        assert out.returncode == 0 and "usage" in out.stdout.lower(), (name, out.stderr[-500:])


def test_interrupted_build_is_refused_then_overwritten(tmp_path):
    """A run that died leaves `<run>.part` behind: the next build refuses to touch it unless
    asked to overwrite, and the overwritten run equals a fresh one."""
    run("build", tmp_path / "fresh", *COMMON, "--data.dataset", TRAIN, "--projection_dim", "4")
    part = tmp_path / "broken.part"
    part.mkdir()
    (part / "gradients.bin").write_bytes(b"\x00" * 100)  # truncated store of the dead run
    (part / "info.json").write_text("{")                 # and a half-written header
    with pytest.raises(FileExistsError, match="already exists"):
        run("build", tmp_path / "broken", *COMMON, "--data.dataset", TRAIN, "--projection_dim", "4")
    assert (part / "gradients.bin").stat().st_size == 100  # nothing was touched
    run("build", tmp_path / "broken", *COMMON, "--data.dataset", TRAIN, "--projection_dim", "4", "--overwrite", "true")
    assert not part.exists()
    a, b = np.asarray(load_gradients(tmp_path / "fresh")), np.asarray(load_gradients(tmp_path / "broken"))
    np.testing.assert_array_equal(a, b)
