"""MAGIC command modes on CPU with a tiny model: one backward per query, per-token data weights,
gradient accumulation and clipping invariances, and the math-SDP switch of the build."""

import numpy as np
import pytest
import torch

from bergson_b200.__main__ import main
from bergson_b200.data import load_gradients, load_scores

MODEL = "native:llama-tiny?vocab_size=256&num_hidden_layers=1"
TRAIN = "synthetic:zipf?n=8&len=12&vocab=256&seed=0&min_len=12"
QUERY = "synthetic:zipf?n=4&len=12&vocab=256&seed=1&min_len=12"
BASE = ["--model", MODEL, "--data.dataset", TRAIN, "--query.dataset", QUERY, "--batch_size", "4", "--lr", "1e-3",
        "--nproc_per_node", "1"]


def run(*args):
    main([str(a) for a in args])


def test_per_query_scores_average_to_the_mean_query_scores(tmp_path):
    """`query_method none` runs one backward replay per query; the mean query loss is linear in the
    per-query losses, so its scores are the average of the per-query ones."""
    run("magic", tmp_path / "mean", *BASE, "--query_method", "mean")
    run("magic", tmp_path / "each", *BASE, "--query_method", "none")
    mean = load_scores(tmp_path / "mean" / "scores")[:].astype(np.float64)
    each = load_scores(tmp_path / "each" / "scores")[:].astype(np.float64)
    assert each.shape == (8, 4) and mean.shape[0] == 8
    np.testing.assert_allclose(each.mean(1), mean.reshape(8), rtol=1e-3, atol=1e-6 * np.abs(mean).max())


def test_per_token_weights_sum_to_the_document_scores(tmp_path):
    """With per-token data weights the metagradient of a document's weight is the sum of the
    metagradients of its tokens' weights."""
    run("magic", tmp_path / "doc", *BASE, "--query_method", "mean")
    run("magic", tmp_path / "tok", *BASE, "--query_method", "mean", "--attribute_tokens", "true")
    doc = load_scores(tmp_path / "doc" / "scores")[:].astype(np.float64).reshape(8)
    from bergson_b200.magic.cli import scores_are_per_token

    assert scores_are_per_token(str(tmp_path / "tok" / "scores"))
    tok = load_scores(tmp_path / "tok" / "scores")
    per_doc = tok.to_grid().double().sum(1).numpy()  # [docs, seq] grid of token scores
    # Token rows follow the (shuffled) training order, document scores the document ids: the two
    # agree as sets of values.
    np.testing.assert_allclose(np.sort(per_doc), np.sort(doc), rtol=1e-3, atol=1e-6 * np.abs(doc).max())


def test_gradient_accumulation_and_micro_batched_backward_leave_scores_unchanged(tmp_path):
    run("magic", tmp_path / "plain", *BASE, "--query_method", "mean", "--max_grad_norm", "0.5")
    run("magic", tmp_path / "accum", *BASE, "--query_method", "mean", "--max_grad_norm", "0.5",
        "--grad_accum_steps", "2", "--double_backward_batch_size", "2")
    a = load_scores(tmp_path / "plain" / "scores")[:].astype(np.float64)
    b = load_scores(tmp_path / "accum" / "scores")[:].astype(np.float64)
    np.testing.assert_allclose(a, b, rtol=2e-3, atol=1e-6 * np.abs(a).max())


def test_force_math_sdp_build_matches_default(tmp_path):
    """The math-SDP switch only changes which attention kernel may run: the store must agree."""
    opt = ["--model", MODEL, "--data.dataset", TRAIN, "--projection_dim", "4", "--token_batch_size", "48",
           "--nproc_per_node", "1"]
    flash, mem = torch.backends.cuda.flash_sdp_enabled(), torch.backends.cuda.mem_efficient_sdp_enabled()
    try:
        run("build", tmp_path / "default", *opt)
        run("build", tmp_path / "math", *opt, "--force_math_sdp", "true")
    finally:
        torch.backends.cuda.enable_flash_sdp(flash)
        torch.backends.cuda.enable_mem_efficient_sdp(mem)
    a, b = np.asarray(load_gradients(tmp_path / "default")), np.asarray(load_gradients(tmp_path / "math"))
    np.testing.assert_allclose(a, b, rtol=1e-4, atol=1e-6)


def test_per_query_columns_are_saved_one_by_one_and_reused(tmp_path):
    """Each query's backward sweep is written as soon as it finishes; a later run over the same
    directory loads the finished columns instead of replaying them, and a padded query batch
    still yields one column per real query."""
    q3 = "synthetic:zipf?n=3&len=12&vocab=256&seed=1&min_len=12"  # 3 queries, batches of 4: one pad row
    base = ["--model", MODEL, "--data.dataset", TRAIN, "--query.dataset", q3, "--batch_size", "4", "--lr", "1e-3",
            "--nproc_per_node", "1", "--query_method", "none"]
    run("magic", tmp_path / "r", *base)
    files = sorted((tmp_path / "r" / "per_query").glob("q*.pt"))
    assert [f.name for f in files] == ["q0.pt", "q1.pt", "q2.pt"]
    first = load_scores(tmp_path / "r" / "scores")[:].astype(np.float64)
    assert first.shape == (8, 3) and not np.allclose(first[:, 0], first[:, 1])
    cols = [torch.load(f, weights_only=True) for f in files]
    np.testing.assert_allclose(first, torch.stack(cols, -1).numpy().astype(np.float64), rtol=1e-3, atol=1e-9)
    # mark a cached column: the second run must pick it up unchanged instead of recomputing it
    torch.save(cols[1] * 0 + 7.0, files[1])
    run("magic", tmp_path / "r", *base, "--resume", "true", "--overwrite", "true")
    again = load_scores(tmp_path / "r" / "scores")[:].astype(np.float64)
    assert np.allclose(again[:, 1], 7.0, rtol=1e-2)
    np.testing.assert_allclose(again[:, [0, 2]], first[:, [0, 2]], rtol=1e-3, atol=1e-9)
