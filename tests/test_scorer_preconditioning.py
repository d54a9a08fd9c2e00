"""Scorer with curvature: one-sided (queries carry H^-1) and split (H^-1/2 on both sides, then
unit norm) preconditioning, score modes, query offsets and the in-memory writer."""

import numpy as np
import torch

from bergson_b200.gradients import GradientProcessor
from bergson_b200.hessians.preconditioner import load_preconditioner
from bergson_b200.score.score import _make_split_hessian
from bergson_b200.score.score_writer import InMemorySequenceScoreWriter, MemmapSequenceScoreWriter
from bergson_b200.score.scorer import Scorer

CPU = torch.device("cpu")


def _h(tmp_path, power, h=None):
    GradientProcessor(hessians={"m": torch.eye(4) * 2.0 if h is None else h}).save(tmp_path / "hessian")
    from bergson_b200.config import InversionConfig

    return load_preconditioner(tmp_path / "hessian", power=power, inversion_cfg=InversionConfig(damping_factor=0.0)).h_inv


def test_no_path_means_no_preconditioner():
    assert load_preconditioner(None, power=-1, device=CPU) is None


def test_one_sided_preconditioning_changes_the_scores_as_h_inverse(tmp_path):
    torch.manual_seed(0)
    q, g = {"m": torch.randn(1, 4)}, {"m": torch.randn(2, 4)}
    h_inv = _h(tmp_path, -1.0)
    torch.testing.assert_close(h_inv["m"], torch.eye(4) / 2, atol=1e-5, rtol=1e-5)
    pre = {"m": q["m"] @ h_inv["m"]}
    w = MemmapSequenceScoreWriter(tmp_path / "with", 2, 1, dtype=torch.float32, distributed=False)
    with_h = Scorer(pre, ["m"], w, CPU, torch.float32).score(g)
    plain = Scorer(q, ["m"], InMemorySequenceScoreWriter(2, 1, dtype=torch.float32), CPU, torch.float32).score(g)
    torch.testing.assert_close(with_h, plain / 2, atol=1e-6, rtol=1e-5)


def test_split_preconditioning_is_h_inv_sqrt_on_both_sides_then_unit_norm(tmp_path):
    torch.manual_seed(0)
    a = torch.randn(4, 4)
    H = a @ a.T + torch.eye(4)
    q, g = {"m": torch.randn(1, 4)}, {"m": torch.randn(2, 4)}
    half = _h(tmp_path, -0.5, H)
    torch.testing.assert_close(half["m"] @ half["m"] @ H, torch.eye(4), atol=1e-4, rtol=1e-4)
    mk = lambda: InMemorySequenceScoreWriter(2, 1, dtype=torch.float32)  # noqa: E731
    split = Scorer({"m": q["m"] @ half["m"]}, ["m"], mk(), CPU, torch.float32, unit_normalize=True,
                   index_transform=_make_split_hessian(half, ["m"], CPU, torch.float32))
    assert not split.supports_rows  # a per-module transform rules out concatenated-row scoring
    got = split.score(g)
    gi = g["m"] @ half["m"]
    want = (gi / gi.norm(dim=1, keepdim=True)) @ (q["m"] @ half["m"]).T
    torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-5)
    unit_only = Scorer(q, ["m"], mk(), CPU, torch.float32, unit_normalize=True).score(g)
    one_sided = Scorer({"m": q["m"] @ (half["m"] @ half["m"])}, ["m"], mk(), CPU, torch.float32).score(g)
    assert not torch.allclose(got, unit_only) and not torch.allclose(got, one_sided)


def test_scores_sum_over_modules_and_land_in_the_offset_columns(tmp_path):
    torch.manual_seed(1)
    sizes = {"a": 3, "b": 5}
    q = {m: torch.randn(2, d) for m, d in sizes.items()}
    g = {m: torch.randn(4, d) for m, d in sizes.items()}
    w = InMemorySequenceScoreWriter(4, 5, dtype=torch.float32)
    s = Scorer(q, ["a", "b"], w, CPU, torch.float32, query_offset=3)
    want = g["a"] @ q["a"].T + g["b"] @ q["b"].T
    torch.testing.assert_close(s.score(g), want, atol=1e-5, rtol=1e-5)
    s([2, 0], {m: v[[2, 0]] for m, v in g.items()})
    out = w.scores.numpy()
    np.testing.assert_allclose(out[[2, 0], 3:], want[[2, 0]].numpy(), rtol=1e-5, atol=1e-5)
    assert np.abs(out[[1, 3]]).sum() == 0 and np.abs(out[:, :3]).sum() == 0


import pytest  # noqa: E402


@pytest.mark.parametrize("unit_normalize", [False, True])
@pytest.mark.parametrize("slices", [[(0, 2), (2, 5)], [(0, 1), (1, 3), (3, 5)]])
def test_scoring_the_queries_in_slices_equals_one_pass(slices, unit_normalize):
    """Slicing the query set bounds memory; it must not change a single score, and unit
    normalisation of the index rows must not be computed per slice."""
    g = torch.Generator().manual_seed(0)
    sizes = {"a": 6, "b": 4}
    queries = {m: torch.randn(5, d, generator=g) for m, d in sizes.items()}
    rows = {m: torch.randn(7, d, generator=g) for m, d in sizes.items()}

    def run(parts):
        w = InMemorySequenceScoreWriter(7, 5, dtype=torch.float32)
        for lo, hi in parts:
            s = Scorer({m: q[lo:hi] for m, q in queries.items()}, list(sizes), w, CPU, torch.float32,
                       unit_normalize=unit_normalize, query_offset=lo)
            s(list(range(7)), rows)
        return w.scores

    whole, sliced = run([(0, 5)]), run(slices)
    torch.testing.assert_close(sliced, whole, rtol=0, atol=1e-6)
    if unit_normalize:
        flat = torch.cat([rows[m] for m in sizes], 1)
        want = (flat / flat.norm(dim=1, keepdim=True)) @ torch.cat([queries[m] for m in sizes], 1).T
        torch.testing.assert_close(whole, want, rtol=1e-5, atol=1e-6)
