"""Concatenated-row scoring must agree with per-module scoring for any module subset and order."""

import pytest
import torch

from bergson_b200.score.scorer import Scorer


class _Sink:
    def __call__(self, indices, scores, query_offset=0):
        self.last = scores


def _setup(score_modules, unit_normalize=False):
    torch.manual_seed(0)
    sizes = {"a": 6, "b": 4, "c": 6}
    grads = {m: torch.randn(5, d) for m, d in sizes.items()}
    queries = {m: torch.randn(3, d) for m, d in sizes.items()}
    spans, off = {}, 0
    for m, d in sizes.items():
        spans[m] = (off, off + d)
        off += d
    rows = torch.cat([grads[m] for m in sizes], dim=1)
    scorer = Scorer(queries, score_modules, _Sink(), torch.device("cpu"), torch.float32,
                    unit_normalize=unit_normalize)
    return scorer, grads, rows, spans, off


@pytest.mark.parametrize("mods", [["a", "b", "c"], ["c", "a"], ["b"], ["c", "b", "a"]])
def test_row_layout_matches_per_module_scores(mods):
    scorer, grads, rows, spans, total = _setup(mods)
    assert scorer.set_row_layout(spans, total)
    torch.testing.assert_close(scorer.score_rows(rows), scorer.score(grads))


def test_row_layout_declines_when_it_would_be_wrong():
    scorer, _, _, spans, total = _setup(["a", "b"], unit_normalize=True)
    assert not scorer.set_row_layout(spans, total)  # norms would include module c
    scorer, _, _, spans, total = _setup(["a", "b", "c"], unit_normalize=True)
    assert scorer.set_row_layout(spans, total)
    scorer, _, _, spans, total = _setup(["a"])
    assert not scorer.set_row_layout({"b": spans["b"]}, total)  # scored module absent from the rows
    assert not scorer.set_row_layout({"a": (0, 5)}, total)  # width mismatch
