"""Reductions of the weighted next-token loss, and the mixing coefficient of query and index
curvature."""

import pytest
import torch
import torch.nn.functional as F

from bergson_b200.utils.math import compute_lambda, weighted_causal_lm_ce

IGNORE = -100


def _batch(B, T=8, V=50, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(B, T, V, generator=g), torch.randint(0, V, (B, T), generator=g)


def _ce(logits, labels, reduction):
    return F.cross_entropy(logits[:, :-1].float().reshape(-1, logits.shape[-1]), labels[:, 1:].reshape(-1),
                           ignore_index=IGNORE, reduction=reduction)


@pytest.mark.parametrize("B", [1, 2, 4, 8])
def test_unit_weights_change_nothing_and_mean_is_the_token_mean(B):
    logits, labels = _batch(B, seed=B)
    plain = weighted_causal_lm_ce(logits, labels)
    torch.testing.assert_close(weighted_causal_lm_ce(logits, labels, example_weight=torch.ones(B)), plain)
    torch.testing.assert_close(plain, _ce(logits, labels, "mean"))


def test_ignored_tokens_are_not_in_the_denominator():
    logits, labels = _batch(4, seed=2)
    labels[1, 3:] = IGNORE
    labels[2, :] = IGNORE  # a row without any supervised token
    want = _ce(logits, labels, "mean")
    torch.testing.assert_close(weighted_causal_lm_ce(logits, labels), want)
    torch.testing.assert_close(weighted_causal_lm_ce(logits, labels, example_weight=torch.ones(4)), want)
    labels[:] = IGNORE
    for red in ("mean", "sum", "sum_of_means"):
        loss = weighted_causal_lm_ce(logits, labels, example_weight=torch.ones(4), reduction=red)
        assert torch.isfinite(loss) and float(loss) == 0.0


def test_weights_scale_their_own_rows_only():
    logits, labels = _batch(2, seed=4)
    base = weighted_causal_lm_ce(logits, labels, example_weight=torch.ones(2))
    bumped = weighted_causal_lm_ce(logits, labels, example_weight=torch.tensor([2.0, 1.0]))
    row0 = weighted_causal_lm_ce(logits, labels, example_weight=torch.tensor([1.0, 0.0]))
    torch.testing.assert_close(bumped - base, row0)  # the denominator counts tokens, not weight mass
    per_token = torch.zeros(2, 8)
    per_token[0, 2] = 1.0  # weight of position t applies to the loss of predicting token t + 1
    one = weighted_causal_lm_ce(logits, labels, example_weight=per_token, reduction="sum")
    torch.testing.assert_close(one, F.cross_entropy(logits[0, 2:3].float(), labels[0, 3:4]))


@pytest.mark.parametrize("weighted", [False, True])
def test_sum_is_a_sum_and_unknown_reductions_fail(weighted):
    logits, labels = _batch(3, seed=6)
    labels[2, 4:] = IGNORE
    kw = {"example_weight": torch.ones(3)} if weighted else {}
    got = weighted_causal_lm_ce(logits, labels, reduction="sum", **kw)
    torch.testing.assert_close(got, _ce(logits, labels, "sum"))
    n_valid = int((labels[:, 1:] != IGNORE).sum())
    torch.testing.assert_close(got, weighted_causal_lm_ce(logits, labels, reduction="mean", **kw) * n_valid)
    per_row = _ce(logits, labels, "none").view(3, -1).sum(1) / (labels[:, 1:] != IGNORE).sum(1)
    torch.testing.assert_close(weighted_causal_lm_ce(logits, labels, reduction="sum_of_means", **kw), per_row.sum())
    with pytest.raises((ValueError, AssertionError), match="Unknown reduction"):
        weighted_causal_lm_ce(logits, labels, reduction="garbage", **kw)


def test_double_precision_logits_stay_double():
    logits, labels = _batch(2, seed=8)
    loss = weighted_causal_lm_ce(logits.double().requires_grad_(True), labels, example_weight=torch.ones(2, dtype=torch.float64))
    assert loss.dtype == torch.float64
    assert weighted_causal_lm_ce(logits.to(torch.bfloat16), labels).dtype == torch.float32
    with pytest.raises(AssertionError, match="vocab size"):
        weighted_causal_lm_ce(logits, labels, vocab_size=49)


def _eig(vals):
    v = torch.tensor(vals, dtype=torch.float32)
    return v, torch.eye(len(vals))


def test_lambda_balances_the_kth_pooled_eigenvalues():
    q = {"a": _eig([4.0, 2.0, 1.0])}
    assert compute_lambda(q, q, target_components=2) == pytest.approx(0.5)  # identical spectra
    assert compute_lambda(q, q, target_components=0) == 1.0
    i = {"a": _eig([8.0, 6.0, 3.0])}
    # k = 2 -> s_q = 2, s_i = 6; lam s_q = (1 - lam) s_i
    lam = compute_lambda(q, i, target_components=2)
    assert lam == pytest.approx(6.0 / 8.0) and lam * 2.0 == pytest.approx((1 - lam) * 6.0)
    assert compute_lambda(q, i, target_components=99) == pytest.approx(3.0 / 4.0)  # clamps to the smallest
    big_index = {"a": _eig([1e6, 1e5, 1e4])}
    assert compute_lambda(q, big_index, target_components=1) > 0.99
    assert compute_lambda(q, {"b": _eig([1.0])}) == 0.99  # nothing in common: the default
    assert compute_lambda({"a": _eig([0.0])}, {"a": _eig([0.0])}, target_components=1) == 0.99


def test_lambda_pools_modules_and_ignores_eigenvectors():
    q = {"a": _eig([5.0, 1.0]), "b": _eig([3.0, 2.0])}
    i = {"a": _eig([10.0, 1.0]), "b": _eig([4.0, 0.5])}
    # pooled and sorted: q = [5, 3, 2, 1], i = [10, 4, 1, 0.5]; k = 3 -> 2 and 1
    assert compute_lambda(q, i, target_components=3) == pytest.approx(1.0 / 3.0)
    rotated = {n: (v, torch.randn_like(e)) for n, (v, e) in q.items()}
    assert compute_lambda(rotated, i, target_components=3) == pytest.approx(1.0 / 3.0)
    for k in range(1, 6):
        assert 0.0 <= compute_lambda(q, i, target_components=k) <= 1.0
    assert compute_lambda({"a": _eig([-1.0, -2.0])}, {"a": _eig([3.0, 1.0])}, target_components=1) == 1.0  # negatives count as 0
