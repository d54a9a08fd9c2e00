"""Builder: every combination of in-memory / on-disk, per-document / per-token, aggregated or
not, and what teardown does under a (mocked) process group."""

from unittest.mock import MagicMock, patch

import numpy as np
import pytest
import torch
from datasets import Dataset

from bergson_b200 import builder as builder_mod
from bergson_b200.builder import Builder
from bergson_b200.config import PreprocessConfig
from bergson_b200.data import load_gradients

SIZES = {"a": 4, "b": 4}


@pytest.fixture
def ds():
    return Dataset.from_dict({"input_ids": [[1, 2, 3, 4, 5]] * 4, "length": [5] * 4})


def _grads(n, seed=0):
    g = torch.Generator().manual_seed(seed)
    return {m: torch.randn(n, d, generator=g) for m, d in SIZES.items()}


def _fake_dist(rank):
    mock = MagicMock()
    mock.is_initialized.return_value = True
    mock.get_rank.return_value = rank
    return patch.object(builder_mod, "dist", mock)


def test_construction(ds, tmp_path):
    b = Builder(ds, SIZES, torch.float32, PreprocessConfig(aggregation="none"))
    assert b.grad_buffer.shape == (4, 8) and b.in_memory_grad_buffer is None
    agg = Builder(ds, SIZES, torch.float32, PreprocessConfig(aggregation="mean"))
    assert agg.grad_buffer.shape == (1, 8) and agg.in_memory_grad_buffer.shape == (1, 8)
    tok = Builder(ds, SIZES, torch.float32, PreprocessConfig(aggregation="none"), attribute_tokens=True)
    assert tok.grad_buffer.shape == (16, 8) and tok.offsets.tolist() == [0, 4, 8, 12, 16]
    disk = Builder(ds, SIZES, torch.bfloat16, PreprocessConfig(aggregation="none"), path=tmp_path)
    assert isinstance(disk.grad_buffer, np.memmap) and load_gradients(tmp_path).shape == (4, 8)


def test_rows_land_at_their_indices_in_memory_and_on_disk(ds, tmp_path):
    g = _grads(2)
    want = torch.cat([g["a"], g["b"]], 1).numpy()
    for path in (None, tmp_path):
        b = Builder(ds, SIZES, torch.float32, PreprocessConfig(aggregation="none"), path=path)
        b([3, 1], g)
        b.teardown()
        np.testing.assert_allclose(np.asarray(b.grad_buffer)[[3, 1]], want, rtol=1e-6)
        assert np.abs(np.asarray(b.grad_buffer)[[0, 2]]).sum() == 0
    np.testing.assert_allclose(np.asarray(load_gradients(tmp_path))[[3, 1]], want, rtol=1e-6)


def test_unit_normalize_without_aggregation(ds):
    g = _grads(4)
    b = Builder(ds, SIZES, torch.float32, PreprocessConfig(aggregation="none", unit_normalize=True))
    b([0, 1, 2, 3], g)
    np.testing.assert_allclose(np.linalg.norm(b.grad_buffer, axis=1), 1.0, rtol=1e-5)


@pytest.mark.parametrize("aggregation", ["mean", "sum"])
def test_aggregated_store_is_the_mean_or_sum_of_all_rows(ds, tmp_path, aggregation):
    g1, g2 = _grads(2, 0), _grads(2, 1)
    b = Builder(ds, SIZES, torch.float32, PreprocessConfig(aggregation=aggregation), path=tmp_path)
    b([0, 1], g1)
    b([2, 3], g2)
    b.teardown()
    total = torch.cat([torch.cat([g["a"], g["b"]], 1) for g in (g1, g2)]).sum(0)
    want = total / 4 if aggregation == "mean" else total
    np.testing.assert_allclose(np.asarray(load_gradients(tmp_path))[0], want.numpy(), rtol=1e-5, atol=1e-6)


def test_only_rank_zero_writes_the_aggregate(ds, tmp_path):
    """The reduction delivers the sum to rank 0 only; other ranks must not write their partial one."""
    for path in (None, tmp_path):
        b = Builder(ds, SIZES, torch.float32, PreprocessConfig(aggregation="mean"), path=path)
        b.in_memory_grad_buffer = torch.ones(1, 8)
        with _fake_dist(rank=1) as d:
            b.teardown()
        d.reduce.assert_called_once()
        assert np.abs(np.asarray(b.grad_buffer, dtype=np.float32)).sum() == 0
    b0 = Builder(ds, SIZES, torch.float32, PreprocessConfig(aggregation="sum"))
    b0.in_memory_grad_buffer = torch.ones(1, 8)
    with _fake_dist(rank=0):
        b0.teardown()
    np.testing.assert_array_equal(b0.grad_buffer, np.ones((1, 8), np.float32))


def test_in_memory_rows_are_summed_over_ranks_but_shared_files_are_not(ds, tmp_path):
    mem = Builder(ds, SIZES, torch.float32, PreprocessConfig(aggregation="none"))
    mem([0, 1], _grads(2))
    with _fake_dist(rank=0) as d:
        mem.teardown()
    d.all_reduce.assert_called_once()  # ranks filled disjoint rows of private buffers
    disk = Builder(ds, SIZES, torch.float32, PreprocessConfig(aggregation="none"), path=tmp_path)
    with _fake_dist(rank=0) as d:
        disk.teardown()
    d.all_reduce.assert_not_called()  # every rank wrote into the same mapped file


def test_in_memory_token_rows_with_scattered_indices(ds):
    b = Builder(ds, SIZES, torch.float32, PreprocessConfig(aggregation="none"), attribute_tokens=True)
    g = _grads(8)  # 4 rows of document 2, then 4 rows of document 0
    b([2, 0], g)
    flat = torch.cat([g["a"], g["b"]], 1).numpy()
    np.testing.assert_allclose(b.grad_buffer[8:12], flat[:4], rtol=1e-6)
    np.testing.assert_allclose(b.grad_buffer[0:4], flat[4:], rtol=1e-6)
    assert np.abs(b.grad_buffer[4:8]).sum() == 0 and np.abs(b.grad_buffer[12:]).sum() == 0
