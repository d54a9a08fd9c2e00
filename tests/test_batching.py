"""Token-budget packing across ranks, padding, and invariance of the stored rows to how the
documents were batched."""

import json

import numpy as np
import pytest
import torch

from bergson_b200.__main__ import main
from bergson_b200.data import _allocate_batches_world, load_gradients, pad_and_tensor

SHORT, LONG, N_SHORT, BUDGET = 25, 1000, 80, 2048


def _lengths():
    return [SHORT] * N_SHORT + [LONG]


@pytest.mark.parametrize("world", [1, 2, 3])
def test_packing_covers_every_document_once_within_the_budget(world):
    lengths = _lengths()
    per_rank = _allocate_batches_world(lengths, BUDGET, world, seed=42)
    assert len(per_rank) == world and len({len(b) for b in per_rank}) == 1  # same number of steps everywhere
    seen = sorted(i for batches in per_rank for b in batches for i in b)
    assert seen == list(range(len(lengths)))
    for batches in per_rank:
        for b in batches:
            assert max(lengths[i] for i in b) * len(b) <= BUDGET


def test_documents_too_short_or_too_long():
    per_rank = _allocate_batches_world([1, 0, 5, 6], 16, 1)
    assert sorted(i for b in per_rank[0] for i in b) == [2, 3]  # fewer than two tokens: no next-token label
    with pytest.raises(RuntimeError, match="too long"):
        _allocate_batches_world([40, 5], 16, 1)
    with pytest.raises(RuntimeError, match="Not enough documents"):
        _allocate_batches_world([5], 16, 2)


def test_max_batch_size_caps_documents_per_batch():
    per_rank = _allocate_batches_world([4] * 20, 1024, 1, max_batch_size=3)
    assert max(len(b) for b in per_rank[0]) <= 3 and sum(len(b) for b in per_rank[0]) == 20


def _pad_worker(rank, local_rank, world, out_dir):
    from bergson_b200.data import allocate_batches
    from bergson_b200.distributed import init_dist

    init_dist(rank, local_rank, world)
    lengths = _lengths()
    worst_local = worst_synced = 0
    for batch in allocate_batches(lengths, BUDGET, seed=42):
        ids = [[1] * lengths[i] for i in batch]
        local = pad_and_tensor(ids, sync_max_len=False)[0]
        synced = pad_and_tensor(ids, sync_max_len=True)[0]
        worst_local = max(worst_local, local.numel())
        worst_synced = max(worst_synced, synced.numel())
        assert synced.shape[1] >= local.shape[1]
    with open(f"{out_dir}/rank{rank}.json", "w") as f:
        json.dump({"local": worst_local, "synced": worst_synced}, f)


def test_local_padding_keeps_the_per_rank_budget_two_ranks(tmp_path):
    """One long document on one rank must not make the other rank pad eighty short ones to
    its length: the build pads per rank; only paths that need equal shapes sync the length."""
    from bergson_b200.config import DistributedConfig
    from bergson_b200.distributed import launch_distributed_run

    launch_distributed_run("pad", _pad_worker, [str(tmp_path)], DistributedConfig(nproc_per_node=2))
    got = [json.load(open(tmp_path / f"rank{r}.json")) for r in range(2)]
    assert all(g["local"] <= BUDGET for g in got), got
    assert max(g["synced"] for g in got) > 4 * BUDGET, got  # what the synchronised length would have cost


def test_pad_and_tensor_masks():
    ids = [[5, 6, 7, 8], [9, 10]]
    labels = [[-100, 6, 7, 8], [9, 10]]
    x, y, loss_mask, coll_mask = pad_and_tensor(ids, labels, padding_value=0)
    assert x.tolist() == [[5, 6, 7, 8], [9, 10, 0, 0]] and y.tolist() == [[-100, 6, 7, 8], [9, 10, -100, -100]]
    assert coll_mask.tolist() == [[True, True, True, False], [True, False, False, False]]  # every real position but the last
    assert loss_mask.tolist() == [[True, True, True, False], [True, False, False, False]]  # position t predicts a supervised token
    x2, _, lm2, _ = pad_and_tensor([[1, 2, 3]], [[-100, -100, 3]])
    assert lm2.tolist() == [[False, True, False]]


MODEL = "native:llama-tiny?vocab_size=256"


@pytest.mark.parametrize("sizes", [(6, 6), (4, 10)])
def test_rows_do_not_depend_on_what_else_is_in_the_store(tmp_path, sizes):
    """Rows of documents built alone equal their rows when built together with others (the
    loss is summed, not averaged, over the batch): same scale and same direction."""
    from datasets import Dataset

    from bergson_b200.data import zipf_token_ids

    na, nb = sizes
    a = zipf_token_ids(na, 14, 256, seed=3, min_length=6)
    b = zipf_token_ids(nb, 20, 256, seed=4, min_length=9)
    for name, rows in (("a", a), ("b", b), ("ab", a + b)):
        Dataset.from_dict({"input_ids": rows}).save_to_disk(str(tmp_path / f"data_{name}"))
        main(["build", str(tmp_path / name), "--model", MODEL, "--data.dataset", str(tmp_path / f"data_{name}"),
              "--projection_dim", "4", "--token_batch_size", "64", "--nproc_per_node", "1"])
    ga, gb, gab = (torch.from_numpy(np.asarray(load_gradients(tmp_path / n)).astype(np.float32)) for n in ("a", "b", "ab"))
    for alone, together in ((ga, gab[:na]), (gb, gab[na:])):
        torch.testing.assert_close(alone.std(), together.std(), rtol=2e-3, atol=0.0)
        cos = torch.nn.functional.cosine_similarity(alone, together, dim=1)
        assert float(cos.min()) > 0.999
