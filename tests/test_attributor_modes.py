"""Attributor: tracing a backward pass as the query, reverse search, curvature on one or both
sides, and approximate indices behind the same calls."""

import pytest
import torch

from bergson_b200 import Attributor, GradientProcessor, InMemoryCollector, collect_gradients
from bergson_b200.collector.collector import CollectorComputer
from bergson_b200.config import FaissConfig, IndexConfig
from bergson_b200.data import allocate_batches

from .helpers import tiny_dataset, tiny_model


@pytest.fixture(scope="module")
def store(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("attr")
    torch.manual_seed(0)
    model = tiny_model("gpt_neox")
    model.requires_grad_(False)
    model.get_input_embeddings().requires_grad_(True)
    ds = tiny_dataset(n=12, length=12)
    cfg = IndexConfig(run_path=str(tmp / "idx"), projection_dim=4, token_batch_size=48)
    cfg.partial_run_path.mkdir(parents=True)
    batches = allocate_batches(ds["length"], 48)
    # one pass that also accumulates the gradient autocorrelation (the dense curvature estimate) ...
    proc = GradientProcessor(projection_dim=4)
    coll = InMemoryCollector(model=model.base_model, data=ds, cfg=cfg, processor=proc, skip_hessians=False)
    CollectorComputer(model=model, data=ds, collector=coll, batches=batches, cfg=cfg).run_with_collector_hooks("mem")
    # ... and the store on disk, with that processor saved beside it
    collect_gradients(model, ds, proc, cfg, batches=batches)
    proc.save(cfg.partial_run_path)
    return model, ds, cfg.partial_run_path


def _trace(attr, model, ds, i, k, **kw):
    x = torch.tensor(ds[i]["input_ids"])[None]
    with attr.trace(model.base_model, k, **kw) as result:
        model(x, labels=x).loss.backward()
    model.zero_grad()
    return result


def test_a_document_finds_itself(store):
    model, ds, path = store
    attr = Attributor(path, device="cpu", unit_norm=True)
    for i in (0, 5):
        r = _trace(attr, model, ds, i, 5)
        assert r.indices.shape == (1, 5) and int(r.indices[0, 0]) == i and float(r.scores[0, 0]) > 0.99
        assert (r.scores[0, :-1] >= r.scores[0, 1:]).all()
    with pytest.raises(ValueError, match="backward"):
        with attr.trace(model.base_model, 3):
            pass
    fresh = attr.trace(model.base_model, 3)
    with fresh as result:
        with pytest.raises(ValueError, match="context"):
            result.scores
        x = torch.tensor(ds[0]["input_ids"])[None]
        model(x, labels=x).loss.backward()
    model.zero_grad()


def test_reverse_returns_the_least_similar(store):
    model, ds, path = store
    attr = Attributor(path, device="cpu", unit_norm=True)
    top = _trace(attr, model, ds, 0, 5)
    low = _trace(attr, model, ds, 0, 5, reverse=True)
    assert float(low.scores[0, 0]) < float(top.scores[0, 0])
    assert int(top.indices[0, 0]) == 0 and 0 not in low.indices[0].tolist()
    assert (low.scores[0, :-1] <= low.scores[0, 1:]).all()
    everything = _trace(attr, model, ds, 0, None)
    assert sorted(everything.indices[0].tolist()) == list(range(len(ds)))
    assert low.indices[0, 0] == everything.indices[0, -1]


@pytest.mark.parametrize("unit_norm", [True, False])
def test_curvature_on_both_sides_or_on_the_query_only(store, unit_norm):
    """unit_norm: H^-1/2 on queries and rows, then cosine; otherwise H^-1 on the query only."""
    model, ds, path = store
    attr = Attributor(path, device="cpu", unit_norm=unit_norm, hessian_path=path)
    assert attr.preconditioner is not None
    r = _trace(attr, model, ds, 0, 5)
    assert int(r.indices[0, 0]) == 0
    if unit_norm:
        assert float(r.scores[0, 0]) > 0.9
    plain = _trace(Attributor(path, device="cpu", unit_norm=unit_norm), model, ds, 0, 5)
    assert not torch.allclose(plain.scores, r.scores)


@pytest.mark.parametrize("factory", ["Flat", "IVF2,SQfp16"])
def test_approximate_indices_answer_the_same_calls(store, factory):
    model, ds, path = store
    exact = _trace(Attributor(path, device="cpu", unit_norm=True), model, ds, 3, 4)
    attr = Attributor(path, device="cpu", unit_norm=True, faiss_cfg=FaissConfig(index_factory=factory, nprobe=2))
    r = _trace(attr, model, ds, 3, 4)
    assert r.indices[0].tolist() == exact.indices[0].tolist()
    torch.testing.assert_close(r.scores.float(), exact.scores.float(), atol=2e-3, rtol=0)
    low = _trace(attr, model, ds, 3, 4, reverse=True)
    assert float(low.scores[0, 0]) < float(r.scores[0, 0]) and 3 not in low.indices[0].tolist()
    # the index was written beside the store and is reused by the next Attributor
    again = Attributor(path, device="cpu", unit_norm=True, faiss_cfg=FaissConfig(index_factory=factory, nprobe=2))
    assert again.faiss_index.ntotal == len(ds)


def test_memory_mapped_index_gives_the_same_neighbours(store):
    """``mmap_index``: the shard's rows stay on disk and are read list by list."""
    import numpy as np

    model, ds, path = store
    cfg = dict(index_factory="IVF2,Flat", nprobe=2, num_shards=2)
    resident = Attributor(path, device="cpu", unit_norm=True, faiss_cfg=FaissConfig(**cfg))
    mapped = Attributor(path, device="cpu", unit_norm=True, faiss_cfg=FaissConfig(**cfg, mmap_index=True))
    assert isinstance(mapped.faiss_index.shards[0].vectors, np.memmap)
    a, b = _trace(resident, model, ds, 2, 5), _trace(mapped, model, ds, 2, 5)
    assert a.indices[0].tolist() == b.indices[0].tolist()
    torch.testing.assert_close(a.scores, b.scores, atol=1e-6, rtol=0)


def test_attributor_over_rows_in_memory_and_module_subsets():
    """``from_rows``: no store on disk; ``modules=`` restricts the inner product to some blocks."""
    g = torch.Generator().manual_seed(0)
    sizes = {"a": 6, "b": 4, "c": 5}
    rows = torch.randn(20, 15, generator=g)
    attr = Attributor.from_rows(rows, sizes, unit_norm=False)
    assert attr.N == 20 and attr.ordered_modules == ["a", "b", "c"] and attr.grads["b"].shape == (20, 4)
    q = {"a": rows[3:5, :6].clone(), "b": rows[3:5, 6:10].clone(), "c": rows[3:5, 10:].clone()}
    s, i = attr.search(q, k=3)
    want = rows @ rows[3:5].T
    assert i[:, 0].tolist() == [3, 4]
    torch.testing.assert_close(s[:, 0], want[[3, 4], [0, 1]], rtol=1e-5, atol=1e-5)
    s_ab, i_ab = attr.search(q, k=20, modules={"a", "b"})
    part = rows[:, :10] @ rows[3:5, :10].T  # only the columns of a and b take part
    order = part.T.argsort(dim=1, descending=True)
    assert i_ab.tolist() == order.tolist()
    torch.testing.assert_close(s_ab, part.T.gather(1, order), rtol=1e-5, atol=1e-5)
    cos = Attributor.from_rows(rows, sizes, unit_norm=True)
    s1, i1 = cos.search(q, k=1)
    assert i1[:, 0].tolist() == [3, 4] and torch.allclose(s1[:, 0], torch.ones(2), atol=1e-5)
    low, _ = cos.search(q, k=2, reverse=True)
    assert (low[:, 0] <= low[:, 1]).all() and (low < s1).all()
