"""In-tree nearest-neighbour indices: every factory against exact search on clustered data."""

import numpy as np
import pytest
import torch

from bergson_b200.query.native_ann import Factory, NativeIndex, parse_factory


def _clustered(n=3000, d=32, clusters=24, seed=0):
    g = np.random.default_rng(seed)
    centres = g.normal(size=(clusters, d)).astype(np.float32) * 4
    x = centres[g.integers(0, clusters, n)] + g.normal(size=(n, d)).astype(np.float32)
    x /= np.linalg.norm(x, axis=1, keepdims=True)
    q = x[g.choice(n, 40, replace=False)] + 0.05 * g.normal(size=(40, d)).astype(np.float32)
    return x, q.astype(np.float32)


def _exact(x, q, k):
    s = q @ x.T
    order = np.argsort(-s, axis=1)[:, :k]
    return np.take_along_axis(s, order, 1), order


def _recall(found, truth):
    return np.mean([len(set(f) & set(t)) / len(t) for f, t in zip(found, truth)])


def test_parse_factory():
    assert parse_factory("Flat") == Factory(0, "fp32")
    assert parse_factory("IVF1024,SQfp16") == Factory(1024, "fp16")
    assert parse_factory("IVF1,SQfp16") == Factory(1, "fp16")
    assert parse_factory("IVF64,PQ8") == Factory(64, "pq", 8)
    assert parse_factory("PQ4x8") == Factory(0, "pq", 4)
    with pytest.raises(ValueError, match="not implemented"):
        parse_factory("HNSW32")


@pytest.mark.parametrize("spec", ["Flat", "SQfp16", "IVF1,SQfp16"])
def test_exhaustive_factories_equal_exact_search(spec):
    x, q = _clustered()
    idx = NativeIndex(x.shape[1], parse_factory(spec))
    assert idx.is_trained
    idx.add(x)
    d, i = idx.search(q, 10)
    ed, ei = _exact(x, q, 10)
    tol = 1e-5 if spec == "Flat" else 2e-3
    np.testing.assert_allclose(d, ed, atol=tol)
    assert _recall(i, ei) > (0.999 if spec == "Flat" else 0.97)


def test_ivf_all_lists_probed_is_exact_and_few_probes_keep_recall(tmp_path):
    x, q = _clustered()
    idx = NativeIndex(x.shape[1], parse_factory("IVF16,Flat"))
    with pytest.raises(RuntimeError):
        idx.add(x)
    idx.train(x[:2000])
    idx.add(x)
    with pytest.raises(RuntimeError):
        idx.add(x)
    assert idx.offsets[-1] == len(x) and sorted(idx.ids.tolist()) == list(range(len(x)))
    ed, ei = _exact(x, q, 10)
    idx.nprobe = 16
    d, i = idx.search(q, 10)
    np.testing.assert_allclose(d, ed, atol=1e-5)
    assert _recall(i, ei) > 0.999
    idx.nprobe = 4
    d4, i4 = idx.search(q, 10)
    assert _recall(i4, ei) > 0.85
    assert (np.diff(d4, axis=1) <= 1e-7).all()  # descending
    # files: reloaded in memory and memory-mapped give the same answers
    idx.save(tmp_path / "0")
    for mmap in (False, True):
        back = NativeIndex.load(tmp_path / "0", mmap=mmap)
        back.nprobe = 4
        d5, i5 = back.search(q, 10)
        np.testing.assert_array_equal(i5, i4)
        np.testing.assert_allclose(d5, d4, atol=1e-6)


def test_fewer_candidates_than_k_are_padded():
    x, q = _clustered(n=200, clusters=8)
    idx = NativeIndex(x.shape[1], parse_factory("IVF32"))
    idx.train(x)
    idx.add(x)
    idx.nprobe = 1
    d, i = idx.search(q, 50)
    assert d.shape == (40, 50) and (i == -1).any()
    assert np.isneginf(d[i == -1]).all() and (i[np.isfinite(d)] >= 0).all()


@pytest.mark.parametrize("spec", ["PQ8", "IVF8,PQ8"])
def test_product_quantiser_ranks_the_true_neighbour_high(spec):
    x, q = _clustered()
    idx = NativeIndex(x.shape[1], parse_factory(spec))
    idx.train(x)
    idx.add(x)
    idx.nprobe = 8
    assert idx.vectors.dtype == torch.uint8 and idx.vectors.shape == (len(x), 8)
    d, i = idx.search(q, 10)
    _, ei = _exact(x, q, 100)
    inside = np.mean([len(set(f) & set(t)) / len(f) for f, t in zip(i, ei)])  # found top-10 within the true top-100
    assert inside > 0.9, inside
    ed = np.take_along_axis(q @ x.T, np.maximum(i, 0), 1)
    assert np.abs(d - ed).max() < 0.25  # scores are those of the decoded rows


def test_attributor_over_ivf_shards(tmp_path):
    import json

    from bergson_b200.config import FaissConfig
    from bergson_b200.query.faiss_index import HAVE_FAISS, FaissIndex

    if HAVE_FAISS:
        pytest.skip("the faiss package provides these factories")
    x, q = _clustered(n=1200)
    store = tmp_path / "store"
    store.mkdir()
    x.astype(np.float16).tofile(store / "gradients.bin")
    with open(store / "info.json", "w") as f:
        json.dump({"grad_sizes": {"w": x.shape[1]}, "num_grads": len(x), "base_dtype": "float16"}, f)
    cfg = FaissConfig(index_factory="IVF8,SQfp16", num_shards=3, nprobe=8)
    FaissIndex.create_index(store, tmp_path / "ann", cfg, "cpu", unit_norm=True, hessians={})
    idx = FaissIndex(tmp_path / "ann")
    assert idx.ntotal == len(x) and idx.backend == "native"
    d, i = idx.search(q, 5)
    ed, ei = _exact(x, q, 5)
    assert _recall(i, ei) > 0.95
    dr, ir = idx.search(q, 5, reverse=True)
    _, er = _exact(x, -q, 5)
    assert _recall(ir, er) > 0.95 and (dr[:, 0] <= d[:, 0]).all()


@pytest.mark.gpu
@pytest.mark.parametrize("spec", ["Flat", "IVF64,SQfp16", "IVF16,PQ32"])
def test_indices_on_the_gpu(spec, tmp_path):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    x, q = _clustered(n=20000, d=64, clusters=64, seed=2)
    idx = NativeIndex(x.shape[1], parse_factory(spec), device="cuda")
    if idx.factory.needs_training:
        idx.train(x)
    idx.add(x)
    idx.nprobe = 16
    assert idx.vectors.is_cuda
    d, i = idx.search(q, 10)
    _, truth = _exact(x, q, 100 if "PQ" in spec else 10)
    if "PQ" in spec:
        assert np.mean([len(set(f) & set(t)) / len(f) for f, t in zip(i, truth)]) > 0.8
    else:
        assert _recall(i, truth) > (0.999 if spec == "Flat" else 0.9)
    idx.save(tmp_path / "0")
    back = NativeIndex.load(tmp_path / "0", device="cuda")
    back.nprobe = 16
    d2, i2 = back.search(q, 10)
    np.testing.assert_array_equal(i2, i)


@pytest.mark.parametrize("spec", ["IVF16,Flat", "IVF16,SQfp16", "IVF8,PQ8"])
def test_masked_scan_and_per_list_loop_find_the_same_neighbours(spec):
    x, q = _clustered()
    idx = NativeIndex(x.shape[1], parse_factory(spec))
    idx.train(x)
    idx.add(x)
    idx.nprobe = 3
    idx.dense_scan = False
    d0, i0 = idx.search(q, 10)
    idx.dense_scan = True
    d1, i1 = idx.search(q, 10)
    np.testing.assert_allclose(d1, d0, atol=1e-5)
    assert np.mean(i0 == i1) > 0.99  # equal scores may swap places
    idx.nprobe, idx.dense_scan = 1, True
    d, i = idx.search(q[:3], 2000)  # more than one list holds: padded the same way
    assert (i == -1).any() and np.isneginf(d[i == -1]).all() and (i[np.isfinite(d)] >= 0).all()


def test_store_helpers_and_multi_part_stores(tmp_path):
    import json

    from bergson_b200.config import FaissConfig
    from bergson_b200.query.faiss_index import (
        HAVE_FAISS, FaissIndex, gradients_loader, index_to_device, normalize_grads, validate_ram)

    x, q = _clustered(n=900)
    unit = normalize_grads(np.vstack([3 * x[:5], np.zeros((1, x.shape[1]), np.float32)]), "cpu", batch_size=4)
    np.testing.assert_allclose(np.linalg.norm(unit[:5], axis=1), 1.0, rtol=1e-5)
    assert np.abs(unit[5]).sum() == 0  # a zero row stays zero instead of becoming NaN
    validate_ram(x[:8], 1000)
    with pytest.raises(AssertionError, match="Not enough RAM"):
        validate_ram(x[:8], 10**15)
    # a store written in three parts: the loader yields them in order and the index spans all of them
    root = tmp_path / "store"
    for i, rows in enumerate(np.array_split(x, 3)):
        d = root / f"shard_{i}"
        d.mkdir(parents=True)
        rows.astype(np.float16).tofile(d / "gradients.bin")
        (d / "info.json").write_text(json.dumps({"grad_sizes": {"w": x.shape[1]}, "num_grads": len(rows), "base_dtype": "float16"}))
    parts = list(gradients_loader(root))
    assert [m.shape[0] for m, _ in parts] == [300, 300, 300] and parts[0][1] == ["w"]
    if HAVE_FAISS:
        return
    FaissIndex.create_index(root, tmp_path / "ann", FaissConfig(index_factory="IVF4,SQfp16", num_shards=2, nprobe=4), "cpu",
                            unit_norm=False, hessians={})
    idx = FaissIndex(tmp_path / "ann")
    assert idx.ntotal == 900
    _, i = idx.search(q, 5)
    _, truth = _exact(x.astype(np.float16).astype(np.float32), q, 5)
    assert _recall(i, truth) > 0.95
    shard = index_to_device(idx.shards[0], "cpu")
    assert shard is idx.shards[0] and shard.device == torch.device("cpu")


def test_nprobe_can_be_changed_after_loading(tmp_path):
    import json

    from bergson_b200.config import FaissConfig
    from bergson_b200.query.faiss_index import HAVE_FAISS, FaissIndex

    if HAVE_FAISS:
        pytest.skip("the faiss package provides these factories")
    x, q = _clustered(n=1200)
    store = tmp_path / "store"
    store.mkdir()
    x.astype(np.float16).tofile(store / "gradients.bin")
    (store / "info.json").write_text(json.dumps({"grad_sizes": {"w": x.shape[1]}, "num_grads": len(x), "base_dtype": "float16"}))
    FaissIndex.create_index(store, tmp_path / "ann", FaissConfig(index_factory="IVF16,Flat", num_shards=2, nprobe=1), "cpu",
                            unit_norm=False, hessians={})
    idx = FaissIndex(tmp_path / "ann")
    assert idx.nprobe == 1 and all(s.nprobe == 1 for s in idx.shards)
    _, truth = _exact(x.astype(np.float16).astype(np.float32), q, 10)
    low = _recall(idx.search(q, 10)[1], truth)
    idx.nprobe = 16
    assert all(s.nprobe == 16 for s in idx.shards)
    assert _recall(idx.search(q, 10)[1], truth) > max(low, 0.99)
