"""A store sharded over two gloo ranks answers queries like a single resident store."""

import numpy as np
import torch

from bergson_b200.config import DistributedConfig
from bergson_b200.data import create_index
from bergson_b200.distributed import init_dist, launch_distributed_run
from bergson_b200.gradients import GradientProcessor


def _make_store(path, rows=37, sizes=None, seed=0):
    sizes = sizes or {"a": 6, "b": 10}
    mm = create_index(path, rows, sizes, np.float32)
    rng = np.random.default_rng(seed)
    mm[:] = rng.standard_normal(mm.shape).astype(np.float32)
    mm.flush()
    GradientProcessor(projection_dim=4).save(path)
    return sizes


def _worker(rank, local_rank, world, path, out_dir, unit_norm):
    from bergson_b200 import Attributor

    init_dist(rank, local_rank, world)
    attr = Attributor(path, device="cpu", unit_norm=unit_norm, sharded=True)
    torch.manual_seed(3)
    queries = {"a": torch.randn(5, 6), "b": torch.randn(5, 10)}
    for reverse in (False, True):
        s, i = attr.search(queries, k=7, reverse=reverse)
        torch.save((s, i), f"{out_dir}/r{rank}_{int(reverse)}.pt")
    s_all, i_all = attr.search(queries, k=None)
    torch.save((s_all, i_all), f"{out_dir}/r{rank}_all.pt")


def test_sharded_store_matches_resident_store(tmp_path):
    from bergson_b200 import Attributor

    store = tmp_path / "store"
    store.mkdir()
    _make_store(store)
    for unit_norm in (False, True):
        out = tmp_path / f"out_{unit_norm}"
        out.mkdir()
        launch_distributed_run("sharded_query", _worker, [str(store), str(out), unit_norm],
                               DistributedConfig(nproc_per_node=2))
        ref = Attributor(store, device="cpu", unit_norm=unit_norm)
        torch.manual_seed(3)
        queries = {"a": torch.randn(5, 6), "b": torch.randn(5, 10)}
        for reverse in (False, True):
            s_ref, i_ref = ref.search(queries, k=7, reverse=reverse)
            for rank in (0, 1):
                s, i = torch.load(out / f"r{rank}_{int(reverse)}.pt")
                torch.testing.assert_close(s, s_ref, rtol=1e-5, atol=1e-6)
                assert torch.equal(i, i_ref)
        s_ref, i_ref = ref.search(queries, k=None)
        s, i = torch.load(out / "r1_all.pt")
        assert s.shape == s_ref.shape == (5, 37)
        torch.testing.assert_close(s, s_ref, rtol=1e-5, atol=1e-6)
        assert torch.equal(i, i_ref)
