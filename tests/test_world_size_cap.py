"""A dataset with fewer documents than ranks shrinks the launch instead of padding the data;
the per-node parent processes still meet at a barrier before anyone reads the result."""

import os
import time

import pytest
import torch.multiprocessing as mp

from bergson_b200.config import DistributedConfig
from bergson_b200.distributed import cap_world_size_to_dataset, find_free_port, parent_barrier


@pytest.mark.parametrize("docs,want", [(1, (1, 1)), (3, (1, 3)), (5, (1, 4)), (0, (1, 1)), (16, (4, 4)), (100, (4, 4))])
def test_cap(docs, want):
    cfg = DistributedConfig(nnode=4, nproc_per_node=4)
    capped = cap_world_size_to_dataset(cfg, dataset_size=docs)
    assert (capped.nnode, capped.nproc_per_node) == want and capped.world_size == want[0] * want[1]
    assert (cfg.nnode, cfg.nproc_per_node, cfg.world_size) == (4, 4, 16)  # the input is not modified
    if docs >= 16:
        assert capped is cfg


def test_single_node_config_is_left_alone():
    cfg = DistributedConfig(nnode=1, nproc_per_node=2)
    assert cap_world_size_to_dataset(cfg, dataset_size=10).world_size == 2


def test_node_rank_sources(monkeypatch):
    for var in ("SLURM_NODEID", "GROUP_RANK", "NODE_RANK"):
        monkeypatch.delenv(var, raising=False)
    with pytest.raises(ValueError, match="node_rank"):
        DistributedConfig(nnode=2, nproc_per_node=2).rank
    assert DistributedConfig(nnode=1, nproc_per_node=2).rank == 0
    monkeypatch.setenv("GROUP_RANK", "1")
    monkeypatch.setenv("LOCAL_RANK", "1")
    cfg = DistributedConfig(nnode=2, nproc_per_node=2)
    assert (cfg.start_rank, cfg.rank) == (2, 3)
    assert DistributedConfig(nnode=2, nproc_per_node=2, node_rank=0).rank == 1  # the explicit field wins


def _node_parent(node: int, nnode: int, port: int, partial, final):
    """What each node's launcher does when a one-document build was capped to one rank:
    node 0 writes and publishes, every node waits at the parents' barrier, then reads."""
    os.environ.update(SLURM_NODEID=str(node), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    orig = DistributedConfig(nnode=nnode, nproc_per_node=4)
    capped = cap_world_size_to_dataset(orig, dataset_size=1)
    if capped.world_size <= 1 and orig._node_rank == 0:
        time.sleep(0.3)
        partial.mkdir(parents=True, exist_ok=True)
        (partial / "config.yaml").write_text("data")
        partial.rename(final)
    if capped.world_size < orig.world_size:
        parent_barrier(orig)
    assert (final / "config.yaml").exists(), f"node {node}: result not visible after the barrier"


def _port_whose_successor_is_free() -> int:
    import socket

    for _ in range(50):  # the parents' barrier listens on MASTER_PORT + 1
        port = find_free_port()
        with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
            try:
                s.bind(("127.0.0.1", port + 1))
                return port
            except OSError:
                continue
    raise RuntimeError("no pair of adjacent free ports found")


def test_parents_wait_for_the_capped_build(tmp_path):
    port = _port_whose_successor_is_free()
    mp.spawn(_node_parent, args=(2, port, tmp_path / "run.part", tmp_path / "run"), nprocs=2, join=True)
    assert (tmp_path / "run" / "config.yaml").read_text() == "data"


def _count_rows(rank, world, dataset):
    import json

    import torch
    import torch.distributed as dist

    mine = torch.tensor([float(len(dataset["rows"][rank::world]))])
    dist.all_reduce(mine)
    with open(f"{dataset['out']}/rank{rank}.json", "w") as f:
        json.dump({"world": world, "total": float(mine)}, f)


def _single(rank, world, dataset):
    dataset["seen"].append((rank, world))


def test_dist_main_runs_a_worker_per_rank(tmp_path):
    import json

    from bergson_b200.distributed import dist_main

    seen = {"seen": []}
    dist_main(seen, _single, nproc=1)  # one device: in this process, no process group
    assert seen["seen"] == [(0, 1)]
    dist_main({"rows": list(range(7)), "out": str(tmp_path)}, _count_rows, nproc=2)
    got = [json.load(open(tmp_path / f"rank{r}.json")) for r in range(2)]
    assert got == [{"world": 2, "total": 7.0}] * 2
