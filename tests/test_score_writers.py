"""Score stores: 16-bit and 32-bit records, written flags, one-shot saves that replace an
existing store, and streaming writers that resume one."""

import json

import numpy as np
import torch

from bergson_b200.data import load_scores, load_scores_loss_signed
from bergson_b200.score.score_writer import MemmapSequenceScoreWriter, save_sequence_scores


def test_bfloat16_records(tmp_path):
    w = MemmapSequenceScoreWriter(tmp_path, 10, 3, dtype=torch.bfloat16, distributed=False)
    b1 = torch.tensor([[1.5, 2.5, 3.5], [4.5, 5.5, 6.5]], dtype=torch.bfloat16)
    b2 = torch.tensor([[7.5, 8.5, 9.5], [10.5, 11.5, 12.5], [13.5, 14.5, 15.5]], dtype=torch.bfloat16)
    w([0, 1], b1)
    w([5, 6, 7], b2)
    w.flush()
    info = json.load(open(tmp_path / "info.json"))
    assert info["num_items"] == 10 and info["num_scores"] == 3 and "bfloat16" in json.dumps(info["dtype"])
    written = np.asarray(w.scores["written_0"])
    assert written.tolist() == [True, True, False, False, False, True, True, True, False, False]
    s = load_scores(tmp_path)
    assert not s.is_written()
    np.testing.assert_array_equal(np.asarray(s[[0, 1]], dtype=np.float32), b1.float().numpy())
    np.testing.assert_array_equal(np.asarray(s[[5, 6, 7]], dtype=np.float32), b2.float().numpy())
    # 16-bit stores come back as fp32 tensors in the loss-signed loader
    full = MemmapSequenceScoreWriter(tmp_path / "full", 4, 1, dtype=torch.bfloat16, distributed=False)
    full([0, 1, 2, 3], torch.tensor([[1.0], [2.0], [3.0], [4.0]]))
    full.flush()
    scores, multi = load_scores_loss_signed(str(tmp_path / "full"))
    assert not multi and scores.dtype == torch.float32 and scores.squeeze(-1).tolist() == [1.0, 2.0, 3.0, 4.0]


def test_float32_records(tmp_path):
    w = MemmapSequenceScoreWriter(tmp_path, 5, 2, dtype=torch.float32, distributed=False)
    w([0, 1], torch.tensor([[1.5, 2.5], [3.5, 4.5]]))
    w.flush()
    np.testing.assert_array_equal(np.asarray(w.scores["score_0"][[0, 1]]), [1.5, 3.5])
    np.testing.assert_array_equal(np.asarray(w.scores["score_1"][[0, 1]]), [2.5, 4.5])


def test_one_shot_save_round_trips_16_bit_and_replaces_a_store(tmp_path):
    src = MemmapSequenceScoreWriter(tmp_path / "src", 4, 1, dtype=torch.bfloat16, distributed=False)
    src([0, 1, 2, 3], torch.tensor([[1.0], [2.0], [3.0], [4.0]]))
    src.flush()
    save_sequence_scores(tmp_path / "dst", load_scores(tmp_path / "src")[:], dtype=torch.bfloat16)
    assert np.asarray(load_scores(tmp_path / "dst")[:], dtype=np.float64).ravel().tolist() == [1.0, 2.0, 3.0, 4.0]
    # fewer score columns than the store that was there: the record size shrinks
    path = tmp_path / "shrink"
    save_sequence_scores(path, np.arange(100, 110, dtype=np.float32).reshape(5, 2))
    save_sequence_scores(path, np.array([1.0, 2.0, 3.0], dtype=np.float32))
    assert json.load(open(path / "info.json"))["num_scores"] == 1
    assert np.asarray(load_scores(path)[:]).ravel().tolist() == [1.0, 2.0, 3.0]
    # another element type
    path = tmp_path / "retype"
    save_sequence_scores(path, np.arange(50, 54, dtype=np.float32), dtype=torch.float32)
    save_sequence_scores(path, np.arange(50, 54, dtype=np.float32), dtype=torch.bfloat16)
    assert np.asarray(load_scores(path)[:], dtype=np.float64).ravel().tolist() == [50.0, 51.0, 52.0, 53.0]


def test_streaming_writer_resumes_an_existing_store(tmp_path):
    """Query columns are filled in slices, each slice reopening the directory."""
    w = MemmapSequenceScoreWriter(tmp_path, 3, 2, dtype=torch.float32, distributed=False)
    w([0, 1, 2], torch.tensor([[1.0], [2.0], [3.0]]), query_offset=0)
    w.flush()
    again = MemmapSequenceScoreWriter(tmp_path, 3, 2, dtype=torch.float32, distributed=False)
    assert not load_scores(tmp_path).is_written()  # column 1 is still missing
    again([0, 1, 2], torch.tensor([[4.0], [5.0], [6.0]]), query_offset=1)
    again.flush()
    s = load_scores(tmp_path)
    assert s.is_written()
    np.testing.assert_array_equal(np.asarray(s[:]), [[1.0, 4.0], [2.0, 5.0], [3.0, 6.0]])
    fresh = MemmapSequenceScoreWriter(tmp_path, 3, 2, dtype=torch.float32, distributed=False, overwrite=True)
    fresh.flush()
    assert not np.asarray(load_scores(tmp_path).mmap["written_0"]).any()


def _rank0_saves(rank, local_rank, world, out_dir):
    """Only rank 0 saves; then every rank meets at a barrier.  A collective hidden inside the
    savers would pair with that barrier on the other rank and leave the group out of step."""
    from pathlib import Path

    import torch.distributed as dist

    from bergson_b200.distributed import init_dist
    from bergson_b200.score.score_writer import save_token_scores

    init_dist(rank, local_rank, world)
    if rank == 0:
        save_sequence_scores(Path(out_dir) / "seq", np.arange(8, dtype=np.float32)[:, None])
        save_token_scores(Path(out_dir) / "tok", np.arange(8, dtype=np.float32)[:, None], np.array([0, 3, 8], dtype=np.int64))
    dist.barrier()
    t = torch.tensor([float(rank)])
    dist.all_reduce(t)
    assert float(t) == 1.0  # the group is still in step


def test_one_shot_savers_are_not_collective(tmp_path):
    from bergson_b200.config import DistributedConfig
    from bergson_b200.distributed import launch_distributed_run

    launch_distributed_run("savers", _rank0_saves, [str(tmp_path)], DistributedConfig(nproc_per_node=2))
    seq = load_scores(tmp_path / "seq")
    assert seq.is_written() and np.asarray(seq[:]).ravel().tolist() == list(range(8))
    tok = load_scores(tmp_path / "tok")
    assert tok.is_written() and tok.offsets.tolist() == [0, 3, 8] and np.asarray(tok[3:8]).ravel().tolist() == [3, 4, 5, 6, 7]
