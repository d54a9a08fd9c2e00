"""Metasmoothness and leave-k-out validation: the closed-form pieces, and both commands end
to end on a tiny random-init model (CPU)."""

import json

import numpy as np
import pytest
import torch

from bergson_b200.__main__ import main
from bergson_b200.magic.metasmoothness import metasmoothness_score

MODEL = "native:llama-tiny?vocab_size=256&num_hidden_layers=1"
TRAIN = "synthetic:zipf?n=16&len=12&vocab=256&seed=0"
QUERY = "synthetic:zipf?n=4&len=12&vocab=256&seed=1"


def run(*args):
    main([str(a) for a in args])


def test_metasmoothness_score_closed_form():
    t0 = torch.zeros(4)
    # Every coordinate keeps its direction: score 1.
    assert metasmoothness_score(t0, torch.tensor([1.0, -1.0, 2.0, 0.5]), torch.tensor([2.0, -2.0, 4.0, 1.0])) == 1.0
    # Every coordinate turns back: score -1.
    assert metasmoothness_score(t0, torch.tensor([1.0, -1.0, 2.0, 0.5]), torch.tensor([0.5, -0.5, 1.0, 0.25])) == -1.0
    # Nothing moved: defined as 1.
    assert metasmoothness_score(t0, t0, t0) == 1.0
    # Mixed: weights are |theta_2h - theta_0| / sum; coordinate 0 (weight 3/4) consistent, coordinate 1 (1/4) not.
    got = metasmoothness_score(torch.zeros(2), torch.tensor([1.0, 2.0]), torch.tensor([3.0, 1.0]))
    assert got == pytest.approx(0.75 - 0.25)


def test_metasmoothness_command(tmp_path):
    run("metasmoothness", tmp_path / "ms", "--model", MODEL, "--data.dataset", TRAIN, "--batch_size", "4", "--lr", "1e-3",
        "--fd_step", "0.05", "--nproc_per_node", "1")
    out = json.loads((tmp_path / "ms" / "metasmoothness.json").read_text())
    assert -1.0 <= out["score"] <= 1.0 and out["fd_step"] == 0.05 and out["total_movement_l1"] > 0
    # A small step on a smooth problem keeps almost every coordinate moving the same way.
    assert out["score"] > 0.5


def test_per_doc_query_losses_scatter_by_document():
    from datasets import Dataset

    from bergson_b200.magic.data_stream import DataStream
    from bergson_b200.validate import per_doc_query_losses

    V = 8
    ids = [[1, 2, 3, 4], [5, 6, 7, 1]]
    # Two sequences, three documents: the second sequence packs documents 1 and 2.
    ds = Dataset.from_dict({"input_ids": ids, "doc_ids": [[0, 0, 0, 0], [1, 1, 2, 2]], "length": [4, 4]})
    stream = DataStream(ds, 2)
    torch.manual_seed(0)
    table = torch.randn(V, V)

    def forward(x):
        return table[x]  # logits depend on the current token only

    got = per_doc_query_losses(forward, stream, 3)
    tok = torch.nn.functional.cross_entropy(table[torch.tensor(ids)][:, :-1].reshape(-1, V),
                                            torch.tensor(ids)[:, 1:].reshape(-1), reduction="none").view(2, 3)
    # Label tokens belong to: seq 0 -> doc 0 (three labels); seq 1 -> docs 1, 2, 2.
    want = torch.stack([tok[0].mean(), tok[1, 0], tok[1, 1:].mean()])
    torch.testing.assert_close(got, want)


def test_bank_loss_cache_key_tracks_what_losses_depend_on():
    from bergson_b200.config.config import ValidationConfig
    from bergson_b200.validate import bank_loss_cache_key

    a = ValidationConfig(run_path="x", model="m")
    b = ValidationConfig(run_path="y", model="m")  # the run path does not enter the key
    assert bank_loss_cache_key(a, False, 10) == bank_loss_cache_key(b, False, 10)
    assert bank_loss_cache_key(a, False, 10) != bank_loss_cache_key(a, True, 10)
    assert bank_loss_cache_key(a, False, 10) != bank_loss_cache_key(a, False, 11)
    b.batch_size = a.batch_size + 1
    assert bank_loss_cache_key(a, False, 10) != bank_loss_cache_key(b, False, 10)


def test_per_doc_query_losses_accepts_a_model_and_matches_its_loss():
    from datasets import Dataset

    from bergson_b200.magic.data_stream import DataStream
    from bergson_b200.validate import per_doc_query_losses

    from .helpers import tiny_model

    torch.manual_seed(0)
    model = tiny_model("llama")
    rows = [[1, 2, 3, 4, 5], [6, 7, 8], [9, 10, 11, 12], [13, 14]]
    stream = DataStream(Dataset.from_dict({"input_ids": rows}), batch_size=2)
    losses = per_doc_query_losses(model, stream, num_docs=4)
    for i, r in enumerate(rows):  # one document per row: its loss when run alone, whatever it was padded with
        x = torch.tensor([r])
        torch.testing.assert_close(losses[i], model(x, labels=x).loss.detach().float(), rtol=1e-4, atol=1e-5)
    # packed rows: a token's loss belongs to the document of its label token
    packed = DataStream(Dataset.from_dict({"input_ids": [[1, 2, 3, 4, 5, 6]], "doc_ids": [[0, 0, 0, 1, 1, 1]]}), batch_size=1,
                        weight_shape=(2,))
    got = per_doc_query_losses(model, packed, num_docs=2)
    x = torch.tensor([[1, 2, 3, 4, 5, 6]])
    tok = torch.nn.functional.cross_entropy(model(x).logits[0, :-1].float(), x[0, 1:], reduction="none")
    label_doc = torch.tensor([0, 0, 1, 1, 1])
    for d in range(2):
        torch.testing.assert_close(got[d], tok[label_doc == d].mean().detach(), rtol=1e-4, atol=1e-5)


def test_stream_serves_per_token_weights_after_a_flat_reweight():
    """Leave-out validation re-weights by flat index into the weights; with per-token weights
    ``[docs, seq_len]`` a flat subset must hit exactly those tokens, a whole row of indices the
    whole document, and per-document weights keep working."""
    from datasets import Dataset

    from bergson_b200.magic.data_stream import DataStream

    data = Dataset.from_dict({"input_ids": [[1, 2, 3, 4], [5, 6, 7, 8]]})
    stream = DataStream(data, batch_size=2, weight_shape=(2, 4))
    stream.requires_grad = False
    stream.weights.view(-1)[torch.tensor([0 * 4 + 2, 1 * 4 + 0])] = 0.0
    want = torch.ones(2, 4)
    want[0, 2] = want[1, 0] = 0.0
    torch.testing.assert_close(stream[0]["example_weight"].cpu(), want)
    stream.weights.data.fill_(1.0)
    stream.weights.view(-1)[torch.arange(4, 8)] = 0.5  # every token of document 1
    torch.testing.assert_close(stream[0]["example_weight"].cpu(), torch.tensor([[1.0] * 4, [0.5] * 4]))
    per_doc = DataStream(data, batch_size=2)
    per_doc.requires_grad = False
    per_doc.weights.view(-1)[torch.tensor([1])] = 0.0
    assert per_doc[0]["example_weight"].cpu().tolist() == [1.0, 0.0]


def test_metasmoothness_over_several_epochs(tmp_path):
    """Epochs are shuffled copies of the documents; a document keeps one data weight across all of
    them, and gradient accumulation and clipping reach the three trainings."""
    run("metasmoothness", tmp_path / "ms", "--model", MODEL, "--data.dataset", TRAIN, "--batch_size", "4", "--lr", "1e-3",
        "--fd_step", "0.05", "--num_epochs", "2", "--grad_accum_steps", "2", "--max_grad_norm", "1.0", "--nproc_per_node", "1")
    out = json.loads((tmp_path / "ms" / "metasmoothness.json").read_text())
    assert -1.0 <= out["score"] <= 1.0 and out["total_movement_l1"] > 0
    one = tmp_path / "one"
    run("metasmoothness", one, "--model", MODEL, "--data.dataset", TRAIN, "--batch_size", "4", "--lr", "1e-3",
        "--fd_step", "0.05", "--num_epochs", "1", "--nproc_per_node", "1")
    single = json.loads((one / "metasmoothness.json").read_text())
    assert out["total_movement_l1"] != single["total_movement_l1"]  # twice the steps, clipped: another trajectory
