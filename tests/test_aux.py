"""Auxiliary components: recall benchmark, finite differences, optimizer-state loaders,
auto batch size model, diagnostics, format templates, in-memory collector, FAISS-less index."""

import json

import numpy as np
import pytest
import torch

from bergson_b200.config import DataConfig, FaissConfig, IndexConfig, RecallConfig, RecallDataConfig
from bergson_b200.gradients import AdafactorNormalizer, AdamNormalizer

from .helpers import tiny_dataset, tiny_model


def test_recall_metrics_with_oracle_scores(tmp_path):
    from datasets import load_from_disk

    from bergson_b200.recall import ensure_recall_datasets, gold_ranks, run_recall
    from bergson_b200.score.score_writer import save_sequence_scores

    data = RecallDataConfig(num_people=6, seed=0, data_dir=str(tmp_path / "data"))
    s_path, q_path = ensure_recall_datasets(data)
    assert ensure_recall_datasets(data) == (s_path, q_path)  # cached
    st, qs = load_from_disk(str(s_path)), load_from_disk(str(q_path))
    assert len(qs) == 24 and len(st) == 24 * 3
    scores = np.zeros((len(st), len(qs)), dtype=np.float32)
    for q, (pid, field) in enumerate(zip(qs["identifier"], qs["field"])):
        for i, (sid, sf) in enumerate(zip(st["identifier"], st["field"])):
            scores[i, q] = 1.0 if (sid, sf) == (pid, field) else -float(i) * 1e-3
    save_sequence_scores(tmp_path / "scores", scores)
    out = run_recall(RecallConfig(run_path=str(tmp_path / "out"), scores=str(tmp_path / "scores"), data=data, k=3))
    assert out["mrr"] == 1.0 and out["recall_at_3"] == 1.0 and out["strict_recall_at_3"] == 1.0
    assert (tmp_path / "out" / "recall.csv").exists() and (tmp_path / "out" / "summary.csv").exists()
    flipped = run_recall(RecallConfig(run_path=str(tmp_path / "o2"), scores=str(tmp_path / "scores"), data=data, k=3,
                                      higher_is_better=False))
    assert flipped["mrr"] < 0.2
    assert gold_ranks(np.array([3.0, 1.0, 3.0, 2.0]), np.array([2, 1])).tolist() == [2, 4]


def test_finite_diff_matches_directional_derivative():
    from bergson_b200.utils.gradcheck import FiniteDiff, compute_effect

    torch.manual_seed(0)
    lin = torch.nn.Linear(4, 3).double()
    x = torch.randn(5, 4, dtype=torch.float64)
    before = lin.weight.detach().clone()
    f = lambda: lin(x).pow(2).sum()  # noqa: E731
    d = {"weight": torch.randn(3, 4, dtype=torch.float64)}
    fd, pred = compute_effect(lin, d, f, eps=1e-5)
    assert abs(fd - pred) / abs(pred) < 1e-6
    assert torch.equal(lin.weight.detach(), before)  # restored exactly (bitwise swap)
    with FiniteDiff(lin, d, 0.5).perturbed(+1):
        torch.testing.assert_close(lin.weight.detach(), before + 0.5 * d["weight"])


def test_optimizer_state_round_trip(tmp_path):
    from bergson_b200.magic import optim
    from bergson_b200.utils.load_from_optimizer import load_from_optimizer, save_second_moments_as_optimizer_pt

    model = tiny_model("gpt2")
    model.requires_grad_(True)
    params = {k: v for k, v in model.named_parameters()}
    opt = optim.adamw(1e-3)
    state = opt.init(params)
    g = torch.Generator().manual_seed(0)
    state["nu"] = {k: torch.rand(v.shape, generator=g) for k, v in params.items()}
    n = save_second_moments_as_optimizer_pt(model, state, tmp_path / "optimizer.pt", step=7, betas=(0.9, 0.99), eps=1e-8)
    assert n == len(params)
    saved = torch.load(tmp_path / "optimizer.pt", weights_only=False)
    assert saved["param_groups"][0]["betas"] == (0.9, 0.99) and int(saved["state"][0]["step"]) == 7
    norms = load_from_optimizer(model, str(tmp_path), include_bias=True)
    name = "h.0.attn.c_attn"  # relative to base_model; Conv1D stores [in, out]
    assert isinstance(norms[name], AdamNormalizer)
    torch.testing.assert_close(norms[name].weight_avg_sq, state["nu"]["transformer.h.0.attn.c_attn.weight"].T)
    torch.testing.assert_close(norms[name].bias_avg_sq, state["nu"]["transformer.h.0.attn.c_attn.bias"])
    # HF-style Adafactor entries, two param groups are rejected when they do not fit the model
    fact = {"state": {0: {"exp_avg_sq_row": torch.rand(8), "exp_avg_sq_col": torch.rand(5), "param_name": "fc.weight"}},
            "param_groups": [{"params": [0]}]}
    torch.save(fact, tmp_path / "fact.pt")
    lin = torch.nn.Sequential()
    lin.fc = torch.nn.Linear(5, 8)
    got = load_from_optimizer(lin, str(tmp_path / "fact.pt"))
    assert isinstance(got["fc"], AdafactorNormalizer) and got["fc"].row.shape == (8,) and got["fc"].col.shape == (5,)


def test_batch_size_prediction_and_cache(tmp_path):
    from bergson_b200.utils.batch_size import _append_to_cache, _check_cache, _get_system_metadata, predict_batch_size

    # 2 GB fixed + 1 MB per token, 80 GB budget
    t = predict_batch_size(2e9 + 1024e6, 1024, 2e9 + 2048e6, 2048, 80e9)
    assert t % 256 == 0 and 77000 < t <= 78000
    assert predict_batch_size(1e9, 256, 1e9, 512, 2e9, max_tokens=4096) == 4096  # flat measurement: capped
    meta = _get_system_metadata(IndexConfig(run_path="x", model="m"))
    assert _check_cache(tmp_path / "c.jsonl", meta) is None
    _append_to_cache(tmp_path / "c.jsonl", meta, 8192)
    assert _check_cache(tmp_path / "c.jsonl", meta) == 8192
    assert _check_cache(tmp_path / "c.jsonl", {**meta, "model": "other"}) is None


def test_diagnose_runs_on_native_model():
    from bergson_b200.diagnose import diagnose
    from bergson_b200.diagnose_config import DiagnoseConfig

    out = diagnose(DiagnoseConfig(model="native:llama-tiny?vocab_size=128", dataset="synthetic:zipf?n=12&len=14&vocab=128&min_len=5",
                                  n_trials=3, precision="fp32", device="cpu", max_len=14, min_len=4, threshold=0.999))
    assert out["special_tokens_ok"] and out["passing"] == "precision=fp32" and out["equal_length_min_cos"] > 0.999


def test_format_template(tmp_path):
    from datasets import Dataset

    from bergson_b200.format import apply_format

    ds = Dataset.from_dict({"question": [" Capital of France? "], "choices": [["Rome", "Paris", "Bern", "Oslo"]], "answer": [1]})
    import bergson_b200

    path = str(__import__("pathlib").Path(bergson_b200.__file__).parent / "templates" / "mcqa.yaml")
    out = apply_format(ds, path)
    assert out["completion"] == ["B"] and out["prompt"][0].startswith("Capital of France?\nA. Rome") and out["prompt"][0].endswith("Answer:")
    (tmp_path / "t.yaml").write_text('doc_to_text: "Q: {{question}}"\n')
    assert apply_format(ds, str(tmp_path / "t.yaml"))["text"] == ["Q:  Capital of France? "]


def test_in_memory_collector_with_scorer_and_flat_index(tmp_path):
    from bergson_b200 import Attributor, GradientProcessor, InMemoryCollector, collect_gradients, load_gradients
    from bergson_b200.collector.collector import CollectorComputer
    from bergson_b200.data import allocate_batches

    torch.manual_seed(0)
    model = tiny_model("gpt_neox")
    model.requires_grad_(False)
    model.get_input_embeddings().requires_grad_(True)
    ds = tiny_dataset(n=10, length=12)
    cfg = IndexConfig(run_path=str(tmp_path / "idx"), projection_dim=4, token_batch_size=48)
    cfg.partial_run_path.mkdir(parents=True)
    batches = allocate_batches(ds["length"], 48)
    proc = GradientProcessor(projection_dim=4)
    coll = InMemoryCollector(model=model.base_model, data=ds, cfg=cfg, processor=proc, skip_hessians=False)
    CollectorComputer(model=model, data=ds, collector=coll, batches=batches, cfg=cfg).run_with_collector_hooks("mem")
    assert set(coll.gradients) == set(coll.shapes()) and next(iter(coll.gradients.values())).shape == (10, 16)
    assert len(proc.hessians) == len(coll.gradients) and len(proc.hessians_eigen) == len(coll.gradients)
    collect_gradients(model, ds, GradientProcessor(projection_dim=4), cfg, batches=batches)
    disk = np.asarray(load_gradients(cfg.partial_run_path))
    mem = torch.cat([coll.gradients[n] for n in coll.shapes()], dim=1).numpy()
    np.testing.assert_allclose(mem, disk, rtol=1e-5, atol=1e-7)
    exact = Attributor(cfg.partial_run_path, unit_norm=True)
    flat = Attributor(cfg.partial_run_path, unit_norm=True, faiss_cfg=FaissConfig(index_factory="Flat", num_shards=2))
    q = {n: torch.from_numpy(disk[:3, lo:hi]) for n, (lo, hi) in exact.offsets.items()}
    s1, i1 = exact.search(q, k=4)
    s2, i2 = flat.search(q, k=4)
    assert i1[:, 0].tolist() == [0, 1, 2] and i2[:, 0].tolist() == [0, 1, 2]
    np.testing.assert_allclose(s1.numpy(), s2.numpy(), atol=1e-4)
