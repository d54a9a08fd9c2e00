"""Collector variants beyond the basic two-sided projection: global projection target, split
heads and per-token rows under optimizer normalisers, query slicing and a two-node build."""

import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from bergson_b200 import GradientProcessor
from bergson_b200.collector.collector import create_projection_matrix
from bergson_b200.collector.gradient_collectors import TraceCollector
from bergson_b200.config import AttentionConfig
from bergson_b200.data import load_gradients, load_scores
from bergson_b200.gradients import AdafactorNormalizer, AdamNormalizer

from .helpers import TwoLayer

ROOT = Path(__file__).resolve().parents[1]


def _collect(model, x, y, processor, mask=None, loss_mask=None, **kw):
    c = TraceCollector(model=model, processor=processor, device="cpu", dtype=torch.float32, **kw)
    with (c.with_batch(mask) if mask is not None else c):
        err = (model(x) - y) ** 2
        (err if loss_mask is None else err * loss_mask[..., None]).sum().backward()
    model.zero_grad()
    return {k: torch.cat(v) for k, v in c.mod_grads.items()}


def _normalizers(model, kind):
    g = torch.Generator().manual_seed(11)
    out = {}
    for name in ("fc1", "fc2"):
        o, i = getattr(model, name).weight.shape
        if kind == "adam":
            out[name] = AdamNormalizer(torch.rand(o, i, generator=g) + 0.5)
        else:
            out[name] = AdafactorNormalizer(torch.rand(o, generator=g) + 0.5, torch.rand(i, generator=g) + 0.5)
    return out


def test_global_projection_sums_projected_modules(tmp_path):
    """projection_target='global': one vector per example, the sum over modules of each module's
    flattened gradient times that module's own [P, d_m] projection."""
    import json

    from bergson_b200.__main__ import main

    common = ["--model", "native:llama-tiny?vocab_size=256&hidden_size=32&intermediate_size=64", "--data.dataset",
              "synthetic:zipf?n=6&len=12&vocab=256&seed=0&min_len=6", "--token_batch_size", "64", "--nproc_per_node", "1"]
    main(["build", str(tmp_path / "full"), "--projection_dim", "0", *common])
    main(["build", str(tmp_path / "glob"), "--projection_dim", "9", "--projection_target", "global", *common])
    full = np.asarray(load_gradients(tmp_path / "full"), dtype=np.float64)
    got = np.asarray(load_gradients(tmp_path / "glob"), dtype=np.float64)
    sizes = json.load(open(tmp_path / "full" / "info.json"))["grad_sizes"]
    assert json.load(open(tmp_path / "glob" / "info.json"))["grad_sizes"] == {"gradients": 9}
    want, off = 0, 0
    for name, d in sizes.items():
        R = create_projection_matrix(f"{name}/single", 9, d, torch.float32, torch.device("cpu"), "rademacher")
        want = want + full[:, off : off + d] @ R.double().numpy().T
        off += d
    np.testing.assert_allclose(got, want, rtol=1e-3, atol=1e-5 * np.abs(want).max())


@pytest.mark.parametrize("kind", ["adam", "adafactor"])
def test_head_split_under_normalizers_matches_row_blocks(kind):
    """A module split into heads must give the rows of the unsplit, normalised gradient."""
    torch.manual_seed(1)
    model = TwoLayer(i=5, h=6, o=2, bias=False)
    x, y = torch.randn(3, 4, 5), torch.randn(3, 4, 2)
    proc = lambda: GradientProcessor(normalizers=_normalizers(model, kind))  # noqa: E731
    whole = _collect(model, x, y, proc(), target_modules={"fc1"})["fc1"].view(3, 6, 5)
    heads = _collect(model, x, y, proc(), target_modules={"fc1"},
                     attention_cfgs={"fc1": AttentionConfig(num_heads=3, head_size=2, head_dim=2)})
    row = _normalizers(model, kind)["fc1"].row if kind == "adafactor" else None
    for h in range(3):
        want = whole[:, 2 * h : 2 * h + 2]
        if row is not None:
            # Adafactor's row scale carries sqrt(mean(row statistics)); a head's normaliser is the
            # slice of the module's, so its mean runs over the head's rows only.
            want = want * (row[2 * h : 2 * h + 2].mean() / row.mean()).sqrt()
        torch.testing.assert_close(heads[f"fc1.head_{h}"].view(3, 2, 5), want, atol=1e-5, rtol=1e-4)


@pytest.mark.parametrize("kind", ["adam", "adafactor", None])
@pytest.mark.parametrize("p", [None, 4])
def test_token_rows_sum_to_sequence_rows_under_normalizers(kind, p):
    torch.manual_seed(2)
    model = TwoLayer()
    x, y = torch.randn(2, 6, 5), torch.randn(2, 6, 2)
    mask = torch.ones(2, 6, dtype=torch.bool)
    mask[1, 4:] = False  # ragged: the second sequence collects four positions
    norms = _normalizers(model, kind) if kind else {}
    # positions outside the mask carry no loss, so they add nothing to the per-sequence rows
    seq = _collect(model, x, y, GradientProcessor(normalizers=norms, projection_dim=p), loss_mask=mask)
    tok = _collect(model, x, y, GradientProcessor(normalizers=norms, projection_dim=p), mask=mask, loss_mask=mask,
                   attribute_tokens=True)
    for name in ("fc1", "fc2"):
        rows = tok[name]
        assert rows.shape[0] == int(mask.sum())
        per_seq = torch.stack([rows[:6].sum(0), rows[6:].sum(0)])
        torch.testing.assert_close(per_seq, seq[name], atol=1e-4, rtol=1e-3)


MODEL = "native:llama-tiny?vocab_size=256"
TRAIN = "synthetic:zipf?n=20&len=16&vocab=256&seed=0&min_len=6"
QUERY = "synthetic:zipf?n=7&len=16&vocab=256&seed=1&min_len=8"


def _cli(*args, env=None):
    out = subprocess.run([sys.executable, "-m", "bergson_b200", *map(str, args)], cwd=ROOT, capture_output=True, text=True,
                         timeout=600, env=env)
    assert out.returncode == 0, out.stderr[-2000:]
    return out


def test_query_slices_equal_single_pass(tmp_path):
    """Scoring in slices of the query set (one data pass per slice) fills the same matrix."""
    common = ["--model", MODEL, "--projection_dim", "4", "--token_batch_size", "64", "--nproc_per_node", "1"]
    _cli("build", tmp_path / "query", "--data.dataset", QUERY, *common)
    _cli("score", tmp_path / "all", "--data.dataset", TRAIN, "--query_path", tmp_path / "query", *common)
    _cli("score", tmp_path / "sliced", "--data.dataset", TRAIN, "--query_path", tmp_path / "query",
         "--query_batch_size", "3", *common)
    a, b = load_scores(tmp_path / "all"), load_scores(tmp_path / "sliced")
    assert b.is_written() and a[:].shape == b[:].shape == (20, 7)
    # the products are the same; only the GEMM blocking (7 vs 3 query columns) reorders fp32 sums
    np.testing.assert_allclose(a[:], b[:], rtol=2e-4, atol=1e-5)


def test_two_node_build_equals_single_node(tmp_path):
    """Two `build --nnode 2` parents on one host (one CPU rank each, loopback rendezvous) write
    the same store as a single-node run."""
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    common = ["--model", MODEL, "--data.dataset", TRAIN, "--projection_dim", "4", "--token_batch_size", "64"]
    _cli("build", tmp_path / "one", *common, "--nproc_per_node", "1")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), CUDA_VISIBLE_DEVICES="")
    procs = []
    for node in (0, 1):
        log = open(tmp_path / f"node{node}.log", "w")
        procs.append((subprocess.Popen(
            [sys.executable, "-m", "bergson_b200", "build", str(tmp_path / "two"), *common, "--nnode", "2",
             "--nproc_per_node", "1", "--node_rank", str(node)], cwd=ROOT, env=env, stdout=log, stderr=subprocess.STDOUT), log))
    for p, log in procs:
        try:
            p.wait(timeout=600)
        finally:
            if p.poll() is None:
                p.kill()
            log.close()
    for node, (p, _) in enumerate(procs):
        assert p.returncode == 0, (tmp_path / f"node{node}.log").read_text()[-2000:]
    a, b = np.asarray(load_gradients(tmp_path / "one")), np.asarray(load_gradients(tmp_path / "two"))
    np.testing.assert_allclose(a, b, rtol=1e-4, atol=1e-6)


def test_shapes_of_global_and_per_module_targets():
    from bergson_b200 import GradientProcessor
    from bergson_b200.collector.gradient_collectors import TraceCollector
    from bergson_b200.config import AttentionConfig

    from .helpers import TwoLayer

    model = TwoLayer(i=5, h=6, o=2)
    mk = lambda proc, **kw: TraceCollector(model=model, processor=proc, device="cpu", dtype=torch.float32, **kw)  # noqa: E731
    assert dict(mk(GradientProcessor(projection_dim=64, projection_target="global")).shapes()) == {"gradients": torch.Size((64,))}
    with pytest.raises(AssertionError):
        mk(GradientProcessor(projection_dim=None, projection_target="global")).shapes()
    per = mk(GradientProcessor(projection_dim=8)).shapes()
    assert set(per) == {"fc1", "fc2"} and all(tuple(s) == (8, 8) for s in per.values())
    full = mk(GradientProcessor(include_bias=True)).shapes()
    assert tuple(full["fc1"]) == (6, 6) and tuple(full["fc2"]) == (2, 7)  # a bias adds one input column
    heads = mk(GradientProcessor(), attention_cfgs={"fc1": AttentionConfig(num_heads=3, head_size=2, head_dim=2)}).shapes()
    assert list(heads) == ["fc1.head_0", "fc1.head_1", "fc1.head_2", "fc2"] and tuple(heads["fc1.head_1"]) == (2, 5)


def test_global_projection_is_a_sum_of_column_blocks():
    """Projecting the concatenated gradient equals summing each module's projection by its own
    column block: why one matrix per module, added up, is a global projection."""
    torch.manual_seed(42)
    g = [torch.randn(3, d) for d in (6, 10, 4)]
    R = create_projection_matrix("test/single", 8, 20, torch.float32, torch.device("cpu"))
    blocks = R.split([6, 10, 4], dim=1)
    torch.testing.assert_close(torch.cat(g, 1) @ R.T, sum(x @ b.T for x, b in zip(g, blocks)))
