"""Wall-clock benchmarks of the user-facing pipelines, the counterparts of the reference's
``benchmarks/benchmark_bergson_cli.py`` (commands run as subprocesses) and
``benchmarks/benchmark_bergson.py run`` (in-memory collection and scoring in one process).

    python benchmarks/bench_pipeline.py cli   --model native:llama-8b?init=device --vocab 128000 --tokens 1e6 [--gpus 1]
    python benchmarks/bench_pipeline.py inmem --model native:pythia-160m?init=device --vocab 50000 --tokens 1e6

``cli`` runs ``build`` (query store), ``build`` (training store), ``reduce`` and ``score`` through
``python -m bergson_b200`` on synthetic Zipf token data of the requested size and prints one JSON
line per command: tokens, wall seconds (process start to exit, model loading included -- what a
user waits for), tokens/s.  ``inmem`` keeps everything in one process: collects the projected
gradients of the training documents with ``InMemoryCollector`` and scores them against the
query gradients held in memory.  Both work on CPU with a tiny model, which is how the test
suite exercises them; the numbers worth keeping come from a GPU.
"""

from __future__ import annotations

import argparse
import json
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def _dataset(tokens: int, seq_len: int, vocab: int, seed: int) -> tuple[str, int]:
    docs = max(2, int(tokens) // seq_len)
    return f"synthetic:zipf?n={docs}&len={seq_len}&vocab={vocab}&seed={seed}&min_len={seq_len}", docs * seq_len


def _run(cmd: list[str]) -> float:
    t0 = time.perf_counter()
    proc = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True)
    dt = time.perf_counter() - t0
    if proc.returncode != 0:
        raise RuntimeError(f"{' '.join(cmd[:6])} ... failed:\n{proc.stderr[-2000:]}")
    return dt


def bench_cli(args) -> list[dict]:
    tmp = Path(args.workdir or tempfile.mkdtemp(prefix="bgn_cli_bench_"))
    train, n_train = _dataset(args.tokens, args.seq_len, args.vocab, 0)
    query, n_query = _dataset(args.query_tokens, args.seq_len, args.vocab, 1)
    common = ["--model", args.model, "--precision", args.precision, "--projection_dim", str(args.projection_dim),
              "--token_batch_size", str(args.token_batch_size), "--nproc_per_node", str(args.gpus), "--overwrite", "true"]
    exe = [sys.executable, "-m", "bergson_b200"]
    plan = [
        ("build_query", n_query, [*exe, "build", str(tmp / "query"), "--data.dataset", query, *common]),
        ("build", n_train, [*exe, "build", str(tmp / "index"), "--data.dataset", train, *common]),
        ("reduce", n_train, [*exe, "reduce", str(tmp / "mean"), "--data.dataset", train, "--aggregation", "mean", *common]),
        # `score` has two precision options (model and scoring): name the model's explicitly
        ("score", n_train, [*exe, "score", str(tmp / "scores"), "--data.dataset", train, "--query_path", str(tmp / "query"),
                            *["--index_cfg.precision" if a == "--precision" else a for a in common]]),
    ]
    out = []
    for name, tokens, cmd in plan:
        seconds = _run(cmd)
        rec = {"bench": "cli", "command": name, "model": args.model, "tokens": tokens, "n_gpus": args.gpus, "seconds": seconds,
               "tokens_per_s": tokens / seconds, "projection_dim": args.projection_dim, "precision": args.precision}
        print(json.dumps(rec), flush=True)
        out.append(rec)
    return out


def bench_inmem(args) -> dict:
    import torch

    from bergson_b200 import GradientProcessor, InMemoryCollector
    from bergson_b200.collector.collector import CollectorComputer
    from bergson_b200.config import IndexConfig
    from bergson_b200.data import allocate_batches, load_data_string
    from bergson_b200.models import load_model
    from bergson_b200.score.score_writer import InMemorySequenceScoreWriter
    from bergson_b200.score.scorer import Scorer
    from bergson_b200.utils.utils import get_device

    device = torch.device(get_device(0) if torch.cuda.is_available() else "cpu")
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[args.precision]
    sync = torch.cuda.synchronize if device.type == "cuda" else (lambda: None)
    model = load_model(args.model, dtype=dtype, device=device)
    model.requires_grad_(False)
    model.get_input_embeddings().requires_grad_(True)
    tmp = Path(args.workdir or tempfile.mkdtemp(prefix="bgn_inmem_bench_"))

    def collect(spec: str, name: str):
        ds = load_data_string(spec)
        ds = ds.add_column("length", [len(r) for r in ds["input_ids"]]) if "length" not in ds.column_names else ds
        cfg = IndexConfig(run_path=str(tmp / name), projection_dim=args.projection_dim, token_batch_size=args.token_batch_size)
        cfg.partial_run_path.mkdir(parents=True, exist_ok=True)
        coll = InMemoryCollector(model=model.base_model, data=ds, cfg=cfg, processor=GradientProcessor(projection_dim=args.projection_dim))
        batches = allocate_batches(ds["length"], args.token_batch_size)
        sync()
        t0 = time.perf_counter()
        CollectorComputer(model=model, data=ds, collector=coll, batches=batches, cfg=cfg).run_with_collector_hooks(name)
        sync()
        return coll, time.perf_counter() - t0, len(ds)

    train, n_train = _dataset(args.tokens, args.seq_len, args.vocab, 0)
    query, n_query = _dataset(args.query_tokens, args.seq_len, args.vocab, 1)
    qcoll, t_query, n_q = collect(query, "query")
    tcoll, t_build, n_t = collect(train, "train")
    modules = list(tcoll.gradients)
    writer = InMemorySequenceScoreWriter(n_t, n_q, dtype=torch.float32)
    scorer = Scorer({m: qcoll.gradients[m].float() for m in modules}, modules, writer, device, torch.float32)
    sync()
    t0 = time.perf_counter()
    scorer(list(range(n_t)), {m: tcoll.gradients[m].to(device) for m in modules})
    sync()
    t_score = time.perf_counter() - t0
    rec = {"bench": "inmem", "model": args.model, "tokens": n_train, "query_tokens": n_query, "device": str(device),
           "build_seconds": t_build, "build_tokens_per_s": n_train / t_build, "query_build_seconds": t_query,
           "score_seconds": t_score, "scores": n_t * n_q, "projection_dim": args.projection_dim, "precision": args.precision,
           "score_checksum": float(writer.scores.double().abs().sum())}
    print(json.dumps(rec), flush=True)
    return rec


def main(argv: list[str] | None = None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("mode", choices=["cli", "inmem"])
    ap.add_argument("--model", default="native:llama-tiny?vocab_size=256")
    ap.add_argument("--tokens", type=float, default=1e5, help="training tokens")
    ap.add_argument("--query-tokens", dest="query_tokens", type=float, default=4096)
    ap.add_argument("--seq-len", dest="seq_len", type=int, default=512)
    ap.add_argument("--vocab", type=int, default=256, help="token ids are drawn below this; keep it within the model's vocabulary")
    ap.add_argument("--projection-dim", dest="projection_dim", type=int, default=16)
    ap.add_argument("--token-batch-size", dest="token_batch_size", type=int, default=8192)
    ap.add_argument("--precision", default="bf16", choices=["bf16", "fp16", "fp32"])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--workdir", default="")
    args = ap.parse_args(argv)
    return bench_cli(args) if args.mode == "cli" else bench_inmem(args)


if __name__ == "__main__":
    main()
