"""Nearest-neighbour search over a synthetic gradient store on one GPU: exact scan against the
in-tree inverted-file indices.

    python benchmarks/bench_ann.py [--rows 1000000] [--dim 256] [--queries 1024] [--k 10]

Rows are unit vectors drawn around 4096 random centres (so that neighbours exist); queries are
perturbed rows.  The store (rows x dim, fp16: 512 MB at the defaults) is larger than L2.  Every
search is timed with CUDA events after three warm-up searches; recall is measured against the
exact fp32 scan.  Prints one JSON line.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=1_000_000)
    ap.add_argument("--dim", type=int, default=256)
    ap.add_argument("--queries", type=int, default=1024)
    ap.add_argument("--k", type=int, default=10)
    ap.add_argument("--reps", type=int, default=5)
    args = ap.parse_args()

    from benchmarks.clocks import ClockSampler
    from bergson_b200.query.native_ann import NativeIndex, parse_factory

    dev = torch.device("cuda", 0)
    g = torch.Generator(dev).manual_seed(0)
    centres = torch.randn(4096, args.dim, device=dev, generator=g) * 3
    which = torch.randint(0, 4096, (args.rows,), device=dev, generator=g)
    x = centres[which] + torch.randn(args.rows, args.dim, device=dev, generator=g)
    x = x / x.norm(dim=1, keepdim=True)
    pick = torch.randperm(args.rows, device=dev, generator=g)[: args.queries]
    q = x[pick] + 0.02 * torch.randn(args.queries, args.dim, device=dev, generator=g)

    def timed(idx):
        for _ in range(3):
            idx.search(q, args.k)
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(args.reps):
            d, i = idx.search(q, args.k)
        t1.record()
        torch.cuda.synchronize()
        return t0.elapsed_time(t1) / args.reps, i

    sampler = ClockSampler(0).start()
    out = {"bench": "ann_search", "rows": args.rows, "dim": args.dim, "queries": args.queries, "k": args.k, "arms": []}
    truth = None
    for spec, nprobe in (("Flat", 0), ("SQfp16", 0), ("IVF1024,SQfp16", 8), ("IVF1024,SQfp16", 32), ("IVF1024,PQ32", 32)):
        idx = NativeIndex(args.dim, parse_factory(spec), device=dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        if idx.factory.needs_training:
            idx.train(x[: 1024 * 256])
        idx.add(x)
        e1.record()
        torch.cuda.synchronize()
        idx.nprobe = nprobe or 1
        ms, found = timed(idx)
        if truth is None:
            truth = found
        recall = float(sum(len(set(a.tolist()) & set(b.tolist())) for a, b in zip(found, truth)) / truth.size)
        out["arms"].append({"index": spec, "nprobe": nprobe or None, "build_s": e0.elapsed_time(e1) / 1e3, "search_ms": ms,
                            "queries_per_s": args.queries / (ms / 1e3), "recall_at_k_vs_exact": recall,
                            "bytes_per_row": int(idx.vectors.element_size() * idx.vectors.shape[1])})
        del idx
        torch.cuda.empty_cache()
    out["clocks"] = sampler.stop()
    print(json.dumps(out))


if __name__ == "__main__":
    main()
