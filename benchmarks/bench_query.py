"""Query throughput against a store resident in GPU memory: top-k of `queries @ store^T`.

    python benchmarks/bench_query.py [--impl ours|reference] [--rows 32768] [--dim 57344]
                                     [--queries 1024] [--k 100]

The store holds random fp16 rows (dimension 224 modules x 256 by default); cosine scoring.
Prints one JSON line with seconds per search and query-row scores per second.
"""

from __future__ import annotations

import argparse
import json
import shutil
import tempfile
from pathlib import Path

from common import cuda_timed, use_reference

import numpy as np
import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--rows", type=int, default=32768)
    ap.add_argument("--dim", type=int, default=57344)
    ap.add_argument("--queries", type=int, default=1024)
    ap.add_argument("--k", type=int, default=100)
    args = ap.parse_args()

    from bergson_b200.data import create_index
    from bergson_b200.gradients import GradientProcessor

    tmp = Path(tempfile.mkdtemp(prefix="query_bench_"))
    modules = args.dim // 256
    sizes = {f"m{i}": 256 for i in range(modules)}
    mm = create_index(tmp, args.rows, sizes, np.float16)
    rng = np.random.default_rng(0)
    for lo in range(0, args.rows, 4096):
        mm[lo : lo + 4096] = rng.standard_normal((min(4096, args.rows - lo), args.dim), dtype=np.float32).astype(np.float16)
    mm.flush()
    GradientProcessor(projection_dim=16).save(tmp)

    if args.impl == "reference":
        if not use_reference():
            print(json.dumps({"impl": "reference", "unavailable": "reference not installed under baseline/_ref"}))
            return
        from bergson import Attributor
    else:
        from bergson_b200 import Attributor

    attr = Attributor(tmp, device="cuda:0", dtype=torch.float16, unit_norm=True)
    q = torch.randn(args.queries, args.dim, device="cuda:0", dtype=torch.float16)
    queries = {f"m{i}": q[:, i * 256 : (i + 1) * 256].contiguous() for i in range(modules)}
    sec = cuda_timed(lambda: attr.search(queries, args.k), warmup=1, iters=3)
    print(json.dumps({"impl": args.impl, "rows": args.rows, "dim": args.dim, "queries": args.queries, "k": args.k,
                      "search_s": sec, "scores_per_s": args.rows * args.queries / sec,
                      "store_gb": args.rows * args.dim * 2 / 1e9}))
    shutil.rmtree(tmp, ignore_errors=True)


if __name__ == "__main__":
    main()
