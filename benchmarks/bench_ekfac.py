"""EK-FAC fitting throughput: K-FAC covariance pass, eigendecomposition, eigenvalue-correction
pass on a random-init GPT-NeoX 12L d768 (bf16 compute, fp32 factors), synthetic Zipf data.

    python benchmarks/bench_ekfac.py [--impl ours|reference] [--docs 64] [--seq-len 1024]

Prints one JSON line with seconds per phase and tokens/s of the two data passes.  The
reference arm runs the unmodified reference collectors on the same in-tree model object.
"""

from __future__ import annotations

import argparse
import json
import shutil
import tempfile
from pathlib import Path

from common import use_reference, wall

import torch

SPEC = dict(model_type="gpt_neox", vocab_size=50304, hidden_size=768, intermediate_size=3072, num_hidden_layers=12,
            num_attention_heads=12, rotary_pct=0.25, max_position_embeddings=2048)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--docs", type=int, default=64)
    ap.add_argument("--seq-len", type=int, default=1024)
    ap.add_argument("--token-batch", type=int, default=16384)
    args = ap.parse_args()

    from bergson_b200.data import allocate_batches, zipf_token_ids
    from bergson_b200.models import build_model
    from bergson_b200.models.registry import args_from_dict
    from datasets import Dataset

    dev = torch.device("cuda:0")
    model = build_model(args_from_dict(SPEC), dtype=torch.bfloat16, device=dev, init_on_device=True)
    model.requires_grad_(False)
    model.get_input_embeddings().requires_grad_(True)
    ids = zipf_token_ids(args.docs, args.seq_len, SPEC["vocab_size"], seed=0)
    ds = Dataset.from_dict({"input_ids": ids, "length": [args.seq_len] * args.docs})
    batches = allocate_batches(ds["length"], args.token_batch)
    tmp = Path(tempfile.mkdtemp(prefix="ekfac_bench_"))

    if args.impl == "reference":
        if not use_reference():
            print(json.dumps({"impl": "reference", "unavailable": "reference not installed under baseline/_ref"}))
            return
        import bergson as pkg
        from bergson.config import HessianConfig
        from bergson.hessians.eigenvectors import compute_eigendecomposition, save_uncorrected_eigenvalues
        from bergson.hessians.hessian_approximations import collect_hessians
    else:
        import bergson_b200 as pkg
        from bergson_b200.config import HessianConfig
        from bergson_b200.hessians.eigenvectors import compute_eigendecomposition, save_uncorrected_eigenvalues
        from bergson_b200.hessians.hessian_approximations import collect_hessians

    cfg = pkg.IndexConfig(run_path=str(tmp / "run"), token_batch_size=args.token_batch)
    cfg.partial_run_path.mkdir(parents=True)
    hcfg = HessianConfig(method="kfac", ev_correction=True, use_dataset_labels=True)
    kw = dict(model=model, data=ds, index_cfg=cfg, batches=batches, hessian_cfg=hcfg)
    collect_hessians(**{**kw, "batches": batches[:1]})  # warm-up (allocator, kernels)
    t_cov = wall(lambda: collect_hessians(**kw))
    total = torch.load(cfg.partial_run_path / "total_processed.pt", weights_only=False)

    def eig():
        a = compute_eigendecomposition(str(cfg.partial_run_path / "activation_sharded"), total)
        g = compute_eigendecomposition(str(cfg.partial_run_path / "gradient_sharded"), total)
        save_uncorrected_eigenvalues(cfg.partial_run_path, a, g, total, 0, 1)

    t_eig = wall(eig)
    t_lam = wall(lambda: collect_hessians(**kw, ev_correction=True))
    tokens = args.docs * args.seq_len
    print(json.dumps({"impl": args.impl, "model": "gpt_neox-12L-d768", "tokens": tokens, "cov_pass_s": t_cov,
                      "eigh_s": t_eig, "lambda_pass_s": t_lam, "fit_s": t_cov + t_eig + t_lam,
                      "cov_tokens_per_s": tokens / t_cov, "lambda_tokens_per_s": tokens / t_lam}))
    shutil.rmtree(tmp, ignore_errors=True)


if __name__ == "__main__":
    main()
