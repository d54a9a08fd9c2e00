"""MAGIC step times on one GPU for either build, with an optional per-operator table.

    python benchmarks/bench_magic.py [--impl ours|reference] [--kernel-table FILE]

Runs the ``magic`` metric of ``benchmarks/extra_metrics.py`` (GPT-2 12L d768, 64 x 512 tokens,
bf16, AdamW: the plain in-place training step and the meta-step = traced step + VJP) and prints
its JSON.  ``--kernel-table`` additionally profiles one meta-step with the torch profiler
(after the timed runs) and writes the per-operator device times to FILE.  The reference arm
needs the package under ``baseline/_ref`` and the stand-ins under ``baseline/shims``.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--kernel-table", default="")
    args = ap.parse_args()
    if args.impl == "reference":
        sys.path[:0] = [str(ROOT / "baseline" / "shims"), str(ROOT / "baseline" / "_ref")]

    import torch

    from benchmarks import extra_metrics as em

    timed = em._magic_run

    def run_and_profile(trainer, state, data, dev, world):
        out = timed(trainer, state, data, dev, world)
        if args.kernel_table:
            from torch.profiler import ProfilerActivity, profile

            st = trainer.step(state, data[0], inplace=True)

            def meta():
                st.detach_()
                st.requires_grad = True
                data.requires_grad = True
                before = st.differentiable_tensors()
                after = trainer.step(st, data[1], trace=True).differentiable_tensors()
                cot = [torch.full_like(t, 1e-3) for t in after]
                torch.autograd.grad(after, before + [data.weights], grad_outputs=cot, allow_unused=True)
                st.requires_grad = False
                data.requires_grad = False

            meta()
            torch.cuda.synchronize()
            with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
                meta()
                torch.cuda.synchronize()
            with open(args.kernel_table, "w") as f:
                f.write(prof.key_averages().table(sort_by="cuda_time_total", row_limit=45, max_name_column_width=80))
        return out

    em._magic_run = run_and_profile
    fn = em.magic_ours if args.impl == "ours" else em.magic_reference
    print(json.dumps(dict(fn(0, 0, 1), impl=args.impl)))


if __name__ == "__main__":
    main()
