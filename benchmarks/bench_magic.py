"""MAGIC step times on one GPU: an ordinary (untraced, in-place) training step and a
meta-step (the step replayed with a graph plus the vector-Jacobian product that carries the
parameter / optimizer-state cotangents to the previous state and to the data weights).

    python benchmarks/bench_magic.py [--seqs 8] [--seq-len 512] [--layers 12]

Model: random-init GPT-2 (d 768, 12 heads, vocab 50257), bf16 parameters, fp32 AdamW state.
Prints one JSON line.  The reference's trainer needs the `torchopt` package, which is not
available offline, so there is no reference arm.
"""

from __future__ import annotations

import argparse
import json

from common import cuda_timed

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seqs", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=512)
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--dtype", choices=["bf16", "fp32"], default="bf16")
    args = ap.parse_args()

    from bergson_b200.data import zipf_token_ids
    from bergson_b200.magic import optim
    from bergson_b200.magic.data_stream import DataStream
    from bergson_b200.magic.trainer import BackwardState, Trainer
    from bergson_b200.models import build_model
    from bergson_b200.models.registry import PRESETS, args_from_dict
    from datasets import Dataset

    dev = torch.device("cuda:0")
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    model = build_model(args_from_dict(dict(PRESETS["gpt2"], num_hidden_layers=args.layers)), dtype=dtype, device=dev,
                        init_on_device=True)
    model.requires_grad_(True)
    model.eval()
    n = args.seqs * 4
    ids = zipf_token_ids(n, args.seq_len, 50257, seed=0)
    data = DataStream(Dataset.from_dict({"input_ids": ids, "length": [args.seq_len] * n}), args.seqs, device=dev)
    trainer, state = Trainer.initialize(model, optim.adamw(lambda s: 3e-4, betas=(0.95, 0.975), eps_root=1e-8,
                                                           weight_decay=0.01))
    holder = {"s": state}

    def plain():
        holder["s"] = trainer.step(holder["s"], data[0], inplace=True)

    t_plain = cuda_timed(plain, warmup=2, iters=5)

    def meta():
        st = holder["s"]
        st.detach_()
        st.requires_grad = True
        data.requires_grad = True
        flat_i = st.differentiable_tensors()
        nxt = trainer.step(st, data[1], trace=True)
        flat_f = nxt.differentiable_tensors()
        cot = [torch.ones_like(t) * 1e-3 for t in flat_f]
        torch.autograd.grad(flat_f, flat_i + [data.weights], grad_outputs=cot, allow_unused=True)

    t_meta = cuda_timed(meta, warmup=1, iters=3)
    tokens = args.seqs * args.seq_len
    print(json.dumps({"model": f"gpt2-{args.layers}L-d768", "dtype": args.dtype, "tokens_per_step": tokens,
                      "train_step_s": t_plain, "meta_step_s": t_meta, "meta_over_train": t_meta / t_plain,
                      "train_tokens_per_s": tokens / t_plain, "meta_tokens_per_s": tokens / t_meta,
                      "peak_mem_gb": torch.cuda.max_memory_allocated() / 1e9}))


if __name__ == "__main__":
    main()
