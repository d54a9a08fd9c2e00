"""Tensor-parallel forward + backward of a Llama stack on N GPUs of one node: the
sequence-parallel path with the collectives inside the GEMM kernels against the same
sharding with NCCL all-reduces (the baseline that the fused kernels have to beat).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \\
        --master-port 29531 benchmarks/bench_tp.py [--layers 8] [--seqs 8] [--seq-len 2048]

Model: random-init Llama blocks (d 4096, 32 heads / 8 KV heads, FFN 14336, vocab 32768), bf16,
frozen weights with gradients flowing to the embeddings (the attribution set-up).  Each arm
is timed with CUDA events after warm-up, maximum over ranks; clocks are sampled during the
timed region.  Rank 0 prints one JSON line.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from datetime import timedelta
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--seqs", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--kernel-table", default="", help="write rank 0's per-kernel device times of one step of each "
                    "arm (torch profiler, taken after the timed region) to this file")
    args = ap.parse_args()

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev, timeout=timedelta(minutes=4))

    from benchmarks.clocks import ClockSampler
    from bergson_b200 import ops
    from bergson_b200.models import build_model
    from bergson_b200.models.registry import PRESETS, args_from_dict
    from bergson_b200.ops import native
    from bergson_b200.parallel import topology
    from bergson_b200.parallel.tensor_parallel import apply_tensor_parallel

    spec = dict(PRESETS["llama-8b"])
    spec.update(model_type="llama", hidden_size=4096, intermediate_size=14336, num_attention_heads=32,
                num_key_value_heads=8, num_hidden_layers=args.layers, vocab_size=32768,
                max_position_embeddings=max(4096, args.seq_len))
    model = build_model(args_from_dict(spec), dtype=torch.bfloat16, device=dev, init_on_device=True, seed=0)
    topology.init_topology(world)
    apply_tensor_parallel(model)
    model.requires_grad_(False)
    model.get_input_embeddings().requires_grad_(True)
    sp = getattr(model, "_seq_parallel", None)
    ids = torch.randint(0, 32768, (args.seqs, args.seq_len), device=dev, generator=torch.Generator(dev).manual_seed(1))
    targets = ids[:, 1:].reshape(-1)

    def step():
        h = model.hidden(ids)[:, :-1]
        logits = model.get_output_embeddings()(h)
        loss = ops.token_cross_entropy(logits.reshape(-1, logits.size(-1)), targets).sum()
        loss.backward()
        model.zero_grad(set_to_none=True)
        return loss

    def timed(label: str) -> dict:
        for _ in range(args.warmup):
            step()
        dist.barrier()
        torch.cuda.synchronize()
        sampler = ClockSampler(local).start()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(args.steps):
            loss = step()
        t1.record()
        dist.barrier()
        torch.cuda.synchronize()
        clocks = sampler.stop()
        ms = torch.tensor([t0.elapsed_time(t1) / args.steps], device=dev, dtype=torch.float64)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        out = {"arm": label, "ms_per_step": float(ms), "loss": float(loss.detach()), "clocks": clocks}
        if args.kernel_table:
            from torch.profiler import ProfilerActivity, profile

            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                step()
                torch.cuda.synchronize()
            if rank == 0:
                with open(args.kernel_table, "a") as f:
                    f.write(f"== {label} ==\n")
                    f.write(prof.key_averages().table(sort_by="cuda_time_total", row_limit=25,
                                                      max_name_column_width=90))
                    f.write("\n")
            dist.barrier()
        return out

    results = []
    if sp is not None:
        results.append(timed("collectives inside the GEMM kernels (peer memory)"))
        results[-1].update(barriers_per_step=sp.barriers // (args.steps + args.warmup),
                           fused_gemms_per_step=sp.fused_gemms // (args.steps + args.warmup))
        model._seq_parallel = None
    results.append(timed("NCCL all-reduce around library-ordered GEMMs"))
    status = int(native.kernel_status(local).item())
    tokens = args.seqs * args.seq_len
    if rank == 0:
        out = {"bench": "tensor_parallel_fwd_bwd", "n_gpus": world, "tokens_per_step": tokens, "layers": args.layers,
               "kernel_status": status, "arms": results}
        for r in results:
            r["tokens_per_s"] = tokens / (r["ms_per_step"] / 1e3)
        if len(results) == 2:
            out["fused_over_nccl"] = results[1]["ms_per_step"] / results[0]["ms_per_step"]
        print(json.dumps(out))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
