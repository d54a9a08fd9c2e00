"""Headline benchmark: gradient-store build throughput (tokens/s).

    python bench.py --gpus N --steps K --warmup W [--impl ours|reference]

Workload (TrackStar build config): random-init Llama 32L d4096 32H/8KV FFN 14336 vocab
128256 RoPE theta 5e5, bf16; synthetic Zipf(s=1.1) sequences of 2048 tokens; per-module
projection_dim 16 with an Adafactor normaliser; rows of 224 x 256 values written to an
on-disk store (fp16 rows in our arm; the reference ties the row dtype to the model dtype).
One "step" is one batch of `--seqs` sequences per rank: forward, backward to the
activations, per-example projected gradients of every Linear, row emission.  Data
parallel, one rank per GPU (weak scaling: the per-rank batch is fixed).

Rank 0 prints one JSON line.  `value` is device-timed (CUDA events, inputs already on
the device, max over ranks); `e2e` is the same metric through the public
`CollectorComputer.step` API including the per-step pinned host->device copy of the
inputs and the device->host read of the step's losses and store rows.
"""

from __future__ import annotations

import argparse
import json
import os
import shutil
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

MODEL = dict(model_type="llama", vocab_size=128256, hidden_size=4096, intermediate_size=14336,
             num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, rope_theta=500000.0,
             max_position_embeddings=8192, rms_norm_eps=1e-5)
SMALL = dict(MODEL, hidden_size=1024, intermediate_size=2816, num_hidden_layers=4, num_attention_heads=8,
             num_key_value_heads=4, vocab_size=32000)
METRIC = "grad_store_build_tokens_per_s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--seqs", type=int, default=8, help="sequences per rank per step")
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--small", action="store_true", help="4-layer d1024 stand-in for quick checks (not a bench value)")
    ap.add_argument("--kernel-table", default="", help="after the timed regions, profile one more step of this "
                    "repository's arm with the torch profiler and write rank 0's per-kernel device times to this file")
    ap.add_argument("--extra", default="query,ekfac,magic",
                    help="comma-separated secondary metrics reported under \"extra\" (query, ekfac; empty for none)")
    return ap.parse_args()


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def make_dataset(world: int, per_rank_batches: int, seqs: int, seq_len: int, vocab: int):
    """Global dataset: every rank gets `per_rank_batches` batches of `seqs` full-length rows."""
    from datasets import Dataset

    from bergson_b200.data import zipf_token_ids

    n = world * per_rank_batches * seqs
    ids = zipf_token_ids(n, seq_len, vocab, seed=0)
    return Dataset.from_dict({"input_ids": ids, "length": [seq_len] * n})


def max_over_ranks(x: float, device) -> float:
    import torch
    import torch.distributed as dist

    if not dist.is_initialized():
        return x
    t = torch.tensor([x], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier_sync(device):
    import torch
    import torch.distributed as dist

    if dist.is_initialized():
        dist.barrier()
    torch.cuda.synchronize(device)


def run_ours(args, rank, local_rank, world):
    import torch

    from bergson_b200 import GradientCollector, GradientProcessor, IndexConfig
    from bergson_b200.collector.collector import CollectorComputer
    from bergson_b200.data import allocate_batches
    from bergson_b200.gradients import AdafactorNormalizer
    from bergson_b200.models import build_model
    from bergson_b200.models.registry import args_from_dict
    from bergson_b200.ops import attribution, native

    device = torch.device("cuda", local_rank)
    spec = SMALL if args.small else MODEL
    model = build_model(args_from_dict(spec), dtype=torch.bfloat16, device=device, init_on_device=True)
    model.requires_grad_(False)
    model.get_input_embeddings().requires_grad_(True)

    W, K, B, S = args.warmup, args.steps, args.seqs, args.seq_len
    per_rank = W + 2 * K + (1 if args.kernel_table else 0)  # warm-up, device-timed, end-to-end (+ profiled) steps
    ds = make_dataset(world, per_rank, B, S, spec["vocab_size"])
    batches = allocate_batches(ds["length"], B * S)
    assert len(batches) == per_rank and all(len(b) == B for b in batches), (len(batches), per_rank)

    g = torch.Generator(device=device).manual_seed(1)
    norms = {
        n: AdafactorNormalizer(torch.rand(m.out_features, generator=g, device=device) + 0.5,
                               torch.rand(m.in_features, generator=g, device=device) + 0.5)
        for n, m in model.base_model.named_modules() if isinstance(m, torch.nn.Linear)
    }
    run_dir = Path(tempfile.gettempdir()) / f"bgn_bench_{os.environ.get('MASTER_PORT', 'single')}"
    if rank == 0:
        shutil.rmtree(run_dir, ignore_errors=True)
        shutil.rmtree(str(run_dir) + ".part", ignore_errors=True)
    barrier_sync(device)
    cfg = IndexConfig(run_path=str(run_dir), projection_dim=16, token_batch_size=B * S, store_dtype="fp16")
    cfg.partial_run_path.mkdir(parents=True, exist_ok=True)
    collector = GradientCollector(model=model.base_model, cfg=cfg, data=ds,
                                  processor=GradientProcessor(norms, projection_dim=16))
    assert collector._fused_enabled, "fused projection path is not active"
    computer = CollectorComputer(model=model, data=ds, collector=collector, batches=batches, cfg=cfg)
    row_bytes = sum(collector.grad_sizes.values()) * 2

    from benchmarks.clocks import ClockSampler

    sampler = ClockSampler(local_rank)
    with collector:
        for b in batches[:W]:
            computer.step(b)
        # ---- device-timed: inputs staged on the device beforehand -----------------------
        staged = [(b, *computer.stage(b)) for b in batches[W : W + K]]
        barrier_sync(device)
        if rank == 0:
            sampler.start()
        native.reset_launch_count()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for b, x, y, mask, batch in staged:
            computer.run_staged(b, x, y, mask, batch)
        t1.record()
        barrier_sync(device)
        dev_ms = max_over_ranks(t0.elapsed_time(t1), device)
        launches = native.launch_count()
        del staged
        # ---- end to end through the public API ------------------------------------------
        barrier_sync(device)
        w0 = time.perf_counter()
        loss_sum = 0.0
        for b in batches[W + K : W + 2 * K]:
            losses = computer.step(b)
            loss_sum += float(losses.sum().cpu())  # device -> host read of the step's result
        collector.builder.flush()  # all rows of the timed steps have reached the store
        barrier_sync(device)
        e2e_s = max_over_ranks(time.perf_counter() - w0, device)
        clocks = sampler.stop() if rank == 0 else None
        if args.kernel_table:  # outside every timed region
            from torch.profiler import ProfilerActivity, profile

            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                computer.step(batches[W + 2 * K])
                torch.cuda.synchronize(device)
            if rank == 0:
                with open(args.kernel_table, "w") as f:
                    f.write(prof.key_averages().table(sort_by="cuda_time_total", row_limit=40,
                                                      max_name_column_width=100))
    status = attribution.kernel_status(local_rank)
    assert status == 0, f"kernel status {status}"
    if rank == 0:
        shutil.rmtree(str(run_dir) + ".part", ignore_errors=True)
    tokens = world * K * B * S
    return {
        "value": tokens / (dev_ms / 1e3), "ms_per_step": dev_ms / K, "gpu_launches": launches,
        "e2e": {"value": tokens / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": 2 * B * S * 8 + B * 8,
                "d2h_bytes_per_step": B * row_bytes + 4, "ms_per_step": e2e_s * 1e3 / K},
        "clocks": clocks, "loss_checksum": loss_sum,
        "arm": {"store": "fp16 rows, pinned staging ring -> memmap", "model_impl": "in-tree Llama on the tcgen05 GEMM"},
        "model": "llama-32L-d4096" if not args.small else "small",
    }


class TimedBatches(list):
    """Batch list whose iterator brackets the timed steps: before batch `warmup` it
    synchronises and records the start, after the last batch it records the end.  The
    reference's own collection loop iterates it, so the timed region is its stock path."""

    def configure(self, warmup: int, device):
        self.warmup, self.device = warmup, device
        self.dev_ms = self.wall_s = None

    def __iter__(self):
        import torch

        t0 = t1 = None
        w0 = 0.0
        for i, b in enumerate(list.__iter__(self)):
            if i == self.warmup:
                barrier_sync(self.device)
                t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0.record()
                w0 = time.perf_counter()
            yield b
        if t0 is not None:
            t1.record()
            barrier_sync(self.device)
            self.wall_s = time.perf_counter() - w0
            self.dev_ms = t0.elapsed_time(t1)


def run_reference(args, rank, local_rank, world):
    """The unmodified reference package from baseline/_ref through its public
    `collect_gradients` on a stock HF Llama of the same architecture."""
    ref_dir, shims = ROOT / "baseline" / "_ref", ROOT / "baseline" / "shims"
    if not (ref_dir / "bergson").exists():
        return {"unavailable": "reference not installed under baseline/_ref"}
    sys.path[:0] = [str(shims), str(ref_dir)]
    import torch

    try:
        import bergson
        from bergson.data import allocate_batches
        from bergson.gradients import AdafactorNormalizer
        from transformers import AutoModelForCausalLM, LlamaConfig
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"reference import failed: {type(e).__name__}: {e}"[:300]}

    device = torch.device("cuda", local_rank)
    spec = SMALL if args.small else MODEL
    hf_cfg = LlamaConfig(**{k: v for k, v in spec.items() if k != "model_type"}, attn_implementation="sdpa")
    torch.manual_seed(0)
    with torch.device(device):
        model = AutoModelForCausalLM.from_config(hf_cfg, dtype=torch.bfloat16)
    model.requires_grad_(False)
    model.get_input_embeddings().requires_grad_(True)

    W, K, B, S = args.warmup, args.steps, args.seqs, args.seq_len
    ds = make_dataset(world, W + K, B, S, spec["vocab_size"])
    batches = TimedBatches(allocate_batches(ds["length"], B * S))
    batches.configure(W, device)
    g = torch.Generator(device=device).manual_seed(1)
    norms = {
        n: AdafactorNormalizer(torch.rand(m.out_features, generator=g, device=device) + 0.5,
                               torch.rand(m.in_features, generator=g, device=device) + 0.5)
        for n, m in model.base_model.named_modules() if isinstance(m, torch.nn.Linear)
    }
    run_dir = Path(tempfile.gettempdir()) / f"ref_bench_{os.environ.get('MASTER_PORT', 'single')}"
    if rank == 0:
        shutil.rmtree(str(run_dir) + ".part", ignore_errors=True)
    barrier_sync(device)
    cfg = bergson.IndexConfig(run_path=str(run_dir), projection_dim=16, token_batch_size=B * S)
    cfg.partial_run_path.mkdir(parents=True, exist_ok=True)
    from benchmarks.clocks import ClockSampler

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    bergson.collect_gradients(model, ds, bergson.GradientProcessor(norms, projection_dim=16), cfg, batches=batches)
    clocks = sampler.stop() if rank == 0 else None
    dev_ms = max_over_ranks(batches.dev_ms, device)
    wall_s = max_over_ranks(batches.wall_s, device)
    if rank == 0:
        shutil.rmtree(str(run_dir) + ".part", ignore_errors=True)
    tokens = world * K * B * S
    row_bytes = 224 * 256 * 2 if not args.small else 28 * 256 * 2
    return {
        "value": tokens / (dev_ms / 1e3), "ms_per_step": dev_ms / K, "gpu_launches": None,
        "e2e": {"value": tokens / wall_s, "unit": "tokens/s", "h2d_bytes_per_step": 2 * B * S * 8,
                "d2h_bytes_per_step": B * row_bytes + 4, "ms_per_step": wall_s * 1e3 / K},
        "clocks": clocks, "arm": {"store": "bf16 rows (model dtype)", "model_impl": "transformers LlamaForCausalLM"},
        "model": "llama-32L-d4096" if not args.small else "small",
    }


def main():
    args = parse_args()
    rank, local_rank, world = dist_env()
    import torch

    if not torch.cuda.is_available():
        if rank == 0:
            print(json.dumps({"impl": args.impl, "unavailable": "no CUDA device"}))
        return
    torch.cuda.set_device(local_rank)
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        from datetime import timedelta

        # A short collective timeout: if one rank of a run fails, the others give up in minutes.
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=timedelta(minutes=4))
    res = (run_reference if args.impl == "reference" else run_ours)(args, rank, local_rank, world)
    extras = None
    which = tuple(w for w in args.extra.split(",") if w)
    if which and "unavailable" not in res and not args.small:
        import gc

        gc.collect()
        torch.cuda.empty_cache()
        from benchmarks.extra_metrics import run_extras

        extras = run_extras(args.impl, rank, local_rank, world, which)
    if rank == 0:
        if "unavailable" in res:
            print(json.dumps({"impl": args.impl, "unavailable": res["unavailable"]}))
        else:
            out = {
                "metric": METRIC, "value": res["value"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
                "data": "synthetic Zipf(s=1.1) token ids, random-init weights", "impl": args.impl,
                "config": {"model": res["model"], "global_batch": world * args.seqs, "seq_len": args.seq_len,
                           "parallelism": f"dp{world}", "projection_dim": 16, "normalizer": "adafactor",
                           "store": "16-bit rows on disk",
                           "l2": "inputs larger than L2 (activations of one step exceed 126 MB many times)"},
                "e2e": res["e2e"], "gpu_launches": res["gpu_launches"], "clocks": res["clocks"], "arm": res["arm"],
            }
            if extras is not None:
                out["extra"] = extras
            print(json.dumps(out))
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
