"""Secondary metrics that ``bench.py`` reports under ``"extra"``: query throughput against a
resident store and EK-FAC fit time, each for this repository (``ours``) and for the unmodified
reference package (``reference``), on ``world`` ranks of one node.

Both are strong-scaling measurements (the total work is fixed, ranks share it), timed on the
device with CUDA events after a warm-up, maximum over ranks.

* ``query``: 1024 queries against 65 536 stored rows of 57 344 fp16 values (224 modules x 256),
  cosine scoring, top-100.  Ours: rows sharded over the ranks, per-rank GEMM + top-k, merged
  across ranks.  Reference: its ``Attributor`` holds the whole store on each rank's GPU.
* ``ekfac``: K-FAC covariances, eigendecomposition and eigenvalue correction for a random-init
  GPT-NeoX 12L d768 on 256 sequences x 1024 synthetic tokens (bf16 compute, fp32 factors).
* ``magic``: one meta-step of the twice-differentiable trainer for a random-init GPT-2 12L d768
  (bf16 parameters, AdamW lr 3e-4) on a global batch of 64 sequences x 512 synthetic tokens,
  data-parallel over the ranks: the step replayed with its graph, then the vector-Jacobian
  product that carries cotangents of the new parameters and optimizer state back to the old
  state and to the 64 data weights.  The plain in-place training step is timed as well.
  The reference's trainer imports ``torchopt``, which is not installed; its arm runs with the
  stand-in under ``baseline/shims/torchopt`` (plain tensor operations, no accelerated op).
"""

from __future__ import annotations

import json
import shutil
import tempfile
from pathlib import Path

QUERY_CFG = dict(rows=65536, dim=57344, queries=1024, k=100)
EKFAC_SPEC = dict(model_type="gpt_neox", vocab_size=50304, hidden_size=768, intermediate_size=3072, num_hidden_layers=12,
                  num_attention_heads=12, rotary_pct=0.25, max_position_embeddings=2048)
EKFAC_CFG = dict(docs=256, seq_len=1024, token_batch=16384)
MAGIC_SPEC = dict(vocab_size=50257, n_positions=1024, n_embd=768, n_layer=12, n_head=12)
# Betas, eps, eps_root and weight decay are the reference TrainingConfig's defaults; eps_root > 0
# keeps d sqrt(v) finite for rows that never received a gradient.
MAGIC_CFG = dict(batch=64, seq_len=512, lr=3e-4, betas=(0.95, 0.975), eps=1e-8, eps_root=1e-8, weight_decay=0.01)


def _max_over_ranks(x: float, device) -> float:
    import torch
    import torch.distributed as dist

    if not dist.is_initialized():
        return x
    t = torch.tensor([x], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _sync(device):
    import torch
    import torch.distributed as dist

    if dist.is_initialized():
        dist.barrier()
    torch.cuda.synchronize(device)


def _timed(fn, device, warmup: int = 1, iters: int = 3) -> float:
    """Milliseconds per call: CUDA events around ``iters`` calls, barrier + sync on both sides."""
    import torch

    for _ in range(warmup):
        fn()
    _sync(device)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(iters):
        fn()
    t1.record()
    _sync(device)
    return _max_over_ranks(t0.elapsed_time(t1) / iters, device)


# --------------------------------------------------------------------------- query


def query_ours(rank: int, local_rank: int, world: int) -> dict:
    import torch

    from bergson_b200 import Attributor
    from bergson_b200.hessians.sharded_computation import shard_bounds

    c = QUERY_CFG
    dev = torch.device("cuda", local_rank)
    lo, hi = shard_bounds(c["rows"], rank, world) if world > 1 else (0, c["rows"])
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    rows = torch.randn(hi - lo, c["dim"], device=dev, dtype=torch.float16, generator=g)
    sizes = {f"m{i}": 256 for i in range(c["dim"] // 256)}
    attr = Attributor.from_rows(rows, sizes, unit_norm=True, sharded=world > 1, row_offset=lo, total_rows=c["rows"])
    gq = torch.Generator(device=dev).manual_seed(99)  # the same queries on every rank
    q = torch.randn(c["queries"], c["dim"], device=dev, dtype=torch.float16, generator=gq)
    queries = {n: q[:, i * 256 : (i + 1) * 256] for i, n in enumerate(sizes)}
    ms = _timed(lambda: attr.search(queries, c["k"]), dev)
    return {"metric": "query_scores_per_s", "value": c["rows"] * c["queries"] / (ms / 1e3), "unit": "scores/s",
            "ms_per_search": ms, "higher_is_better": True, "scaling": "strong", "config": dict(c, store="fp16, resident",
                                                                                                 scoring="cosine, top-k")}


def query_reference(rank: int, local_rank: int, world: int) -> dict:
    import numpy as np
    import torch

    from bergson import Attributor
    from bergson.data import create_index
    from bergson.gradients import GradientProcessor

    c = QUERY_CFG
    dev = torch.device("cuda", local_rank)
    base = Path("/dev/shm") if Path("/dev/shm").is_dir() else Path(tempfile.gettempdir())
    # One store shared by all ranks: the reference's create_index is collective (rank 0 creates the
    # file, a barrier, every rank maps it), and its Attributor has no sharding -- each rank loads
    # the whole store onto its own GPU and answers the same queries.
    tmp = base / "ref_query_store"
    if rank == 0:
        shutil.rmtree(tmp, ignore_errors=True)
        tmp.mkdir(parents=True)
    _sync(dev)
    try:
        sizes = {f"m{i}": 256 for i in range(c["dim"] // 256)}
        mm = create_index(tmp, c["rows"], sizes, np.float16)
        if rank == 0:
            g = torch.Generator(device=dev).manual_seed(1234)
            for lo in range(0, c["rows"], 8192):
                n = min(8192, c["rows"] - lo)
                mm[lo : lo + n] = torch.randn(n, c["dim"], device=dev, dtype=torch.float16, generator=g).cpu().numpy()
            mm.flush()
            GradientProcessor(projection_dim=16).save(tmp)
        del mm
        _sync(dev)
        attr = Attributor(tmp, device=str(dev), dtype=torch.float16, unit_norm=True)
        gq = torch.Generator(device=dev).manual_seed(99)
        q = torch.randn(c["queries"], c["dim"], device=dev, dtype=torch.float16, generator=gq)
        queries = {n: q[:, i * 256 : (i + 1) * 256].contiguous() for i, n in enumerate(sizes)}
        ms = _timed(lambda: attr.search(queries, c["k"]), dev)
    finally:
        _sync(dev)
        if rank == 0:
            shutil.rmtree(tmp, ignore_errors=True)
    return {"metric": "query_scores_per_s", "value": c["rows"] * c["queries"] / (ms / 1e3), "unit": "scores/s",
            "ms_per_search": ms, "higher_is_better": True, "scaling": "strong", "config": dict(c, store="fp16, resident",
                                                                                                 scoring="cosine, top-k")}


# --------------------------------------------------------------------------- EK-FAC fit


def _ekfac_data(world: int, vocab: int):
    from datasets import Dataset

    from bergson_b200.data import zipf_token_ids

    c = EKFAC_CFG
    ids = zipf_token_ids(c["docs"], c["seq_len"], vocab, seed=0)
    return Dataset.from_dict({"input_ids": ids, "length": [c["seq_len"]] * c["docs"]})


def _ekfac_run(pkg, model, ds, batches, tmp: Path, dev, rank: int, world: int) -> dict:
    """Covariance pass, eigendecomposition, eigenvalue-correction pass through ``pkg``'s own
    functions; device-timed per phase."""
    import torch

    from_cfg = pkg.config.HessianConfig
    from_h = pkg.hessians
    collect = from_h.hessian_approximations.collect_hessians
    eig = from_h.eigenvectors

    cfg = pkg.IndexConfig(run_path=str(tmp / "run"), token_batch_size=EKFAC_CFG["token_batch"])
    if rank == 0:
        cfg.partial_run_path.mkdir(parents=True, exist_ok=True)
    _sync(dev)
    hcfg = from_cfg(method="kfac", ev_correction=True, use_dataset_labels=True)
    kw = dict(model=model, data=ds, index_cfg=cfg, batches=batches, hessian_cfg=hcfg)
    collect(**{**kw, "batches": batches[:1]})  # warm-up: allocator, kernels, tensor maps

    def phase(fn):
        _sync(dev)
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        fn()
        t1.record()
        _sync(dev)
        return _max_over_ranks(t0.elapsed_time(t1) / 1e3, dev)

    t_cov = phase(lambda: collect(**kw))
    total = torch.load(cfg.partial_run_path / "total_processed.pt", weights_only=False)

    def decompose():
        a = eig.compute_eigendecomposition(str(cfg.partial_run_path / "activation_sharded"), total)
        g = eig.compute_eigendecomposition(str(cfg.partial_run_path / "gradient_sharded"), total)
        eig.save_uncorrected_eigenvalues(cfg.partial_run_path, a, g, total, rank, world)

    t_eig = phase(decompose)
    t_lam = phase(lambda: collect(**kw, ev_correction=True))
    tokens = EKFAC_CFG["docs"] * EKFAC_CFG["seq_len"]
    fit = t_cov + t_eig + t_lam
    return {"metric": "ekfac_fit_s", "value": fit, "unit": "s", "higher_is_better": False, "scaling": "strong",
            "cov_pass_s": t_cov, "eigh_s": t_eig, "lambda_pass_s": t_lam, "tokens": tokens,
            "config": dict(EKFAC_CFG, model="gpt_neox-12L-d768", compute="bf16", factors="fp32")}


def ekfac_ours(rank: int, local_rank: int, world: int) -> dict:
    import torch

    import bergson_b200 as pkg
    import bergson_b200.config  # noqa: F401
    import bergson_b200.hessians.eigenvectors  # noqa: F401
    import bergson_b200.hessians.hessian_approximations  # noqa: F401
    from bergson_b200.data import allocate_batches
    from bergson_b200.models import build_model
    from bergson_b200.models.registry import args_from_dict

    dev = torch.device("cuda", local_rank)
    model = build_model(args_from_dict(EKFAC_SPEC), dtype=torch.bfloat16, device=dev, init_on_device=True)
    model.requires_grad_(False)
    model.get_input_embeddings().requires_grad_(True)
    ds = _ekfac_data(world, EKFAC_SPEC["vocab_size"])
    batches = allocate_batches(ds["length"], EKFAC_CFG["token_batch"])
    tmp = Path(tempfile.gettempdir()) / "bgn_ekfac_bench"
    if rank == 0:
        shutil.rmtree(tmp, ignore_errors=True)
    try:
        return _ekfac_run(pkg, model, ds, batches, tmp, dev, rank, world)
    finally:
        _sync(dev)
        if rank == 0:
            shutil.rmtree(tmp, ignore_errors=True)


def ekfac_reference(rank: int, local_rank: int, world: int) -> dict:
    import torch
    from transformers import AutoModelForCausalLM, GPTNeoXConfig

    import bergson as pkg
    import bergson.config  # noqa: F401
    import bergson.hessians.eigenvectors  # noqa: F401
    import bergson.hessians.hessian_approximations  # noqa: F401
    from bergson.data import allocate_batches

    dev = torch.device("cuda", local_rank)
    s = EKFAC_SPEC
    hf = GPTNeoXConfig(vocab_size=s["vocab_size"], hidden_size=s["hidden_size"], intermediate_size=s["intermediate_size"],
                       num_hidden_layers=s["num_hidden_layers"], num_attention_heads=s["num_attention_heads"],
                       rotary_pct=s["rotary_pct"], max_position_embeddings=s["max_position_embeddings"],
                       attn_implementation="sdpa")
    torch.manual_seed(0)
    with torch.device(dev):
        model = AutoModelForCausalLM.from_config(hf, dtype=torch.bfloat16)
    model.requires_grad_(False)
    model.get_input_embeddings().requires_grad_(True)
    ds = _ekfac_data(world, s["vocab_size"])
    batches = allocate_batches(ds["length"], EKFAC_CFG["token_batch"])
    tmp = Path(tempfile.gettempdir()) / "ref_ekfac_bench"
    if rank == 0:
        shutil.rmtree(tmp, ignore_errors=True)
    try:
        return _ekfac_run(pkg, model, ds, batches, tmp, dev, rank, world)
    finally:
        _sync(dev)
        if rank == 0:
            shutil.rmtree(tmp, ignore_errors=True)


# --------------------------------------------------------------------------- MAGIC


def _magic_data(vocab: int):
    """Four global batches of synthetic Zipf tokens (the same ids for both arms)."""
    import numpy as np
    from datasets import Dataset

    n, length = MAGIC_CFG["batch"] * 4, MAGIC_CFG["seq_len"]
    rng = np.random.default_rng(0)
    ids = np.minimum(rng.zipf(1.1, size=(n, length)), vocab) - 1
    return Dataset.from_dict({"input_ids": ids.tolist(), "length": [length] * n})


def _magic_run(trainer, state, data, dev, world: int) -> dict:
    """Times ``Trainer.step`` in place and a traced step plus its VJP (the same calls for both
    packages: their trainers expose the same interface)."""
    import torch

    holder = {"s": state, "loss": 0.0}

    def train_step():
        holder["s"] = trainer.step(holder["s"], data[0], inplace=True)

    train_ms = _timed(train_step, dev, warmup=2, iters=4)

    def meta_step():
        st = holder["s"]
        st.detach_()
        st.requires_grad = True
        data.requires_grad = True
        before = st.differentiable_tensors()
        after = trainer.step(st, data[1], trace=True).differentiable_tensors()
        cot = [torch.full_like(t, 1e-3) for t in after]
        grads = torch.autograd.grad(after, before + [data.weights], grad_outputs=cot, allow_unused=True)
        holder["loss"] = float(grads[-1].float().abs().sum())  # device -> host read of the weight gradient
        st.requires_grad = False
        data.requires_grad = False

    torch.cuda.reset_peak_memory_stats(dev)
    meta_ms = _timed(meta_step, dev, warmup=1, iters=3)
    tokens = MAGIC_CFG["batch"] * MAGIC_CFG["seq_len"]
    return {"metric": "magic_meta_step_s", "value": meta_ms / 1e3, "unit": "s", "higher_is_better": False,
            "scaling": "strong", "train_step_s": train_ms / 1e3, "meta_over_train": meta_ms / train_ms,
            "meta_tokens_per_s": tokens / (meta_ms / 1e3), "weight_grad_abs_sum": holder["loss"],
            "peak_mem_gb": torch.cuda.max_memory_allocated(dev) / 1e9,
            "config": {"model": "gpt2-12L-d768 random init", "global_batch": MAGIC_CFG["batch"],
                       "seq_len": MAGIC_CFG["seq_len"], "dtype": "bf16", "optimizer": "adamw",
                       "parallelism": f"dp{world}"}}


def magic_ours(rank: int, local_rank: int, world: int) -> dict:
    import torch

    from bergson_b200.magic import optim
    from bergson_b200.magic.data_stream import DataStream
    from bergson_b200.magic.trainer import Trainer
    from bergson_b200.models import build_model
    from bergson_b200.models.registry import PRESETS, args_from_dict

    dev = torch.device("cuda", local_rank)
    s = MAGIC_SPEC
    spec = dict(PRESETS["gpt2"], vocab_size=s["vocab_size"], hidden_size=s["n_embd"], num_hidden_layers=s["n_layer"],
                num_attention_heads=s["n_head"], max_position_embeddings=s["n_positions"])
    model = build_model(args_from_dict(spec), dtype=torch.bfloat16, device=dev, init_on_device=True)
    model.requires_grad_(True)
    model.eval()
    c = MAGIC_CFG
    opt = optim.adamw(lambda step: c["lr"], betas=c["betas"], eps=c["eps"], eps_root=c["eps_root"],
                      weight_decay=c["weight_decay"])
    trainer, state = Trainer.initialize(model, opt)
    data = DataStream(_magic_data(s["vocab_size"]), c["batch"], device=dev)
    return _magic_run(trainer, state, data, dev, world)


def magic_reference(rank: int, local_rank: int, world: int) -> dict:
    from functools import partial

    import torch
    import torchopt
    from transformers import AutoModelForCausalLM, GPT2Config

    from bergson.magic.data_stream import DataStream
    from bergson.magic.trainer import Trainer
    from bergson.utils import weighted_causal_lm_ce

    dev = torch.device("cuda", local_rank)
    s = MAGIC_SPEC
    # What the reference's prepare_trainer builds: eager attention, dropout off in eval mode,
    # the weighted cross-entropy as the model's loss function.
    hf = GPT2Config(vocab_size=s["vocab_size"], n_positions=s["n_positions"], n_embd=s["n_embd"], n_layer=s["n_layer"],
                    n_head=s["n_head"], attn_implementation="eager")
    torch.manual_seed(0)
    with torch.device(dev):
        model = AutoModelForCausalLM.from_config(hf, dtype=torch.bfloat16)
    model.loss_function = partial(weighted_causal_lm_ce, reduction="mean")
    model.requires_grad_(True)
    model.eval()
    c = MAGIC_CFG
    opt = torchopt.adamw(lambda step: c["lr"], betas=c["betas"], eps=c["eps"], eps_root=c["eps_root"],
                         weight_decay=c["weight_decay"])
    trainer, state = Trainer.initialize(model, opt)
    data = DataStream(_magic_data(s["vocab_size"]), c["batch"], device=dev)
    out = _magic_run(trainer, state, data, dev, world)
    out["torchopt"] = getattr(torchopt, "__version__", "?")
    return out


def run_extras(impl: str, rank: int, local_rank: int, world: int, which=("query", "ekfac")) -> dict:
    """``{"query": {...}, "ekfac": {...}}``; a metric that fails reports its error instead of
    taking the headline down with it."""
    table = {"ours": {"query": query_ours, "ekfac": ekfac_ours, "magic": magic_ours},
             "reference": {"query": query_reference, "ekfac": ekfac_reference, "magic": magic_reference}}[impl]
    out = {}
    for name in which:
        try:
            out[name] = table[name](rank, local_rank, world)
        except Exception as e:  # noqa: BLE001 - reported in the JSON line
            import traceback

            out[name] = {"error": f"{type(e).__name__}: {e}"[:300], "where": traceback.format_exc()[-400:]}
        import torch

        torch.cuda.empty_cache()
    return out


if __name__ == "__main__":
    import sys

    sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
    print(json.dumps(run_extras("ours", 0, 0, 1)))
