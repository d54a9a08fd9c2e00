"""One tiny forward + backward of the flagship path (gradient-store build with the fused
projection kernels) on a CUDA device, checked against the torch path."""

from __future__ import annotations

import tempfile
from pathlib import Path

import numpy as np
import torch


def run_smoke(device: torch.device) -> None:
    from . import GradientProcessor, IndexConfig, collect_gradients, load_gradients
    from .data import allocate_batches, synthetic_dataset
    from .gradients import AdafactorNormalizer
    from .models import build_model
    from .models.registry import PRESETS, args_from_dict
    from .ops import attribution, native

    args = args_from_dict(dict(PRESETS["llama-tiny"], hidden_size=128, intermediate_size=256, vocab_size=1024))
    model = build_model(args, dtype=torch.bfloat16, device=device)
    model.requires_grad_(False)
    model.get_input_embeddings().requires_grad_(True)
    ds = synthetic_dataset("synthetic:zipf?n=12&len=160&vocab=1024&seed=0&min_len=90")
    batches = allocate_batches(ds["length"], 640)
    g = torch.Generator().manual_seed(0)
    norms = {
        n: AdafactorNormalizer((torch.rand(m.out_features, generator=g) + 0.5).to(device),
                               (torch.rand(m.in_features, generator=g) + 0.5).to(device))
        for n, m in model.base_model.named_modules() if isinstance(m, torch.nn.Linear)
    }
    stores = {}
    with tempfile.TemporaryDirectory() as tmp:
        for fused in (True, False):
            cfg = IndexConfig(run_path=str(Path(tmp) / f"fused_{fused}"), projection_dim=16, token_batch_size=640,
                              store_dtype="fp32", fused_collection=fused)
            cfg.partial_run_path.mkdir(parents=True)
            native.reset_launch_count()
            collect_gradients(model, ds, GradientProcessor(norms, projection_dim=16), cfg, batches=batches)
            torch.cuda.synchronize(device)
            stores[fused] = np.array(load_gradients(cfg.partial_run_path))
            if fused:
                launches = native.launch_count()
    assert attribution.kernel_status(device.index or 0) == 0, "a kernel gave up on a bounded wait"
    a, b = stores[True], stores[False]
    scale = np.abs(b).max()
    err = np.abs(a - b).max() / scale
    assert np.isfinite(a).all() and scale > 0, "store is empty or not finite"
    assert err < 3e-2, f"fused store deviates from the torch path: rel err {err:.3e}"
    print(f"smoke ok: store {a.shape}, fused-vs-torch max rel err {err:.2e}, {launches} kernel launches")
