"""Per-operator times of the EK-FAC covariance pass (torch profiler, CPU and device side).

    python benchmarks/profile_ekfac_cov.py [OUT.txt]

Model and data are those of the ``ekfac`` metric of ``benchmarks/extra_metrics.py`` (GPT-NeoX 12L
d768, 256 x 1024 tokens, token batches of 16384).  Prints the wall time of one full pass
(16 batches, teardown included) and writes two tables for a 4-batch pass (teardown included, so
its share is larger than in the full pass): operators by device time and by host time.
"""
import shutil
import sys
import tempfile
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
import torch
from torch.profiler import ProfilerActivity, profile
from benchmarks import extra_metrics as em
import bergson_b200 as pkg
from bergson_b200.data import allocate_batches
from bergson_b200.models import build_model
from bergson_b200.models.registry import args_from_dict
from bergson_b200.hessians.hessian_approximations import collect_hessians


def main():
    dev = torch.device("cuda", 0)
    model = build_model(args_from_dict(em.EKFAC_SPEC), dtype=torch.bfloat16, device=dev, init_on_device=True)
    model.requires_grad_(False)
    model.get_input_embeddings().requires_grad_(True)
    ds = em._ekfac_data(1, em.EKFAC_SPEC["vocab_size"])
    batches = allocate_batches(ds["length"], em.EKFAC_CFG["token_batch"])
    tmp = Path(tempfile.mkdtemp())
    cfg = pkg.IndexConfig(run_path=str(tmp / "run"), token_batch_size=em.EKFAC_CFG["token_batch"])
    cfg.partial_run_path.mkdir(parents=True, exist_ok=True)
    hcfg = pkg.config.HessianConfig(method="kfac", ev_correction=True, use_dataset_labels=True)
    kw = dict(model=model, data=ds, index_cfg=cfg, hessian_cfg=hcfg)
    collect_hessians(**kw, batches=batches[:1])
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    collect_hessians(**kw, batches=batches)
    torch.cuda.synchronize()
    print("cov pass wall", time.perf_counter() - t0, "batches", len(batches))
    with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
        collect_hessians(**kw, batches=batches[:4])
        torch.cuda.synchronize()
    out = Path(sys.argv[1] if len(sys.argv) > 1 else "ekfac_cov_profile.txt")
    out.parent.mkdir(parents=True, exist_ok=True)
    with open(out, "w") as f:
        f.write(prof.key_averages().table(sort_by="cuda_time_total", row_limit=30, max_name_column_width=70))
        f.write("\n\n")
        f.write(prof.key_averages().table(sort_by="self_cpu_time_total", row_limit=25, max_name_column_width=70))
    shutil.rmtree(tmp, ignore_errors=True)


if __name__ == "__main__":
    main()
