"""Apply a factored inverse Hessian to a stored gradient set (IVHP) and write the result
as an fp32 store (reference ``bergson/hessians/apply_hessian.py``)."""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from pathlib import Path
from typing import Literal

import numpy as np
import torch
import torch.distributed as dist

from ..collector.collector import create_projection_matrix
from ..config import InversionConfig
from ..config.parsing import Serializable
from ..data import column_offsets, create_index, load_gradients
from ..distributed import init_dist
from ..utils.logger import get_logger
from ..utils.utils import get_device, numpy_to_tensor
from .preconditioner import DiagonalFactoredPreconditioner, FactoredPreconditioner


@dataclass
class EkfacConfig(Serializable):
    hessian_method_path: str = ""
    """Directory holding the factor shards."""
    gradient_path: str = ""
    """Store with the gradients to transform."""
    run_path: str = ""
    """Output store."""
    ev_correction: bool = False
    """Use the EK-FAC corrected eigenvalues."""
    apply_batch_size: int = 32
    """Gradients moved to the device and transformed at a time."""
    projection_dim: int = 0
    """If > 0, compress every module's output to ``[p, p]``: ``P_out (H^-1 G) P_in^T``."""
    projection_type: Literal["normal", "rademacher"] = "rademacher"
    projection_scale: Literal["jl", "row_norm"] = "jl"
    preconditioner_path: str = ""
    """Safetensors of per-module ``[out, in]`` optimizer preconditioner grids."""
    debug: bool = False


class EkfacApplicator:
    """``inversion_cfg`` selects a standard inversion, ``apply_fn`` a custom eigenvalue
    function; both only together with ``preconditioner_path`` (elementwise multiplier
    first, then the EK-FAC inverse)."""

    def __init__(self, cfg: EkfacConfig, inversion_cfg: InversionConfig | None = None, apply_fn=None):
        if inversion_cfg is not None and apply_fn is not None and not cfg.preconditioner_path:
            raise ValueError("Pass either inversion_cfg or apply_fn, not both.")
        if cfg.projection_dim > 0 and cfg.ev_correction:
            raise ValueError("projection_dim compression is not supported with EK-FAC (ev_correction=True); "
                             "set ev_correction=False or projection_dim=0.")
        self.cfg, self.inversion_cfg, self.apply_fn = cfg, inversion_cfg, apply_fn
        self.path, self.gradient_path = cfg.hessian_method_path, cfg.gradient_path
        self.logger = get_logger("EkfacApplicator", level="DEBUG" if cfg.debug else "INFO")
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world_size = dist.get_world_size() if dist.is_initialized() else 1
        self.device = get_device(self.rank)

    def _preconditioners(self):
        cfg = self.cfg
        common = dict(rank=self.rank, device=self.device, ev_correction=cfg.ev_correction)
        if cfg.preconditioner_path:
            if self.apply_fn is None:
                raise ValueError("preconditioner_path requires apply_fn.")
            diag = DiagonalFactoredPreconditioner.from_shards(self.path, cfg.preconditioner_path,
                                                              apply_fn=self.apply_fn, **common)
            if self.inversion_cfg is None:
                return [], diag
            return [diag], FactoredPreconditioner.from_shards(self.path, inversion_cfg=self.inversion_cfg, **common)
        return [], FactoredPreconditioner.from_shards(
            self.path, inversion_cfg=None if self.apply_fn is not None else self.inversion_cfg,
            apply_fn=self.apply_fn, **common)

    def compute_ivhp_sharded(self):
        chain, pre = self._preconditioners()
        o_dims = {n: pre.eigen_g[n].shape[1] for n in pre.eigen_a}
        i_dims = {n: pre.eigen_a[n].shape[1] for n in pre.eigen_a}
        p = self.cfg.projection_dim
        sizes = {n: p * p if p > 0 else o_dims[n] * i_dims[n] for n in pre.eigen_a}
        mm = load_gradients(self.gradient_path)
        with open(os.path.join(self.gradient_path, "info.json")) as f:
            in_off = column_offsets(json.load(f)["grad_sizes"])
        n_q = mm.shape[0]
        out = create_index(Path(self.cfg.run_path), num_grads=n_q, grad_sizes=sizes, dtype=np.float32)
        out_off = column_offsets(sizes)
        self.logger.info(f"Loaded gradients for {n_q} queries and computing IVHP...")
        for lo in range(0, n_q, self.cfg.apply_batch_size):
            hi = min(lo + self.cfg.apply_batch_size, n_q)
            grads = {
                n: numpy_to_tensor(np.ascontiguousarray(mm[lo:hi, in_off[n][0] : in_off[n][1]])).to(self.device, torch.float32)
                for n in pre.eigen_a
            }
            for c in chain:
                grads = c.apply(grads)
            res = pre.apply(grads)
            if p > 0:
                for n, flat in res.items():
                    if n not in o_dims:
                        continue
                    g = flat.view(-1, o_dims[n], i_dims[n])
                    L = create_projection_matrix(f"{n}/left", p, o_dims[n], g.dtype, g.device,
                                                 self.cfg.projection_type, self.cfg.projection_scale)
                    R = create_projection_matrix(f"{n}/right", p, i_dims[n], g.dtype, g.device,
                                                 self.cfg.projection_type, self.cfg.projection_scale)
                    res[n] = L @ g @ R.T
            if self.rank == 0:  # every rank holds the full result; one writer is enough
                for n, t in res.items():
                    a, b = out_off[n]
                    out[lo:hi, a:b] = t.flatten(1).cpu().numpy()
        out.flush()
        if dist.is_initialized():
            dist.barrier()
        self.logger.info(f"Saved IVHP gradients to {self.cfg.run_path}")


def apply_worker(rank: int, local_rank: int, world_size: int, cfg: EkfacConfig, inversion_cfg: InversionConfig):
    init_dist(rank, local_rank, world_size)
    EkfacApplicator(cfg, inversion_cfg=inversion_cfg).compute_ivhp_sharded()
