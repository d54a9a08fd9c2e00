"""Functional, twice-differentiable trainer (MAGIC).

``Trainer`` is stateless; everything that changes lives in ``TrainerState`` (parameter
dict, optimizer-state pytree, buffers, batch index, CPU and CUDA RNG states).  ``step``
computes (micro-batched) gradients of the weighted loss, synchronises them
(differentiable all-reduce, or reduce-scatter under parameter sharding), clips, and
applies a functional optimizer update.  ``train`` checkpoints the state *before* the steps
chosen by ``save_mode``; ``backward`` sweeps the trajectory in reverse, re-materialising
states from checkpoints and pulling ``(d/dparams, d/dopt_state, d/dweights)`` through
each traced step (reference ``bergson/magic/trainer.py:80-1099``).

Model ops run on the any-order-differentiable path (``ops.composable``) whenever a graph
through the step is required.
"""

from __future__ import annotations

import json
import math
import os
import threading
import time
from collections.abc import Callable
from contextlib import contextmanager, nullcontext
from dataclasses import dataclass, field
from pathlib import Path
from shutil import rmtree
from typing import Any

import psutil
import torch
import torch.distributed as dist
from torch import nn
from torch.func import functional_call
from tqdm.auto import tqdm

from .. import ops
from ..config.config import SaveMode, TrainingConfig
from ..data import sorted_checkpoints
from ..utils.utils import get_device
from ..utils.worker_utils import setup_model_and_peft
from . import optim
from .collectives import all_reduce_sum
from .data_stream import DataStream
from .fsdp import LazyGather, gather_params, simple_fsdp
from .grad_accum import (
    accumulate_grads,
    maybe_get_cuda_rng_state,
    maybe_set_cuda_rng_state,
    microbatch_step_vjp,
    rng_restore,
    rng_snapshot,
)
from .optim import GradientTransformation, OptState, tree_flatten_with_path, tree_iter, tree_map
from .rtl_tqdm import RtlTqdm

LR_HISTORY_FILENAME = "log_history.json"


def write_lr_history(save_dir, schedule: Callable[[int], float], num_steps: int) -> Path:
    """Per-step learning rates as ``[{"step", "learning_rate"}]`` beside the checkpoints."""
    save_dir = Path(save_dir)
    save_dir.mkdir(parents=True, exist_ok=True)
    path = save_dir / LR_HISTORY_FILENAME
    with open(path, "w") as f:
        json.dump([{"step": s, "learning_rate": float(schedule(s))} for s in range(num_steps)], f)
    return path


def next_save_index(current: int, n: int, save_mode: SaveMode, save_interval: int = 0) -> int:
    """The checkpoint index after ``current`` in a run of ``n`` steps (always > current).

    ``all``: every step; ``interval``: every ``save_interval``; ``sqrt``: every
    ``isqrt(n)`` steps, then every step inside the last chunk; ``log``: halve the remainder.
    """
    if save_mode == "all":
        return current + 1
    if save_mode == "interval":
        if save_interval <= 0:
            raise ValueError("save_mode='interval' requires save_interval > 0.")
        return current + save_interval
    if save_mode == "sqrt":
        chunk = math.isqrt(n)
        return current + 1 if current >= n - chunk else current + chunk
    if save_mode == "log":
        return max(1, (n - current) // 2) + current
    raise ValueError(f"Unsupported save mode: {save_mode}")


class SaveFuture:
    """Handle of a checkpoint being written by a background thread."""

    def __init__(self, thread: threading.Thread | None, box: dict, name: str = ""):
        self.thread, self.box, self.name = thread, box, name

    def result(self):
        if self.thread is not None:
            self.thread.join()
            self.thread = None
        if "error" in self.box:
            raise self.box["error"]
        return self.box.get("value")


@dataclass
class BackwardState:
    param_grads: dict[str, torch.Tensor]
    opt_grads: list[torch.Tensor]
    """Cotangents of the floating-point optimizer-state leaves, in flatten order."""
    weight_grads: torch.Tensor


@dataclass
class TrainerState:
    params: dict[str, torch.Tensor]
    opt_state: OptState
    buffers: dict[str, torch.Tensor]
    batch_index: int = 0
    cuda_rng_state: torch.Tensor = field(default_factory=maybe_get_cuda_rng_state)
    cpu_rng_state: torch.Tensor = field(default_factory=torch.random.get_rng_state)

    def copy_(self, other: "TrainerState"):
        for k in self.params:
            self.params[k].copy_(other.params[k])
        for k in self.buffers:
            self.buffers[k].copy_(other.buffers[k])

        def leaf(dst, src):
            if isinstance(dst, torch.Tensor):
                dst.copy_(src)
                return dst
            return src

        self.opt_state = tree_map(leaf, self.opt_state, other.opt_state)
        self.batch_index = other.batch_index
        self.cuda_rng_state.copy_(other.cuda_rng_state)
        self.cpu_rng_state.copy_(other.cpu_rng_state)

    def to(self, device) -> "TrainerState":
        """Snapshot on ``device`` (always a copy, so later in-place steps cannot touch it)."""
        mv = lambda t: t.to(device, copy=True) if isinstance(t, torch.Tensor) else t  # noqa: E731

        def mv_opt(t):
            # Integer leaves (the step count) stay on the host: the schedule and the bias
            # correction read them every step, and a device copy would cost a sync each time.
            if isinstance(t, torch.Tensor) and not t.is_floating_point():
                return t.to("cpu", copy=True)
            return mv(t)

        return TrainerState({k: mv(p) for k, p in self.params.items()}, tree_map(mv_opt, self.opt_state),
                            {k: mv(b) for k, b in self.buffers.items()}, self.batch_index,
                            self.cuda_rng_state.clone(), self.cpu_rng_state.clone())

    @contextmanager
    def activate(self, model: nn.Module):
        """Run ``model`` with this state's parameters and buffers in place of its own and with
        this state's random-number streams; yields the tensors acting as parameters (their
        autograd history intact, so gradients taken inside reach the state).  The model's own
        parameters and the ambient random state come back on exit
        (reference ``bergson/magic/trainer.py:302-310``)."""
        from .swap import swap_parameters

        ambient = rng_snapshot()
        rng_restore((self.cpu_rng_state, self.cuda_rng_state))
        try:
            with swap_parameters(model, self.params, self.buffers, strict=True) as active:
                yield active
        finally:
            rng_restore(ambient)

    def state_dict(self) -> dict:
        """Flat dict: parameter and buffer names, ``.batch_index``, ``.cuda_rng_state``,
        ``.cpu_rng_state`` and ``opt_state/<path>`` leaves."""
        state = {**self.params, **self.buffers, ".batch_index": torch.tensor(self.batch_index),
                 ".cuda_rng_state": self.cuda_rng_state, ".cpu_rng_state": self.cpu_rng_state}
        for path, leaf in tree_flatten_with_path(self.opt_state):
            state["opt_state/" + ".".join(map(str, path))] = leaf
        return state

    def _rank_file(self, path: str) -> str:
        rank = dist.get_rank() if dist.is_initialized() else 0
        return os.path.join(path, f"__{rank}_0.pt")

    def save(self, path: str, debug_pbar=None) -> SaveFuture:
        """Write ``<path>/`` asynchronously: one tensor file per rank, then ``.metadata``
        (written last by rank 0's writer; a checkpoint without it is incomplete)."""
        os.makedirs(path, exist_ok=True)
        snap = {k: (v.detach().to("cpu", copy=True) if isinstance(v, torch.Tensor) else v)
                for k, v in self.state_dict().items()}
        rank = dist.get_rank() if dist.is_initialized() else 0
        world = dist.get_world_size() if dist.is_initialized() else 1
        target = self._rank_file(path)
        box: dict = {}

        def write():
            try:
                tmp = target + ".tmp"
                torch.save(snap, tmp)
                os.replace(tmp, target)
                if rank == 0:
                    deadline = time.monotonic() + 600
                    while time.monotonic() < deadline:
                        if all(os.path.exists(os.path.join(path, f"__{r}_0.pt")) for r in range(world)):
                            break
                        time.sleep(0.01)
                    with open(os.path.join(path, ".metadata"), "w") as f:
                        json.dump({"world_size": world, "keys": sorted(snap)}, f)
            except BaseException as e:  # noqa: BLE001
                box["error"] = e

        t = threading.Thread(target=write, daemon=True)
        t.start()
        return SaveFuture(t, box, name=path if debug_pbar is not None else "")

    def load(self, path: str):
        """Load this rank's tensors from a checkpoint directory (in place)."""
        deadline = time.monotonic() + 600
        while not os.path.exists(os.path.join(path, ".metadata")) and time.monotonic() < deadline:
            time.sleep(0.01)
        saved = torch.load(self._rank_file(path), map_location="cpu", weights_only=True)
        for k, v in self.state_dict().items():
            if k == ".batch_index":
                self.batch_index = int(saved[k])
            elif isinstance(v, torch.Tensor):
                v.data.copy_(saved[k])

    def detach_(self) -> "TrainerState":
        self.params = {k: p.detach() for k, p in self.params.items()}
        self.opt_state = tree_map(
            lambda t: t.detach() if isinstance(t, torch.Tensor) and t.is_floating_point() else t, self.opt_state)
        return self

    @property
    def requires_grad(self) -> bool:
        return any(t.requires_grad for t in self.differentiable_tensors())

    @requires_grad.setter
    def requires_grad(self, value: bool):
        for t in self.differentiable_tensors():
            t.requires_grad = value

    def differentiable_tensors(self) -> list[torch.Tensor]:
        opt = [t for t in tree_iter(self.opt_state) if isinstance(t, torch.Tensor) and t.is_floating_point()]
        return list(self.params.values()) + opt

    def size_in_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.state_dict().values() if isinstance(t, torch.Tensor))


class Trainer:
    """Stateless trainer for ``model`` and a functional ``optimizer``."""

    @classmethod
    def initialize(cls, model: nn.Module, optimizer: GradientTransformation, *, fsdp: bool = False):
        """Returns ``(trainer, initial_state)``.  Only trainable parameters enter the state;
        frozen ones stay in the module.  With ``fsdp`` every parameter is stored as this
        rank's row block."""
        params = {k: v.detach().clone() for k, v in model.named_parameters() if v.requires_grad}
        buffers = {k: v.detach().clone() for k, v in model.named_buffers()}
        shapes = None
        if fsdp and dist.is_initialized():
            params, shapes = simple_fsdp(params)
        state = TrainerState(params, optimizer.init(params), buffers)
        return cls(model, optimizer, param_shapes=shapes), state

    def __init__(self, model: nn.Module, optimizer: GradientTransformation, *, param_shapes=None):
        self.model = model
        self.optimizer = optimizer
        self.param_shapes = param_shapes  # full shapes when parameters are sharded
        self.lazy_gather = os.environ.get("BERGSON_B200_FSDP_GATHER", "module") != "all"
        self.gather_count = 0
        self._last_loss = 0.0

    # -- forward --------------------------------------------------------------------------

    def call_model(self, params: dict, inputs: dict, buffers: dict | None = None):
        if self.param_shapes is not None and self.lazy_gather:
            # Sharded parameters are gathered around each owning module's forward (and again when
            # the backward pass needs them), never all at once.
            with LazyGather(self.model, params, self.param_shapes) as lazy:
                out = functional_call(self.model, dict(buffers or {}), args=(), kwargs=inputs)
            self.gather_count += lazy.gathers
            return out
        full = gather_params(params, self.param_shapes) if self.param_shapes is not None else params
        return functional_call(self.model, {**full, **(buffers or {})}, args=(), kwargs=inputs)

    @staticmethod
    def _loss_scale(fsdp: bool) -> float:
        """Sharded parameters sum gradients over ranks; the mean comes from the loss."""
        return 1.0 / dist.get_world_size() if fsdp and dist.is_initialized() else 1.0

    def _ops_mode(self, trace: bool):
        # Kernels of the fused path implement first-order backward only.
        return ops.composable() if trace else nullcontext()

    # -- one step -------------------------------------------------------------------------

    def step(self, state: TrainerState, inputs: dict[str, Any], *, inplace: bool = False, trace: bool = False,
             fsdp: bool = False, max_grad_norm: float | None = None, grad_accum_steps: int = 1) -> TrainerState:
        """One optimizer step from ``state`` on ``inputs``; ``trace`` keeps the autograd
        graph from the incoming state (and the data weights) to the returned state."""
        rng_restore((state.cpu_rng_state, state.cuda_rng_state))
        params = state.params if trace else {k: v.detach().requires_grad_(True) for k, v in state.params.items()}
        call = lambda p, mb: self.call_model(p, mb, state.buffers)  # noqa: E731
        with self._ops_mode(trace):
            grads, self._last_loss = accumulate_grads(call, params, inputs, grad_accum_steps, create_graph=trace,
                                                      loss_scale=self._loss_scale(fsdp))
        return self._apply_update(state, grads, inplace=inplace, trace=trace, fsdp=fsdp, max_grad_norm=max_grad_norm)

    def _apply_update(self, state: TrainerState, grads: dict, *, inplace: bool = False, trace: bool = False,
                      fsdp: bool = False, max_grad_norm: float | None = None) -> TrainerState:
        """Synchronise, clip and apply ``grads``."""
        grads = {k: g for k, g in grads.items() if g is not None}
        if dist.is_initialized() and not fsdp:
            world = dist.get_world_size()
            if trace:
                grads = {k: all_reduce_sum(g / world) for k, g in grads.items()}
            else:
                for g in grads.values():
                    dist.all_reduce(g, op=dist.ReduceOp.AVG)
        coef = None
        fused_step = inplace and not trace and self.optimizer.step_inplace is not None
        if max_grad_norm and fused_step:
            # One multi-tensor reduction; the coefficient is applied inside the optimizer kernel.
            reduce = _all_reduce_ if fsdp and dist.is_initialized() else None
            coef = optim.global_norm_coef(list(grads.values()), max_grad_norm, reduce=reduce)
        if fused_step and (coef is not None or not max_grad_norm):
            stepped = self.optimizer.step_inplace(grads, state.opt_state, state.params, coef)
            if stepped is not None:
                return TrainerState(stepped[0], stepped[1], state.buffers, state.batch_index + 1)
        if max_grad_norm and coef is not None:
            torch._foreach_mul_(list(grads.values()), coef.to(next(iter(grads.values())).dtype))
        elif max_grad_norm:
            sq = sum(g.float().pow(2).sum() for g in grads.values())
            if fsdp and dist.is_initialized():
                sq = all_reduce_sum(sq) if trace else _all_reduce_(sq)
            coef = (max_grad_norm / (sq.sqrt() + 1e-6)).clamp(max=1.0)
            if trace:
                grads = {k: g * coef.to(g.dtype) for k, g in grads.items()}
            else:
                for g in grads.values():
                    g.mul_(coef.to(g.dtype))
        if not inplace and self.optimizer.step_traced is not None:
            stepped = self.optimizer.step_traced(grads, state.opt_state, state.params)
            if stepped is not None:
                return TrainerState(stepped[0], stepped[1], state.buffers, state.batch_index + 1)
        updates, new_opt = self.optimizer.update(grads, state.opt_state, params=state.params, inplace=inplace)
        new_params = optim.apply_updates(state.params, updates, inplace=inplace)
        return TrainerState(new_params, new_opt, state.buffers, state.batch_index + 1)

    def metagrad_step(self, fwd_state: TrainerState, inputs: dict, bwd_state: BackwardState,
                      data_weights: torch.Tensor, *, fsdp: bool = False, max_grad_norm: float | None = None,
                      grad_accum_steps: int = 1, double_backward_batch_size: int | None = None) -> BackwardState:
        """Micro-batched VJP through one step (peak memory of one micro-batch)."""
        call = lambda p, mb: self.call_model(p, mb, fwd_state.buffers)  # noqa: E731
        with ops.composable():
            pg, og, wc = microbatch_step_vjp(
                call, self._apply_update, fwd_state, inputs, bwd_state.param_grads, bwd_state.opt_grads, data_weights,
                model_training=self.model.training, loss_scale=self._loss_scale(fsdp), fsdp=fsdp,
                max_grad_norm=max_grad_norm,
                grad_accum_steps=grad_accum_steps, double_backward_batch_size=double_backward_batch_size)
        return BackwardState(pg, og, wc + bwd_state.weight_grads)

    # -- training loop ----------------------------------------------------------------------

    def resume(self, state: TrainerState, save_dir: str) -> TrainerState:
        """Load the newest complete checkpoint; incomplete ones (no ``.metadata``) are removed."""
        valid = []
        for idx, path in sorted_checkpoints(save_dir):
            if os.path.exists(os.path.join(path, ".metadata")):
                valid.append((idx, path))
            elif not dist.is_initialized() or dist.get_rank() == 0:
                rmtree(path) if os.path.isdir(path) else os.remove(path)
        if valid:
            idx, path = valid[-1]
            state.load(path)
            state.batch_index = idx
            state.detach_()
        return state

    def _save_checkpoint(self, state: TrainerState, save_dir: str, i: int, optimizer_cfg: dict | None, pbar=None):
        p = os.path.join(save_dir, f"step_{i}.ckpt")
        if optimizer_cfg is not None:
            from ..utils.load_from_optimizer import save_second_moments_as_optimizer_pt

            os.makedirs(p, exist_ok=True)
            save_second_moments_as_optimizer_pt(self.model, state.opt_state, os.path.join(p, "optimizer.pt"), step=i,
                                                **optimizer_cfg)
        return state.save(p, debug_pbar=pbar)

    def train(self, state: TrainerState, data: DataStream, *, debug: bool = False, inplace: bool = False,
              save_dir: str | None = None, save_mode: SaveMode = "sqrt", trace: bool = False,
              log_fn: Callable[[int, float], None] | None = None, resume: bool = False, fsdp: bool = False,
              max_grad_norm: float | None = None, grad_accum_steps: int = 1, optimizer_cfg: dict | None = None,
              save_interval: int = 0) -> TrainerState:
        """Run every batch of ``data``; the state *before* step i is checkpointed when i is
        on the ``save_mode`` schedule (at most one write in flight)."""
        if save_dir is not None:
            os.makedirs(save_dir, exist_ok=True)
        n, next_save, start = len(data), 0, 0
        if resume and save_dir is not None:
            state = self.resume(state, save_dir)
            start = state.batch_index
            while next_save < start:
                next_save = next_save_index(next_save, n, save_mode, save_interval)
        pending: SaveFuture | None = None
        main = not dist.is_initialized() or dist.get_rank() == 0
        pbar = tqdm(range(start, n), desc="Training", disable=not main)
        try:
            for i in pbar:
                if save_dir and i == next_save:
                    if pending is not None:
                        pending.result()
                    pending = self._save_checkpoint(state, save_dir, i, optimizer_cfg, pbar if debug else None)
                    next_save = next_save_index(next_save, n, save_mode, save_interval)
                state = self.step(state, data[i], inplace=inplace, trace=trace, fsdp=fsdp,
                                  max_grad_norm=max_grad_norm, grad_accum_steps=grad_accum_steps)
                state.cpu_rng_state, state.cuda_rng_state = rng_snapshot()
                if log_fn is not None:
                    log_fn(i, self._last_loss)
        except BaseException:
            if pending is not None:
                try:
                    pending.result()
                except Exception:  # noqa: BLE001 - the original error matters more
                    pass
            raise
        if pending is not None:
            pending.result()
        if save_dir and save_mode == "interval" and next_save == n:
            self._save_checkpoint(state, save_dir, n, optimizer_cfg).result()
        return state


def _all_reduce_(t: torch.Tensor) -> torch.Tensor:
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return t


def _save_backward_state(bwd: BackwardState, path: str, expected_idx: int, last_idx: int) -> None:
    tmp = path + ".tmp"
    torch.save({"expected_idx": expected_idx, "last_idx": last_idx, "param_grads": bwd.param_grads,
                "opt_grads": bwd.opt_grads, "weight_grads": bwd.weight_grads}, tmp)
    os.replace(tmp, path)


def _load_backward_state(path: str, ckpt_list, device, main: bool):
    saved = torch.load(path, map_location=device, weights_only=True)
    bwd = BackwardState(saved["param_grads"], saved["opt_grads"], saved["weight_grads"])
    expected, last = saved["expected_idx"], saved["last_idx"]
    valid = []
    for idx, p in ckpt_list:
        if idx > expected:
            continue
        if os.path.exists(os.path.join(p, ".metadata")):
            valid.append((idx, p))
        elif os.path.isdir(p) and main:
            rmtree(p)
    if not valid and expected >= 0:
        raise RuntimeError(f"Cannot resume backward: no valid checkpoints found for step {expected}")
    if main:
        print(f"Resuming backward pass from step {expected}")
    return bwd, valid, expected, last


def _backward(self: Trainer, ckpt_dir: str, data: DataStream, bwd_state: BackwardState, fwd_state: TrainerState, *,
              cleanup: bool = True, debug: bool = False, inplace: bool = False, fsdp: bool = False,
              resume: bool = False, save_every: int = 0, save_mode: SaveMode = "sqrt",
              max_grad_norm: float | None = None, grad_accum_steps: int = 1,
              double_backward_batch_size: int | None = None) -> BackwardState:
    """Reverse sweep over the trajectory stored in ``ckpt_dir``.

    For the step expected next, the newest checkpoint at or before it is loaded and the
    missing steps are replayed untraced (stashing intermediate states in host RAM when it
    fits, else on disk); then that step is re-run traced and the cotangents of the next
    state are pulled back to the current state and to the data weights.
    """
    ckpts = sorted_checkpoints(ckpt_dir)
    paths = [p for _, p in ckpts]
    preserve = {paths[-1]} if cleanup else set(paths)
    ckpt_list: list[tuple[int, Any]] = list(ckpts)
    state_size = fwd_state.size_in_bytes()
    main = not dist.is_initialized() or dist.get_rank() == 0
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    bwd_path = os.path.join(ckpt_dir, f"backward_rank{rank}.pt")

    if resume and os.path.exists(bwd_path):
        bwd_state, ckpt_list, expected, last = _load_backward_state(bwd_path, ckpt_list, data.device, main)
    else:
        expected, _ = ckpt_list[-1]
        last = expected
    bar = RtlTqdm(desc="Backward", total=last + 1, initial=last - expected, disable=not main, smoothing=0)
    futures: list[SaveFuture] = []

    def follow(idx: int, target: int) -> int:
        return (target - idx) // 2 + idx if save_mode == "log" else min(target, idx + 1)

    while ckpt_list:
        for f in futures:
            f.result()
        futures.clear()
        idx, ckpt = ckpt_list[-1]
        fwd_state.detach_()
        t0 = time.monotonic()
        fwd_state.load(ckpt) if isinstance(ckpt, str) else fwd_state.copy_(ckpt)
        fwd_state.batch_index = idx
        if dist.is_initialized() and isinstance(ckpt, str):
            dist.barrier()  # every rank has read its file before rank 0 may delete the directory
        if debug and main:
            bar.write(f"Loaded checkpoint {ckpt if isinstance(ckpt, str) else idx} in {time.monotonic() - t0:.2f}s")
        if idx == expected:
            del ckpt_list[-1]
            if isinstance(ckpt, str) and main and ckpt not in preserve:
                rmtree(ckpt) if os.path.isdir(ckpt) else os.remove(ckpt)

        nxt = follow(idx, expected)
        while idx < expected:
            fwd_state = self.step(fwd_state, data[fwd_state.batch_index], inplace=inplace, trace=False, fsdp=fsdp,
                                  max_grad_norm=max_grad_norm, grad_accum_steps=grad_accum_steps)
            idx += 1
            if idx == nxt and idx < expected:
                if psutil.virtual_memory().available > world * state_size:
                    ckpt_list.append((idx, fwd_state.to("cpu").detach_()))
                else:
                    p = os.path.join(ckpt_dir, f"step_{idx}.ckpt")
                    ckpt_list.append((idx, p))
                    futures.append(fwd_state.save(p))
                nxt = follow(idx, expected)
        expected = idx - 1

        fwd_state.detach_()
        fwd_state.requires_grad = True
        data.requires_grad = True
        batch = data[fwd_state.batch_index]
        if grad_accum_steps > 1:
            bwd_state = self.metagrad_step(fwd_state, batch, bwd_state, data.weights, fsdp=fsdp,
                                           max_grad_norm=max_grad_norm, grad_accum_steps=grad_accum_steps,
                                           double_backward_batch_size=double_backward_batch_size)
        else:
            flat_i = fwd_state.differentiable_tensors()
            state_f = self.step(fwd_state, batch, trace=True, fsdp=fsdp, max_grad_norm=max_grad_norm)
            flat_f = state_f.differentiable_tensors()
            keys = list(bwd_state.param_grads)
            cot = list(bwd_state.param_grads.values()) + bwd_state.opt_grads
            w_prev = bwd_state.weight_grads
            del bwd_state
            res = list(torch.autograd.grad(flat_f, flat_i + [data.weights], grad_outputs=cot, allow_unused=True))
            res = [r if r is not None else torch.zeros_like(t) for r, t in zip(res, flat_i + [data.weights])]
            w_step = res[-1]
            if dist.is_initialized() and not fsdp:
                # The averaged gradient contains each document with weight 1/world.
                w_step = w_step / world
            bwd_state = BackwardState({k: res[i] for i, k in enumerate(keys)}, res[len(keys) : -1], w_step + w_prev)
            del state_f, flat_f
        bar.update()
        if save_every > 0 and (last - expected) % save_every == 0:
            _save_backward_state(bwd_state, bwd_path, expected, last)

    for f in futures:
        f.result()
    if os.path.exists(bwd_path):
        os.remove(bwd_path)
    bar.close()
    return bwd_state


Trainer.backward = _backward  # type: ignore[attr-defined]
Trainer.save_backward_state = staticmethod(_save_backward_state)  # type: ignore[attr-defined]


def prepare_trainer(cfg: TrainingConfig, rank: int, schedule: Callable):
    """Model, optimizer, trainer and initial state for ``cfg``."""
    model, target_modules = setup_model_and_peft(cfg, attn_implementation="eager", apply_fsdp=False)
    model.to(get_device(rank))
    model.train() if cfg.train_mode else model.eval()
    if target_modules:
        model.requires_grad_(False)
        for name in target_modules:
            model.get_submodule(name).requires_grad_(True)
    else:
        model.requires_grad_(True)
    if cfg.grad_checkpointing:
        model.gradient_checkpointing_enable(gradient_checkpointing_kwargs=dict(use_reentrant=False))
    if cfg.optimizer == "adamw":
        opt = optim.adamw(schedule, betas=(cfg.adam_beta1, cfg.adam_beta2), eps=cfg.adam_eps, eps_root=cfg.eps_root,
                          weight_decay=cfg.weight_decay)
    elif cfg.optimizer == "muon":
        opt = optim.muon(schedule, momentum=cfg.adam_beta1, adamw_betas=(cfg.adam_beta1, cfg.adam_beta2),
                         adamw_eps_root=cfg.eps_root, weight_decay=cfg.weight_decay)
    elif cfg.optimizer == "sgd":
        opt = optim.sgd(schedule, momentum=cfg.adam_beta1, weight_decay=cfg.weight_decay)
    else:
        raise ValueError(f"Unsupported optimizer: {cfg.optimizer}")
    if cfg.fsdp and cfg.optimizer == "muon" and dist.is_initialized():
        raise ValueError("Muon orthogonalises whole matrices and cannot run on row-sharded parameters; "
                         "use adamw or sgd with fsdp.")
    trainer, state = Trainer.initialize(model, opt, fsdp=cfg.fsdp and dist.is_initialized())
    return trainer, state, model
