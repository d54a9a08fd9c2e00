"""Running Grams ``H_m = sum_rows r_m^T r_m`` of per-example (or per-token) gradient blocks.

The accumulator is fed whole batches.  When every module's block has the same width (the
usual case: ``projection_dim**2`` columns each) the blocks of a batch are viewed as one
``[rows, modules, width]`` tensor and all Grams advance in a single batched product into a
stacked ``[modules, width, width]`` buffer; otherwise each module is updated on its own.
``finish`` hands the sums to ``process_autocorrelation_matrices`` (mean over rows, sum over
ranks, fp64 eigendecomposition) and stores the result on the processor.
"""

from __future__ import annotations

import torch
from torch import Tensor

from ..gradients import GradientProcessor
from ..process_autocorrelation import process_autocorrelation_matrices


class GramAccumulator:
    def __init__(self, sizes: dict[str, int]):
        self.sizes = dict(sizes)
        self.names = list(sizes)
        widths = set(sizes.values())
        self.uniform = len(widths) == 1 and len(self.names) > 1
        self._stack: Tensor | None = None
        self._single: dict[str, Tensor] = {}

    def add_blocks(self, blocks: dict[str, Tensor]) -> None:
        """``blocks[name]``: ``[rows, width_name]`` for (a subset of) the modules."""
        if self.uniform and len(blocks) == len(self.names):
            self.add_rows(torch.cat([blocks[n].float() for n in self.names], dim=1))
            return
        for name, b in blocks.items():
            b = b.float()
            if name in self._single:
                self._single[name].addmm_(b.mT, b)
            else:
                self._single[name] = b.mT @ b

    def add_rows(self, rows: Tensor) -> None:
        """``rows``: ``[n, sum(widths)]`` with the modules' blocks side by side in ``sizes`` order."""
        rows = rows.float()
        if not self.uniform:
            off = 0
            for name in self.names:
                w = self.sizes[name]
                self.add_blocks({name: rows[:, off : off + w]})
                off += w
            return
        w = self.sizes[self.names[0]]
        x = rows.view(rows.shape[0], len(self.names), w).transpose(0, 1)  # [modules, n, width]
        if self._stack is None:
            self._stack = torch.bmm(x.mT, x)
        else:
            self._stack.baddbmm_(x.mT, x)

    def sums(self) -> dict[str, Tensor]:
        out = dict(self._single)
        if self._stack is not None:
            for k, name in enumerate(self.names):
                out[name] = out[name] + self._stack[k] if name in out else self._stack[k]
        return out

    def finish(self, processor: GradientProcessor, num_rows: int, rank: int) -> None:
        sums = self.sums()
        if sums:
            process_autocorrelation_matrices(processor, sums, num_rows, self.sizes, rank)
