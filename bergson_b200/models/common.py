"""Shared pieces of the in-tree causal-LM families.

The families mirror the HF module names (``gpt_neox.layers.N.attention.query_key_value``,
``model.layers.N.self_attn.q_proj``, ``transformer.h.N.attn.c_attn`` ...) because the
gradient store's column names and the optimizer-normaliser keys are module names
relative to ``base_model`` (reference ``bergson/collector/collector.py:160-183``).
"""

from __future__ import annotations

from dataclasses import asdict, dataclass, field
from typing import Any

import torch
import torch.nn as nn
from torch import Tensor

from ..utils.math import weighted_causal_lm_ce


@dataclass
class ModelArgs:
    """Architecture hyper-parameters (HF ``config.json`` key names)."""

    model_type: str = "llama"
    vocab_size: int = 32000
    hidden_size: int = 512
    intermediate_size: int = 2048
    num_hidden_layers: int = 4
    num_attention_heads: int = 8
    num_key_value_heads: int | None = None
    max_position_embeddings: int = 2048
    rope_theta: float = 10000.0
    rotary_pct: float = 1.0
    rms_norm_eps: float = 1e-5
    layer_norm_eps: float = 1e-5
    use_parallel_residual: bool = True
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    mlp_bias: bool = False
    initializer_range: float = 0.02
    hidden_dropout: float = 0.0
    extra: dict[str, Any] = field(default_factory=dict)

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @property
    def kv_heads(self) -> int:
        return self.num_key_value_heads or self.num_attention_heads

    def to_dict(self) -> dict[str, Any]:
        d = asdict(self)
        d.update(d.pop("extra"))
        return d

    # HF configs are attribute bags; a few callers use ``getattr(config, key)``.
    def __getattr__(self, name):
        extra = self.__dict__.get("extra", {})
        if name in extra:
            return extra[name]
        raise AttributeError(name)


@dataclass
class CausalLMOutput:
    """Forward result; indexable like an HF ``ModelOutput`` (by field name, or by position
    over the fields that are set, loss first)."""

    logits: Tensor | None = None
    loss: Tensor | None = None
    hidden_states: Tensor | None = None

    def _present(self) -> list[tuple[str, Tensor]]:
        order = ("loss", "logits", "hidden_states")
        return [(k, getattr(self, k)) for k in order if getattr(self, k) is not None]

    def __getitem__(self, key):
        if isinstance(key, str):
            return getattr(self, key)
        return self._present()[key][1]

    def keys(self):
        return [k for k, _ in self._present()]

    def __contains__(self, key) -> bool:
        return key in self.keys()


class Backbone(nn.Module):
    """Base of the ``base_model`` sub-modules; mirrors HF's ``device`` / ``dtype``."""

    @property
    def device(self) -> torch.device:
        return next(self.parameters()).device

    @property
    def dtype(self) -> torch.dtype:
        return next(self.parameters()).dtype


class NativeCausalLM(nn.Module):
    """Base class: HF-like surface (``config``, ``base_model``, ``device``, ``dtype``,
    ``get_input_embeddings``, ``loss_function``, ``forward(...).logits``)."""

    base_model_prefix = "model"
    config: ModelArgs

    def __init__(self, config: ModelArgs):
        super().__init__()
        self.config = config
        self.loss_function = weighted_causal_lm_ce
        self.gradient_checkpointing = False

    @property
    def base_model(self) -> nn.Module:
        return getattr(self, self.base_model_prefix)

    @property
    def device(self) -> torch.device:
        return next(self.parameters()).device

    @property
    def dtype(self) -> torch.dtype:
        return next(self.parameters()).dtype

    def get_input_embeddings(self) -> nn.Module:
        raise NotImplementedError

    def get_output_embeddings(self) -> nn.Module:
        raise NotImplementedError

    def gradient_checkpointing_enable(self, **_):
        self.gradient_checkpointing = True

    def hidden(self, input_ids: Tensor) -> Tensor:
        """Final-norm hidden states ``[B, S, d]``."""
        raise NotImplementedError

    def forward(self, input_ids: Tensor, labels: Tensor | None = None, **kwargs) -> CausalLMOutput:
        h = self.hidden(input_ids)
        head = self.get_output_embeddings()
        V = self.config.vocab_size
        ours = getattr(self.loss_function, "func", self.loss_function) is weighted_causal_lm_ce
        if (labels is not None and V % 8 and ours and getattr(head, "bias", None) is None
                and not head._forward_hooks):
            # A vocabulary that is not a multiple of 8 is padded for the head's GEMM; the loss
            # runs on the padded width (the extra columns cannot win any probability) and the
            # logits handed back are the view without them.
            from ..ops.linear import linear_keep_padding

            padded = linear_keep_padding(h, head.weight)
            if padded is not None:
                loss = self.loss_function(padded, labels, vocab_size=V, padded_vocab=True, **kwargs)
                return CausalLMOutput(logits=padded[..., :V], loss=loss)
        logits = head(h)
        loss = None
        if labels is not None:
            loss = self.loss_function(
                logits, labels, vocab_size=V, **kwargs
            )
        return CausalLMOutput(logits=logits, loss=loss)

    def _init_weights(self, std: float) -> None:
        for m in self.modules():
            if isinstance(m, nn.Linear):
                nn.init.normal_(m.weight, 0.0, std)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)
            elif isinstance(m, nn.Embedding):
                nn.init.normal_(m.weight, 0.0, std)
            elif isinstance(m, Conv1D):
                nn.init.normal_(m.weight, 0.0, std)
                nn.init.zeros_(m.bias)

    def save_pretrained(self, path, **_):
        """Write ``config.json`` + ``model.safetensors`` (HF layout, same tensor names)."""
        import json
        from pathlib import Path

        from safetensors.torch import save_file

        path = Path(path)
        path.mkdir(parents=True, exist_ok=True)
        cfg = self.config.to_dict()
        cfg["architectures"] = [type(self).__name__]
        with open(path / "config.json", "w") as f:
            json.dump(cfg, f, indent=2)
        seen: dict[int, str] = {}
        tensors = {}
        for k, v in self.state_dict().items():
            if v.data_ptr() in seen:  # tied weights are stored once
                continue
            seen[v.data_ptr()] = k
            tensors[k] = v.detach().cpu().contiguous()
        save_file(tensors, str(path / "model.safetensors"))


class Conv1D(nn.Module):
    """GPT-2 style linear layer whose weight is stored ``[in, out]``
    (``nx`` inputs, ``nf`` outputs), numerically ``x @ W + b``."""

    def __init__(self, nf: int, nx: int):
        super().__init__()
        self.nf, self.nx = nf, nx
        self.weight = nn.Parameter(torch.empty(nx, nf))
        self.bias = nn.Parameter(torch.zeros(nf))

    def forward(self, x: Tensor) -> Tensor:
        from ..ops.linear import linear

        return linear(x, self.weight, self.bias, layout="io", module=self, tap=getattr(self, "_tap", None))

    def extra_repr(self) -> str:
        return f"nf={self.nf}, nx={self.nx}"


def maybe_checkpoint(module: NativeCausalLM, fn, *args):
    if module.gradient_checkpointing and torch.is_grad_enabled():
        from torch.utils.checkpoint import checkpoint

        return checkpoint(fn, *args, use_reentrant=False)
    return fn(*args)
