"""GPT-2 family: learned positions, LayerNorm, Conv1D projections (weights stored
``[in, out]``), tanh-GELU MLP, output head tied to the token embedding."""

from __future__ import annotations

import torch
import torch.nn as nn
from torch import Tensor

from .. import ops
from .common import Backbone, Conv1D, ModelArgs, NativeCausalLM, maybe_checkpoint


class _LN(nn.LayerNorm):
    def forward(self, x: Tensor) -> Tensor:
        return ops.layer_norm(x, self.weight, self.bias, self.eps)


class GPT2Attention(nn.Module):
    def __init__(self, cfg: ModelArgs):
        super().__init__()
        d = cfg.hidden_size
        self.num_heads, self.head_dim = cfg.num_attention_heads, cfg.head_dim
        self.c_attn = Conv1D(3 * d, d)
        self.c_proj = Conv1D(d, d)

    def forward(self, x: Tensor) -> Tensor:
        B, S, d = x.shape
        q, k, v = self.c_attn(x).split(d, dim=2)
        shape = (B, S, self.num_heads, self.head_dim)
        o = ops.causal_attention(
            q.view(shape).transpose(1, 2), k.view(shape).transpose(1, 2), v.view(shape).transpose(1, 2)
        )
        return self.c_proj(o.transpose(1, 2).reshape(B, S, d))


class GPT2MLP(nn.Module):
    def __init__(self, cfg: ModelArgs):
        super().__init__()
        self.c_fc = Conv1D(cfg.intermediate_size, cfg.hidden_size)
        self.c_proj = Conv1D(cfg.hidden_size, cfg.intermediate_size)

    def forward(self, x: Tensor) -> Tensor:
        return self.c_proj(ops.gelu(self.c_fc(x), approximate="tanh"))


class GPT2Block(nn.Module):
    def __init__(self, cfg: ModelArgs):
        super().__init__()
        self.ln_1 = _LN(cfg.hidden_size, eps=cfg.layer_norm_eps)
        self.attn = GPT2Attention(cfg)
        self.ln_2 = _LN(cfg.hidden_size, eps=cfg.layer_norm_eps)
        self.mlp = GPT2MLP(cfg)

    def forward(self, x: Tensor) -> Tensor:
        x = x + self.attn(self.ln_1(x))
        return x + self.mlp(self.ln_2(x))


class GPT2Model(Backbone):
    def __init__(self, cfg: ModelArgs):
        super().__init__()
        self.wte = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.wpe = nn.Embedding(cfg.max_position_embeddings, cfg.hidden_size)
        self.h = nn.ModuleList(GPT2Block(cfg) for _ in range(cfg.num_hidden_layers))
        self.ln_f = _LN(cfg.hidden_size, eps=cfg.layer_norm_eps)


class GPT2LMHeadModel(NativeCausalLM):
    base_model_prefix = "transformer"

    def __init__(self, cfg: ModelArgs):
        super().__init__(cfg)
        self.transformer = GPT2Model(cfg)
        self.lm_head = ops.Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
        self._init_weights(cfg.initializer_range)
        self.lm_head.weight = self.transformer.wte.weight

    def get_input_embeddings(self):
        return self.transformer.wte

    def get_output_embeddings(self):
        return self.lm_head

    def hidden(self, input_ids: Tensor) -> Tensor:
        t = self.transformer
        pos = torch.arange(input_ids.shape[1], device=input_ids.device)
        x = t.wte(input_ids) + t.wpe(pos)[None]
        for block in t.h:
            x = maybe_checkpoint(self, block, x)
        return t.ln_f(x)
