"""Llama family: RMSNorm, RoPE (rotate-half), grouped-query attention, SwiGLU."""

from __future__ import annotations

import torch
import torch.nn as nn
from torch import Tensor

from .. import ops
from .common import Backbone, ModelArgs, NativeCausalLM, maybe_checkpoint


class LlamaRMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.variance_epsilon = eps

    def forward(self, x: Tensor) -> Tensor:
        return ops.rms_norm(x, self.weight, self.variance_epsilon)


class LlamaAttention(nn.Module):
    def __init__(self, cfg: ModelArgs):
        super().__init__()
        d, hd = cfg.hidden_size, cfg.head_dim
        self.num_heads, self.kv_heads, self.head_dim = cfg.num_attention_heads, cfg.kv_heads, hd
        self.q_proj = ops.Linear(d, self.num_heads * hd, bias=cfg.attention_bias)
        self.k_proj = ops.Linear(d, self.kv_heads * hd, bias=cfg.attention_bias)
        self.v_proj = ops.Linear(d, self.kv_heads * hd, bias=cfg.attention_bias)
        self.o_proj = ops.Linear(self.num_heads * hd, d, bias=cfg.attention_bias)
        self.tp_group = None  # set by parallel.tensor_parallel.apply_tensor_parallel

    def forward(self, x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
        B, S, _ = x.shape
        if self.tp_group is not None:
            from ..parallel.tensor_parallel import copy_to_group, reduce_from_group

            x = copy_to_group(x, self.tp_group)
        q = self.q_proj(x).view(B, S, self.num_heads, self.head_dim)
        k = self.k_proj(x).view(B, S, self.kv_heads, self.head_dim)
        v = self.v_proj(x).view(B, S, self.kv_heads, self.head_dim)
        q = ops.rotary(q, cos, sin, self.head_dim)
        k = ops.rotary(k, cos, sin, self.head_dim)
        o = ops.causal_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
        out = self.o_proj(o.transpose(1, 2).reshape(B, S, -1))
        return reduce_from_group(out, self.tp_group) if self.tp_group is not None else out


class LlamaMLP(nn.Module):
    def __init__(self, cfg: ModelArgs):
        super().__init__()
        d, f = cfg.hidden_size, cfg.intermediate_size
        self.gate_proj = ops.Linear(d, f, bias=cfg.mlp_bias)
        self.up_proj = ops.Linear(d, f, bias=cfg.mlp_bias)
        self.down_proj = ops.Linear(f, d, bias=cfg.mlp_bias)
        self.tp_group = None  # set by parallel.tensor_parallel.apply_tensor_parallel

    def forward(self, x: Tensor) -> Tensor:
        if self.tp_group is None:
            return self.down_proj(ops.swiglu(self.gate_proj(x), self.up_proj(x)))
        from ..parallel.tensor_parallel import copy_to_group, reduce_from_group

        x = copy_to_group(x, self.tp_group)
        return reduce_from_group(self.down_proj(ops.swiglu(self.gate_proj(x), self.up_proj(x))), self.tp_group)


class LlamaDecoderLayer(nn.Module):
    def __init__(self, cfg: ModelArgs):
        super().__init__()
        self.self_attn = LlamaAttention(cfg)
        self.mlp = LlamaMLP(cfg)
        self.input_layernorm = LlamaRMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.post_attention_layernorm = LlamaRMSNorm(cfg.hidden_size, cfg.rms_norm_eps)

    def forward(self, x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
        x = x + self.self_attn(self.input_layernorm(x), cos, sin)
        return x + self.mlp(self.post_attention_layernorm(x))


class LlamaModel(Backbone):
    def __init__(self, cfg: ModelArgs):
        super().__init__()
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.layers = nn.ModuleList(LlamaDecoderLayer(cfg) for _ in range(cfg.num_hidden_layers))
        self.norm = LlamaRMSNorm(cfg.hidden_size, cfg.rms_norm_eps)


class LlamaForCausalLM(NativeCausalLM):
    base_model_prefix = "model"

    def __init__(self, cfg: ModelArgs):
        super().__init__(cfg)
        self.model = LlamaModel(cfg)
        self.lm_head = ops.Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
        self._init_weights(cfg.initializer_range)
        if cfg.tie_word_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight

    def get_input_embeddings(self):
        return self.model.embed_tokens

    def get_output_embeddings(self):
        return self.lm_head

    def hidden(self, input_ids: Tensor) -> Tensor:
        m = self.model
        x = m.embed_tokens(input_ids)
        cos, sin = ops.rotary_tables(
            input_ids.shape[1], self.config.head_dim, self.config.rope_theta, x.device
        )
        for layer in m.layers:
            x = maybe_checkpoint(self, layer, x, cos, sin)
        return m.norm(x)
