"""GPT-NeoX / Pythia family: LayerNorm, fused QKV with per-head ``[q|k|v]`` layout,
rotary on the first ``rotary_pct`` of each head, GELU MLP, parallel residual."""

from __future__ import annotations

import torch
import torch.nn as nn
from torch import Tensor

from .. import ops
from .common import Backbone, ModelArgs, NativeCausalLM, maybe_checkpoint


class _LN(nn.LayerNorm):
    def forward(self, x: Tensor) -> Tensor:
        return ops.layer_norm(x, self.weight, self.bias, self.eps)


class NeoXAttention(nn.Module):
    def __init__(self, cfg: ModelArgs):
        super().__init__()
        d = cfg.hidden_size
        self.num_heads = cfg.num_attention_heads
        self.head_dim = cfg.head_dim
        self.rot_dim = int(self.head_dim * cfg.rotary_pct)
        self.theta = cfg.rope_theta
        self.query_key_value = ops.Linear(d, 3 * d, bias=True)
        self.dense = ops.Linear(d, d, bias=True)

    def forward(self, x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
        B, S, _ = x.shape
        qkv = self.query_key_value(x).view(B, S, self.num_heads, 3 * self.head_dim)
        q, k, v = qkv.split(self.head_dim, dim=-1)  # each [B, S, H, D]
        q = ops.rotary(q, cos, sin, self.rot_dim)
        k = ops.rotary(k, cos, sin, self.rot_dim)
        o = ops.causal_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
        return self.dense(o.transpose(1, 2).reshape(B, S, -1))


class NeoXMLP(nn.Module):
    def __init__(self, cfg: ModelArgs):
        super().__init__()
        self.dense_h_to_4h = ops.Linear(cfg.hidden_size, cfg.intermediate_size)
        self.dense_4h_to_h = ops.Linear(cfg.intermediate_size, cfg.hidden_size)

    def forward(self, x: Tensor) -> Tensor:
        return self.dense_4h_to_h(ops.gelu(self.dense_h_to_4h(x)))


class NeoXLayer(nn.Module):
    def __init__(self, cfg: ModelArgs):
        super().__init__()
        self.parallel = cfg.use_parallel_residual
        self.input_layernorm = _LN(cfg.hidden_size, eps=cfg.layer_norm_eps)
        self.post_attention_layernorm = _LN(cfg.hidden_size, eps=cfg.layer_norm_eps)
        self.attention = NeoXAttention(cfg)
        self.mlp = NeoXMLP(cfg)

    def forward(self, x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
        a = self.attention(self.input_layernorm(x), cos, sin)
        if self.parallel:
            return x + a + self.mlp(self.post_attention_layernorm(x))
        x = x + a
        return x + self.mlp(self.post_attention_layernorm(x))


class NeoXModel(Backbone):
    def __init__(self, cfg: ModelArgs):
        super().__init__()
        self.embed_in = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.layers = nn.ModuleList(NeoXLayer(cfg) for _ in range(cfg.num_hidden_layers))
        self.final_layer_norm = _LN(cfg.hidden_size, eps=cfg.layer_norm_eps)


class GPTNeoXForCausalLM(NativeCausalLM):
    base_model_prefix = "gpt_neox"

    def __init__(self, cfg: ModelArgs):
        super().__init__(cfg)
        self.gpt_neox = NeoXModel(cfg)
        self.embed_out = ops.Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
        self._init_weights(cfg.initializer_range)

    def get_input_embeddings(self):
        return self.gpt_neox.embed_in

    def get_output_embeddings(self):
        return self.embed_out

    def hidden(self, input_ids: Tensor) -> Tensor:
        m = self.gpt_neox
        x = m.embed_in(input_ids)
        rot = m.layers[0].attention.rot_dim
        cos, sin = ops.rotary_tables(input_ids.shape[1], rot, self.config.rope_theta, x.device)
        for layer in m.layers:
            x = maybe_checkpoint(self, layer, x, cos, sin)
        return m.final_layer_norm(x)
