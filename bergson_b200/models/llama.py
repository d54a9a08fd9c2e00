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

    def forward_seq_parallel(self, h: Tensor, residual: Tensor, cos: Tensor, sin: Tensor, sp, lead) -> Tensor:
        """``residual + o_proj(attention(...))`` on token shards ``[T / W, d]``: q/k/v gather the
        tokens inside their GEMMs, o_proj reduce-scatters from its epilogue."""
        from ..parallel.sequence_parallel import Published, gather_linear, scatter_linear

        B, S = lead
        pub = Published(sp, h)
        q = gather_linear(pub, self.q_proj, lead).view(B, S, self.num_heads, self.head_dim)
        k = gather_linear(pub, self.k_proj, lead).view(B, S, self.kv_heads, self.head_dim)
        v = gather_linear(pub, self.v_proj, lead).view(B, S, self.kv_heads, self.head_dim)
        pub.release()
        q = ops.rotary(q, cos, sin, self.head_dim)
        k = ops.rotary(k, cos, sin, self.head_dim)
        o = ops.causal_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
        return scatter_linear(o.transpose(1, 2).reshape(B * S, -1), self.o_proj, sp, lead, residual)


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

    def forward_seq_parallel(self, h: Tensor, residual: Tensor, sp, lead) -> Tensor:
        from ..parallel.sequence_parallel import Published, gather_linear, scatter_linear

        pub = Published(sp, h)
        a = ops.swiglu(gather_linear(pub, self.gate_proj, lead), gather_linear(pub, self.up_proj, lead))
        pub.release()
        return scatter_linear(a, self.down_proj, sp, lead, residual)


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

    def forward_seq_parallel(self, x: Tensor, cos: Tensor, sin: Tensor, sp, lead) -> Tensor:
        """The block on a token shard ``[T / W, d]`` (norms and residuals are per token)."""
        x = self.self_attn.forward_seq_parallel(self.input_layernorm(x), x, cos, sin, sp, lead)
        return self.mlp.forward_seq_parallel(self.post_attention_layernorm(x), x, sp, lead)


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
        sp = self._seq_parallel_for(input_ids)
        if sp is not None:
            return self._hidden_seq_parallel(input_ids, sp)
        x = m.embed_tokens(input_ids)
        cos, sin = ops.rotary_tables(
            input_ids.shape[1], self.config.head_dim, self.config.rope_theta, x.device
        )
        for layer in m.layers:
            x = maybe_checkpoint(self, layer, x, cos, sin)
        return m.norm(x)

    def _seq_parallel_for(self, input_ids: Tensor):
        """The sequence-parallel context when this call can take the fused tensor-parallel path:
        16-bit CUDA weights, a token count that splits into 128-row blocks per rank, frozen
        sharded weights, and no hook-based collector on the sharded projections.  The reason for
        staying on the all-reduce path is printed once."""
        sp = getattr(self, "_seq_parallel", None)
        if sp is None:
            return None
        reason = self._seq_parallel_obstacle(sp, input_ids)
        if reason is None:
            return sp
        seen = self.__dict__.setdefault("_sp_reasons", set())
        if reason not in seen:
            seen.add(reason)
            if sp.rank == 0:
                print(f"tensor parallel: all-reduce path for this call ({reason})", flush=True)
        return None

    def _seq_parallel_obstacle(self, sp, input_ids: Tensor) -> str | None:
        from ..ops.functional import _composable
        from ..parallel.sequence_parallel import hooks_compatible

        if self.gradient_checkpointing:
            return "gradient checkpointing"
        if _composable():
            return "graph will be differentiated again"
        w = self.model.layers[0].self_attn.q_proj.weight
        if not w.is_cuda:
            return "weights are not on a GPU"
        if not sp.fits(input_ids.numel(), self.config.hidden_size, w.dtype):
            return (f"{input_ids.numel()} tokens of {w.dtype} do not split into 128-row blocks over "
                    f"{sp.world} ranks")
        sharded = [m for layer in self.model.layers for m in (
            layer.self_attn.q_proj, layer.self_attn.k_proj, layer.self_attn.v_proj, layer.self_attn.o_proj,
            layer.mlp.gate_proj, layer.mlp.up_proj, layer.mlp.down_proj)]
        if any(m.weight.requires_grad or m.bias is not None for m in sharded):
            return "trainable or biased projections"
        if not hooks_compatible(sharded):
            return "a hook-based collector is attached"
        return None

    def _hidden_seq_parallel(self, input_ids: Tensor, sp) -> Tensor:
        """Final-norm hidden states with the blocks run on token shards (collectives inside the
        GEMM kernels); the shards are gathered once at the end because the head is replicated."""
        from ..parallel.sequence_parallel import gather_tokens

        m = self.model
        B, S = input_ids.shape
        lead = (B, S)
        rows = B * S // sp.world
        sp.ensure(B * S, self.config.hidden_size, m.embed_tokens.weight.dtype)
        if not getattr(sp, "_announced", False):
            sp._announced = True
            if sp.rank == 0:
                print(f"tensor parallel: sequence-parallel blocks over {sp.world} ranks, all-gather and "
                      "reduce-scatter inside the GEMM kernels (peer memory)", flush=True)
        # This rank's tokens only: the residual stream stays sharded over tokens between blocks.
        x = m.embed_tokens(input_ids.reshape(-1)[sp.rank * rows : (sp.rank + 1) * rows])
        cos, sin = ops.rotary_tables(S, self.config.head_dim, self.config.rope_theta, x.device)
        for layer in m.layers:
            x = layer.forward_seq_parallel(x, cos, sin, sp, lead)
        return gather_tokens(m.norm(x), sp).view(B, S, -1)
