"""In-tree causal-LM families and the loader that maps a model string to one."""

from .common import CausalLMOutput, Conv1D, ModelArgs, NativeCausalLM
from .gpt2 import GPT2LMHeadModel
from .gpt_neox import GPTNeoXForCausalLM
from .llama import LlamaForCausalLM
from .registry import FAMILIES, PRESETS, build_model, load_model, parse_native_spec

__all__ = [
    "CausalLMOutput",
    "Conv1D",
    "ModelArgs",
    "NativeCausalLM",
    "GPT2LMHeadModel",
    "GPTNeoXForCausalLM",
    "LlamaForCausalLM",
    "FAMILIES",
    "PRESETS",
    "build_model",
    "load_model",
    "parse_native_spec",
]
