"""Model construction from a string.

* ``native:<family>?hidden_size=128&num_hidden_layers=6&...`` or
  ``native:<preset>`` builds a random-init in-tree model (seeded);
* a local directory with ``config.json`` whose ``model_type`` is one of the in-tree
  families loads that family and, when present, its ``*.safetensors`` weights;
* anything else falls back to ``transformers.AutoModelForCausalLM`` (generic hook
  path; needs the weights to be available locally or from the hub).
"""

from __future__ import annotations

import json
from pathlib import Path
from urllib.parse import parse_qsl

import torch

from .common import ModelArgs, NativeCausalLM
from .gpt2 import GPT2LMHeadModel
from .gpt_neox import GPTNeoXForCausalLM
from .llama import LlamaForCausalLM

FAMILIES: dict[str, type[NativeCausalLM]] = {
    "gpt_neox": GPTNeoXForCausalLM,
    "llama": LlamaForCausalLM,
    "gpt2": GPT2LMHeadModel,
}

PRESETS: dict[str, dict] = {
    # plumbing config: GPT-NeoX 6L d128, 4 heads, rotary 25 %, FFN 512
    "neox-tiny": dict(model_type="gpt_neox", vocab_size=50304, hidden_size=128, intermediate_size=512,
                      num_hidden_layers=6, num_attention_heads=4, rotary_pct=0.25, max_position_embeddings=2048),
    "pythia-160m": dict(model_type="gpt_neox", vocab_size=50304, hidden_size=768, intermediate_size=3072,
                        num_hidden_layers=12, num_attention_heads=12, rotary_pct=0.25, max_position_embeddings=2048),
    "llama-8b": dict(model_type="llama", vocab_size=128256, hidden_size=4096, intermediate_size=14336,
                     num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, rope_theta=500000.0,
                     max_position_embeddings=8192),
    "llama-70b": dict(model_type="llama", vocab_size=128256, hidden_size=8192, intermediate_size=28672,
                      num_hidden_layers=80, num_attention_heads=64, num_key_value_heads=8, rope_theta=500000.0,
                      max_position_embeddings=8192),
    "llama-tiny": dict(model_type="llama", vocab_size=512, hidden_size=64, intermediate_size=128,
                       num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=512),
    "gpt2": dict(model_type="gpt2", vocab_size=50257, hidden_size=768, intermediate_size=3072,
                 num_hidden_layers=12, num_attention_heads=12, max_position_embeddings=1024,
                 tie_word_embeddings=True),
    "gpt2-tiny": dict(model_type="gpt2", vocab_size=512, hidden_size=64, intermediate_size=256,
                      num_hidden_layers=2, num_attention_heads=4, max_position_embeddings=256,
                      tie_word_embeddings=True),
}

_HF_ALIASES = {
    # GPT-2's config.json uses its own key names.
    "n_embd": "hidden_size",
    "n_layer": "num_hidden_layers",
    "n_head": "num_attention_heads",
    "n_positions": "max_position_embeddings",
    "n_inner": "intermediate_size",
    "layer_norm_epsilon": "layer_norm_eps",
    "rotary_emb_base": "rope_theta",
}


def _convert(v: str):
    for cast in (int, float):
        try:
            return cast(v)
        except ValueError:
            pass
    if v.lower() in ("true", "false"):
        return v.lower() == "true"
    return v


def args_from_dict(d: dict) -> ModelArgs:
    d = {_HF_ALIASES.get(k, k): v for k, v in d.items()}
    if isinstance(d.get("rope_parameters"), dict):
        d.setdefault("rope_theta", d["rope_parameters"].get("rope_theta", 10000.0))
        if "partial_rotary_factor" in d["rope_parameters"]:
            d.setdefault("rotary_pct", d["rope_parameters"]["partial_rotary_factor"])
    known = {f for f in ModelArgs.__dataclass_fields__ if f != "extra"}
    kw = {k: v for k, v in d.items() if k in known and v is not None}
    extra = {k: v for k, v in d.items() if k not in known}
    args = ModelArgs(**kw, extra=extra)
    if args.model_type == "gpt2" and "intermediate_size" not in kw:
        args.intermediate_size = 4 * args.hidden_size
    if args.model_type == "gpt2":
        args.tie_word_embeddings = True
    return args


def parse_native_spec(spec: str) -> tuple[ModelArgs, int]:
    """``native:<family-or-preset>?k=v&...`` -> (ModelArgs, init seed)."""
    assert spec.startswith("native:"), spec
    body = spec[len("native:"):]
    name, _, query = body.partition("?")
    opts = {k: _convert(v) for k, v in parse_qsl(query)}
    seed = int(opts.pop("seed", 0))
    opts.pop("init", None)
    if name in PRESETS:
        base = dict(PRESETS[name])
    elif name in FAMILIES:
        base = {"model_type": name}
    else:
        raise ValueError(f"Unknown native model {name!r}; families {sorted(FAMILIES)}, presets {sorted(PRESETS)}")
    base.update(opts)
    return args_from_dict(base), seed


def build_model(args: ModelArgs, *, dtype=torch.float32, device="cpu", seed: int = 0,
                init_on_device: bool = False) -> NativeCausalLM:
    """Random-init model.  By default initialisation is drawn on CPU in fp32 from ``seed``
    so the weights do not depend on the target device or dtype; ``init_on_device`` draws
    them directly on ``device`` in ``dtype`` (fast for multi-billion-parameter models,
    reproducible per device type)."""
    cls = FAMILIES[args.model_type]
    if init_on_device and torch.device(device).type == "cuda":
        prev = torch.get_default_dtype()
        torch.set_default_dtype(dtype)
        try:
            with torch.device(device), torch.random.fork_rng(devices=[torch.device(device)]):
                torch.manual_seed(seed)
                model = cls(args)
        finally:
            torch.set_default_dtype(prev)
        return model
    with torch.random.fork_rng(devices=[]):
        torch.manual_seed(seed)
        model = cls(args)
    return model.to(device=device, dtype=dtype)


def load_model(name: str, *, dtype=torch.float32, device="cpu", revision=None, **hf_kwargs):
    """Resolve a model string (see module docstring)."""
    if name.startswith("native:"):
        args, seed = parse_native_spec(name)
        return build_model(args, dtype=dtype, device=device, seed=seed, init_on_device="init=device" in name)
    path = Path(name)
    if (path / "config.json").exists():
        with open(path / "config.json") as f:
            raw = json.load(f)
        if raw.get("model_type") in FAMILIES and not hf_kwargs.pop("force_hf", False):
            model = build_model(args_from_dict(raw), dtype=torch.float32, device="cpu")
            shards = sorted(path.glob("*.safetensors"))
            if shards:
                from safetensors.torch import load_file

                state = {}
                for s in shards:
                    state.update(load_file(str(s)))
                missing, unexpected = model.load_state_dict(state, strict=False)
                missing = [m for m in missing if "lm_head" not in m and "embed_out" not in m]
                if missing:
                    raise RuntimeError(f"Checkpoint at {path} lacks tensors: {missing[:8]}")
            return model.to(device=device, dtype=dtype)
    from transformers import AutoModelForCausalLM

    return AutoModelForCausalLM.from_pretrained(
        name, dtype=dtype, revision=revision, device_map={"": str(device)}, **hf_kwargs
    )
