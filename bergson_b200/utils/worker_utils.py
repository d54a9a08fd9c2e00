"""Per-worker set-up: model, processor, data pipeline
(reference ``bergson/utils/worker_utils.py``)."""

from __future__ import annotations

import shutil
import warnings
from functools import partial
from pathlib import Path

import numpy as np
import torch
from datasets import Dataset

from ..config.config import AttributionConfig, DataConfig, IndexConfig, ModelConfig
from ..data import load_data_string, tokenize, tokenize_and_chunk
from ..gradients import GradientProcessor, Normalizer
from ..models import NativeCausalLM, load_model
from ..models.registry import parse_native_spec
from .math import weighted_causal_lm_ce
from .utils import assert_type, get_device, get_layer_list, simple_parse_kwargs_string

BIG_NUM = np.iinfo(np.int64).max

_DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32, "fp64": torch.float64}


def validate_run_path(index_cfg: IndexConfig):
    """Refuse to overwrite an existing run unless ``overwrite``.  The check runs on global rank
    0 only; with several nodes the other nodes' parents wait for it at a barrier, so that none
    of them can create the (shared) partial directory before it has been checked."""
    multi_node = index_cfg.distributed.nnode > 1
    try:
        if index_cfg.distributed.rank == 0:
            for path in (Path(index_cfg.run_path), Path(index_cfg.partial_run_path)):
                if not path.exists():
                    continue
                if index_cfg.overwrite:
                    shutil.rmtree(path)
                else:
                    raise FileExistsError(f"Run path {path} already exists. Use --overwrite to overwrite it.")
    finally:
        if multi_node:
            from ..distributed import parent_barrier

            parent_barrier(index_cfg.distributed)


def create_processor(model, cfg: IndexConfig, target_modules: set[str] | None = None) -> GradientProcessor:
    rank = cfg.distributed.rank
    normalizers: dict[str, Normalizer] = {}
    if cfg.optimizer_state:
        from .load_from_optimizer import load_from_optimizer

        normalizers = load_from_optimizer(model, cfg.optimizer_state, include_bias=cfg.include_bias,
                                          target_modules=target_modules)
    processor = GradientProcessor(
        normalizers,
        projection_dim=cfg.projection_dim or None,
        reshape_to_square=cfg.reshape_to_square,
        projection_type=cfg.projection_type,
        projection_scale=cfg.projection_scale,
        projection_target=cfg.projection_target,
        include_bias=cfg.include_bias,
    )
    if rank == 0:
        processor.save(cfg.partial_run_path)
    return processor


def apply_force_math_sdp(cfg: ModelConfig) -> None:
    if not getattr(cfg, "force_math_sdp", False):
        return
    torch.backends.cuda.enable_flash_sdp(False)
    torch.backends.cuda.enable_mem_efficient_sdp(False)
    print("force_math_sdp: disabled flash and memory-efficient SDPA backends")


def setup_model_and_peft(cfg: ModelConfig, device_map_auto: bool = False, apply_fsdp: bool = True, **model_kwargs):
    """Load the model (in-tree family or HF), install the weighted CE loss, freeze all
    parameters except the input embeddings (so that backward reaches every layer
    without computing weight gradients), optionally shard with FSDP."""
    apply_force_math_sdp(cfg)
    local_rank = cfg.distributed.local_rank
    if cfg.precision in _DTYPES:
        dtype = _DTYPES[cfg.precision]
    elif cfg.precision in ("int4", "int8"):
        dtype = torch.bfloat16
    elif cfg.precision == "auto":
        dtype = "auto"
    else:
        raise ValueError(f"Unsupported precision: {cfg.precision}")
    device = "cpu" if (cfg.fsdp or not torch.cuda.is_available()) else get_device(local_rank)
    model_kwargs.update(simple_parse_kwargs_string(cfg.model_kwargs))
    target_modules = None

    native = cfg.model.startswith("native:") or (
        (Path(cfg.model) / "config.json").exists() and not (Path(cfg.model) / "adapter_config.json").exists()
    )
    if native and cfg.precision not in ("int4", "int8") and not cfg.peft_init_kwargs:
        model_kwargs.pop("attn_implementation", None)
        model = load_model(cfg.model, dtype=torch.float32 if dtype == "auto" else dtype, device=device,
                           revision=cfg.revision, **model_kwargs)
    else:
        model, target_modules = _load_hf_model(cfg, dtype, device, device_map_auto, model_kwargs)

    if getattr(cfg, "tensor_parallel", 1) > 1:
        from ..parallel import topology
        from ..parallel.tensor_parallel import apply_tensor_parallel

        topology.init_topology(cfg.tensor_parallel)
        apply_tensor_parallel(model)

    reduction = getattr(cfg, "loss_reduction", "mean")
    model.loss_function = partial(weighted_causal_lm_ce, reduction=reduction)
    model.requires_grad_(False)
    model.get_input_embeddings().requires_grad_(True)

    if cfg.fsdp and apply_fsdp:
        from torch.distributed.fsdp import fully_shard

        for layer in get_layer_list(model):
            fully_shard(layer)
        fully_shard(model)
    return model, target_modules


def _load_hf_model(cfg: ModelConfig, dtype, device, device_map_auto: bool, model_kwargs: dict):
    from transformers import AutoModelForCausalLM

    quant = None
    if cfg.precision in ("int4", "int8"):
        from transformers import BitsAndBytesConfig

        quant = BitsAndBytesConfig(
            load_in_4bit=cfg.precision == "int4", load_in_8bit=cfg.precision == "int8",
            bnb_4bit_compute_dtype=dtype, bnb_4bit_quant_storage=dtype, bnb_4bit_quant_type="nf4",
            bnb_4bit_use_double_quant=True,
        )
    peft_cfg = None
    try:
        from peft import PeftConfig

        try:
            peft_cfg = PeftConfig.from_pretrained(cfg.model)
        except ValueError:
            peft_cfg = None
    except ImportError:
        PeftConfig = None  # noqa: N806
    assert not (cfg.peft_init_kwargs and peft_cfg), f"peft_init_args is set but '{cfg.model}' is already a PEFT adapter."
    base = peft_cfg.base_model_name_or_path if peft_cfg else cfg.model
    device_map = "auto" if device_map_auto else {"": device}
    model = AutoModelForCausalLM.from_pretrained(base, device_map=device_map, quantization_config=quant, dtype=dtype,
                                                 revision=cfg.revision, **model_kwargs)
    target_modules = None
    if cfg.peft_init_kwargs or peft_cfg:
        from peft import PeftModel, PeftType, get_peft_model
        from peft.mapping import PEFT_TYPE_TO_CONFIG_MAPPING

        from .peft import extract_peft_target_modules

        if cfg.peft_init_kwargs:
            kw = simple_parse_kwargs_string(cfg.peft_init_kwargs)
            ptype = PeftType(kw.pop("peft_type", "LORA"))
            model = get_peft_model(model, PEFT_TYPE_TO_CONFIG_MAPPING[ptype](**kw))
        else:
            model = PeftModel.from_pretrained(model, cfg.model, device_map=device_map, autocast_adapter_dtype=False)
        target_modules = extract_peft_target_modules(model)
    return model, target_modules


def extract_peft_target_modules(model) -> set[str]:
    """Adapter module names of a PEFT model (needs the optional ``peft`` package)."""
    from .peft import extract_peft_target_modules as impl

    return impl(model)


def estimate_advantage(ds: Dataset, cfg: DataConfig):
    """Dr. GRPO advantage: reward minus the mean reward of rollouts sharing the prompt."""
    import pandas as pd

    df = assert_type(pd.DataFrame, ds.select_columns([cfg.prompt_column, cfg.reward_column]).to_pandas())
    adv = df[cfg.reward_column] - df.groupby(cfg.prompt_column)[cfg.reward_column].transform("mean")
    return adv.tolist()


def filter_by_max_tokens(ds: Dataset, cfg: AttributionConfig) -> Dataset:
    """Take a prefix of at most ``max_tokens`` tokens, or tile the rows up to it."""
    if cfg.max_tokens is None:
        return ds
    lengths = ds["length"]
    total = sum(lengths)
    if total >= cfg.max_tokens:
        keep, used = [], 0
        for i, n in enumerate(lengths):
            if used + n > cfg.max_tokens:
                break
            keep.append(i)
            used += n
        if keep:
            print(f"Filtered dataset to {len(keep)} examples ({used} tokens) due to max_tokens limit.")
            return ds.select(keep)
        print("Warning: No examples fit within max_tokens limit.")
        return ds
    reps = cfg.max_tokens // total
    idx, used = list(range(len(ds))) * reps, total * reps
    for i, n in enumerate(lengths):
        if used + n > cfg.max_tokens:
            break
        idx.append(i)
        used += n
    print(f"Tiled dataset ~{reps}x to {len(idx)} examples ({used} tokens) to reach max_tokens={cfg.max_tokens}.")
    return ds.select(idx)


def max_tokens_for_model(tokenizer, model_str: str, revision: str | None) -> int:
    """min(tokenizer.model_max_length, config.max_position_embeddings)."""
    if model_str.startswith("native:"):
        return parse_native_spec(model_str)[0].max_position_embeddings
    from transformers import AutoConfig

    try:
        from peft import PeftConfig

        p = PeftConfig.from_pretrained(model_str)
        if p.base_model_name_or_path:
            model_str = p.base_model_name_or_path
    except Exception:
        pass
    mc = AutoConfig.from_pretrained(model_str, revision=revision)
    return min(getattr(tokenizer, "model_max_length", BIG_NUM), getattr(mc, "max_position_embeddings", BIG_NUM))


def _load_tokenizer(cfg: AttributionConfig):
    from transformers import AutoTokenizer

    return AutoTokenizer.from_pretrained(cfg.tokenizer or cfg.model)


def setup_data_pipeline(cfg: AttributionConfig, data_cfg: DataConfig | None = None) -> tuple[Dataset, int]:
    """Load, format, tokenise (unless ``input_ids`` is already present), add ``length``
    and ``advantage`` columns, apply ``max_tokens``, drop unused columns."""
    data_cfg = data_cfg or cfg.data
    ds = load_data_string(data_cfg.dataset, data_cfg.split, data_cfg.subset, data_cfg.data_kwargs)
    pretokenized = "input_ids" in (ds.column_names or [])
    tokenizer = None
    if not pretokenized or data_cfg.chunk_length > 0:
        tokenizer = _load_tokenizer(cfg)
    if tokenizer is not None or cfg.model.startswith("native:"):
        max_model_len = max_tokens_for_model(tokenizer, cfg.model, cfg.revision)
    else:
        try:
            max_model_len = max_tokens_for_model(None, cfg.model, cfg.revision)
        except Exception:
            max_model_len = BIG_NUM

    if data_cfg.chunk_length > 0:
        if data_cfg.chunk_length > max_model_len:
            raise ValueError(f"chunk_length {data_cfg.chunk_length} exceeds model's maximum context length {max_model_len}")
        return tokenize_and_chunk(ds, tokenizer, chunk_size=data_cfg.chunk_length), len(ds)

    token_bs = getattr(cfg, "token_batch_size", BIG_NUM)
    if BIG_NUM > token_bs > max_model_len:
        raise ValueError(
            f"Token batch size {token_bs} exceeds model max length ({max_model_len}). "
            f"Use --token_batch_size {max_model_len} or smaller."
        )
    max_length = min(max_model_len, token_bs)
    remove = set(ds.column_names) if cfg.drop_columns else set()
    tok_cfg = data_cfg
    if data_cfg.format_template:
        from ..format import apply_format

        ds = apply_format(ds, data_cfg.format_template)
        has_completion = "completion" in ds.column_names
        tok_cfg = DataConfig(prompt_column="prompt" if has_completion else "text",
                             completion_column="completion" if has_completion else "", truncation=data_cfg.truncation)
    if not pretokenized:
        ds = ds.map(tokenize, batched=True, fn_kwargs=dict(args=tok_cfg, tokenizer=tokenizer, max_length=max_length))
    if "length" not in ds.column_names:
        ds = ds.map(lambda b: {"length": [len(x) for x in b["input_ids"]]}, batched=True)
    if not data_cfg.truncation:
        longest = max(ds["length"])
        if longest > max_model_len:
            warnings.warn(f"Dataset contains a document longer than the model can handle ({longest} > {max_model_len}). "
                          "Consider using --truncation.")
        elif longest > token_bs:
            warnings.warn(f"Dataset contains a document longer than token_batch_size ({longest} > {token_bs}). "
                          "Consider increasing --token_batch_size or using --truncation.")
    if data_cfg.reward_column:
        rewards = np.array(ds[data_cfg.reward_column], dtype=np.float64)
        nan = np.isnan(rewards)
        if nan.any():
            if not data_cfg.skip_nan_rewards:
                raise ValueError(f"Reward column '{data_cfg.reward_column}' contains NaN values")
            print(f"Warning: Filtering out {nan.sum()} rows with NaN rewards")
            ds = ds.filter(lambda _, i: not nan[i], with_indices=True)
        ds = ds.add_column("advantage", estimate_advantage(ds, data_cfg), new_fingerprint="advantage")
    if cfg.max_tokens is not None:
        ds = filter_by_max_tokens(ds, cfg)
    remove = (remove - {"length", "input_ids", "labels"}) & set(ds.column_names)
    if remove:
        ds = ds.remove_columns(list(remove))
    return ds, len(ds)
