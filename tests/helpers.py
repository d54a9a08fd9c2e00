"""Shared fixtures-as-functions for the CPU tests."""

import torch
import torch.nn as nn
from datasets import Dataset

from bergson_b200.config import IndexConfig
from bergson_b200.models import build_model
from bergson_b200.models.registry import PRESETS, args_from_dict


class TwoLayer(nn.Module):
    """fc1 -> relu -> fc2 on [N, S, I] inputs; ``device`` like an HF model."""

    def __init__(self, i=5, h=3, o=2, bias=True):
        super().__init__()
        self.fc1 = nn.Linear(i, h, bias=bias)
        self.relu = nn.ReLU()
        self.fc2 = nn.Linear(h, o, bias=bias)

    @property
    def device(self):
        return self.fc1.weight.device

    def forward(self, x):
        return self.fc2(self.relu(self.fc1(x)))


def tiny_model(family="gpt_neox", dtype=torch.float32, **over):
    base = dict(PRESETS[{"gpt_neox": "neox-tiny", "llama": "llama-tiny", "gpt2": "gpt2-tiny"}[family]])
    base.update(dict(vocab_size=128, num_hidden_layers=2), **over)
    if family == "gpt_neox":
        base.update(hidden_size=32, intermediate_size=64, num_attention_heads=4)
    return build_model(args_from_dict(base), dtype=dtype)


def tiny_dataset(n=8, length=12, vocab=128, seed=0, ragged=True):
    g = torch.Generator().manual_seed(seed)
    ids = []
    for i in range(n):
        L = int(torch.randint(4, length + 1, (1,), generator=g)) if ragged else length
        ids.append(torch.randint(0, vocab, (L,), generator=g).tolist())
    return Dataset.from_dict({"input_ids": ids, "length": [len(x) for x in ids]})


def index_cfg(run_path, **kw):
    base = dict(run_path=str(run_path), model="native:unused", token_batch_size=64)
    base.update(kw)
    return IndexConfig(**base)
