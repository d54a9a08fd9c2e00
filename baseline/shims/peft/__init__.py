"""Stand-in for ``peft``: the names the reference imports; no adapter support."""

import enum


class PeftModel:  # only used in isinstance checks and annotations
    pass


class PeftConfig:
    @classmethod
    def from_pretrained(cls, *a, **k):
        raise ValueError("peft is not installed")


class PeftType(str, enum.Enum):
    LORA = "LORA"


def get_peft_model(*a, **k):
    raise ImportError("peft is not installed")


def get_peft_model_state_dict(*a, **k):
    raise ImportError("peft is not installed")
