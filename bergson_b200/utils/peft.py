"""PEFT adapter helpers (optional dependency)."""

from __future__ import annotations


def set_peft_enabled(model, enabled: bool) -> None:
    """Enable or disable every adapter layer of a PEFT model."""
    for m in model.modules():
        if hasattr(m, "enable_adapters") and callable(m.enable_adapters) and m is not model:
            try:
                m.enable_adapters(enabled)
            except TypeError:
                pass


def extract_peft_target_modules(model) -> set[str]:
    """Names (relative to ``base_model``) of the adapter sub-modules."""
    from peft import get_peft_model_state_dict

    out: set[str] = set()
    state = get_peft_model_state_dict(model=model)
    for adapter in model.peft_config.keys():
        for name in state:
            candidate = f"{name.removesuffix('.weight')}.{adapter}".removeprefix("base_model.")
            try:
                model.get_submodule(candidate)
                out.add(candidate)
            except AttributeError:
                print(f"Adapter parameter '{candidate}' not found in the model.")
    return out


def detect_peft_modules(model) -> set[str]:
    """Like ``extract_peft_target_modules`` but strict: an adapter parameter without a matching
    sub-module is an error rather than a printed note (reference ``bergson/utils/peft.py:5-30``)."""
    from peft import get_peft_model_state_dict

    out: set[str] = set()
    state = get_peft_model_state_dict(model)
    for adapter in model.peft_config:
        for name in state:
            candidate = f"{name.removesuffix('.weight')}.{adapter}".removeprefix("base_model.")
            try:
                model.get_submodule(candidate)
            except AttributeError as e:
                raise RuntimeError(f"Adapter parameter '{candidate}' not found in the model.") from e
            out.add(candidate)
    return out
