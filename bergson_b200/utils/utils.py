"""Small helpers shared across the package: dtype bridges between torch and numpy
(bf16 via ml_dtypes), device/backend selection, the ``a=b,c=d|e`` kwargs
mini-language (reference ``bergson/utils/utils.py:57-273``)."""

from __future__ import annotations

import os
import random
import warnings
from typing import Any, Type, TypeVar

import ml_dtypes
import numpy as np
import torch
from torch import Tensor, nn

T = TypeVar("T")
np_bfloat16 = np.dtype(ml_dtypes.bfloat16)

_PRECISIONS = {
    "bf16": torch.bfloat16,
    "fp16": torch.float16,
    "fp32": torch.float32,
    "fp64": torch.float64,
}
_DTYPE_RANK = {torch.float64: 0, torch.float32: 1, torch.float16: 2, torch.bfloat16: 3}


def assert_type(typ: Type[T], obj: Any) -> T:
    if not isinstance(obj, typ):
        raise TypeError(f"Expected {typ.__name__}, got {type(obj).__name__}")
    return obj


def get_layer_list(model) -> nn.ModuleList:
    """The ``nn.ModuleList`` holding the transformer blocks."""
    n = assert_type(int, model.config.num_hidden_layers)
    found = [
        m
        for m in model.base_model.modules()
        if isinstance(m, nn.ModuleList) and len(m) == n
    ]
    assert len(found) == 1, "Could not find the list of layers."
    return found[0]


def setup_reproducibility(seed: int = 42) -> None:
    """Fix seeds and force deterministic algorithms (debug mode)."""
    print("WARNING: Running in debug mode, much slower performance expected.")
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    os.environ["PYTHONHASHSEED"] = str(seed)
    os.environ["CUDA_LAUNCH_BLOCKING"] = "1"
    os.environ["CUBLAS_WORKSPACE_CONFIG"] = ":4096:8"
    torch.backends.cudnn.deterministic = True
    torch.backends.cudnn.benchmark = False
    torch.use_deterministic_algorithms(True)


def handle_arg_string(arg: str):
    """Parse one value of the kwargs mini-language (``|`` separates list items)."""
    if "|" in arg:
        return [handle_arg_string(v) for v in arg.split("|")]
    for cast in (int, float):
        try:
            return cast(arg)
        except ValueError:
            pass
    low = arg.lower()
    if low in ("true", "false"):
        return low == "true"
    return arg


def simple_parse_kwargs_string(args_string: str) -> dict:
    """``"a=1,b=x|y"`` -> ``{"a": 1, "b": ["x", "y"]}``."""
    out: dict[str, Any] = {}
    if not args_string.strip():
        return out
    for elem in args_string.split(","):
        key, sep, val = elem.partition("=")
        key, val = key.strip(), val.strip()
        if not (key and sep):
            raise ValueError(f"Invalid argument: '{elem}'. Expected format key=value.")
        if not key.isidentifier():
            raise ValueError(f"Invalid key: '{key}'. Must be a valid identifier.")
        out[key] = handle_arg_string(val)
    return out


def get_gradient_dtype(model) -> torch.dtype:
    """Dtype of the trainable floating-point parameters (widest if mixed)."""
    dtypes = {
        p.dtype for p in model.parameters() if p.requires_grad and p.dtype.is_floating_point
    }
    if not dtypes:
        dtypes = {p.dtype for p in model.parameters() if p.dtype.is_floating_point}
    assert dtypes, "No floating-point parameters found"
    return sorted(dtypes, key=lambda d: _DTYPE_RANK.get(d, 99))[0]


def tensor_to_numpy(tensor: Tensor) -> np.ndarray:
    """CPU tensor -> numpy, bit-exact for bfloat16."""
    if tensor.dtype != torch.bfloat16:
        return tensor.numpy()
    return tensor.view(torch.uint16).numpy().view(np_bfloat16)


def numpy_to_tensor(arr: np.ndarray) -> Tensor:
    """numpy -> tensor, bit-exact for ml_dtypes bfloat16 (and 2-byte void views)."""
    if arr.dtype == np_bfloat16 or arr.dtype.str == "|V2":
        return torch.from_numpy(arr.view(np.uint16).copy()).view(torch.bfloat16)
    if not arr.flags.writeable:
        # A read-only memory map: the tensor is only ever read, so torch's warning about writes
        # through a non-writable array does not apply.
        with warnings.catch_warnings():
            warnings.filterwarnings("ignore", message="The given NumPy array is not writable")
            return torch.from_numpy(arr)
    return torch.from_numpy(arr)


def convert_dtype_to_np(dtype: torch.dtype) -> np.dtype:
    table = {
        torch.float16: np.dtype(np.float16),
        torch.float32: np.dtype(np.float32),
        torch.float64: np.dtype(np.float64),
        torch.bfloat16: np_bfloat16,
    }
    if dtype not in table:
        raise ValueError(f"Unsupported torch dtype: {dtype}")
    return table[dtype]


def convert_dtype_to_torch(dtype) -> torch.dtype:
    dtype = np.dtype(dtype)
    table = {
        np.dtype(np.float16): torch.float16,
        np.dtype(np.float32): torch.float32,
        np.dtype(np.float64): torch.float64,
        np_bfloat16: torch.bfloat16,
    }
    if dtype not in table:
        raise ValueError(f"Unsupported numpy dtype: {dtype}")
    return table[dtype]


def convert_precision_to_torch(precision: str) -> torch.dtype:
    if precision not in _PRECISIONS:
        raise ValueError(f"Precision {precision!r} has no torch dtype.")
    return _PRECISIONS[precision]


def get_device_index(rank: int = 0) -> int:
    """CUDA index for a local rank; 0 when the process sees a single GPU."""
    if torch.cuda.is_available() and torch.cuda.device_count() == 1:
        return 0
    return rank


def get_device(rank: int = 0) -> str:
    return f"cuda:{get_device_index(rank)}" if torch.cuda.is_available() else "cpu"


def current_device() -> torch.device:
    if not torch.cuda.is_available():
        return torch.device("cpu")
    return torch.device("cuda", torch.cuda.current_device())


def dist_backend(mixed: bool = False) -> str:
    if not torch.cuda.is_available():
        return "gloo"
    return "cpu:gloo,cuda:nccl" if mixed else "nccl"


def dist_device_id(rank: int = 0) -> torch.device | None:
    return torch.device(get_device(rank)) if torch.cuda.is_available() else None
