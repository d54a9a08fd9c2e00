"""Loader and thin typed wrappers of the in-tree sm_100a extension.

The extension is compiled in-tree by ``bergson_b200.ops.build`` (``nvcc -gencode
arch=compute_100a,code=sm_100a``) into ``bergson_b200/ops/_build``.  On a machine
with a GPU a missing or unloadable extension is an error, not a silent fallback:
``available()`` raises there unless ``BERGSON_B200_ALLOW_FALLBACK=1`` is set.
"""

from __future__ import annotations

import importlib.util
import os
from pathlib import Path

import torch

_BUILD_DIR = Path(__file__).resolve().parent / "_build"
_EXT_NAME = "bergson_b200_C"
_mod = None
_load_error: Exception | None = None


def extension_path() -> Path:
    return _BUILD_DIR / f"{_EXT_NAME}.so"


def _load():
    global _mod, _load_error
    if _mod is not None or _load_error is not None:
        return _mod
    so = extension_path()
    try:
        if not so.exists():
            raise FileNotFoundError(
                f"{so} not found; build it with `python -m bergson_b200.ops.build`"
            )
        spec = importlib.util.spec_from_file_location(_EXT_NAME, so)
        assert spec and spec.loader
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _mod = mod
    except Exception as e:  # noqa: BLE001 - reported below
        _load_error = e
    return _mod


def available() -> bool:
    """Whether the fused kernels can run in this process."""
    if not torch.cuda.is_available():
        return False
    if os.environ.get("BERGSON_B200_DISABLE_NATIVE") == "1":
        return False
    mod = _load()
    if mod is None:
        if os.environ.get("BERGSON_B200_ALLOW_FALLBACK") == "1":
            return False
        raise RuntimeError(
            "A CUDA device is present but the bergson_b200 sm_100a extension could not "
            f"be loaded ({_load_error!r}). Build it with `python -m bergson_b200.ops.build` "
            "or set BERGSON_B200_ALLOW_FALLBACK=1 to run the slow torch path."
        )
    return True


def ext():
    """The loaded extension module (raises if unavailable)."""
    mod = _load()
    if mod is None:
        raise RuntimeError(f"bergson_b200 extension unavailable: {_load_error!r}")
    return mod


_launches = 0
# Number of kernel launches behind one call of each extension function (helpers such as the
# reduction of per-block partial sums are torch ops and are not counted).
_KERNELS_PER_CALL = {"kernel_status": 0}


def launch_count() -> int:
    """Kernel launches issued through this module since the last ``reset_launch_count``."""
    return _launches


def reset_launch_count() -> None:
    global _launches
    _launches = 0


def __getattr__(name: str):
    # ``native.rmsnorm_fwd(...)`` forwards to the extension's function of that name and
    # counts the launch.
    fn = getattr(ext(), name)
    per_call = _KERNELS_PER_CALL.get(name, 1)

    def counted(*args, **kwargs):
        global _launches
        _launches += per_call
        return fn(*args, **kwargs)

    counted.__name__ = name
    globals()[name] = counted
    return counted
