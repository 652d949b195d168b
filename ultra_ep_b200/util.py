"""Environment readers and dtype helpers used by the configuration layer."""

from __future__ import annotations

import os

import torch

_TRUTHY = {"1", "true", "yes", "on"}
_FALSY = {"0", "false", "no", "off"}


def check_dtype(name: str, dtype) -> torch.dtype:
    if not isinstance(dtype, torch.dtype):
        raise TypeError(f"{name} must be a torch.dtype, got {type(dtype).__name__}")
    return dtype


def dtype_element_size(dtype: torch.dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


def print_rank_0(message) -> None:
    import torch.distributed as dist

    if dist.is_initialized() and dist.get_rank() == 0:
        print(message, flush=True)


def read_env(name: str):
    """The variable's value stripped of blanks, or None when unset or empty."""
    raw = os.environ.get(name)
    if raw is None:
        return None
    raw = raw.strip()
    return raw or None


def read_bool_env(name: str, default: bool) -> bool:
    raw = read_env(name)
    if raw is None:
        return default
    low = raw.lower()
    if low in _TRUTHY:
        return True
    if low in _FALSY:
        return False
    raise ValueError(f"{name} must be one of: 0/1, true/false, yes/no, on/off")


def read_int_env(name: str, default: int) -> int:
    raw = read_env(name)
    return default if raw is None else int(raw)


def read_float_env(name: str, default: float) -> float:
    raw = read_env(name)
    return default if raw is None else float(raw)


def read_str_env(name: str, default: str) -> str:
    raw = read_env(name)
    return default if raw is None else raw
