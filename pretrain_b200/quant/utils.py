"""Format predicates and rule matching (counterparts of src/quant/utils.py)."""

from __future__ import annotations

import fnmatch
from typing import Optional

import torch

from . import FP8_FORMATS, INT8_SERIES, MXFP8_FORMATS, NVFP4_FORMATS
from .config import QuantConfig

_E5M2_NAMES = {"fp8_e5m2", "mxfp8_e5m2"}


def is_fp8(fmt: str) -> bool:
    return fmt in FP8_FORMATS


def is_mxfp8(fmt: str) -> bool:
    return fmt in MXFP8_FORMATS


def is_nvfp4(fmt: str) -> bool:
    return fmt in NVFP4_FORMATS


def is_int8s(fmt: str) -> bool:
    return fmt in INT8_SERIES


def is_quantized(fmt: str) -> bool:
    return is_fp8(fmt) or is_mxfp8(fmt) or is_nvfp4(fmt) or is_int8s(fmt)


def str_to_dtype_fp8(fmt: str) -> Optional[torch.dtype]:
    """Element dtype of an fp8 or mxfp8 format name (None for anything else)."""
    if not (is_fp8(fmt) or is_mxfp8(fmt)):
        return None
    return torch.float8_e5m2 if fmt in _E5M2_NAMES else torch.float8_e4m3fn


def str_to_qmax_int8s(fmt: str) -> Optional[int]:
    return (1 << (int(fmt[3:]) - 1)) - 1 if is_int8s(fmt) else None


def _matches(fqn: str, patterns) -> bool:
    leaf = fqn.rsplit(".", 1)[-1]
    return any(fnmatch.fnmatch(fqn, p) or fnmatch.fnmatch(leaf, p) for p in patterns)


def should_quantize(fqn: str, cfg: QuantConfig) -> bool:
    """A module is taken when it matches ``include`` (if any is given) and no ``exclude``
    pattern; patterns match the full name or its last component."""
    if cfg.include and not _matches(fqn, cfg.include):
        return False
    return not _matches(fqn, cfg.exclude)


def resolve_rule(fqn: str, rules) -> Optional[QuantConfig]:
    """First enabled rule that takes the module."""
    return next((r for r in rules if r.enabled and should_quantize(fqn, r)), None)
