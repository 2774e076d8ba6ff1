"""``apply_quantization``: swap eligible ``nn.Linear`` modules for ``QuantLinear`` by rule
(counterpart of src/quant/convert.py).  Run it before ``torch.compile``."""

from __future__ import annotations

import warnings

import torch.nn as nn

from . import QUANT_PASSTHROUGH, fp8
from .linear import QuantLinear
from .utils import resolve_rule


def _quantizes(rule) -> bool:
    return any(fmt not in QUANT_PASSTHROUGH for fmt in rule.dtype.values())


def _check_hardware(rules) -> None:
    """Every quantized format of this build runs on sm_100 only; anything else is an error —
    there is no fallback path."""
    for rule in rules:
        if not rule.enabled:
            continue
        for fmt in rule.dtype.values():
            if fmt in QUANT_PASSTHROUGH:
                continue
            if not fp8.is_supported():
                raise RuntimeError(f"quant dtype {fmt!r} requires {fp8.HARDWARE_REQUIREMENT}. "
                                   "Disable quant or run on supported hardware.")


def apply_quantization(model: nn.Module, config) -> nn.Module:
    """In place.  ``config.training.quant`` is the rule list; each Linear takes the first enabled
    rule whose include/exclude patterns accept its qualified name.  Linears whose weight is
    tied to an embedding are left alone (with a warning).  No-op when no rule is enabled."""
    rules = config.training.quant
    if not any(rule.enabled for rule in rules):
        return model
    _check_hardware(rules)

    tied = {id(m.weight) for m in model.modules() if isinstance(m, nn.Embedding)}
    swaps = []
    for parent_name, parent in model.named_modules():
        for child_name, child in parent.named_children():
            if not isinstance(child, nn.Linear):
                continue
            fqn = f"{parent_name}.{child_name}" if parent_name else child_name
            rule = resolve_rule(fqn, rules)
            if rule is None or not _quantizes(rule):
                continue
            if id(child.weight) in tied:
                warnings.warn(f"quant: skipping {fqn!r} — its weight is tied to an embedding; "
                              "swapping would break the tie.")
                continue
            swaps.append((parent, child_name, child, rule))
    for parent, child_name, child, rule in swaps:
        setattr(parent, child_name, QuantLinear.from_linear(child, rule))
    return model
