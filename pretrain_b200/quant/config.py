"""``QuantConfig`` with the fields, defaults and validation errors of the reference's
(src/utils/config.py:285-325), extended by ``blockwise`` granularity, and the rule-list
normalisation the reference's ``TrainingConfig`` applies (src/utils/config.py:366-376)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

from . import (BLOCK_SIZE, FP8_FORMATS, QUANT_DTYPE_RECIPES, QUANT_FORMATS, QUANT_GRANULARITY, QUANT_OPERANDS)


@dataclass
class QuantConfig:
    enabled: bool = False
    dtype_recipe: Optional[str] = None
    dtype: dict = field(default_factory=dict)      # operand -> format
    scaling: dict = field(default_factory=dict)    # {granularity, block_size}
    include: List[str] = field(default_factory=list)
    exclude: List[str] = field(default_factory=lambda: ["lm_head"])

    def __post_init__(self):
        if not self.enabled:
            return
        if self.dtype_recipe is not None:
            recipe = QUANT_DTYPE_RECIPES.get(self.dtype_recipe)
            if recipe is None:
                raise ValueError(f"unknown quant dtype_recipe: {self.dtype_recipe!r}; "
                                 f"expected one of {sorted(QUANT_DTYPE_RECIPES)}")
            for operand, fmt in recipe.items():
                self.dtype.setdefault(operand, fmt)      # an explicit per-operand format wins

        block_fmts = [f for f in self.dtype.values() if f in BLOCK_SIZE]
        self.scaling.setdefault("granularity", "blockwise" if block_fmts else "tensorwise")
        granularity = self.scaling["granularity"]
        if granularity not in QUANT_GRANULARITY:
            raise ValueError(f"unknown quant granularity: {granularity!r}; expected one of {sorted(QUANT_GRANULARITY)}")

        for operand, fmt in self.dtype.items():
            if operand not in QUANT_OPERANDS:
                raise ValueError(f"unknown quant dtype key: {operand!r}; expected one of {sorted(QUANT_OPERANDS)}")
            if fmt not in QUANT_FORMATS:
                raise ValueError(f"unknown quant fmt for {operand}: {fmt!r}; expected one of {sorted(QUANT_FORMATS)}")

        if granularity == "blockwise":
            # plain fp8 formats under blockwise scaling mean their MX form
            for operand, fmt in list(self.dtype.items()):
                if fmt in FP8_FORMATS:
                    self.dtype[operand] = "mxfp8_e5m2" if fmt == "fp8_e5m2" else "mxfp8_e4m3"
            sizes = {BLOCK_SIZE[f] for f in self.dtype.values() if f in BLOCK_SIZE}
            if len(sizes) > 1:
                raise ValueError(f"quant formats with different block sizes in one rule: {sorted(sizes)}")
            implied = sizes.pop() if sizes else 32
            if self.scaling.setdefault("block_size", implied) != implied:
                raise ValueError(f"quant block_size {self.scaling['block_size']!r} does not match the "
                                 f"format's block size {implied}")
        elif block_fmts:
            raise ValueError(f"quant formats {sorted(set(block_fmts))} need granularity 'blockwise', got {granularity!r}")


def normalize_quant_rules(quant, mixed_precision: str = "bf16") -> list:
    """dict | QuantConfig | list of either -> list of QuantConfig; operands an enabled rule leaves
    unset take the AMP dtype ("fp32" when mixed precision is off)."""
    rules = quant if isinstance(quant, list) else [quant]
    amp = "fp32" if mixed_precision == "no" else mixed_precision
    out = []
    for rule in rules:
        if isinstance(rule, dict):
            rule = QuantConfig(**rule)
        if rule.enabled:
            for operand in QUANT_OPERANDS:
                rule.dtype.setdefault(operand, amp)
        out.append(rule)
    return out


@dataclass
class TrainingConfig:
    """The slice of the reference's ``TrainingConfig`` that the quantized-linear path reads
    (src/utils/config.py:349, :366-376): the AMP dtype and the ``quant`` rule list."""

    mixed_precision: str = "bf16"
    quant: object = field(default_factory=QuantConfig)

    def __post_init__(self):
        self.quant = normalize_quant_rules(self.quant, self.mixed_precision)
