"""Quantized-linear front end with the call signatures of gongyisheng/pretrain's ``src/quant``.

Keyword tables the config validates against.  They hold everything the reference's tables hold
(src/quant/__init__.py:15-44) plus the block-scaled formats its TODOs name: MXFP8 (``mxfp8``,
``mxfp8_e4m3``, ``mxfp8_e5m2``: 32-element blocks, E8M0 scales), NVFP4 (``nvfp4`` / ``fp4_nv``:
16-element blocks, E4M3 scales + fp32 tensor scale), granularity ``blockwise`` and the recipes
``mxfp8`` and ``nvfp4``.  Import-light on purpose: the config module imports this one.
"""

QUANT_PASSTHROUGH = frozenset({"fp32", "fp16", "bf16"})

FP8_FORMATS = frozenset({"fp8", "fp8_e4m3", "fp8_e5m2"})
MXFP8_FORMATS = frozenset({"mxfp8", "mxfp8_e4m3", "mxfp8_e5m2"})
NVFP4_FORMATS = frozenset({"nvfp4", "fp4_nv"})
INT8_SERIES = frozenset({"int8", "int7", "int6", "int5", "int4"})

QUANT_FORMATS = QUANT_PASSTHROUGH | FP8_FORMATS | MXFP8_FORMATS | NVFP4_FORMATS | INT8_SERIES

QUANT_GRANULARITY = frozenset({"tensorwise", "rowwise", "blockwise"})

QUANT_OPERANDS = ("weight", "act", "input_grad", "weight_grad")


def _uniform(fmt):
    return {operand: fmt for operand in QUANT_OPERANDS}


QUANT_DTYPE_RECIPES = {
    "fp8": {"weight": "fp8_e4m3", "act": "fp8_e4m3", "input_grad": "fp8_e5m2", "weight_grad": "fp8_e5m2"},
    "mxfp8": {"weight": "mxfp8_e4m3", "act": "mxfp8_e4m3", "input_grad": "mxfp8_e5m2", "weight_grad": "mxfp8_e5m2"},
    "nvfp4": _uniform("nvfp4"),
    **{fmt: _uniform(fmt) for fmt in sorted(INT8_SERIES)},
}

# block length implied by a block-scaled format
BLOCK_SIZE = {**{f: 32 for f in MXFP8_FORMATS}, **{f: 16 for f in NVFP4_FORMATS}}
