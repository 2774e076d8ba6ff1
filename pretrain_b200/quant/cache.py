"""Quantized copies of a weight, kept on the parameter between the steps that write it.

The reference re-quantizes every weight in every forward and again in every backward
(src/quant/linear.py:73-76,98); here a parameter's codes are made once and reused until the
parameter changes.  "Changes" is detected through the tensor's version counter, its storage
address and its dtype - which covers every in-place op and ``optimizer.step()`` of the stock
optimizers, but NOT a write through ``param.data`` (``p.data.add_(...)``, ``p.data.copy_(...)``,
``p.data[i] = ...``): those leave the version counter alone.  Three things cover that case:

* ``post_step()`` of ``QuantLinear`` and ``SparseMoEBlock`` drops the copies; the reference's
  training loop calls ``model.post_step()`` after every optimizer step
  (src/training/trainer.py:367, src/model/transformer.py:144-147), so under that loop the copies
  never outlive a step whatever the optimizer does;
* ``invalidate(module_or_parameter)`` drops them on request (after an EMA swap, a manual
  ``.data`` edit, loading a checkpoint into ``.data``);
* ``B200Q_WEIGHT_CACHE=0`` in the environment turns the reuse off altogether.
"""

from __future__ import annotations

import os

import torch
import torch.nn as nn

_PREFIX = "_b200q_"


def enabled() -> bool:
    return os.environ.get("B200Q_WEIGHT_CACHE", "1") != "0"


def cached(param: torch.Tensor, slot: str, key, make):
    """`make()` once per state of `param`: the result is kept in attribute ``_b200q_<slot>`` of the
    parameter together with (version, address, dtype, key) and reused while those match.  Tensors
    that are not parameters, and every call under ``torch.compile``, are not cached."""
    if torch.compiler.is_compiling() or not isinstance(param, nn.Parameter) or not enabled():
        return make()
    full = (param._version, param.data_ptr(), param.dtype, key)
    name = _PREFIX + slot
    hit = getattr(param, name, None)
    if hit is None or hit[0] != full:
        with torch.no_grad():
            hit = (full, make())
        setattr(param, name, hit)
    return hit[1]


def invalidate(obj) -> int:
    """Drop every cached quantized copy held by a parameter, or by all parameters of a module.
    Returns how many were dropped."""
    params = obj.parameters() if isinstance(obj, nn.Module) else [obj]
    dropped = 0
    for p in params:
        for name in [n for n in vars(p) if n.startswith(_PREFIX)]:
            delattr(p, name)
            dropped += 1
    return dropped
