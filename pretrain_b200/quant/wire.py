"""Pre-quantized weights as a file / wire format: the codes and scale factors the kernels consume, written once and
loaded without touching the high-precision master weights.

The reference checkpoints only ``model.state_dict()`` (src/training/trainer.py:524-570) and re-quantizes every weight in
every forward (src/quant/linear.py:73-76).  This module adds, beside that and without changing it (``QuantLinear`` keeps
``weight`` / ``bias`` as its only state-dict entries), a container for the QUANTIZED form of the weights - for serving a
trained model without its bf16 weights on the wire, or for handing codes from the rank that quantized them to its peers.

Layout of a file (little endian):

    bytes 0..7    magic  b"B200QW" + two version bytes (0, 1)
    bytes 8..15   N = length of the JSON header in bytes
    bytes 16..    JSON header (UTF-8), zero-padded so that the payload starts on a multiple of 256
    payload       the blobs named by the header, each starting on a multiple of 256 relative to the payload start

    header = {"version": 1, "tensors": {name: entry}}
    entry  = {"format":  "mxfp8_e4m3" | "mxfp8_e5m2" | "nvfp4" | "fp8_e4m3" | "fp8_e5m2",
              "shape":   [rows, cols]        the weight as nn.Linear stores it, (out_features, in_features), or
                                             (experts * out, in) for an expert stack; blocks / scales run along cols
              "codes":   {"offset", "nbytes"}   rows x cols code bytes (cols / 2 for nvfp4: element 2i in the low nibble)
              "sf":      {"offset", "nbytes", "layout": "swizzle_128x4"}   block formats: E8M0 / E4M3 scale bytes in the
                                             128 x 4 tiled layout of include/b200q.h
              "scales":  {"offset", "nbytes"}   fp8 formats: one fp32 scale per row
              "tensor_scale": float | null}     nvfp4: the fp32 tensor scale

Codes and scale factors are exactly what ``b200q_quantize_*`` writes (axis = 1, swizzled scale factors), so a loaded
entry is an operand of ``b200q_gemm_*`` as it is."""

from __future__ import annotations

import io
import json
import struct
from dataclasses import dataclass
from typing import BinaryIO, Dict, Optional, Union

import torch

MAGIC = b"B200QW\x00\x01"
_ALIGN = 256
_E2M1 = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
_FP8 = {"mxfp8_e4m3": torch.float8_e4m3fn, "mxfp8_e5m2": torch.float8_e5m2, "mxfp8": torch.float8_e4m3fn,
        "fp8_e4m3": torch.float8_e4m3fn, "fp8_e5m2": torch.float8_e5m2, "fp8": torch.float8_e4m3fn}
_CANON = {"mxfp8": "mxfp8_e4m3", "fp8": "fp8_e4m3", "fp4_nv": "nvfp4"}
FORMATS = ("mxfp8_e4m3", "mxfp8_e5m2", "nvfp4", "fp8_e4m3", "fp8_e5m2")


@dataclass
class QuantizedWeight:
    """One weight in its quantized form.  ``codes`` uint8 (rows, cols) or (rows, cols / 2); ``sf`` uint8 flat swizzled
    buffer (block formats); ``scales`` fp32 (rows,) (fp8 formats); ``tensor_scale`` fp32 (1,) (nvfp4)."""
    format: str
    shape: tuple
    codes: torch.Tensor
    sf: Optional[torch.Tensor] = None
    scales: Optional[torch.Tensor] = None
    tensor_scale: Optional[torch.Tensor] = None

    def to(self, device) -> "QuantizedWeight":
        mv = lambda t: None if t is None else t.to(device)
        return QuantizedWeight(self.format, tuple(self.shape), mv(self.codes), mv(self.sf), mv(self.scales), mv(self.tensor_scale))


def canonical_format(fmt: str) -> str:
    fmt = _CANON.get(fmt, fmt)
    if fmt not in FORMATS:
        raise ValueError(f"no quantized weight format {fmt!r} (one of {', '.join(FORMATS)})")
    return fmt


def quantize_weight(weight: torch.Tensor, fmt: str) -> QuantizedWeight:
    """Quantize a 2-D weight (rows = out_features, blocks / scales along in_features) on the GPU kernels."""
    from .. import ops
    fmt = canonical_format(fmt)
    w = weight.detach()
    if w.dim() == 3:                                   # an expert stack (E, out, in) is stored as (E * out, in)
        w = w.reshape(-1, w.shape[-1])
    w = w.to(torch.bfloat16)
    if fmt.startswith("mxfp8"):
        codes, sf = ops.quantize_mxfp8(w, 1, ops.fmt_of(_FP8[fmt]), ops.SF_SWIZZLED)
        return QuantizedWeight(fmt, tuple(w.shape), codes, sf=sf)
    if fmt == "nvfp4":
        codes, sf, ts = ops.quantize_nvfp4(w, 1, None, ops.SF_SWIZZLED)
        return QuantizedWeight(fmt, tuple(w.shape), codes, sf=sf, tensor_scale=ts)
    codes, scales = ops.quantize_fp8(w, ops.fmt_of(_FP8[fmt]), 1)
    return QuantizedWeight(fmt, tuple(w.shape), codes, scales=scales)


def _unswizzle(sf: torch.Tensor, rows: int, nblk: int) -> torch.Tensor:
    kt = (nblk + 3) // 4
    r = torch.arange(rows, device=sf.device).unsqueeze(1)
    kb = torch.arange(nblk, device=sf.device).unsqueeze(0)
    return sf[((r // 128) * kt + kb // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + kb % 4]


def dequantize_weight(qw: QuantizedWeight, dtype=torch.bfloat16) -> torch.Tensor:
    """The values the codes stand for, in plain torch (any device): for checking a file, or for a consumer that has
    no block-scaled GEMM."""
    rows, cols = qw.shape
    fmt = qw.format
    if fmt.startswith("mxfp8"):
        sf = _unswizzle(qw.sf, rows, cols // 32)
        scale = torch.exp2(sf.float() - 127.0)
        v = qw.codes.view(_FP8[fmt]).float().view(rows, cols // 32, 32) * scale.unsqueeze(-1)
    elif fmt == "nvfp4":
        lut = torch.tensor(_E2M1 + [-x for x in _E2M1], device=qw.codes.device)
        vals = torch.stack((lut[(qw.codes & 0xF).long()], lut[(qw.codes >> 4).long()]), dim=-1).view(rows, cols)
        eff = _unswizzle(qw.sf, rows, cols // 16).view(torch.float8_e4m3fn).float() * qw.tensor_scale.float()
        v = vals.view(rows, cols // 16, 16) * eff.unsqueeze(-1)
    else:
        v = qw.codes.view(_FP8[fmt]).float() * qw.scales.float().view(-1, 1)
    return v.reshape(rows, cols).to(dtype)


def _pad(n: int) -> int:
    return (-n) % _ALIGN


def dump(tensors: Dict[str, QuantizedWeight], f: BinaryIO) -> None:
    """Write the container (see the module docstring) to a binary stream."""
    header, blobs, offset = {"version": 1, "tensors": {}}, [], 0

    def place(t: torch.Tensor) -> dict:
        nonlocal offset
        raw = t.detach().contiguous().cpu().view(torch.uint8).reshape(-1).numpy().tobytes()
        rec = {"offset": offset, "nbytes": len(raw)}
        blobs.append(raw + b"\x00" * _pad(len(raw)))
        offset += len(raw) + _pad(len(raw))
        return rec

    for name, qw in tensors.items():
        fmt = canonical_format(qw.format)
        entry = {"format": fmt, "shape": [int(s) for s in qw.shape], "codes": place(qw.codes),
                 "tensor_scale": None if qw.tensor_scale is None else float(qw.tensor_scale.float().item())}
        if qw.sf is not None:
            entry["sf"] = dict(place(qw.sf), layout="swizzle_128x4")
        if qw.scales is not None:
            entry["scales"] = place(qw.scales.float())
        header["tensors"][name] = entry
    hdr = json.dumps(header, sort_keys=True).encode()
    hdr += b" " * _pad(16 + len(hdr))
    f.write(MAGIC + struct.pack("<Q", len(hdr)) + hdr)
    for b in blobs:
        f.write(b)


def parse(data: Union[bytes, memoryview], device="cpu") -> Dict[str, QuantizedWeight]:
    """Read a container from bytes; raises ValueError on anything that is not one."""
    data = memoryview(data)
    if len(data) < 16 or bytes(data[:8]) != MAGIC:
        raise ValueError("not a b200q quantized-weight container (bad magic or version)")
    (n,) = struct.unpack("<Q", data[8:16])
    if 16 + n > len(data):
        raise ValueError("truncated container: header runs past the end")
    header = json.loads(bytes(data[16:16 + n]).decode())
    if header.get("version") != 1:
        raise ValueError(f"unsupported container version {header.get('version')!r}")
    base = 16 + n

    def blob(rec, dtype=torch.uint8) -> torch.Tensor:
        lo, hi = base + rec["offset"], base + rec["offset"] + rec["nbytes"]
        if hi > len(data):
            raise ValueError("truncated container: a blob runs past the end")
        t = torch.frombuffer(bytearray(data[lo:hi]), dtype=torch.uint8)
        return (t.view(dtype) if dtype != torch.uint8 else t).to(device)

    out = {}
    for name, e in header["tensors"].items():
        fmt = canonical_format(e["format"])
        rows, cols = e["shape"]
        codes = blob(e["codes"]).view(rows, cols // 2 if fmt == "nvfp4" else cols)
        out[name] = QuantizedWeight(
            fmt, (rows, cols), codes, sf=blob(e["sf"]) if "sf" in e else None,
            scales=blob(e["scales"], torch.float32) if "scales" in e else None,
            tensor_scale=None if e.get("tensor_scale") is None else torch.tensor([e["tensor_scale"]], dtype=torch.float32, device=device))
    return out


def save(tensors: Dict[str, QuantizedWeight], path: str) -> None:
    with open(path, "wb") as f:
        dump(tensors, f)


def load(path: str, device="cpu") -> Dict[str, QuantizedWeight]:
    with open(path, "rb") as f:
        return parse(f.read(), device)


def dumps(tensors: Dict[str, QuantizedWeight]) -> bytes:
    buf = io.BytesIO()
    dump(tensors, buf)
    return buf.getvalue()


def export_model(model: torch.nn.Module) -> Dict[str, QuantizedWeight]:
    """Quantized form of every weight the quantized layers of `model` would quantize at run time: each ``QuantLinear``'s
    weight in its rule's weight format, named as in the state dict (``<module>.weight``).  Layers whose weight format has
    no container form (the int8 series, passthrough formats) are left out."""
    from .linear import QuantLinear
    out = {}
    for name, mod in model.named_modules():
        if isinstance(mod, QuantLinear):
            fmt = _CANON.get(mod.cfg.dtype["weight"], mod.cfg.dtype["weight"])
            if fmt in FORMATS:
                out[f"{name}.weight" if name else "weight"] = quantize_weight(mod.weight, fmt)
    return out


def attach_to_model(model: torch.nn.Module, tensors: Dict[str, QuantizedWeight]) -> int:
    """Hand loaded entries to the ``QuantLinear`` modules they belong to (``QuantLinear.attach_quantized``): their
    gradient-free forward then multiplies by these codes instead of quantizing the master weight.  Returns how many
    were attached; the state dict is not touched."""
    from .linear import QuantLinear
    n = 0
    for name, mod in model.named_modules():
        key = f"{name}.weight" if name else "weight"
        if isinstance(mod, QuantLinear) and key in tensors:
            mod.attach_quantized(tensors[key])
            n += 1
    return n
