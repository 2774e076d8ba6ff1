"""Helpers for the GPU parity tests: device-side dequantisation (plain torch, fp32) of the
byte formats, used as the dequantize-then-matmul reference at sizes the CPU oracle is too
slow for.  Test infrastructure only."""

import torch

_E2M1 = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]


def sf_index(outer: int, nblk: int, device):
    kt = (nblk + 3) // 4
    r = torch.arange(outer, device=device).unsqueeze(1)
    kb = torch.arange(nblk, device=device).unsqueeze(0)
    return ((r // 128) * kt + kb // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + kb % 4


def unswizzle(sf_buf, outer, nblk):
    return sf_buf[sf_index(outer, nblk, sf_buf.device)]


def swizzle(sf_nat):
    outer, nblk = sf_nat.shape
    out = torch.zeros(((outer + 127) // 128) * ((nblk + 3) // 4) * 512, dtype=torch.uint8, device=sf_nat.device)
    out[sf_index(outer, nblk, sf_nat.device).reshape(-1)] = sf_nat.reshape(-1)
    return out


def deq_fp8(codes, dtype):
    return codes.view(dtype).float()


def deq_mxfp8(codes, sf_buf, dtype=torch.float8_e4m3fn, swizzled=True):
    outer, c = codes.shape
    sf = unswizzle(sf_buf, outer, c // 32) if swizzled else sf_buf.view(outer, c // 32)
    scale = torch.exp2(sf.float() - 127.0)
    return (codes.view(dtype).float().view(outer, c // 32, 32) * scale.unsqueeze(-1)).view(outer, c)


def deq_nvfp4(packed, sf_buf, ts, swizzled=True):
    outer, half = packed.shape
    c = half * 2
    lut = torch.tensor(_E2M1 + [-v for v in _E2M1], device=packed.device)
    vals = torch.stack((lut[(packed & 0xF).long()], lut[(packed >> 4).long()]), dim=-1).view(outer, c)
    sf = unswizzle(sf_buf, outer, c // 16) if swizzled else sf_buf.view(outer, c // 16)
    eff = sf.view(torch.float8_e4m3fn).float() * ts.float()
    return (vals.view(outer, c // 16, 16) * eff.unsqueeze(-1)).view(outer, c)


def matmul_fp32(a, b):
    """A . B^T with true fp32 accumulation (TF32 off)."""
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        return a.float() @ b.float().t()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def rel_errors(out, ref):
    out, ref = out.float(), ref.float()
    return ((out - ref).abs().max() / ref.abs().max()).item(), ((out - ref).norm() / ref.norm()).item()
