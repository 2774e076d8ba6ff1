"""The pre-quantized weight container (pretrain_b200/quant/wire.py): byte layout and round trip on the CPU; on the GPU,
codes that went through a file multiply to the same bits as freshly quantized ones, and the nn.Linear-compatible state
dict (what the reference checkpoints, src/training/trainer.py:524-570) is untouched."""

import io
import json
import struct

import pytest
import torch
import torch.nn as nn

from pretrain_b200.quant import wire

E4 = torch.float8_e4m3fn


def _synthetic():
    g = torch.Generator().manual_seed(0)
    u8 = lambda *s: torch.randint(0, 127, s, generator=g, dtype=torch.int32).to(torch.uint8)
    rows, cols = 160, 96
    sfn = lambda nblk: ((rows + 127) // 128) * ((nblk + 3) // 4) * 512
    return {
        "blk.0.up.weight": wire.QuantizedWeight("mxfp8_e4m3", (rows, cols), u8(rows, cols), sf=u8(sfn(cols // 32))),
        "blk.0.down.weight": wire.QuantizedWeight("nvfp4", (rows, cols), u8(rows, cols // 2), sf=u8(sfn(cols // 16)),
                                                  tensor_scale=torch.tensor([0.0123])),
        "head.weight": wire.QuantizedWeight("fp8_e5m2", (rows, cols), u8(rows, cols), scales=torch.rand(rows, generator=g)),
    }


def test_container_round_trip_and_layout():
    tensors = _synthetic()
    data = wire.dumps(tensors)
    assert data[:8] == b"B200QW\x00\x01"
    (n,) = struct.unpack("<Q", data[8:16])
    assert (16 + n) % 256 == 0
    header = json.loads(data[16:16 + n].decode())
    assert header["version"] == 1 and sorted(header["tensors"]) == sorted(tensors)
    for e in header["tensors"].values():
        for key in ("codes", "sf", "scales"):
            if key in e:
                assert e[key]["offset"] % 256 == 0
    assert header["tensors"]["blk.0.up.weight"]["sf"]["layout"] == "swizzle_128x4"
    back = wire.parse(data)
    for name, qw in tensors.items():
        got = back[name]
        assert got.format == qw.format and tuple(got.shape) == tuple(qw.shape) and torch.equal(got.codes, qw.codes)
        for field in ("sf", "scales", "tensor_scale"):
            a, b = getattr(got, field), getattr(qw, field)
            assert (a is None) == (b is None) and (a is None or torch.equal(a, b))
    # a file on disk is the same bytes
    buf = io.BytesIO()
    wire.dump(tensors, buf)
    assert buf.getvalue() == data


def test_container_rejects_what_it_is_not():
    data = wire.dumps(_synthetic())
    with pytest.raises(ValueError, match="magic"):
        wire.parse(b"B200QW\x00\x02" + data[8:])
    with pytest.raises(ValueError, match="truncated"):
        wire.parse(data[:-300])
    with pytest.raises(ValueError, match="truncated"):
        wire.parse(data[:40])
    with pytest.raises(ValueError):
        wire.canonical_format("int8")


def test_dequantize_follows_the_format_definitions():
    rows, cols = 128, 64
    codes = torch.full((rows, cols), 0x38, dtype=torch.uint8)              # E4M3 1.0
    sf = torch.zeros(512, dtype=torch.uint8)
    nat = torch.full((rows, 2), 127, dtype=torch.uint8)
    nat[5, 1] = 130                                                        # one block scaled by 2^3
    r = torch.arange(rows).unsqueeze(1); kb = torch.arange(2).unsqueeze(0)
    sf[((r // 128) * 1 + kb // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + kb % 4] = nat
    w = wire.dequantize_weight(wire.QuantizedWeight("mxfp8_e4m3", (rows, cols), codes, sf=sf), torch.float32)
    want = torch.ones(rows, cols); want[5, 32:] = 8.0
    assert torch.equal(w, want)
    packed = torch.full((rows, cols // 2), 0x2A, dtype=torch.uint8)        # low nibble 0xA = -1.0, high nibble 0x2 = +1.0
    sf4 = torch.full((512,), 0x38, dtype=torch.uint8)
    w4 = wire.dequantize_weight(wire.QuantizedWeight("nvfp4", (rows, cols), packed, sf=sf4, tensor_scale=torch.tensor([0.5])), torch.float32)
    assert torch.equal(w4[:, 0::2], torch.full((rows, cols // 2), -0.5)) and torch.equal(w4[:, 1::2], torch.full((rows, cols // 2), 0.5))
    w8 = wire.dequantize_weight(wire.QuantizedWeight("fp8_e4m3", (rows, cols), codes, scales=torch.arange(rows).float()), torch.float32)
    assert torch.equal(w8, torch.arange(rows).float().view(-1, 1).expand(rows, cols))


@pytest.mark.gpu
@pytest.mark.parametrize("recipe,granularity", [("mxfp8", None), ("nvfp4", None), ("fp8", "rowwise")])
def test_weights_through_a_file_give_the_same_bits(tmp_path, recipe, granularity):
    from pretrain_b200 import build
    from pretrain_b200.quant.config import TrainingConfig
    from pretrain_b200.quant.convert import apply_quantization
    build.build()
    torch.manual_seed(0)
    q = {"enabled": True, "dtype_recipe": recipe}
    if granularity:
        q["scaling"] = {"granularity": granularity}
    cfg = type("Cfg", (), {"training": TrainingConfig(quant=q)})()
    model = nn.Sequential(nn.Linear(256, 384, bias=True), nn.Linear(384, 128, bias=False)).cuda().bfloat16()
    keys_before = list(model.state_dict())
    apply_quantization(model, cfg)
    x = torch.randn(64, 256, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        want = model(x)
    tensors = wire.export_model(model)
    assert sorted(tensors) == ["0.weight", "1.weight"]
    path = str(tmp_path / "w.b200q")
    wire.save(tensors, path)
    loaded = wire.load(path, "cuda")
    for k in tensors:
        assert torch.equal(loaded[k].codes, tensors[k].codes)
        deq = wire.dequantize_weight(loaded[k]).float()
        ref = model.state_dict()[k].float()
        assert ((deq - ref).norm() / ref.norm()).item() < (0.12 if recipe == "nvfp4" else 0.05)
    assert wire.attach_to_model(model, loaded) == 2
    with torch.no_grad():
        got = model(x)
    assert torch.equal(got, want)                                     # same codes, same GEMM: same bits
    assert list(model.state_dict()) == keys_before                    # still the nn.Linear state dict
    assert all(v.dtype == torch.bfloat16 for v in model.state_dict().values())
    # training ignores the attachment, and a weight update drops it
    model(x.requires_grad_(True)).float().sum().backward()
    with torch.no_grad():
        model[0].weight.add_(0.01)
        model(x.detach())
    assert model[0]._packed is None and model[1]._packed is not None
    model[1].post_step()
    assert model[1]._packed is None
