"""Host logic of the quantized-linear front end (config, rule matching, converter): the cases
the reference's own tests cover (tests/fast/utils/test_config.py:712-872,
tests/fast/quant/test_utils.py, tests/fast/quant/test_converter.py), plus the block-scaled
extensions.  No GPU needed."""

from types import SimpleNamespace

import pytest
import torch
import torch.nn as nn

from pretrain_b200.quant import QUANT_DTYPE_RECIPES, QUANT_FORMATS, QUANT_GRANULARITY
from pretrain_b200.quant.config import QuantConfig, TrainingConfig
from pretrain_b200.quant.convert import apply_quantization
from pretrain_b200.quant.linear import QuantLinear
from pretrain_b200.quant.utils import (is_fp8, is_mxfp8, is_nvfp4, is_quantized, resolve_rule, should_quantize,
                                       str_to_dtype_fp8, str_to_qmax_int8s)


def _only(tc):
    assert len(tc.quant) == 1
    return tc.quant[0]


def test_defaults_disabled_and_inert():
    q = QuantConfig()
    assert q.enabled is False and q.exclude == ["lm_head"] and q.include == []
    assert q.dtype == {} and q.scaling == {}
    QuantConfig(enabled=False, dtype={"weight": "not_a_fmt"})     # not validated when off


def test_operand_defaults_follow_mixed_precision():
    r = _only(TrainingConfig(mixed_precision="bf16", quant={"enabled": True}))
    assert r.dtype == {k: "bf16" for k in ("weight", "act", "input_grad", "weight_grad")}
    assert _only(TrainingConfig(mixed_precision="no", quant={"enabled": True})).dtype["weight"] == "fp32"
    r2 = _only(TrainingConfig(quant={"enabled": True, "dtype": {"weight": "fp8"}}))
    assert r2.dtype == {"weight": "fp8", "act": "bf16", "input_grad": "bf16", "weight_grad": "bf16"}
    assert _only(TrainingConfig(quant={"enabled": False})).dtype == {}


def test_fp8_recipe_and_overrides():
    q = QuantConfig(enabled=True, dtype_recipe="fp8")
    assert q.dtype == {"weight": "fp8_e4m3", "act": "fp8_e4m3", "input_grad": "fp8_e5m2", "weight_grad": "fp8_e5m2"}
    assert q.scaling["granularity"] == "tensorwise"
    q = QuantConfig(enabled=True, dtype_recipe="fp8", dtype={"weight_grad": "bf16"})
    assert q.dtype["weight"] == "fp8_e4m3" and q.dtype["weight_grad"] == "bf16" and q.dtype["input_grad"] == "fp8_e5m2"
    q = QuantConfig(enabled=True, dtype_recipe="fp8", scaling={"granularity": "rowwise"})
    assert q.scaling["granularity"] == "rowwise"


def test_validation_errors():
    with pytest.raises(ValueError, match="dtype_recipe"):
        QuantConfig(enabled=True, dtype_recipe="fp3")
    with pytest.raises(ValueError, match="unknown quant fmt"):
        QuantConfig(enabled=True, dtype={"weight": "not_a_fmt"})
    with pytest.raises(ValueError, match="dtype key"):
        QuantConfig(enabled=True, dtype={"grad_weight": "bf16"})
    with pytest.raises(ValueError, match="granularity"):
        QuantConfig(enabled=True, dtype_recipe="fp8", scaling={"granularity": "row"})


def test_rule_list_normalisation():
    tc = TrainingConfig(quant=[{"enabled": True, "dtype_recipe": "fp8", "include": ["*.mlp.*"]},
                               {"enabled": True, "dtype": {"weight": "fp8"}, "include": ["*.attn.*"]}])
    assert len(tc.quant) == 2 and tc.quant[0].include == ["*.mlp.*"]
    assert tc.quant[1].dtype == {"weight": "fp8", "act": "bf16", "input_grad": "bf16", "weight_grad": "bf16"}
    r = TrainingConfig(quant={"enabled": True, "dtype_recipe": "fp8"}).quant[0]
    assert r.dtype["input_grad"] == r.dtype["weight_grad"] == "fp8_e5m2" and "grad" not in r.dtype


def test_block_scaled_extensions():
    assert {"mxfp8", "nvfp4"} <= set(QUANT_DTYPE_RECIPES) and "blockwise" in QUANT_GRANULARITY
    assert {"mxfp8_e4m3", "mxfp8_e5m2", "nvfp4", "fp4_nv"} <= QUANT_FORMATS
    q = QuantConfig(enabled=True, dtype_recipe="mxfp8")
    assert q.scaling == {"granularity": "blockwise", "block_size": 32}
    assert q.dtype["weight"] == "mxfp8_e4m3" and q.dtype["input_grad"] == "mxfp8_e5m2"
    q = QuantConfig(enabled=True, dtype_recipe="nvfp4")
    assert q.scaling == {"granularity": "blockwise", "block_size": 16}
    # plain fp8 names under blockwise scaling are read as their MX forms
    q = QuantConfig(enabled=True, dtype_recipe="fp8", scaling={"granularity": "blockwise", "block_size": 32})
    assert q.dtype["act"] == "mxfp8_e4m3" and q.dtype["weight_grad"] == "mxfp8_e5m2"
    with pytest.raises(ValueError, match="block_size"):
        QuantConfig(enabled=True, dtype_recipe="mxfp8", scaling={"granularity": "blockwise", "block_size": 64})
    with pytest.raises(ValueError, match="blockwise"):
        QuantConfig(enabled=True, dtype_recipe="nvfp4", scaling={"granularity": "rowwise"})


def test_format_predicates():
    assert is_fp8("fp8") and is_fp8("fp8_e5m2") and not is_fp8("mxfp8")
    assert is_mxfp8("mxfp8_e5m2") and is_nvfp4("fp4_nv") and not is_quantized("bf16")
    assert str_to_dtype_fp8("fp8") == torch.float8_e4m3fn and str_to_dtype_fp8("mxfp8_e5m2") == torch.float8_e5m2
    assert str_to_dtype_fp8("bf16") is None
    assert [str_to_qmax_int8s(f) for f in ("int8", "int7", "int4")] == [127, 63, 7]


def test_rule_matching():
    cfg = QuantConfig(enabled=True, dtype_recipe="fp8")
    assert should_quantize("blocks.0.mlp.down_proj", cfg) and not should_quantize("lm_head", cfg)
    cfg = QuantConfig(enabled=True, dtype_recipe="fp8", include=["*.mlp.*"], exclude=["down_proj"])
    assert should_quantize("blocks.0.mlp.gate_up_proj", cfg)
    assert not should_quantize("blocks.0.mlp.down_proj", cfg)       # exclude wins, leaf-name match
    assert not should_quantize("blocks.0.attn.q_proj", cfg)
    off = QuantConfig(enabled=False)
    mlp = QuantConfig(enabled=True, dtype_recipe="fp8", include=["*.mlp.*"])
    rest = QuantConfig(enabled=True, dtype_recipe="mxfp8")
    assert resolve_rule("blocks.1.mlp.down_proj", [off, mlp, rest]) is mlp
    assert resolve_rule("blocks.1.attn.o_proj", [off, mlp, rest]) is rest
    assert resolve_rule("lm_head", [off, mlp, rest]) is None


class _Tiny(nn.Module):
    def __init__(self, tie=False):
        super().__init__()
        self.embed = nn.Embedding(32, 16)
        self.blocks = nn.ModuleList([nn.ModuleDict({"mlp": nn.Sequential(nn.Linear(16, 64), nn.Linear(64, 16)),
                                                    "attn": nn.ModuleDict({"q_proj": nn.Linear(16, 16, bias=False)})})])
        self.lm_head = nn.Linear(16, 32, bias=False)
        self.proj_tied = nn.Linear(16, 32, bias=False)
        if tie:
            self.proj_tied.weight = self.embed.weight


def _cfg(quant):
    return SimpleNamespace(training=TrainingConfig(quant=quant))


def test_converter_disabled_is_noop_and_passthrough_rule_swaps_nothing():
    m = apply_quantization(_Tiny(), _cfg({"enabled": False}))
    assert not any(isinstance(x, QuantLinear) for x in m.modules())
    m = apply_quantization(_Tiny(), _cfg({"enabled": True}))         # every operand passthrough
    assert not any(isinstance(x, QuantLinear) for x in m.modules())


@pytest.mark.skipif(torch.cuda.is_available() and torch.cuda.get_device_capability()[0] == 10, reason="needs a non-B200 host")
def test_converter_raises_without_capable_gpu():
    with pytest.raises(RuntimeError, match="requires"):
        apply_quantization(_Tiny(), _cfg({"enabled": True, "dtype_recipe": "mxfp8"}))
    with pytest.raises(RuntimeError, match="requires"):
        apply_quantization(_Tiny(), _cfg({"enabled": True, "dtype_recipe": "int8"}))


def test_converter_swaps_by_rule(monkeypatch):
    from pretrain_b200.quant import fp8
    monkeypatch.setattr(fp8, "is_supported", lambda: True)
    m = _Tiny(tie=True)
    w0 = m.blocks[0]["mlp"][0].weight.detach().clone()
    with pytest.warns(UserWarning, match="tied"):
        apply_quantization(m, _cfg([{"enabled": True, "dtype_recipe": "nvfp4", "include": ["*.mlp.*"]},
                                    {"enabled": True, "dtype_recipe": "fp8", "scaling": {"granularity": "rowwise"}}]))
    mlp0, q = m.blocks[0]["mlp"][0], m.blocks[0]["attn"]["q_proj"]
    assert isinstance(mlp0, QuantLinear) and mlp0.cfg.dtype["weight"] == "nvfp4"
    assert isinstance(q, QuantLinear) and q.cfg.dtype["weight"] == "fp8_e4m3" and q.bias is None
    assert torch.equal(mlp0.weight, w0) and mlp0.bias is not None
    assert type(m.lm_head) is nn.Linear                    # default exclude
    assert type(m.proj_tied) is nn.Linear                  # tie guard
    assert set(mlp0.state_dict()) == {"weight", "bias"}    # state-dict compatible with nn.Linear


def test_moe_block_host_state_matches_the_reference_layout():
    """Buffers, parameter names and the load-balancing bookkeeping of the MoE block (src/layers/mlp.py:182-239,
    324-500; the reference's tests/fast/layers/test_mlp.py checks the same names and the sign rule)."""
    from pretrain_b200.layers.mlp import ExpertBias, ExpertLoad, MoERouter, SparseMoEBlock
    blk = SparseMoEBlock(64, intermediate_size=32, n_routed_experts=4, n_routed_experts_per_token=2, n_shared_experts=2,
                         aux_loss=False, expert_bias=True, expert_bias_update_rate=0.01)
    assert sorted(n for n, _ in blk.named_buffers()) == ["expert_load.eval_load", "expert_load.train_load", "router.expert_bias.bias"]
    assert sorted(n for n, _ in blk.named_parameters()) == ["expert_down", "expert_gate_up", "router.gate.weight",
                                                            "shared_expert.down_proj.weight", "shared_expert.gate_up_proj.weight"]
    assert blk.shared_expert.down_proj.in_features == 2 * 32
    assert SparseMoEBlock(64, intermediate_size=32, n_routed_experts=4, n_routed_experts_per_token=2, dropout=0.25).expert_dropout.p == 0.25
    assert "expert_load.train_load" not in blk.state_dict() and "router.expert_bias.bias" in blk.state_dict()
    with pytest.raises(ValueError):
        SparseMoEBlock(64, intermediate_size=32, n_routed_experts=4, n_routed_experts_per_token=2, aux_loss=True, expert_bias=True)
    # sign rule: overloaded experts go down, underloaded ones up, by exactly the rate
    eb = ExpertBias(4, 0.01)
    eb.update(torch.tensor([10, 0, 5, 5]))
    assert torch.allclose(eb.bias, torch.tensor([-0.01, 0.01, 0.0, 0.0]))
    assert eb.half().bias.dtype == torch.float32                       # pinned to fp32 through casts
    load = ExpertLoad(4)
    load.record_load(torch.tensor([1, 2, 3, 4]), True)
    load.record_load(torch.tensor([1, 0, 0, 0]), True)
    load.record_load(torch.tensor([9, 9, 9, 9]), False)
    assert load.train_load.tolist() == [2, 2, 3, 4] and load.eval_load.tolist() == [9, 9, 9, 9]
    # post_step feeds the accumulated load to the bias and clears it
    blk.expert_load.record_load(torch.tensor([8, 0, 4, 4]), True)
    blk.post_step()
    assert torch.allclose(blk.router.expert_bias.bias, torch.tensor([-0.01, 0.01, 0.0, 0.0]))
    assert blk.expert_load.train_load.sum().item() == 0
    # the router has no torch path: on a CPU tensor it raises instead of switching implementation
    r = MoERouter(16, 4, 2, expert_bias=True, router_score_fn="softmax")
    with pytest.raises(RuntimeError, match="no CPU path"):
        r(torch.randn(32, 16))


def test_flop_and_parameter_accounting_of_the_mlp_blocks():
    """The class methods the reference's model statistics call (src/layers/mlp.py:152-176, 309-322, 510-587); the
    expected numbers were produced by the reference's own methods for the same arguments."""
    from pretrain_b200.layers.mlp import MLP_REGISTRY, DenseMLPBlock, MoERouter, SparseMoEBlock
    assert MLP_REGISTRY == {"dense": DenseMLPBlock, "moe": SparseMoEBlock}
    assert DenseMLPBlock.compute_flops(64, intermediate_size=96) == 6 * 64 * 96
    assert DenseMLPBlock.compute_flops(64, intermediate_size=96, gated=False, bias=True) == 4 * 64 * 96 + 96 + 64
    assert DenseMLPBlock.compute_parameters(64, intermediate_size=96, bias=True) == 3 * 64 * 96 + 2 * 96 + 64
    assert MoERouter.compute_flops(64, 8, expert_bias=True) == 2 * 64 * 8 + 8 and MoERouter.compute_parameters(64, 8, expert_bias=True) == 64 * 8
    kw = dict(intermediate_size=96, n_routed_experts=8)
    assert SparseMoEBlock.compute_flops(64, n_shared_experts=2, expert_bias=True, bias=True, **kw) == 149448
    assert SparseMoEBlock.compute_parameters(64, active=True, **kw) == 37376
    assert SparseMoEBlock.compute_parameters(64, **kw) == 64 * 8 + 8 * 3 * 64 * 96
    blk = SparseMoEBlock(64, intermediate_size=32, n_routed_experts=4, n_routed_experts_per_token=2, aux_loss=False)
    blk.expert_load.record_load(torch.tensor([1, 2, 3, 4]), True)
    blk.expert_load.record_load(torch.tensor([5, 5, 5, 5]), False)
    assert blk.forward_meta()["expert_load"].tolist() == [1, 2, 3, 4]
    assert blk.eval().forward_meta()["expert_load"].tolist() == [5, 5, 5, 5]


def test_activation_registries_cover_the_reference_names():
    """Names of src/layers/activation.py:130-158 and the rule that a squared variant squares the unary activation
    before the gate multiplies in."""
    import torch.nn.functional as F
    from pretrain_b200.layers.mlp import GATED_ACTIVATIONS, UNGATED_ACTIVATIONS, gated_mlp, silu_glu, ungated_mlp
    assert set(UNGATED_ACTIVATIONS) == {"relu", "gelu", "silu", "leaky_relu", "relu2", "gelu2", "silu2", "leaky_relu2"}
    assert set(GATED_ACTIVATIONS) == set(UNGATED_ACTIVATIONS) | {"bilinear", "bilinear2", "powlu"}
    assert GATED_ACTIVATIONS["silu"] is silu_glu                    # the one with a fused kernel
    g, u = torch.randn(8, 16), torch.randn(8, 16)
    assert torch.equal(UNGATED_ACTIVATIONS["leaky_relu2"](g), F.leaky_relu(g, 0.01) ** 2)
    assert torch.equal(GATED_ACTIVATIONS["silu2"](g, u), F.silu(g) ** 2 * u)
    assert torch.equal(GATED_ACTIVATIONS["bilinear2"](g, u), g ** 2 * u)
    p = GATED_ACTIVATIONS["powlu"](g, torch.ones_like(g))
    neg = g <= 0
    assert torch.allclose(p[neg], (g * g * torch.sigmoid(g))[neg]) and torch.isfinite(p).all()
    x, wgu, wd = torch.randn(2, 3, 16), torch.randn(24, 16), torch.randn(16, 12)
    gate, up = (x @ wgu.t()).chunk(2, -1)
    assert torch.allclose(gated_mlp(x, wgu, wd, silu_glu), (F.silu(gate) * up) @ wd.t())
    assert torch.allclose(ungated_mlp(x, wgu[:12], wd, F.relu, torch.ones(12)), F.relu(x @ wgu[:12].t() + 1) @ wd.t())


def test_weight_cache_sees_version_bumps_and_can_be_invalidated(monkeypatch):
    """The quantized-weight cache: reused while the parameter is untouched, rebuilt after an in-place op; a write
    through ``.data`` is invisible to it (no version bump), which is what ``invalidate`` / ``post_step`` and the
    B200Q_WEIGHT_CACHE=0 switch are for."""
    import torch.nn as nn
    from pretrain_b200.quant import cache
    monkeypatch.delenv("B200Q_WEIGHT_CACHE", raising=False)
    p = nn.Parameter(torch.ones(4, 4))
    made = []

    def make():
        made.append(p.detach().clone())
        return made[-1]

    assert cache.cached(p, "mx", "k", make) is made[0] and cache.cached(p, "mx", "k", make) is made[0]
    with torch.no_grad():
        p.add_(1.0)                                           # bumps the version: seen
    assert cache.cached(p, "mx", "k", make) is made[1] and made[1][0, 0] == 2
    p.data.add_(1.0)                                          # does not: the stale copy is served
    assert cache.cached(p, "mx", "k", make) is made[1]
    assert cache.invalidate(p) == 1
    assert cache.cached(p, "mx", "k", make) is made[2] and made[2][0, 0] == 3
    assert cache.cached(p, "mx", "other key", make) is made[3]
    lin = nn.Linear(4, 4)
    cache.cached(lin.weight, "fp8", 0, make)
    cache.cached(lin.weight, "mx", 0, make)
    assert cache.invalidate(lin) == 2 and cache.invalidate(lin) == 0
    monkeypatch.setenv("B200Q_WEIGHT_CACHE", "0")             # switch: every call re-quantizes
    n = len(made)
    cache.cached(p, "mx", "k", make); cache.cached(p, "mx", "k", make)
    assert len(made) == n + 2
    assert cache.cached(torch.ones(2), "mx", "k", lambda: 7) == 7      # plain tensors are never cached


def test_quant_linear_post_step_drops_the_cached_weight_copies():
    """QuantLinear.post_step is what the reference's loop calls after optimizer.step() (src/training/trainer.py:367)."""
    from pretrain_b200.quant import cache
    from pretrain_b200.quant.config import TrainingConfig
    from pretrain_b200.quant.linear import QuantLinear
    cfg = TrainingConfig(quant={"enabled": True, "dtype_recipe": "mxfp8"}).quant[0]
    q = QuantLinear(32, 32, False, cfg)
    cache.cached(q.weight, "mx", 0, lambda: 1)
    assert hasattr(q.weight, "_b200q_mx")
    q.post_step()
    assert not hasattr(q.weight, "_b200q_mx")
