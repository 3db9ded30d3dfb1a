"""Model registry and the built-in models (reference: tests/test_registry.py)."""

import pytest
import torch
import torch.nn as nn

from composed_mixture_of_experts_engine_b200.models import (ModelRegistry, MoEDecoder, ToyMoEModel, build_model,
                                                            build_model_from_config, list_registered_models,
                                                            register_model)
from composed_mixture_of_experts_engine_b200.parallel import build_topology
from composed_mixture_of_experts_engine_b200.utils.config import MoEConfig

pytestmark = pytest.mark.cpu


def _cfg(**model):
    base = dict(hidden_dim=32, num_layers=2, num_experts=4, top_k=2, ffn_dim=64, vocab_size=128, sequence_length=8,
                dtype="float32")
    base.update(model)
    return MoEConfig.from_dict({"model": base, "training": dict(max_steps=5, warmup_steps=0)})


def test_builtins_registered():
    assert {"toy_moe", "moe_decoder"} <= set(list_registered_models())


def test_duplicate_and_unknown():
    with pytest.raises(ValueError) as ei:
        register_model("toy_moe")(nn.Module)
    assert "ToyMoEModel" in str(ei.value)
    with pytest.raises(KeyError) as ei:
        ModelRegistry.get("nope")
    assert "toy_moe" in str(ei.value)


def test_decorator_and_factory():
    @register_model("tiny_test_model")
    class Tiny(nn.Module):
        def __init__(self, cfg, topology):
            super().__init__()
            self.l = nn.Linear(cfg.model.hidden_dim, 2)

    try:
        m = build_model_from_config(_cfg(), build_topology(1, 1, device_type="cpu"), arch="tiny_test_model")
        assert isinstance(m, Tiny) and next(m.parameters()).device.type == "cpu"
    finally:
        ModelRegistry.unregister("tiny_test_model")


def test_toy_model_forward_backward_and_counts():
    topo = build_topology(1, 1, device_type="cpu")
    m = build_model(_cfg(), topo)
    assert isinstance(m, ToyMoEModel)
    ids = torch.randint(0, 128, (2, 8))
    logits = m(ids)
    assert logits.shape == (2, 8, 128)
    logits.float().mean().backward()
    c = m.count_parameters()
    assert c["total"] == sum(p.numel() for p in m.parameters())
    assert c["moe_experts"] == 2 * 4 * 3 * 32 * 64 and c["moe_router"] == 2 * 32 * 4
    assert hasattr(m.blocks[0], "norm") and hasattr(m.blocks[0].moe, "router")


def test_decoder_loss_equals_logits_path():
    torch.manual_seed(0)
    topo = build_topology(1, 1, device_type="cpu")
    m = build_model(_cfg(arch="moe_decoder", num_heads=2, aux_loss_coeff=0.01, init_std=0.02), topo)
    assert isinstance(m, MoEDecoder)
    ids, tgt = torch.randint(0, 128, (2, 8)), torch.randint(0, 128, (2, 8))
    want = torch.nn.functional.cross_entropy(m(ids).view(-1, 128), tgt.view(-1))
    assert float(m.loss(ids, tgt)) == pytest.approx(float(want), rel=1e-5)
    aux, z = m.aux_losses()
    assert float(aux) > 0 and float(z) > 0


def test_decoder_is_causal():
    torch.manual_seed(1)
    m = build_model(_cfg(arch="moe_decoder", num_heads=2), build_topology(1, 1, device_type="cpu"))
    ids = torch.randint(0, 128, (1, 8))
    ids2 = ids.clone()
    ids2[0, -1] = (ids2[0, -1] + 1) % 128
    a, b = m(ids), m(ids2)
    assert torch.allclose(a[0, :-1], b[0, :-1], atol=1e-6) and not torch.allclose(a[0, -1], b[0, -1])


def test_sm100_attention_shape_gate_is_off_by_default(monkeypatch):
    """The hand-written attention kernels are opt-in and only take sequence lengths that are multiples of 128 and
    head dimensions 64 / 128; everything else stays on the library path."""
    import torch

    from composed_mixture_of_experts_engine_b200.ops import attention_sm100 as A

    monkeypatch.delenv("CMOE_ATTN_SM100", raising=False)
    assert not A.enabled()
    monkeypatch.setenv("CMOE_ATTN_SM100", "1")
    assert A.enabled()
    assert A.shape_supported(4096, 16, 16, 128) and A.shape_supported(256, 32, 8, 64)
    assert not A.shape_supported(100, 4, 4, 64) and not A.shape_supported(256, 4, 3, 64)
    q = torch.randn(1, 128, 2, 64)  # CPU tensors never qualify
    assert not A.supported(q, q, q)
