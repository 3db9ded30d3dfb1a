"""Registering a model class and building it from a config."""
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
import torch
import torch.nn as nn

from composed_mixture_of_experts_engine_b200.models import (ModelRegistry, build_model_from_config,
                                                            list_registered_models, register_model)
from composed_mixture_of_experts_engine_b200.parallel import DistributedMoELayer, build_topology
from composed_mixture_of_experts_engine_b200.utils.config import MoEConfig


@register_model("two_layer_moe")
class TwoLayerMoE(nn.Module):
    def __init__(self, cfg, topology):
        super().__init__()
        m = cfg.model
        self.embed = nn.Embedding(m.vocab_size, m.hidden_dim)
        self.moe = nn.ModuleList([DistributedMoELayer(m.hidden_dim, m.ffn_dim, m.num_experts, m.top_k, topology)
                                  for _ in range(2)])
        self.head = nn.Linear(m.hidden_dim, m.vocab_size, bias=False)

    def forward(self, ids):
        x = self.embed(ids)
        for layer in self.moe:
            x = x + layer(x)
        return self.head(x)


print("registered:", list_registered_models())
cfg = MoEConfig.from_dict({"model": dict(hidden_dim=64, num_layers=2, num_experts=4, top_k=2, ffn_dim=128,
                                         vocab_size=256, sequence_length=16, dtype="float32"),
                           "training": dict(max_steps=10, warmup_steps=0)})
topo = build_topology(1, 1, device_type="cpu")
for arch in ("toy_moe", "moe_decoder", "two_layer_moe"):
    model = build_model_from_config(cfg, topo, arch=arch)
    out = model(torch.randint(0, 256, (2, 16)))
    print(f"{arch:14s} params={sum(p.numel() for p in model.parameters()):8d} output={tuple(out.shape)}")
# the two mistakes the registry catches: registering a name twice, asking for a name nobody registered
try:
    register_model("two_layer_moe")(TwoLayerMoE)
except ValueError as exc:
    print("duplicate ->", exc)
try:
    build_model_from_config(cfg, topo, arch="no_such_model")
except KeyError as exc:
    print("unknown   ->", str(exc)[:100])
ModelRegistry.unregister("two_layer_moe")
