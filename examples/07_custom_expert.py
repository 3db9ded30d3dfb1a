"""Custom experts: subclass the layer and replace ``self.experts``; routing, dispatch and combine stay the same."""
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
import torch
import torch.nn as nn

from composed_mixture_of_experts_engine_b200.parallel import DistributedMoELayer


class GeluExpert(nn.Module):
    """A plain two-layer GELU MLP instead of the SwiGLU expert."""

    def __init__(self, hidden: int, ffn: int):
        super().__init__()
        self.up, self.down = nn.Linear(hidden, ffn), nn.Linear(ffn, hidden)

    def forward(self, x):
        return self.down(torch.nn.functional.gelu(self.up(x)))


class GeluMoELayer(DistributedMoELayer):
    def __init__(self, hidden_dim, ffn_dim, num_experts, top_k, **kw):
        super().__init__(hidden_dim, ffn_dim, num_experts, top_k, **kw)
        # replacing the module list switches the layer to its generic per-expert path
        self.experts = nn.ModuleList([GeluExpert(hidden_dim, ffn_dim) for _ in self.local_expert_ids])


torch.manual_seed(0)
layer = GeluMoELayer(64, 128, num_experts=4, top_k=2)
x = torch.randn(2, 10, 64, requires_grad=True)
y = layer(x)
y.pow(2).mean().backward()
print("output", tuple(y.shape), "| expert-0 up grad", float(layer.experts[0].up.weight.grad.norm()))

# check against the definition y_t = sum_k w[t,k] * Expert_{idx[t,k]}(x_t)
flat = x.detach().reshape(-1, 64)
idx, w, _ = layer.router(flat)
want = torch.zeros_like(flat)
for t in range(flat.shape[0]):
    for k in range(2):
        want[t] += w[t, k] * layer.experts[int(idx[t, k])](flat[t])
print("matches the per-token definition:", bool(torch.allclose(y.detach().reshape(-1, 64), want, atol=1e-5)))
