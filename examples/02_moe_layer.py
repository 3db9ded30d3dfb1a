"""A Mixture-of-Experts layer: forward, backward, telemetry, capacity dropping."""
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
import torch

from composed_mixture_of_experts_engine_b200.parallel import DistributedMoELayer

torch.manual_seed(0)
device = "cuda" if torch.cuda.is_available() else "cpu"
dtype = torch.bfloat16 if device == "cuda" else torch.float32

layer = DistributedMoELayer(hidden_dim=256, ffn_dim=512, num_experts=8, top_k=2, dtype=dtype).to(device)
layer.enable_timing(True)
x = torch.randn(4, 64, 256, device=device, dtype=dtype, requires_grad=True)
y = layer(x)
y.float().pow(2).mean().backward()
print("output", tuple(y.shape), "finite", bool(torch.isfinite(y).all()))
print("local experts", layer.local_expert_ids, "| expert compute ms", round(layer.last_expert_compute_ms, 3))
print("grad norms: x", float(x.grad.float().norm()), "w13", float(layer.w13.grad.float().norm()))

tight = DistributedMoELayer(256, 512, 8, 2, capacity_factor=0.5, capacity_dropping=True, dtype=dtype).to(device)
tight(x.detach())
print("dropped fraction with capacity_factor=0.5:", round(tight.last_dropped_token_fraction, 3))

# which rank owns which expert (a single process owns all of them; under expert parallelism each rank owns a
# contiguous block), and how the layer's cost grows with the token count
print("expert -> rank:", {e: layer._expert_to_rank(e) for e in range(0, 8, 2)} if hasattr(layer, "_expert_to_rank")
      else "all local")
import time

for tokens in (256, 1024, 4096):
    xb = torch.randn(tokens, 256, device=device, dtype=dtype)
    layer(xb)  # warm-up
    if device == "cuda":
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    layer(xb)
    if device == "cuda":
        torch.cuda.synchronize()
    print(f"{tokens:>5} tokens: {(time.perf_counter() - t0) * 1e3:.2f} ms")
