"""Top-k routing: functional entry point, module, statistics and gradients."""
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
import torch

from composed_mixture_of_experts_engine_b200.ops import MoERouter, moe_topk_route

torch.manual_seed(0)
device = "cuda" if torch.cuda.is_available() else "cpu"
dtype = torch.bfloat16 if device == "cuda" else torch.float32
N, H, E, K = 1024, 512, 64, 2

tokens = torch.randn(N, H, device=device, dtype=dtype)
gate_w = (torch.randn(H, E, device=device) / H**0.5).to(dtype)
idx, w = moe_topk_route(tokens, gate_w, K)
print("indices", tuple(idx.shape), idx.dtype, "weights", tuple(w.shape), "row sums", float(w.float().sum(-1).mean()))

router = MoERouter(H, E, top_k=K, dtype=dtype).to(device)
router.profile_timing = True
x = tokens.clone().requires_grad_(True)
idx, w, counts = router(x)
loss = w.float().pow(2).sum() + 0.01 * router.last_aux_loss + 1e-3 * router.last_z_loss
loss.backward()
prof = router.last_profile
print(f"backend={prof.backend} fused={prof.used_fused_kernel} kernel_ms={prof.kernel_ms:.3f}")
print(f"imbalance={prof.expert_load_imbalance:.3f} z_loss={prof.router_z_loss:.3f} aux={prof.aux_loss:.3f}")
print("tokens per expert: mean", prof.tokens_per_expert_mean, "std", round(prof.tokens_per_expert_std, 2))
print("grad norms: tokens", float(x.grad.float().norm()), "gate", float(router.gate_w.grad.float().norm()))
assert int(counts.sum()) == N * K

# the validating interface the MoE layer talks to: one RouterStats record per call, plus the capacity budget
from composed_mixture_of_experts_engine_b200.parallel import MoERouterInterface

iface = MoERouterInterface(hidden_dim=H, num_experts=E, top_k=K, capacity_factor=1.25, dtype=dtype).to(device)
stats = iface(tokens)
print("RouterStats:", tuple(stats.expert_indices.shape), "counts sum", int(stats.dispatch_counts.sum()),
      "imbalance", round(float(stats.load_imbalance), 3))
for n in (256, 4096, 65536):
    print(f"capacity budget for {n:>6} tokens: {iface.capacity_budget(n)} rows per expert")

# a small latency sweep (median of a few calls; CUDA events on a GPU, the wall clock on CPU)
import time

for n, h, e, k in ((512, 256, 16, 2), (2048, 1024, 64, 2), (4096, 2048, 64, 8)):
    xs = torch.randn(n, h, device=device, dtype=dtype)
    gw = (torch.randn(h, e, device=device) / h**0.5).to(dtype)
    times = []
    for _ in range(5):
        if device == "cuda":
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            moe_topk_route(xs, gw, k)
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        else:
            t0 = time.perf_counter()
            moe_topk_route(xs, gw, k)
            times.append((time.perf_counter() - t0) * 1e3)
    ms = sorted(times)[len(times) // 2]
    print(f"N={n:<5} H={h:<5} E={e:<3} K={k}: {ms:.3f} ms, {n / ms / 1e3:.2f} M tokens/s")
