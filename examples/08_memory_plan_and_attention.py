"""Per-GPU memory plan of the shipped configurations, and the two attention paths of the decoder.

The plan needs no GPU.  The attention comparison runs only when a B200 is present: it calls the packed RoPE +
attention op once through the library kernel and once through the hand-written tcgen05 kernels
(``CMOE_ATTN_SM100=1``) and prints the largest difference.  The reference has neither a planner nor attention.
"""

import os
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from composed_mixture_of_experts_engine_b200.utils.config import MoEConfig  # noqa: E402
from composed_mixture_of_experts_engine_b200.utils.memory import format_plan, plan_memory  # noqa: E402

for name in ("olmoe_1b7b.yaml", "mixtral_8x7b.yaml"):
    cfg = MoEConfig.from_yaml(ROOT / "configs" / name)
    print(f"== {name}")
    print(format_plan(plan_memory(cfg)))

if torch.cuda.is_available():
    from composed_mixture_of_experts_engine_b200.ops import functional as OF

    B, S, nh, nkv, hd = 2, 512, 8, 2, 128
    cos, sin = OF.rope_tables(S, hd, 10000.0, torch.device("cuda"))
    qkv = torch.randn(B, S, nh + 2 * nkv, hd, device="cuda").to(torch.bfloat16)
    outs = {}
    for flag in ("0", "1"):
        os.environ["CMOE_ATTN_SM100"] = flag
        outs[flag] = OF.rope_causal_attention(qkv.clone(), cos, sin, nh, nkv).float()
    print("library vs hand-written attention, max |diff|:", float((outs["0"] - outs["1"]).abs().max()))
else:
    print("no GPU: skipping the attention comparison")
print("\nExample 08 complete")
