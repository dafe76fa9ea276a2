"""One small case of the gated delta-rule kernel for an `ncu` capture: `python profiles/delta_rule_case.py prefill|decode`
(16 heads over 4 query/key heads, 128 x 128 states: a 4 x 2048-token prompt step, or a single-token step of 64 sequences)."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "nano-vllm_b200"))

from nanovllm import mixops  # noqa: E402

H, G, d, dev = 16, 4, 128, "cuda"
S, q = (4, 2048) if sys.argv[1] == "prefill" else (64, 1)
n = S * q
if q > 1:
    cu = torch.arange(0, S + 1, dtype=torch.int32, device=dev) * q
    sp = mixops.StepSpans(S, q, cu, cu, None)
else:
    sp = mixops.StepSpans(S, 1, None, None, torch.full((S,), 100, dtype=torch.int32, device=dev))
x = torch.randn(n, (2 * G + H) * d, device=dev).bfloat16()
ba = torch.randn(n, 2 * H, device=dev)
rate, bias = -torch.rand(H, device=dev), torch.zeros(H, device=dev)
state = torch.zeros(S, H, d, d, device=dev)
slots = torch.arange(S, dtype=torch.int32, device=dev)
for _ in range(4):
    o = mixops.gated_delta(x, 0, G * d, 2 * G * d, ba, rate, bias, state, slots, sp, H, G, d, d, d ** -0.5)
torch.cuda.synchronize()
print("ok", float(o.abs().mean()))
