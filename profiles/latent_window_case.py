"""One small case of the windowed latent attention kernel for an `ncu` capture: `python profiles/latent_window_case.py prefill|decode`
(16 heads over cached rows of 256 + 64 elements, no sink, half-split rotation: a 4 x 2048-token prompt step or a single-token step
over 64 x 4096 cached tokens, both with a 1024-token window)."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "nano-vllm_b200"))

from nanovllm import mixops  # noqa: E402
from nanovllm.layers.rotary_embedding import build_banded_cos_sin  # noqa: E402

H, R, d, rd, bs, dev, win = 16, 256, 128, 64, 256, "cuda", 1024
S, q, k = (4, 2048, 2048) if sys.argv[1] == "prefill" else (64, 1, 4096)
nblk = S * (k // bs)
cache = torch.randn(nblk * bs, R + rd, device=dev).bfloat16()
bt = torch.arange(nblk, dtype=torch.int32, device=dev).view(S, -1)
q_lat, q_raw = torch.randn(H, S * q, R, device=dev).bfloat16(), torch.randn(S * q, H, d + rd, device=dev).bfloat16()
table = build_banded_cos_sin(rd, 8192, 5e4, None, dev)
if q > 1:
    cu = torch.arange(0, S + 1, dtype=torch.int32, device=dev)
    sp = mixops.StepSpans(S, q, cu * q, cu * k, None)
else:
    sp = mixops.StepSpans(S, 1, None, None, torch.full((S,), k, dtype=torch.int32, device=dev))
for _ in range(4):
    o = mixops.latent_attention(q_lat, q_raw, d, cache, bt, bs, sp, None, table, 0.07, window=win, layout=mixops.ROT_HALVES)
torch.cuda.synchronize()
print("ok", float(o.float().abs().mean()))
