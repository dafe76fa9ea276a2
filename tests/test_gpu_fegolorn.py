"""Fegolorn on the GPU against the plain implementation (oracle/fegolorn_ref.py, float64, whole sequences, no cache):
every mechanism alone, then whole models through the engine's runner, scheduler bookkeeping and cache / state manager --
prompts, token-by-token decoding, portions, mixed batches, reused pages and slots -- and greedy generation through LLM."""
import math

import pytest
import torch

import fegolorn_helpers as fh
from oracle import fegolorn_ref as ref
from test_gpu_musavik import paged, portions_batches_and_dirty_slots, spans_decode
from test_gpu_tafopel import Replay, rel_err, spans_varlen

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 3e-4, "bfloat16": 6e-2}
F64 = torch.float64


# ---------------------------------------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cols", [44, 200, 1500])
def test_sublayer_close_gates_norms_scales_and_opens_the_next(dtype, cols):
    """x += ls * rms(y * sigmoid(gate)) * g_out, then rms(x) * g_in of the sublayer that follows; the gate arrives as a column slice of
    a wider projection; y in the activation type or fp32 (the expert sum); rows wider than a thread's registers hold."""
    from nanovllm.layers.layernorm import GatedScaledSandwich
    g = torch.Generator().manual_seed(cols)
    n, eps = 7, 3e-5
    a, b = GatedScaledSandwich(cols, eps, DT[dtype], "cuda"), GatedScaledSandwich(cols, eps, DT[dtype], "cuda")
    g_out, g_in = torch.tensor(0.8125), torch.tensor(1.375)
    ls = (0.5 + torch.rand(cols, generator=g)).to(torch.bfloat16)
    a.load("out", g_out), a.load("ls", ls), b.load("in", g_in)
    x = torch.randn(n, cols, generator=g) * 3
    wide = (torch.randn(n, cols + 9, generator=g) * 2).to(DT[dtype])
    for y in ((torch.randn(n, cols, generator=g) * 5).to(DT[dtype]), torch.randn(n, cols, generator=g) * 5):
        for gate in (wide.cuda()[:, 9:], None):
            xd = x.cuda().clone()
            h = a.close(xd, y.cuda(), gate, then=b)
            t = y.double() * (torch.sigmoid(wide[:, 9:].double()) if gate is not None else 1.0)
            want = x.double() + ref.rms(t, eps) * g_out.double() * ls.double()
            assert rel_err(xd, want) < 2e-6
            assert rel_err(h, ref.rms(want, eps) * g_in.double()) < (3e-6 if dtype == "float32" else 4e-3)
            xd2 = x.cuda().clone()
            assert a.close(xd2, y.cuda(), gate) is None and torch.equal(xd2, xd)
    assert rel_err(b.open(x.cuda()), ref.rms(x.double(), eps) * g_in.double()) < (3e-6 if dtype == "float32" else 4e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("ff,limit", [(40, 0.8), (96, 1.0), (7, 2.5)])
def test_clamped_gated_feed_forward(dtype, ff, limit):
    """Inputs large enough that both clamps act: the gate is cut from above only, the other branch on both sides, and (u + 1) not u."""
    from nanovllm.layers.moe import ClampedGluFF
    g = torch.Generator().manual_seed(ff)
    width, n = 48, 33
    mlp = {"kind": "dense", "ff": ff, "limit": limit}
    W = {k: fh.random_tensor(k, s, g).to(torch.bfloat16) for k, s in fh.mlp_shapes(mlp, width).items()}
    layer = ClampedGluFF(width, mlp, DT[dtype], "cuda", extra_rows=width)
    for k, w in W.items():
        assert layer.load(k, w)
    rg, rb = torch.randn(width, width, generator=g).to(torch.bfloat16), torch.randn(width, generator=g).to(torch.bfloat16)
    layer.w_extra.copy_(rg), layer.b_extra.copy_(rb)
    h = (torch.randn(n, width, generator=g) * 3).to(DT[dtype])
    pre = h.double() @ W["gate"].double().T
    assert (pre > limit).any() and (pre < -limit).any()
    y, gate = layer.forward(h.cuda())
    tol = 2e-5 if dtype == "float32" else 2e-2
    assert rel_err(y, ref.clamped_glu(h.double(), W, limit)) < tol
    assert rel_err(gate, h.double() @ rg.double().T + rb.double()) < tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(6, 2, 24, 16), (3, 3, 20, 0), (1, 1, 12, 28), (8, 3, 64, 48), (12, 4, 32, 8)])
def test_experts_chosen_by_logit_and_weighted_over_the_chosen(dtype, shape):
    """The router bias decides the choice (a large bias on one expert puts it in every token's set), the weights are the softmax over
    the chosen logits alone (all experts chosen: over all; one: weight 1), the shared expert is added unweighted."""
    from nanovllm.layers.moe import BiasedTopKExpertsFF
    E, top, ff, sh = shape
    g = torch.Generator().manual_seed(sum(shape))
    width, n = 64, 41
    mlp = fh.moe(E, top, ff, sh)
    W = {k: fh.random_tensor(k, s, g).to(torch.bfloat16) for k, s in fh.mlp_shapes(mlp, width).items()}
    W["router.b"][E - 1] = 40.0
    layer = BiasedTopKExpertsFF(width, mlp, DT[dtype], "cuda", extra_rows=0)
    for k, w in W.items():
        assert layer.load(k, w), k
    h = torch.randn(n, width, generator=g).to(DT[dtype])
    z = h.double() @ W["router"].double().T + W["router.b"].double()
    assert bool((z.topk(top, -1).indices == E - 1).any(-1).all())
    y, gate = layer.forward(h.cuda())
    assert gate is None and y.dtype == torch.float32
    assert rel_err(y, ref.routed_experts(h.double(), W, mlp)) < (2e-5 if dtype == "float32" else 2e-2)


def plain_rotated_value_attention(q, k, v, H, G, scale, base, pos_of_row):
    """float64, one sequence: keys and values of all positions, queries of the rows asked for; values turn by their own position and
    every head's sum turns back by the query's."""
    L, vd = k.shape[0], v.shape[-1]
    fv = ref.frequencies(vd, base)
    vr = ref.rotate(v, torch.arange(L), fv, "interleaved")
    out = []
    for r, i in enumerate(pos_of_row):
        o = []
        for h in range(H):
            s = (k[:i + 1, h // (H // G)] @ q[r, h]) * scale
            o.append(torch.softmax(s, 0) @ vr[:i + 1, h // (H // G)])
        out.append(ref.rotate(torch.stack(o)[None], torch.tensor([i]), fv, "interleaved", sign=-1.0)[0])
    return torch.stack(out)                                                        # [rows, H, vd]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("bs,shape", [(16, (4, 2, 32, 32)), (64, (10, 2, 64, 64)), (16, (3, 3, 10, 6))])
def test_values_carry_their_position_and_the_sum_is_turned_back(dtype, bs, shape):
    """Store (value pairs turned by the token's position), causal attention, and the turn back by the query's position, with one key
    made to dominate a head: that head must return the planted value turned by (its position - the query's position) -- a key at
    position 0, at page borders and hundreds of tokens back, seen from the last row of a portion and from a decoded token, over
    scrambled pages with a stale dominating row behind the sequence's end."""
    from nanovllm import mixops
    from nanovllm.layers.rotary_embedding import build_banded_cos_sin
    H, G, d, vd = shape
    L, base, scale = 330, 40.0, 0.2
    g = torch.Generator().manual_seed(bs + sum(shape))
    pages = torch.randperm(40, generator=g)[:(L + bs - 1) // bs + 1]
    vtab = build_banded_cos_sin(vd, 512, base, None, "cuda")
    bt = pages[None, :].to(torch.int32).cuda().contiguous()
    for star in (0, bs - 1, bs, 129, L - 2):
        x = torch.randn(L, H * d + G * d + G * vd, generator=g)
        x[:, H * d:H * d + G * d] *= 0.3
        for pos in sorted({star, star + 1, L - 1}):
            xx = x.clone()
            u = xx[pos, d * (H - 1):d * H] / xx[pos, d * (H - 1):d * H].norm()
            xx[star, H * d + (G - 1) * d:H * d + G * d] = 40.0 * u                # the last head of position `pos` looks straight at `star`
            xx[pos, d * (H - 1):d * H] = 8.0 * u
            xd = xx.to(DT[dtype])
            cache = torch.zeros(40 * bs, G * (d + vd), dtype=DT[dtype])
            cache[:, (G - 1) * d:G * d] = (60.0 * u).to(DT[dtype])                 # stale rows would win if they were read
            cache[:, G * d:] = 1e3
            cache = cache.cuda()
            slots = torch.tensor([int(pages[j // bs]) * bs + j % bs for j in range(L)], dtype=torch.int32).cuda()
            proj = xd.cuda().clone()
            mixops.headnorm_rope_store(proj, 0, H * d, H * d + G * d, H, G, d, vd, None, None, False, None, torch.arange(L).cuda(), slots,
                                       cache, 1e-6, v_cos_sin=vtab)
            q64, k64, v64 = xd.double()[:, :H * d].view(L, H, d), xd.double()[:, H * d:H * d + G * d].view(L, G, d), xd.double()[:, H * d + G * d:].view(L, G, vd)
            want = plain_rotated_value_attention(q64[pos:pos + 1], k64, v64, H, G, scale, base, [pos])[0]
            turned = ref.rotate(v64[star:star + 1, G - 1:G], torch.tensor([star - pos]), ref.frequencies(vd, base), "interleaved")[0, 0]
            assert (want[H - 1] - turned).abs().max().item() < 1e-3               # the test itself: the planted value, turned by the distance
            for decode in (False, True):
                for kw in (dict(fma=True), dict()):
                    if decode and pos == 0:
                        continue
                    first = pos if decode else max(0, pos - 20)
                    sp = spans_decode([pos + 1]) if decode else spans_varlen([pos + 1 - first], [pos + 1])
                    acc = mixops.window_attention(proj[first:pos + 1], cache, bt, bs, sp, H, G, d, vd, scale, None, 0, out_f32=dtype == "bfloat16", **kw)
                    o = mixops.head_rotate_gate(acc.view(-1, H, vd), DT[dtype], vtab, torch.arange(first, pos + 1).cuda(), sign=-1.0)
                    assert rel_err(o[-1].view(H, vd), want) < (1e-4 if dtype == "float32" else 2e-2), (star, pos, decode, kw)


def plain_latent_rows(q, rows, rank, scale, window, pos_of_row):
    """float64: q [r, H, rank + rot], cache rows [L, rank + rot] (keys; the first `rank` columns are the values) -> [r, H, rank]."""
    out = []
    for r, i in enumerate(pos_of_row):
        lo = max(0, i - window + 1) if window else 0
        s = torch.einsum("hd,jd->hj", q[r], rows[lo:i + 1]) * scale
        out.append(torch.softmax(s, -1) @ rows[lo:i + 1, :rank])
    return torch.stack(out)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("bs,window,H,rank,rot", [(16, 50, 3, 24, 8), (64, 64, 8, 64, 32), (64, 65, 16, 128, 32), (16, 1, 2, 16, 4), (16, 0, 5, 40, 8),
                                                  (64, 200, 4, 96, 64)])
def test_latent_attention_sees_exactly_its_window(dtype, bs, window, H, rank, rot):
    """One cached row is made to dominate a head: the head must return that row's latent exactly while the row is among the last
    `window` positions and must not feel it one position later.  The row sits at position 0, at page borders and far back; the query
    is the last row of a portion or a single decoded token (keys split over CTAs there); pages are scrambled and a stale dominating
    row lies behind the sequence's end.  No sink enters the softmax."""
    from nanovllm import mixops
    from nanovllm.layers.rotary_embedding import build_banded_cos_sin
    L, D, scale = 330, rank + rot, 0.2
    g = torch.Generator().manual_seed(bs + window + H)
    pages = torch.randperm(40, generator=g)[:(L + bs - 1) // bs + 1]
    table = build_banded_cos_sin(rot, 512, 1e9, None, "cuda")                 # a base so large that only pair 0 turns visibly; q_rot is zero anyway
    bt = pages[None, :].to(torch.int32).cuda().contiguous()
    w = window or L + 1
    for star in sorted({0, bs - 1, bs, 129, L - 2}):
        rows = torch.randn(L, D, generator=g) * 0.3
        q = torch.randn(L, H, D, generator=g)
        q[:, :, rank:] = 0.0
        for pos in sorted({star, star + 1, star + w - 1, star + w, L - 1} & set(range(star, L))):
            qq, rr = q.clone(), rows.clone()
            u = qq[pos, 1 % H, :rank] / qq[pos, 1 % H, :rank].norm()
            rr[star, :rank] = 40.0 * u
            qq[pos, 1 % H, :rank] = 8.0 * u
            stale = torch.cat([60.0 * u, torch.zeros(rot)])
            cache = paged(rr, pages, bs, dtype, 40, stale=stale)
            kv = torch.stack([cache[int(pages[j // bs]) * bs + j % bs] for j in range(pos + 1)]).double()
            qd = qq.to(DT[dtype])
            want = plain_latent_rows(qd[pos:pos + 1].double(), kv, rank, scale, window, [pos])[0]
            seen = pos - star < w
            near = (want[1 % H] - kv[star, :rank]).abs().max().item() < 1e-3
            assert near == seen, (star, pos)                                  # the test itself distinguishes the two cases
            for decode in (False, True):
                for kw in (dict(fma=True), dict()):
                    if decode and pos == 0:
                        continue
                    first = pos if decode else max(0, pos - 20)
                    sp = spans_decode([pos + 1]) if decode else spans_varlen([pos + 1 - first], [pos + 1])
                    qr = qd[first:pos + 1].cuda().contiguous()
                    q_lat = qr[:, :, :rank].transpose(0, 1).contiguous()
                    o = mixops.latent_attention(q_lat, qr, rank, cache.cuda(), bt, bs, sp, None, table, scale, window=window,
                                                layout=mixops.ROT_HALVES, **kw)
                    assert rel_err(o[:, -1], want) < (1e-4 if dtype == "float32" else 2e-2), (star, pos, decode, kw)


class _Mixer:
    """A mixer whose forward also returns its gate columns, as a layer that returns the mixer output alone."""

    def __init__(self, mixer):
        self.m, self.dtype = mixer, mixer.dtype
        self.bind, self.unbind = mixer.bind, mixer.unbind

    def forward(self, h, pos, ctx, sp, inst=0):
        return self.m.forward(h, pos, ctx, sp, inst)[0]


def _mixer(layer, dtype, width, seed, extra=0):
    from nanovllm.layers.latent_attention import GatedWindowLatentAttention
    from nanovllm.layers.window_attention import RotatedValueAttention
    g = torch.Generator().manual_seed(seed)
    W = {k: fh.random_tensor("mix." + k, s, g).to(torch.bfloat16) for k, s in fh.mixer_shapes(layer, width).items()}
    cls = RotatedValueAttention if layer["type"] == "attention" else GatedWindowLatentAttention
    m = cls(width, layer["mixer"], 1e-5, DT[dtype], "cuda", 512, extra_rows=extra)
    for k, w in W.items():
        assert m.load(k, w), k
    return m, W


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("layer", [fh.attention(scaling=(4.0, 1.0, 4.0, 64)), fh.attention(heads=5, kv_heads=1, dim=64, vdim=32, rot_dims=16, base=1e4),
                                   fh.attention(heads=2, kv_heads=2, dim=6, vdim=10, rot_dims=6, scaling=(2.0, 2.0, 8.0, 40), window=20),
                                   fh.attention(heads=4, kv_heads=4, dim=32, vdim=64, rot_dims=0)])
def test_attention_layer_whole_in_portions_in_batches_and_in_used_pages(dtype, layer):
    """Head norms with one shared weight, banded partial rotation (all three bands occur), rotated values, against the plain layer."""
    width = 48
    m, W = _mixer(layer, dtype, width, 3)
    portions_batches_and_dirty_slots(_Mixer(m), lambda h: ref.attention(h, W, layer["mixer"], 1e-5), width, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("layer", [fh.latent(), fh.latent(heads=8, dim=32, rot_dim=32, vdim=32, kv_rank=64, window=65, base=1e4),
                                   fh.latent(heads=1, dim=12, rot_dim=6, vdim=10, kv_rank=20, window=1),
                                   fh.latent(heads=5, dim=4, rot_dim=2, vdim=6, kv_rank=10, window=0, scaling=(2.0, 1.0, 2.0, 16)),
                                   fh.latent(heads=16, dim=16, rot_dim=32, vdim=16, kv_rank=128, window=64)])
def test_latent_layer_whole_in_portions_in_batches_and_in_used_pages(dtype, layer):
    """Half-split rotation of the shared key part and of the queries' rotated part, the latent's norm, window, output gate."""
    width = 48
    m, W = _mixer(layer, dtype, width, 4)
    portions_batches_and_dirty_slots(_Mixer(m), lambda h: ref.latent_attention(h, W, layer["mixer"], 1e-5), width, dtype)


def test_band_edges_of_the_frequency_scaling():
    from nanovllm.layers.rotary_embedding import banded_frequencies
    for dims, base, sc in ((8, 5000.0, (4.0, 1.0, 4.0, 64)), (64, 5e5, (4.0, 1.0, 8.0, 1024)), (6, 40.0, (2.0, 2.0, 8.0, 40)), (16, 300.0, None)):
        scaling = dict(zip(("factor", "low", "high", "original"), sc)) if sc else None
        got, want = banded_frequencies(dims, base, scaling), ref.frequencies(dims, base, scaling)
        assert torch.allclose(got, want, rtol=1e-12, atol=0)
    f = ref.frequencies(8, 5000.0, dict(factor=4.0, low=1.0, high=4.0, original=64))
    plain = ref.frequencies(8, 5000.0)
    ratio = (f / plain).tolist()
    assert ratio[0] == 1.0 and abs(ratio[-1] - 0.25) < 1e-12 and any(0.25 < r < 1.0 for r in ratio)     # kept, slowed, and blended pairs


def test_soft_cap():
    from nanovllm import mixops
    x = torch.linspace(-200, 200, 4001)
    got = mixops.softcap_(x.cuda().clone(), 20.0)
    assert rel_err(got, 20.0 * torch.tanh(x.double() / 20.0)) < 1e-6


# ---------------------------------------------------------------------------------------------------------------------------
# whole models through the engine
# ---------------------------------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def checkpoints(tmp_path_factory):
    root = tmp_path_factory.mktemp("fegolorn")
    out = {}
    for name, cfg in (("a", fh.config_a()), ("b", fh.config_b()), ("c", fh.config_c())):
        W = fh.random_weights(cfg, 21)
        out[name] = (fh.write_checkpoint(str(root / name), cfg, W), cfg, W)
    return out


@pytest.fixture(scope="module")
def engines(checkpoints):
    made = {}

    def get(name, dtype):
        if (name, dtype) not in made:
            made[(name, dtype)] = Replay(checkpoints[name][0], dtype)
        return made[(name, dtype)]
    yield get
    for e in made.values():
        e.runner.exit()


def oracle_logits(checkpoints, name, toks):
    _, cfg, W = checkpoints[name]
    return ref.forward(cfg, W, toks)


def assert_logits(got, want, dtype, tag=None):
    """fp32: the RMS error over everything.  bf16: a token whose best experts are nearly tied may take the other one, so the bound is
    on the median over positions, with a loose one on the sum."""
    got, want = got.double().cpu(), want.double().cpu()
    if dtype == "float32":
        assert rel_err(got, want) < TOL[dtype], tag
    else:
        per_pos = ((got - want) ** 2).mean(1).sqrt() / (want ** 2).mean(1).sqrt()
        assert per_pos.median().item() < TOL[dtype] and rel_err(got, want) < 0.3, (tag, per_pos.median().item(), rel_err(got, want))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_whole_prompt_and_first_tokens(engines, checkpoints, name, dtype):
    e = engines(name, dtype)
    vocab = checkpoints[name][1]["vocab"]
    for i, n in enumerate((1, 2, 17, 150)):
        toks = fh.tokens(n, vocab, i)
        got = e.step([("p", toks)])["p"]
        e.end("p")
        assert_logits(got, oracle_logits(checkpoints, name, toks), dtype, n)


def test_the_stream_after_every_layer(checkpoints):
    """The residual stream after each layer (a layer that borrows weights counts as a layer) against the plain implementation."""
    e = Replay(checkpoints["a"][0], "float32", eager=True)
    _, cfg, W = checkpoints["a"]
    toks = fh.tokens(45, cfg["vocab"], 3)
    want = []
    ref.forward(cfg, W, toks, want)
    model, taps = e.runner.model, []
    plain_forward = model.forward
    type(model).__call__ = lambda self, ids, pos: plain_forward(ids, pos, taps)
    try:
        e.step([("p", toks)])
    finally:
        type(model).__call__ = type(model).forward
    e.runner.exit()
    assert len(taps) == len(want) == len(cfg["layers"])
    for r, (a, b) in enumerate(zip(taps, want)):
        assert rel_err(a, b) < 1e-4, r


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b"])
def test_long_decoding_matches_the_prompt_path(engines, checkpoints, name, dtype):
    """One prompt token, then 170 tokens one by one through the decode graphs, across ten pages and several windows."""
    e = engines(name, dtype)
    toks = fh.tokens(171, checkpoints[name][1]["vocab"], 5)
    want = oracle_logits(checkpoints, name, toks)
    got = [e.step([("d", toks[:1])])["d"]]
    for t in toks[1:]:
        got.append(e.step([("d", [t])])["d"])
    e.end("d")
    got = torch.cat(got)
    assert_logits(got, want, dtype)
    assert_logits(got[-20:], want[-20:], dtype, "far end")   # no drift at the far end


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_portions_of_many_sizes(engines, checkpoints, name, dtype):
    e = engines(name, dtype)
    cuts = (2, 3, 2, 31, 16, 2, 1, 1, 48, 15, 1, 5, 33)
    toks = fh.tokens(sum(cuts), checkpoints[name][1]["vocab"], 6)
    got, at = [], 0
    for n in cuts:
        got.append(e.step([("c", toks[at:at + n])])["c"])
        at += n
    e.end("c")
    assert_logits(torch.cat(got), oracle_logits(checkpoints, name, toks), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b"])
def test_unequal_requests_in_one_batch_and_reused_pages_and_slots(engines, checkpoints, name, dtype):
    """Four requests of unequal length, portions beside single tokens; two of them end early and a fifth and sixth take over
    their pages and state slots (the previous token of the pair embedding lives there) while the others go on.  Every request must
    come out as if it had run alone."""
    e = engines(name, dtype)
    vocab = checkpoints[name][1]["vocab"]
    T = {k: fh.tokens(n, vocab, 10 + i) for i, (k, n) in enumerate(dict(a=90, b=37, c=9, d=140, e=70, f=44).items())}
    plan = [
        [("a", 40), ("b", 2)], [("a", 1), ("b", 30), ("c", 9)], [("a", 1), ("b", 1), ("d", 64)], [("a", 1), ("b", 1), ("d", 1)],
        [("a", 17), ("b", 3), ("d", 2)], [("a", 1), ("d", 1)], [("a", 29), ("d", 72)],
        # b and c are done: e and f arrive in their places
        [("e", 33), ("f", 1), ("d", 0)], [("e", 1), ("f", 43)], [("e", 36)],
    ]
    got = {k: [] for k in T}
    at = {k: 0 for k in T}
    ended = set()
    for step in plan:
        entries = [(k, T[k][at[k]:at[k] + n]) for k, n in step if n]
        for k, n in step:
            at[k] += n
        for k, lg in e.step(entries).items():
            got[k].append(lg)
        for k in T:
            if at[k] == len(T[k]) and k in e.live and k not in ended:
                e.end(k)
                ended.add(k)
    assert ended == set(T)
    for k in T:
        assert_logits(torch.cat(got[k]), oracle_logits(checkpoints, name, T[k]), dtype, k)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_wider_model_over_64_token_pages(checkpoints, dtype):
    """The configuration with tensor-core sizes over pages as long as the key tile: a 333-token prompt in portions that end beside
    page borders and window edges, then single tokens, next to a second request that arrives in the middle."""
    e = Replay(checkpoints["c"][0], dtype, pool_tokens=768, block=64, seqs=3)
    vocab = checkpoints["c"][1]["vocab"]
    a, b = fh.tokens(333, vocab, 81), fh.tokens(90, vocab, 82)
    got = {"a": [], "b": []}
    at = {"a": 0, "b": 0}
    for step in ([("a", 63)], [("a", 2)], [("a", 64), ("b", 1)], [("a", 1), ("b", 70)], [("a", 130), ("b", 1)], [("a", 1), ("b", 18)], [("a", 60)],
                 *[[("a", 1)] for _ in range(12)]):
        entries = [(k, (a if k == "a" else b)[at[k]:at[k] + n]) for k, n in step]
        for k, n in step:
            at[k] += n
        for k, lg in e.step(entries).items():
            got[k].append(lg)
    e.runner.exit()
    assert at == {"a": 333, "b": 90}
    for k, toks in (("a", a), ("b", b)):
        assert_logits(torch.cat(got[k]), oracle_logits(checkpoints, "c", toks), dtype, k)


def test_batch_does_not_change_a_request_beyond_rounding(engines, checkpoints):
    e = engines("a", "float32")
    vocab = checkpoints["a"][1]["vocab"]
    x, y = fh.tokens(50, vocab, 30), fh.tokens(21, vocab, 31)
    alone = e.step([("x", x)])["x"]
    e.end("x")
    both = e.step([("y", y), ("x", x)])["x"]
    e.end("x"), e.end("y")
    assert rel_err(both, alone) < 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(checkpoints, dtype):
    """LLM.generate on a checkpoint without a tokenizer: scheduler, block and slot manager, decode graphs, sampler.  Teacher-forced
    against the plain implementation: each generated token is its argmax, or loses to it by less than the format's rounding."""
    from nanovllm import LLM, SamplingParams
    path, cfg, W = checkpoints["a"]
    llm = LLM(path, dtype=dtype, max_num_seqs=3, max_model_len=256, max_num_batched_tokens=96, kvcache_block_size=16,
              num_kvcache_blocks=24, gpu_memory_utilization=0.5)
    prompts = [fh.tokens(n, cfg["vocab"], 40 + i) for i, n in enumerate((5, 61, 1, 100, 18))]      # more requests than slots, chunked prompts
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True), use_tqdm=False)
    llm.exit()
    assert [len(o["token_ids"]) for o in outs] == [24] * 5
    tol = 1e-3 if dtype == "float32" else 0.15
    for p, o in zip(prompts, outs):
        seq = p + o["token_ids"]
        lg = ref.forward(cfg, W, seq[:-1])
        for i, tok in enumerate(o["token_ids"]):
            row = lg[len(p) - 1 + i]
            assert (row.max() - row[tok]).item() <= tol * row.std().item(), (len(p), i)


def test_replay_command_line(checkpoints, tmp_path):
    """bin/trace_run end to end: JSON steps on stdin, logits files and 'done' lines out."""
    import json
    import os
    import subprocess
    import numpy as np
    path, cfg, W = checkpoints["b"]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    toks = fh.tokens(40, cfg["vocab"], 50)
    steps = [{"step": 0, "entries": [{"id": "q", "tokens": toks[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "q", "tokens": toks[30:31], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "q", "tokens": toks[31:32], "want": [0]}, {"id": "r", "tokens": toks[:3], "want": [2]}], "end": ["r"]},
             {"step": 3, "entries": [{"id": "q", "tokens": toks[32:], "want": [7]}], "end": ["q"]}]
    out = tmp_path / "out"
    r = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", path, "--dtype", "float32", "--out", str(out), "--max-tokens", "128"],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    want = ref.forward(cfg, W, toks)
    V = cfg["vocab"]
    g0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, V))
    g2 = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(-1, V))
    g3 = torch.from_numpy(np.fromfile(out / "3.f32", dtype="<f4").reshape(-1, V))
    assert not (out / "1.f32").exists()
    assert rel_err(g0, want[[0, 29]]) < TOL["float32"] and rel_err(g2, want[[31, 2]]) < TOL["float32"] and rel_err(g3, want[[39]]) < TOL["float32"]
