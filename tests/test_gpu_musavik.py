"""Musavik on the GPU against the plain implementation (oracle/musavik_ref.py, float64, whole sequences, no cache):
every mechanism alone, then whole models through the engine's runner, scheduler bookkeeping and cache / state manager --
prompts, token-by-token decoding, portions, mixed batches, reused pages and slots -- and greedy generation through LLM."""
import math
from types import SimpleNamespace

import pytest
import torch

import musavik_helpers as mh
from oracle import musavik_ref as ref
from test_gpu_tafopel import Replay, rel_err, spans_varlen

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 3e-4, "bfloat16": 6e-2}
F64 = torch.float64


def spans_decode(k_lens):
    from nanovllm import mixops
    return mixops.StepSpans(len(k_lens), 1, None, None, torch.tensor(k_lens, dtype=torch.int32, device="cuda"))


# ---------------------------------------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pair_embedding_takes_the_previous_token_from_the_prompt_or_the_slot(dtype):
    """Rows in the middle of a portion pair with the row before; the first row of a later portion pairs with the token its state
    slot holds; position 0 takes the extra last row whatever a reused slot holds; afterwards the slot holds the portion's last token."""
    from nanovllm import mixops
    g = torch.Generator().manual_seed(1)
    vocab, width, buckets, mp, mc, scale = 90, 40, 31, 13, 5, 1.75
    cfg = {"embedding": {"scale": scale, "bigram": {"buckets": buckets, "mul_prev": mp, "mul_cur": mc}}}
    W = {"embed": torch.randn(vocab, width, generator=g).to(DT[dtype]), "bigram": torch.randn(buckets + 1, width, generator=g).to(DT[dtype])}
    seqs = [mh.tokens(n, vocab, 60 + n) for n in (9, 1, 14)]
    want = [ref.embedding(W, cfg, s) for s in seqs]
    prev = torch.full((5,), 77, dtype=torch.int64, device="cuda")              # stale tokens of earlier owners
    slots = torch.tensor([3, 0, 4], dtype=torch.int32, device="cuda")
    tab, pair = W["embed"].cuda(), W["bigram"].cuda()
    # step 1 (varlen): 4 tokens of sequence 0, all of sequence 1, 6 of sequence 2
    ids = torch.tensor(seqs[0][:4] + seqs[1] + seqs[2][:6], dtype=torch.int64, device="cuda")
    copy = torch.empty(11, width, dtype=DT[dtype], device="cuda")
    x = mixops.embed_pair(ids, tab, scale, spans_varlen([4, 1, 6], [4, 1, 6]), pair, buckets, mp, mc, prev, slots, copy=copy)
    tol = 1e-6 if dtype == "float32" else 1e-6
    assert rel_err(x, torch.cat([want[0][:4], want[1], want[2][:6]])) < tol and torch.equal(copy, x.to(DT[dtype]))
    assert prev.tolist() == [seqs[1][-1], 77, 77, seqs[0][3], seqs[2][5]]
    # step 2 (varlen): the rest of sequence 2 beside one token of sequence 0
    ids = torch.tensor(seqs[2][6:] + seqs[0][4:5], dtype=torch.int64, device="cuda")
    x = mixops.embed_pair(ids, tab, scale, spans_varlen([8, 1], [14, 5]), pair, buckets, mp, mc, prev, slots[[2, 0]].contiguous())
    assert rel_err(x, torch.cat([want[2][6:], want[0][4:5]])) < tol
    # step 3 (single tokens, with a padding row)
    ids = torch.tensor([seqs[0][5], 0], dtype=torch.int64, device="cuda")
    x = mixops.embed_pair(ids, tab, scale, spans_decode([6, 0]), pair, buckets, mp, mc, prev, slots[[0, 1]].contiguous())
    assert rel_err(x[:1], want[0][5:6]) < tol and bool((x[1] == 0).all())
    assert prev[3].item() == seqs[0][5] and prev[0].item() == seqs[1][-1]
    # no pair table: the scaled embedding alone
    x = mixops.embed_pair(ids[:1], tab, scale, spans_decode([6]))
    assert rel_err(x, W["embed"].double()[seqs[0][5]][None] * scale) < tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cols", [44, 200, 1000])
def test_norms_on_both_sides_of_a_sublayer(dtype, cols):
    from nanovllm.layers.layernorm import SandwichNorm
    g = torch.Generator().manual_seed(cols)
    a, b = SandwichNorm(cols, 1e-5, DT[dtype], "cuda"), SandwichNorm(cols, 1e-5, DT[dtype], "cuda")
    for n in (a, b):
        n.w_in.copy_(0.3 * torch.randn(cols, generator=g))
        n.w_out.copy_(0.3 * torch.randn(cols, generator=g))
    x = torch.randn(7, cols, generator=g) * 3 + 1.5
    y = (torch.randn(7, cols, generator=g) * 5).to(DT[dtype])
    xd = x.cuda()
    tol = 2e-6 if dtype == "float32" else 4e-3
    assert rel_err(a.open(xd), ref.zc_norm(x.double(), a.w_in.double().cpu(), 1e-5)) < tol
    nxt = a.close(xd, y.cuda(), then=b)
    want = x.double() + ref.zc_norm(y.double(), a.w_out.double().cpu(), 1e-5)
    assert rel_err(xd, want) < 2e-6                                         # the stream itself stays fp32 in both formats
    assert rel_err(nxt, ref.zc_norm(xd.double().cpu(), b.w_in.double().cpu(), 1e-5)) < tol
    copy = torch.empty(7, cols, dtype=DT[dtype], device="cuda")
    assert b.close(xd, y.cuda(), copy=copy) is None
    assert torch.equal(copy, xd.to(DT[dtype]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_biased_dense_feed_forward(dtype):
    from nanovllm.layers.moe import BiasedDenseFF
    g = torch.Generator().manual_seed(4)
    width, ffw = 40, 72
    W = {"up": torch.randn(ffw, width, generator=g) * 0.3, "up.b": torch.randn(ffw, generator=g), "down": torch.randn(width, ffw, generator=g) * 0.2,
         "down.b": torch.randn(width, generator=g)}
    W = {k: v.to(DT[dtype]) for k, v in W.items()}
    ff = BiasedDenseFF(width, {"ff": ffw}, DT[dtype], "cuda")
    for k, v in W.items():
        assert ff.load(k, v)
    h = torch.randn(13, width, generator=g).to(DT[dtype])
    assert rel_err(ff.forward(h.cuda()), ref.dense_ff(W, "", h.double())) < (1e-5 if dtype == "float32" else 1.5e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(3, 1, 16, 24, 8), (4, 2, 64, 32, 64), (2, 2, 10, 7, 4), (5, 5, 32, 128, 0)])
def test_head_norms_rotation_and_cache_rows(dtype, shape):
    """Per-head statistics (heads of very different size), one weight vector for all heads, rotation of the first dims only with
    the pair (2i, 2i+1), at positions up to the thousands; values leave with unit RMS; a token with slot -1 stores nothing."""
    from nanovllm import mixops
    from nanovllm.layers.rotary_embedding import build_interleaved_cos_sin
    H, G, d, vd, dims = shape
    g = torch.Generator().manual_seed(sum(shape))
    n, base, eps = 9, 777.0, 1e-5
    cols = H * d + G * d + G * vd + 5                                           # other columns follow and stay untouched
    x = (torch.randn(n, cols, generator=g) * torch.linspace(0.2, 4.0, cols)).to(DT[dtype])
    wq, wk = (1 + 0.3 * torch.randn(d, generator=g)).to(DT[dtype]), (1 + 0.3 * torch.randn(d, generator=g)).to(DT[dtype])
    pos = torch.tensor([0, 1, 2, 63, 64, 500, 1999, 3, 1000], dtype=torch.int64)
    slots = torch.tensor([4, 0, 17, -1, 3, 9, 8, 30, 1], dtype=torch.int32)
    cache = torch.full((32, G * (d + vd)), 7.0, dtype=DT[dtype], device="cuda")
    table = build_interleaved_cos_sin(dims, 2048, base, None, "cuda") if dims else None
    xd = x.cuda().clone()
    mixops.headnorm_rope_store(xd, 0, H * d, H * d + G * d, H, G, d, vd, wq.cuda(), wk.cuda(), True, table, pos.cuda(), slots.cuda(), cache, eps)

    def turned(y, w):                                                            # plain: norm, weight, then rotate every token by its own position
        y = ref.unit_rms(y, eps) * w.double()
        if not dims:
            return y
        out = torch.empty_like(y)
        for t in range(n):
            full = torch.zeros(int(pos[t]) + 1, y.shape[1], y.shape[2], dtype=F64)
            full[-1] = y[t]
            out[t] = ref.rotate_pairs(full, dims, base)[-1]
        return out
    xx = x.double()
    tol = 3e-6 if dtype == "float32" else 4e-3
    assert rel_err(xd[:, :H * d], turned(xx[:, :H * d].view(n, H, d), wq).reshape(n, -1)) < tol
    wantk = turned(xx[:, H * d:H * d + G * d].view(n, G, d), wk).reshape(n, -1)
    wantv = ref.unit_rms(xx[:, H * d + G * d:H * d + G * d + G * vd].view(n, G, vd), eps).reshape(n, -1)
    for t, s in enumerate(slots.tolist()):
        if s >= 0:
            assert rel_err(cache[s, :G * d], wantk[t]) < tol and rel_err(cache[s, G * d:], wantv[t]) < tol
    untouched = [s for s in range(32) if s not in slots.tolist()]
    assert bool((cache[untouched] == 7.0).all())
    assert torch.equal(xd[:, H * d:].cpu(), x[:, H * d:])                       # only the queries change in place


def paged(rows, pages, bs, dtype, total_pages, stale=None):
    """rows [L, D] -> cache [total_pages * bs, D] with token j at pages[j // bs] * bs + j % bs; the rest holds `stale`."""
    cache = torch.zeros(total_pages * bs, rows.shape[1], dtype=DT[dtype]) if stale is None else stale.to(DT[dtype]).repeat(total_pages * bs, 1)
    for j in range(rows.shape[0]):
        cache[int(pages[j // bs]) * bs + j % bs] = rows[j].to(DT[dtype])
    return cache


def plain_mixed_attention(q, k, v, H, G, scale, window, keep, T, rows):
    """float64: softmax per head over the visible keys, the heads' weights mixed by T, then the values of the head's own group."""
    L = k.shape[0]
    see = ref.visible(L, window if window else L + 1, keep if window else 0)
    P = []
    for h in range(H):
        s = (q[:, h] @ k[:, h // (H // G)].T) * scale
        P.append(torch.softmax(torch.where(see, s, torch.full_like(s, -math.inf)), -1))
    mixed = torch.einsum("hg,gij->hij", T.double(), torch.stack(P))
    return torch.stack([mixed[h] @ v[:, h // (H // G)] for h in range(H)], 1)[rows]      # [rows, H, vd]


PATHS = [dict(fma=True), dict(), dict(splits=3)]          # fp32-pipe kernel, tensor-core kernel, tensor-core kernel with the keys split


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("bs,window,keep", [(16, 50, 3), (64, 64, 1), (64, 200, 70), (16, 30, 64), (16, 1, 2)])
def test_attention_sees_the_window_and_the_kept_first_tokens(dtype, bs, window, keep):
    """One key is made to dominate head 1: the head's own weights must then sit on that key exactly while it is inside the window
    or among the kept first tokens, and must not feel it one position later / one token further in.  The key sits at position 0,
    at the last kept position and the first one that is not kept, at page borders and far back; the query is the last row of a
    portion or a single decoded token; pages are scrambled and hold a stale dominating row beyond the sequence's end."""
    from nanovllm import mixops
    H, G, d, vd, L = 4, 2, 32, 32, 330
    g = torch.Generator().manual_seed(bs + window + keep)
    npages = (L + bs - 1) // bs + 1
    pages = torch.randperm(40, generator=g)[:npages]
    eye = torch.eye(H)
    for star in sorted({0, keep - 1, keep, bs - 1, bs, 129, L - 2}):
        q = torch.randn(L, H * d, generator=g)
        k = torch.randn(L, G * d, generator=g) * 0.3
        v = torch.randn(L, G * vd, generator=g)
        for pos in sorted({star, star + 1, star + window - 1, star + window, L - 1} & set(range(star, L))):
            qq, kk = q.clone(), k.clone()
            u = qq[pos, d:2 * d] / qq[pos, d:2 * d].norm()
            kk[star, :d] = 40.0 * u                           # head 1 (key/value head 0) of position `pos` looks straight at it
            qq[pos, d:2 * d] = 8.0 * u
            stale = torch.cat([60.0 * u.repeat(G), torch.full((G * vd,), 1e3)])
            cache = paged(torch.cat([kk, v], 1), pages, bs, dtype, 40, stale=stale)
            kv_t = torch.stack([cache[int(pages[j // bs]) * bs + j % bs] for j in range(pos + 1)]).double()
            qd = qq.to(DT[dtype]).double()
            want = plain_mixed_attention(qd[:pos + 1].view(-1, H, d), kv_t[:, :G * d].reshape(-1, G, d), kv_t[:, G * d:].reshape(-1, G, vd),
                                         H, G, 0.2, window, keep, eye, [pos])[0]
            seen = pos - star < window or star < keep
            near = (want[1] - kv_t[star, G * d:G * d + vd]).abs().max().item() < 1e-3
            assert near == seen, (star, pos)                   # the test itself distinguishes the two cases
            bt = pages[None, :].to(torch.int32).cuda().contiguous()
            for decode in (False, True):
                for kw in PATHS:
                    if decode:
                        qrows, sp = qq[pos:pos + 1], spans_decode([pos + 1])
                    else:
                        first = max(0, pos - 20)
                        qrows, sp = qq[first:pos + 1], spans_varlen([pos + 1 - first], [pos + 1])
                    acc = mixops.window_attention(qrows.to(DT[dtype]).cuda(), cache.cuda(), bt, bs, sp, H, G, d, vd, 0.2, None, window,
                                                  keep_first=keep, all_values=True, out_f32=True, **kw)
                    own = torch.stack([acc[-1, h, h // (H // G)] for h in range(H)]).double().cpu()
                    assert rel_err(own, want) < (1e-4 if dtype == "float32" else 2e-2), (star, pos, decode, kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(6, 2, 64, 64), (3, 1, 8, 24), (8, 8, 32, 32), (4, 2, 64, 128), (16, 1, 128, 32)])
def test_head_mixing_after_the_softmax(dtype, shape):
    """Every head's weights on every value head, then the mix: against the plain softmax, mix and product, for a prompt portion
    behind cached tokens and for single tokens, with a mixing matrix far from the identity and a gate; the result lands scaled in a
    column slice of a wider buffer."""
    from nanovllm import mixops
    H, G, d, vd = shape
    g = torch.Generator().manual_seed(sum(shape))
    L, bs, window, keep, scale = 150, 16, 40, 6, 0.3
    pages = torch.randperm(20, generator=g)[:(L + bs - 1) // bs]
    q, k, v = torch.randn(L, H * d, generator=g), torch.randn(L, G * d, generator=g), torch.randn(L, G * vd, generator=g)
    T = (torch.eye(H) * 0.5 + torch.randn(H, H, generator=g) * 0.6).float()
    gate = torch.randn(L, H * vd, generator=g).to(DT[dtype])
    cache = paged(torch.cat([k, v], 1), pages, bs, dtype, 20)
    kv = torch.stack([cache[int(pages[j // bs]) * bs + j % bs] for j in range(L)]).double()
    qd = q.to(DT[dtype])
    bt = pages[None, :].to(torch.int32).cuda().contiguous()
    want = plain_mixed_attention(qd.double().view(L, H, d), kv[:, :G * d].reshape(L, G, d), kv[:, G * d:].reshape(L, G, vd), H, G, scale, window,
                                 keep, T, list(range(L))) * torch.sigmoid(gate.double()).view(L, H, vd) * 1.7
    tol = 1e-4 if dtype == "float32" else 2.5e-2
    for first, last, decode in ((0, 100, False), (100, 149, False), (149, 150, True), (60, 61, True)):
        sp = spans_decode([last]) if decode else spans_varlen([last - first], [last])
        acc = mixops.window_attention(qd[first:last].cuda(), cache.cuda(), bt, bs, sp, H, G, d, vd, scale, None, window, keep_first=keep,
                                      all_values=True, out_f32=dtype != "float32")
        assert acc.shape == (last - first, H, G, vd)
        wide = torch.full((last - first, H * vd + 24), 5.0, dtype=DT[dtype], device="cuda")
        mixops.head_mix_gate(acc, T.cuda(), gate[first:last].cuda(), DT[dtype], out=wide[:, 8:8 + H * vd], out_scale=1.7)
        assert rel_err(wide[:, 8:8 + H * vd], want[first:last].reshape(last - first, -1)) < tol, (first, last)
        assert bool((wide[:, :8] == 5.0).all()) and bool((wide[:, 8 + H * vd:] == 5.0).all())


def _load(layer, W, pre, width):
    for leaf in layer.weight_shapes(width):
        assert layer.load(leaf, W[pre + leaf]), leaf
    return layer


def run_parts(layer, parts, bs, inst=0):
    """parts: [(h rows [n, width] on the host, tokens behind them, state slot, page list)] -> the layer's outputs, one per part,
    all parts in ONE step (a single-token step when every part brings one token behind cached ones)."""
    from nanovllm import mixops
    q_lens, k_lens = [p[0].shape[0] for p in parts], [p[1] + p[0].shape[0] for p in parts]
    decode = all(n == 1 and k > 1 for n, k in zip(q_lens, k_lens))
    sp = spans_decode(k_lens) if decode else spans_varlen(q_lens, k_lens)
    pos = torch.cat([torch.arange(p[1], p[1] + p[0].shape[0]) for p in parts]).to(torch.int64).cuda()
    width = max(len(p[3]) for p in parts)
    bt = torch.full((len(parts), width), -1, dtype=torch.int32)
    slot_map = []
    for r, p in enumerate(parts):
        bt[r, :len(p[3])] = torch.tensor(p[3], dtype=torch.int32)
        slot_map += [p[3][j // bs] * bs + j % bs for j in range(p[1], p[1] + p[0].shape[0])]
    ctx = SimpleNamespace(state_slots=torch.tensor([p[2] for p in parts], dtype=torch.int32, device="cuda"), block_tables=bt.cuda(),
                          slot_mapping=torch.tensor(slot_map, dtype=torch.int32, device="cuda"))
    h = torch.cat([p[0] for p in parts]).to(layer.dtype).cuda()
    out = layer.forward(h, pos, ctx, sp, inst)
    return list(out.split(q_lens))


def portions_batches_and_dirty_slots(layer, plain, width, dtype, bs=16, L=150, tol=None):
    """Three sequences through `layer`: whole, in portions of many sizes down to two tokens and single tokens, and side by side in one
    batch, in slots and pages that hold another sequence's leftovers, against `plain` (float64, whole sequence)."""
    g = torch.Generator().manual_seed(9)
    hs = [torch.randn(n, width, generator=g).to(DT[dtype]) for n in (L, 37, 9)]
    want = [plain(h.double()) for h in hs]
    tol = tol or (2e-4 if dtype == "float32" else 3e-2)
    layer.bind(40, bs, 4, 2)
    pg = lambda first, n: list(range(first, first + (n + bs - 1) // bs))
    # whole, alone (also dirties slot 1 and pages 0..): state left behind must not leak into the next owner
    got = run_parts(layer, [(hs[0], 0, 1, pg(0, L))], bs)
    assert rel_err(got[0], want[0]) < tol
    # portions, in the slot and pages just used by another sequence, second pass's states untouched by the first's
    for inst in (0, 1):
        outs, at = [], 0
        for n in (2, 3, 2, 31, 16, 2, 1, 1, 48, 15, 1, 5, 14, 9):
            outs.append(run_parts(layer, [(hs[0][at:at + n], at, 1, pg(0, L))], bs, inst)[0])
            at += n
        assert at == L and rel_err(torch.cat(outs), want[0]) < tol, inst
    # three unequal sequences in one batch, portions beside single tokens
    plan = [[(0, 60), (1, 2)], [(0, 1), (1, 30), (2, 9)], [(0, 1), (1, 1)], [(0, 1), (1, 1)], [(0, 87), (1, 3)]]
    at, outs = [0, 0, 0], [[], [], []]
    pages = [pg(20, L), pg(0, 37), pg(5, 9)]
    slots = [0, 3, 1]
    for step in plan:
        got = run_parts(layer, [(hs[s][at[s]:at[s] + n], at[s], slots[s], pages[s]) for s, n in step], bs)
        for (s, n), o in zip(step, got):
            outs[s].append(o)
            at[s] += n
    assert at == [L, 37, 9]
    for s in range(3):
        assert rel_err(torch.cat(outs[s]), want[s]) < tol, s
    layer.unbind()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("m", [dict(width=48, blocks=3, conv=4), dict(width=70, blocks=1, conv=1), dict(width=256, blocks=2, conv=2),
                               dict(width=36, blocks=36, conv=6)])
def test_gated_diagonal_recurrence_layer(dtype, m):
    from nanovllm.layers.diag_recurrence import GatedDiagonalRecurrence
    width = 40
    cfg = mh.config([({"type": "rglru", "mixer": m}, None)], width=width)
    W = mh.random_weights(cfg, 3)
    layer = _load(GatedDiagonalRecurrence(width, m, DT[dtype], "cuda"), {k: v.to(DT[dtype]) for k, v in W.items()}, "l0.mix.", width)
    portions_batches_and_dirty_slots(layer, lambda h: ref.rglru(W, "l0.mix.", m, h), width, dtype)
    # a portion long enough for the chunk-parallel form (chunks of 64 tokens), behind cached tokens and in a batch
    g = torch.Generator().manual_seed(5)
    h = torch.randn(400, width, generator=g).to(DT[dtype])
    want = ref.rglru(W, "l0.mix.", m, h.double())
    layer.bind(25, 16, 3, 1)
    pages = list(range(25))
    a = run_parts(layer, [(h[:7], 0, 2, pages)], 16)[0]
    b, c = run_parts(layer, [(h[7:391], 7, 2, pages), (h[:200], 0, 0, pages)], 16)
    d = run_parts(layer, [(h[391:], 391, 2, pages)], 16)[0]
    tol = 2e-4 if dtype == "float32" else 3e-2
    assert rel_err(torch.cat([a, b, d]), want) < tol and rel_err(c, want[:200]) < tol


def test_a_slow_channel_remembers_and_a_fast_one_forgets():
    """lam decides the memory: with a large negative lam the state carries an early input for hundreds of tokens, with a large
    positive one it is gone after one; r = 1 everywhere (large gate bias) makes the decay exactly exp(-8 softplus(lam))."""
    from nanovllm.layers.diag_recurrence import GatedDiagonalRecurrence
    m, width = dict(width=2, blocks=1, conv=1), 2
    layer = GatedDiagonalRecurrence(width, m, torch.float32, "cuda")
    z, one = torch.zeros, torch.ones
    W = {"y": torch.eye(2) * 50, "y.b": one(2), "x": torch.eye(2), "x.b": z(2), "conv": one(2, 1), "conv.b": z(2), "ra": z(1, 2, 2), "ra.b": one(1, 2) * 30,
         "ri": z(1, 2, 2), "ri.b": one(1, 2) * 30, "lam": torch.tensor([-9.0, 3.0]), "o": torch.eye(2)}
    _load(layer, W, "", width)
    layer.bind(19, 16, 1, 1)
    pages = list(range(19))
    h = torch.zeros(300, 2)
    h[0] = 1.0                                                       # one write, then silence; the bias of y keeps the read-out open
    out = torch.cat([run_parts(layer, [(h[:150], 0, 0, pages)], 16)[0], run_parts(layer, [(h[150:], 150, 0, pages)], 16)[0]]).cpu()
    want = ref.rglru({k: v for k, v in W.items()}, "", m, h.double())
    assert rel_err(out, want) < 1e-4
    a = math.exp(-8 * math.log1p(math.exp(-9.0)))
    ratio = (out[299, 0] / out[1, 0]).item()                         # what is left of token 0's write, 298 steps on
    assert abs(ratio / a ** 298 - 1.0) < 1e-3 and 0.7 < a ** 298 < 0.8 and out[5, 1].abs().item() < 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("m", [mh.right(), mh.right(heads=1, kv_heads=1, dim=10, vdim=6, conv=1), mh.right(heads=6, kv_heads=2, dim=20, vdim=40, conv=5),
                               mh.right(heads=2, kv_heads=1, dim=128, vdim=64, conv=2), mh.right(heads=2, kv_heads=2, dim=64, vdim=33, conv=3)])
def test_gated_delta_layer(dtype, m):
    from nanovllm.layers.gated_delta import GatedDeltaMixer
    width, eps = 40, 1e-5
    cfg = mh.config([(mh.parallel(mh.left(), m), None)], width=width)
    W = mh.random_weights(cfg, 4)
    layer = _load(GatedDeltaMixer(width, m, eps, DT[dtype], "cuda"), {k: v.to(DT[dtype]) for k, v in W.items()}, "l0.mix.right.", width)
    portions_batches_and_dirty_slots(layer, lambda h: ref.gated_delta(W, "l0.mix.right.", m, h, eps), width, dtype,
                                     tol=3e-4 if dtype == "float32" else 4e-2)


def test_the_delta_rule_overwrites_what_a_key_held():
    """With beta = 1 and no decay, writing a second value under the same key replaces the first: the read-out returns the new
    value only (a plain additive memory would return the sum), and an orthogonal key's value is left alone."""
    from nanovllm import mixops
    d, vd = 8, 32
    k1, k2 = torch.zeros(d), torch.zeros(d)
    k1[0], k2[3] = 1.0, 1.0
    g = torch.Generator().manual_seed(2)
    v = torch.randn(4, vd, generator=g)
    keys = torch.stack([k1, k2, k1, k1])
    qs = torch.stack([k1, k2, k1, k2])
    x = torch.cat([qs, keys, v], 1).cuda()
    ba = torch.tensor([[40.0, -40.0]] * 4, device="cuda")            # sigmoid(40) = 1; softplus(-40) = 0: no decay
    state = torch.full((1, 1, vd, d), 3.0, device="cuda")            # a new sequence ignores what the slot holds
    out = mixops.gated_delta(x, 0, d, 2 * d, ba, torch.tensor([-1.0], device="cuda"), torch.zeros(1, device="cuda"), state,
                             torch.zeros(1, dtype=torch.int32, device="cuda"), spans_varlen([4], [4]), 1, 1, d, vd, 1.0)[:, 0].cpu()
    assert rel_err(out[0], v[0]) < 1e-5 and rel_err(out[1], v[1]) < 1e-5
    assert rel_err(out[2], v[2]) < 1e-5                              # overwritten, not v[0] + v[2]
    assert rel_err(out[3], v[1]) < 1e-5                              # the other key's value survived both rewrites


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", [0, 1, 2])
def test_parallel_mixer_layer(dtype, which):
    """Both mixers on one input through the merged projections, over scrambled pages: small heads on the fp32 pipe, tensor-core
    heads with a window around the key tile, kept first tokens beyond the window size."""
    from nanovllm.layers.gated_delta import GatedDeltaMixer
    from nanovllm.layers.parallel_mixer import ParallelMixer
    from nanovllm.layers.window_attention import MixedHeadWindowAttention
    m = [mh.parallel()["mixer"], mh.config_c()["layers"][0]["mixer"], mh.config_c()["layers"][2]["mixer"]][which]
    width, eps = 48, 1e-5
    cfg = mh.config([({"type": "parallel", "mixer": m}, None)], width=width)
    W = mh.random_weights(cfg, 6)
    layer = ParallelMixer(width, MixedHeadWindowAttention, m["left"], GatedDeltaMixer, m["right"], m["left_scale"], m["right_scale"], DT[dtype],
                          "cuda", eps=eps, max_position=512)
    _load(layer, {k: v.to(DT[dtype]) for k, v in W.items()}, "l0.mix.", width)
    portions_batches_and_dirty_slots(layer, lambda h: ref.parallel_mixer(W, "l0.mix.", m, h, eps), width, dtype,
                                     tol=3e-4 if dtype == "float32" else 4e-2)


# ---------------------------------------------------------------------------------------------------------------------------
# whole models through the engine
# ---------------------------------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def checkpoints(tmp_path_factory):
    root = tmp_path_factory.mktemp("musavik")
    out = {}
    for name, cfg in (("a", mh.config_a()), ("b", mh.config_b()), ("c", mh.config_c())):
        W = mh.random_weights(cfg, 21)
        out[name] = (mh.write_checkpoint(str(root / name), cfg, W), cfg, W)
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
    """fp32: the RMS error over everything.  bf16: rounding of a projection's operands is relative to the terms of its sums, so a
    token whose small query or key of a dozen elements is then made a unit vector can come out several times worse than its
    neighbours in these tiny random models; the bound is therefore on the median over positions, with a loose one on the sum."""
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
        toks = mh.tokens(n, vocab, i)
        got = e.step([("p", toks)])["p"]
        e.end("p")
        assert_logits(got, oracle_logits(checkpoints, name, toks), dtype, n)


def test_the_stream_after_every_layer_run(checkpoints):
    """The residual stream after each run of each layer (repeated layers count every time) against the plain implementation."""
    from nanovllm.utils.context import set_context
    e = Replay(checkpoints["a"][0], "float32", eager=True)
    _, cfg, W = checkpoints["a"]
    toks = mh.tokens(45, cfg["vocab"], 3)
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
    assert len(taps) == len(want) == 1 + 3 * 2 + 1
    for r, (a, b) in enumerate(zip(taps, want)):
        assert rel_err(a, b) < 1e-4, r


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b"])
def test_long_decoding_matches_the_prompt_path(engines, checkpoints, name, dtype):
    """One prompt token, then 170 tokens one by one through the decode graphs, across ten pages and several windows."""
    e = engines(name, dtype)
    toks = mh.tokens(171, checkpoints[name][1]["vocab"], 5)
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
    toks = mh.tokens(sum(cuts), checkpoints[name][1]["vocab"], 6)
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
    their pages and state slots while the others go on.  Every request must come out as if it had run alone."""
    e = engines(name, dtype)
    vocab = checkpoints[name][1]["vocab"]
    T = {k: mh.tokens(n, vocab, 10 + i) for i, (k, n) in enumerate(dict(a=90, b=37, c=9, d=140, e=70, f=44).items())}
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
    """The configuration with tensor-core head sizes over pages as long as the key tile: a 333-token prompt in portions that end
    beside page borders and window edges, then single tokens, next to a second request that arrives in the middle."""
    e = Replay(checkpoints["c"][0], dtype, pool_tokens=768, block=64, seqs=3)
    vocab = checkpoints["c"][1]["vocab"]
    a, b = mh.tokens(333, vocab, 81), mh.tokens(90, vocab, 82)
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
    x, y = mh.tokens(50, vocab, 30), mh.tokens(21, vocab, 31)
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
    prompts = [mh.tokens(n, cfg["vocab"], 40 + i) for i, n in enumerate((5, 61, 1, 100, 18))]      # more requests than slots, chunked prompts
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
    toks = mh.tokens(40, cfg["vocab"], 50)
    steps = [{"step": 0, "entries": [{"id": "q", "tokens": toks[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "q", "tokens": toks[30:31], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "q", "tokens": toks[31:32], "want": [0]}, {"id": "r", "tokens": toks[:3], "want": [2]}], "end": ["r"]},
             {"step": 3, "entries": [{"id": "q", "tokens": toks[32:], "want": [7]}], "end": ["q"]}]
    out = tmp_path / "out"
    r = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", path, "--dtype", "float32", "--out", str(out), "--max-tokens", "128"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    want = ref.forward(cfg, W, toks)
    rd = lambda i: torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"]))
    assert not (out / "1.f32").exists()
    assert rel_err(rd(0), want[[0, 29]]) < 3e-4 and rel_err(rd(2), torch.stack([want[31], want[2]])) < 3e-4 and rel_err(rd(3), want[[39]]) < 3e-4
