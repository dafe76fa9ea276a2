"""Host side of the Fegolorn path (no GPU): configuration reader and registry, layers that borrow weights, checkpoint tensor names
and shapes, the folded norm weights, and a few properties of the plain implementation the GPU tests lean on."""
import json

import pytest
import torch

import fegolorn_helpers as fh
from oracle import fegolorn_ref as ref


def _model(cfg):
    from nanovllm.models.fegolorn import FegolornConfig, FegolornForCausalLM
    return FegolornForCausalLM(FegolornConfig(cfg), device="cpu", max_position=64)


def test_registry_reads_the_configuration(tmp_path):
    from nanovllm.models.fegolorn import FegolornConfig, FegolornForCausalLM
    from nanovllm.models.registry import model_class, read_config
    cfg = fh.config_a()
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    c = read_config(str(tmp_path))
    assert isinstance(c, FegolornConfig) and model_class(c) is FegolornForCausalLM
    assert (c.vocab_size, c.hidden_size, c.norm_eps, c.embed_scale, c.logit_softcap) == (97, 64, 2e-5, 2.5, 12.0)
    assert c.pair == {"buckets": 53, "mul_prev": 7, "mul_cur": 11} and c.num_hidden_layers == 6
    b = FegolornConfig(fh.config_b())
    assert b.pair is None and b.embed_scale == 1.0 and b.logit_softcap == 0.0


def test_layers_that_borrow_weights_get_caches_of_their_own():
    from nanovllm.models.fegolorn import FegolornConfig
    c = FegolornConfig(fh.config_a())
    assert c.runs == [(0, 0), (1, 0), (1, 1), (3, 0), (0, 1), (1, 2)] and c.copies == {0: 2, 1: 3, 3: 1}
    assert len(set(c.runs)) == len(c.runs)
    m = _model(fh.config_a())
    assert sorted(m.blocks) == [0, 1, 3]
    elems = 2 * (24 + 8) + 3 * 2 * (16 + 8) + (16 + 4)
    assert m.cache_block_bytes(16) == elems * 16 * 2 and m.state_slot_bytes() == 8


def test_bad_configurations_are_refused():
    from nanovllm.models.fegolorn import FegolornConfig
    cfg = fh.config_a()
    cfg["layers"][0]["type"] = "lstm"
    with pytest.raises(ValueError):
        FegolornConfig(cfg)
    cfg = fh.config_a()
    cfg["layers"][1]["mlp"]["kind"] = "glu"
    with pytest.raises(ValueError):
        FegolornConfig(cfg)
    cfg = fh.config_a()
    cfg["layers"][2]["weights_of"] = 4                                       # a later layer
    with pytest.raises(ValueError):
        FegolornConfig(cfg)
    cfg = fh.config_a()
    cfg["layers"][5]["weights_of"] = 2                                       # a layer that borrows itself
    with pytest.raises(ValueError):
        FegolornConfig(cfg)
    cfg = fh.config_a()
    cfg["layers"][2]["type"] = "latent_attention"                            # not the mixer of the layer it borrows from
    with pytest.raises(ValueError):
        FegolornConfig(cfg)


@pytest.mark.parametrize("cfg", [fh.config_a(), fh.config_b(), fh.config_c()])
def test_checkpoint_tensor_names_and_shapes(cfg):
    """Every tensor the helpers write is taken, under its name, and none is missing; the norms' single numbers load from 0-d tensors."""
    m = _model(cfg)
    want = {k: (tuple(v) or (1,)) for k, v in fh.shapes(cfg).items()}
    assert {k: tuple(v) for k, v in m.weight_shapes().items()} == want
    for name, w in fh.random_weights(cfg, 3).items():
        m.load_hf_tensor(name, w)
    with pytest.raises(KeyError):
        m.load_hf_tensor("l0.mix.sink", torch.zeros(3))
    borrowed = [i for i, l in enumerate(cfg["layers"]) if l.get("weights_of") is not None]
    for i in borrowed:
        with pytest.raises(KeyError):
            m.load_hf_tensor(f"l{i}.norm1", torch.ones(()))


def test_norm_numbers_and_column_scales_are_folded_in_fp32():
    from nanovllm.layers.layernorm import GatedScaledSandwich
    s = GatedScaledSandwich(5, 1e-5, torch.bfloat16, "cpu")
    ls = torch.tensor([0.5, 1.0, 1.5, 2.0, 0.25], dtype=torch.bfloat16)
    s.load("ls", ls)
    assert torch.equal(s.w_out, ls.float())
    s.load("out", torch.tensor(0.8125, dtype=torch.bfloat16))
    assert torch.equal(s.w_out, ls.float() * 0.8125)
    s.load("ls", 2 * ls)                                                     # either order
    assert torch.equal(s.w_out, 2 * ls.float() * 0.8125)
    s.load("in", torch.tensor(1.375))
    assert torch.equal(s.w_in32, torch.full((5,), 1.375)) and s.w_in.dtype == torch.bfloat16 and torch.equal(s.w_in.float(), s.w_in32)


def test_frequency_bands():
    from nanovllm.layers.rotary_embedding import banded_frequencies, build_banded_cos_sin
    sc = dict(factor=4.0, low=1.0, high=4.0, original=64)
    f, plain = banded_frequencies(8, 5000.0, sc), banded_frequencies(8, 5000.0)
    assert torch.allclose(f, ref.frequencies(8, 5000.0, sc), rtol=1e-13, atol=0)
    assert f[0] == plain[0] and torch.isclose(f[3], plain[3] / 4) and plain[1] / 4 < f[1] < plain[1]
    t = build_banded_cos_sin(8, 50, 5000.0, sc)
    assert t.shape == (50, 8) and t.dtype == torch.float32
    assert torch.allclose(t[7, :4].double(), (7 * f).cos(), atol=1e-7) and torch.allclose(t[7, 4:].double(), (7 * f).sin(), atol=1e-7)


def test_plain_rotations_are_inverse_and_relative():
    """What the GPU tests of the rotated values lean on: turning by p and back is the identity, and the two layouts pair differently."""
    g = torch.Generator().manual_seed(1)
    x = torch.randn(6, 2, 8, generator=g, dtype=torch.float64)
    pos = torch.tensor([0, 1, 5, 64, 500, 1999])
    f = ref.frequencies(8, 100.0)
    for layout in ("interleaved", "halves"):
        y = ref.rotate(x, pos, f, layout)
        assert torch.allclose(ref.rotate(y, pos, f, layout, sign=-1.0), x, atol=1e-12)
        assert torch.equal(y[0], x[0]) and not torch.allclose(y[1], x[1])
    a, b = ref.rotate(x, pos, f, "interleaved"), ref.rotate(x, pos, f, "halves")
    assert not torch.allclose(a, b) and torch.allclose(a.norm(dim=-1), x.norm(dim=-1)) and torch.allclose(b.norm(dim=-1), x.norm(dim=-1))
    swap = [0, 4, 1, 5, 2, 6, 3, 7]                                          # element 2i of one layout is element i of the other
    assert torch.allclose(ref.rotate(x[..., swap], pos, f, "interleaved"), b[..., swap], atol=1e-12)
    part = ref.rotate(x, pos, ref.frequencies(4, 100.0), "interleaved")
    assert torch.equal(part[..., 4:], x[..., 4:])


def test_plain_model_properties():
    """Tokens later in the sequence do not change earlier logits; the pair table's last row serves the first token; a layer that
    borrows weights changes the result when its source's weights change."""
    cfg = fh.config_a()
    W = fh.random_weights(cfg, 5)
    toks = fh.tokens(40, cfg["vocab"], 1)
    full = ref.forward(cfg, W, toks)
    assert torch.allclose(ref.forward(cfg, W, toks[:25]), full[:25], atol=1e-9)
    assert float(full.abs().max()) < cfg["logit_softcap"]
    W2 = dict(W)
    W2["bigram"] = W["bigram"].clone()
    W2["bigram"][-1] += 1.0
    changed = ref.forward(cfg, W2, toks)
    assert not torch.allclose(changed[0], full[0])
    W3 = dict(W)
    W3["bigram"] = W["bigram"].clone()
    W3["bigram"][:-1] += 1.0
    assert torch.allclose(ref.forward(cfg, W3, toks[:1]), full[:1], atol=1e-12)
