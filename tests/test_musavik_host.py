"""Host side of the Musavik path (no GPU): configuration reader and registry, execution order of repeated layers, checkpoint
tensor names and shapes, and a few properties of the plain implementation the GPU tests lean on."""
import json

import pytest
import torch

import musavik_helpers as mh
from oracle import musavik_ref as ref


def _model(cfg):
    from nanovllm.models.musavik import MusavikConfig, MusavikForCausalLM
    return MusavikForCausalLM(MusavikConfig(cfg), device="cpu", max_position=64)


def test_registry_reads_the_configuration(tmp_path):
    from nanovllm.models.musavik import MusavikConfig, MusavikForCausalLM
    from nanovllm.models.registry import model_class, read_config
    cfg = mh.config_a()
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    c = read_config(str(tmp_path))
    assert isinstance(c, MusavikConfig) and model_class(c) is MusavikForCausalLM
    assert (c.vocab_size, c.hidden_size, c.norm_eps, c.embed_scale) == (97, 64, 2e-5, 2.5)
    assert c.pair == {"buckets": 53, "mul_prev": 7, "mul_cur": 11} and c.num_hidden_layers == 4
    b = MusavikConfig(mh.config_b())
    assert b.pair is None and b.embed_scale == 1.0
    assert MusavikConfig(mh.config_c()).loop is None


@pytest.mark.parametrize("cfg", [mh.config_a(), mh.config_b(), mh.config_c()])
def test_execution_order_of_repeated_layers(cfg):
    from nanovllm.models.musavik import layer_runs
    runs = layer_runs(len(cfg["layers"]), cfg.get("loop"))
    assert [(i, opens) for i, _, opens in runs] == ref.layer_runs(cfg)
    # every (layer, pass) pair occurs once: each pass has a cache and state of its own
    assert len({(i, k) for i, k, _ in runs}) == len(runs)


def test_execution_order_by_hand():
    from nanovllm.models.musavik import MusavikConfig, layer_runs
    assert layer_runs(5, {"start": 1, "stop": 3, "times": 3}) == [(0, 0, False), (1, 0, True), (2, 0, False), (1, 1, True), (2, 1, False),
                                                                (1, 2, True), (2, 2, False), (3, 0, False), (4, 0, False)]
    assert layer_runs(2, {"start": 0, "stop": 2, "times": 1}) == [(0, 0, True), (1, 0, False)]
    assert layer_runs(3, None) == [(0, 0, False), (1, 0, False), (2, 0, False)]
    c = MusavikConfig(mh.config_a())
    assert [c.passes_of(i) for i in range(4)] == [1, 3, 3, 1]
    for bad in ({"start": 2, "stop": 2, "times": 2}, {"start": 0, "stop": 9, "times": 2}, {"start": 0, "stop": 1, "times": 0}):
        with pytest.raises(ValueError):
            layer_runs(4, bad)


def test_bad_configurations_are_refused():
    from nanovllm.models.musavik import MusavikConfig
    cfg = mh.config_a()
    cfg["layers"][0]["type"] = "lstm"
    with pytest.raises(ValueError):
        MusavikConfig(cfg)
    cfg = mh.config_a()
    cfg["layers"][1]["mlp"]["kind"] = "moe"
    with pytest.raises(ValueError):
        MusavikConfig(cfg)


@pytest.mark.parametrize("cfg", [mh.config_a(), mh.config_b(), mh.config_c()])
def test_checkpoint_tensor_names_and_shapes(cfg):
    m = _model(cfg)
    assert {k: tuple(v) for k, v in m.weight_shapes().items()} == mh.shapes(cfg)
    W = mh.random_weights(cfg, 1)
    for name, w in W.items():
        m.load_hf_tensor(name, w)
    with pytest.raises(KeyError):
        m.load_hf_tensor("l0.mix.nothing", torch.zeros(1))
    with pytest.raises(KeyError):
        m.load_hf_tensor("l99.norm1", torch.zeros(1))
    per_pass = [b.mixer.state_slot_bytes() for b in m.blocks]
    assert m.state_slot_bytes() == sum(p * b.passes for p, b in zip(per_pass, m.blocks)) + 8


def test_merged_projections_hold_both_mixers_tensors():
    """The parallel mixer's two input projections and two output projections live in one weight each; loading by name fills the
    right rows and columns."""
    cfg = mh.config_a()
    m = _model(cfg)
    W = mh.random_weights(cfg, 2)
    for name, w in W.items():
        m.load_hf_tensor(name, w)
    pm = m.blocks[1].mixer
    l, r = cfg["layers"][1]["mixer"]["left"], cfg["layers"][1]["mixer"]["right"]
    rows = [("left.q", l["heads"] * l["dim"]), ("left.k", l["kv_heads"] * l["dim"]), ("left.v", l["kv_heads"] * l["vdim"]), ("left.g", l["heads"] * l["vdim"]),
            ("right.q", r["kv_heads"] * r["dim"]), ("right.k", r["kv_heads"] * r["dim"]), ("right.v", r["heads"] * r["vdim"]), ("right.g", r["heads"] * r["vdim"])]
    at = 0
    for leaf, n in rows:
        assert torch.equal(pm.w_in[at:at + n], W["l1.mix." + leaf]), leaf
        at += n
    assert at == pm.w_in.shape[0]
    assert torch.equal(pm.w_o, torch.cat([W["l1.mix.left.o"], W["l1.mix.right.o"]], 1))
    assert torch.equal(pm.b_in[:rows[0][1]], W["l1.mix.left.q.b"]) and bool((pm.b_in[sum(n for _, n in rows[:3]):] == 0).all())


def test_plain_implementation_is_causal_and_windows_are_exact():
    cfg = mh.config_a()
    W = mh.random_weights(cfg, 5)
    toks = mh.tokens(40, cfg["vocab"], 1)
    full = ref.forward(cfg, W, toks)
    assert torch.allclose(ref.forward(cfg, W, toks[:23]), full[:23], atol=1e-9)
    see = ref.visible(12, 4, 2)
    assert see[9].tolist() == [True, True, False, False, False, False, True, True, True, True, False, False]
    assert see[3].tolist() == [True, True, True, True] + [False] * 8
    # the pair embedding depends on the previous token, and the first token takes the extra row
    a, b = ref.embedding(W, cfg, [5, 9]), ref.embedding(W, cfg, [6, 9])
    assert not torch.allclose(a[1], b[1]) and torch.allclose(ref.embedding(W, cfg, [9])[0] - W["embed"].double()[9] * 2.5, W["bigram"].double()[53])


def test_state_slots_and_pages_change_hands():
    """The block manager gives a finished sequence's pages and state slot to the next one (lowest free slot first)."""
    from nanovllm.engine.block_manager import BlockManager
    from nanovllm.engine.sequence import Sequence
    Sequence.block_size = 16
    bm = BlockManager(6, 16, num_state_slots=2, prefix_cache=False)
    a, b, c = Sequence(list(range(40))), Sequence(list(range(20))), Sequence(list(range(30)))
    bm.extend(a), bm.extend(b)
    assert (a.state_slot, b.state_slot) == (0, 1) and len(a.block_table) == 3 and len(b.block_table) == 2
    assert not bm.can_extend(c)                       # no slot left
    held = list(a.block_table)
    bm.deallocate(a)
    assert bm.can_extend(c)
    bm.extend(c)
    assert c.state_slot == 0 and set(c.block_table) & set(held)
