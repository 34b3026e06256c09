"""Host-side parts of the Radupel decoder: the configuration reader and its plan, the tensor names and shapes, the run order
with a looped stretch (each pass with a cache entry of its own, every pass but the first taking the embedding's output in
again), what the layers keep, and the plain implementation's own mechanisms against brute force."""
import copy

import numpy as np
import pytest
import torch

import plain_radupel as plain
import radupel_models as M
from edgelm_b200.cache import CompositeEntry, SequenceCache
from edgelm_b200.config import ConfigError, config_class_for
from edgelm_b200.engine.model import DecoderModel
from edgelm_b200.parts import KVNeed, StateNeed


@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
def test_plan_names_every_tensor_with_its_shape(name):
    cfg = M.CONFIGS[name]
    conf = config_class_for(cfg).from_dict(cfg)
    assert type(conf).__name__ == "RadupelConfig"
    W = M.tensors_for(cfg, 0)
    want = DecoderModel(conf.plan(), torch.float32).expected_weights()
    assert {k: tuple(v) for k, v in want.items()} == {k: tuple(v.shape) for k, v in W.items()}
    again = config_class_for(conf.to_dict()).from_dict(conf.to_dict())
    assert again.plan() == conf.plan()


def test_the_plan_reads_every_constant():
    plan = config_class_for(M.CFG_A).from_dict(M.CFG_A).plan()
    assert plan.hidden_size == 64 and plan.vocab_size == 173 and plan.residual_streams == 1
    assert plan.head["softcap"] == 12.0 and plan.head["tied_to"] == "embed"
    assert [(e.layer, e.add_embedding) for e in plan.schedule] == [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    assert all(l.block == "parallel_prenorm" and l.mixer.kind == "parallel" for l in plan.layers)
    mix = plan.layers[0].mixer
    assert mix["left_scale"] == 1.3 and mix["right_scale"] == 0.7
    att = mix["left"]
    assert att.kind == "masked_attention" and att["mask"] is None and att["rot_pairs"] == "half" and att["head_gate"] is True and att["bias"] is False
    assert att["rot_dims"] == 8 and att["rot_base"] == 700.0 and att["scale"] == 0.3 and att["v_head_dim"] == 24 and att["conv"] == 2
    assert att["num_heads"] == 4 and att["num_kv_heads"] == 2 and att["head_dim"] == 16
    lin = mix["right"]
    assert lin.kind == "decay_linear_attention" and lin["heads"] == 2 and lin["head_dim"] == 24 and lin["v_head_dim"] == 16
    assert lin["decay"] == (0.9, 0.998) and lin["eps"] == 1e-5 and lin["activation"] == "silu"
    assert plan.layers[0].ffn.kind == "swiglu" and plan.layers[0].ffn["bias"] == ".b" and plan.layers[0].ffn["intermediate_size"] == 40
    ffn = plan.layers[1].ffn
    assert ffn.kind == "moe" and ffn["experts"] == 6 and ffn["top"] == 3 and ffn["intermediate_size"] == 24 and ffn["glu"] == (1.5, 1.702, 1.0)
    assert ffn["router"] == {"kind": "scored", "identity": 3, "groups": 3, "keep": 2, "scale": 1.7}
    assert ffn["shared"].kind == "clamped_glu" and ffn["shared"]["intermediate_size"] == 32 and ffn["shared"]["limit"] == 1.0 and ffn["shared"]["alpha"] == 1.702
    assert plan.layers[2].ffn is None and plan.layers[2].ffn_norm is None
    last = plan.layers[3]
    assert last.mixer["left"]["conv"] is None and last.mixer["left"]["rot_dims"] == 0
    assert last.ffn["router"] == {"kind": "scored", "identity": 0, "groups": 1, "keep": 1, "scale": 1.0} and last.ffn["shared"] is None
    b = config_class_for(M.CFG_B).from_dict(M.CFG_B).plan()
    assert b.head["softcap"] is None and [(e.layer, e.add_embedding) for e in b.schedule] == [(0, False), (1, False), (2, False)]
    c = config_class_for(M.CFG_C).from_dict(M.CFG_C).plan()
    assert [(e.layer, e.add_embedding) for e in c.schedule] == [(0, False), (1, False), (0, True), (1, False), (2, False)]
    assert c.first_runs(3).schedule[2].add_embedding


def test_refusals():
    for change, text in ((lambda c: c["layers"][0].update(type="attention"), "not part of this architecture"),
                         (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "kind 'glu'"),
                         (lambda c: c["layers"][0]["mixer"]["left"].pop("scale"), "'scale' is missing"),
                         (lambda c: c["layers"][0]["mixer"].pop("left_scale"), "'left_scale' is missing"),
                         (lambda c: c["layers"][0]["mixer"]["right"].update(decay=[0.5]), "one number per head"),
                         (lambda c: c["layers"][0]["mixer"]["right"].update(decay=[0.5, 1.5]), "decays"),
                         (lambda c: c.pop("norm"), "'norm'"),
                         (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "multiple"),
                         (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=18), "rotated dimensions"),
                         (lambda c: c["layers"][1]["mlp"]["router"].update(top=10), "of 6 experts"),
                         (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "groups"),
                         (lambda c: c["layers"][1]["mlp"]["expert"].update(limit=0.0), "limit"),
                         (lambda c: c.update(logit_softcap=-1.0), "logit_softcap"),
                         (lambda c: c["loop"].update(stop=5), "loop"),
                         (lambda c: c["loop"].update(times=0), "loop")):
        cfg = copy.deepcopy(M.CFG_A)
        change(cfg)
        with pytest.raises(ConfigError, match=text):
            DecoderModel(config_class_for(cfg).from_dict(cfg).plan(), torch.float32)


def test_what_the_layer_runs_keep():
    """Every run of a looped layer has an entry of its own: pages and a convolution's tail for the softmax attention, a
    matrix per head for the linear attention; a layer without a convolution keeps no tail."""
    model = DecoderModel(config_class_for(M.CFG_A).from_dict(M.CFG_A).plan(), torch.bfloat16)
    assert model.keeps_embedding
    needs = model.cache_needs()
    assert len(needs) == 8
    first = dict(needs[0].items)
    assert dict(first["left"].items) == {"kv": KVNeed(2, 16, None, v_head_dim=24), "conv": StateNeed((1, 4 * 16 + 2 * 16 + 2 * 24))}
    assert first["right"] == StateNeed((2, 16, 24))
    for run in (1, 3, 5):
        n = dict(needs[run].items)
        assert dict(n["left"].items) == {"kv": KVNeed(1, 8, None, v_head_dim=8), "conv": StateNeed((3, 8 * 8 + 8 + 8))} and n["right"] == StateNeed((3, 8, 40))
    last = dict(needs[7].items)
    assert last["left"] == KVNeed(1, 12, None, v_head_dim=20) and last["right"] == StateNeed((4, 8, 8))
    cache = SequenceCache(needs, max_tokens=256, max_positions=1 << 20)
    assert all(isinstance(e, CompositeEntry) for e in cache.entries)
    passes = [cache.entries[run]["right"] for run in (1, 3, 5)]
    assert len({id(e.group) for e in passes}) == 1 and sorted(e.index for e in passes) == [0, 1, 2]     # three passes, three states
    assert sorted(cache.entries[run]["left"]["kv"].index for run in (1, 3, 5)) == [0, 1, 2]
    s = cache.open()
    cache.reserve(s, 130)
    cache.advance(s, 130)
    cache.check()
    assert all(g.n_held[s] == 3 for g in cache.kv_groups)
    cache.close(s)
    cache.check()
    assert not DecoderModel(config_class_for(M.CFG_B).from_dict(M.CFG_B).plan(), torch.float32).keeps_embedding


def test_a_second_norm_without_a_feed_forward_may_be_stored():
    model = DecoderModel(config_class_for(M.CFG_A).from_dict(M.CFG_A).plan(), torch.float32)
    assert "l2.norm2" in model.ignorable_weights() and "l2.norm2" not in model.expected_weights() and "l0.norm2" not in model.ignorable_weights()


def test_plain_mechanisms_against_brute_force():
    g = np.random.default_rng(3)
    # the convolution: row t by hand, zeros before the first row, the last column is the current token's
    u, taps = g.normal(size=(6, 2)), g.normal(size=(2, 3))
    y = plain.causal_conv(u, taps)
    assert np.allclose(y[0], taps[:, 2] * u[0]) and np.allclose(y[1], taps[:, 1] * u[0] + taps[:, 2] * u[1])
    assert np.allclose(y[4], taps[:, 0] * u[2] + taps[:, 1] * u[3] + taps[:, 2] * u[4])
    # half-split pairs: dimension i turns with i + dims / 2, the rest passes, position 0 is the identity
    x = g.normal(size=(3, 1, 6))
    r = plain.rotate_half_pairs(x, np.array([0, 3, 11]), 4, 100.0)
    a = 11 * 100.0 ** (-2.0 / 4)
    assert np.allclose(r[0], x[0]) and np.allclose(r[..., 4:], x[..., 4:])
    assert np.allclose(r[2, 0, 1], x[2, 0, 1] * np.cos(a) - x[2, 0, 3] * np.sin(a))
    assert np.allclose(r[2, 0, 3], x[2, 0, 3] * np.cos(a) + x[2, 0, 1] * np.sin(a))
    # the linear attention as a sum over earlier tokens: o_t = sum_(s <= t) decay^(t - s) (q_t . k_s) v_s
    q, k, v = g.normal(size=(5, 1, 3)), g.normal(size=(5, 1, 3)), g.normal(size=(5, 1, 2))
    o = plain.decayed_linear_attention(q, k, v, np.array([0.8]))
    assert np.allclose(o[3, 0], sum(0.8 ** (3 - s) * (q[3, 0] @ k[s, 0]) * v[s, 0] for s in range(4)))
    # the gate per head multiplies the whole head: with a wide-open gate on head 0 and a shut one on head 1 only head 0 is left
    m = {"heads": 2, "kv_heads": 1, "dim": 2, "vdim": 2, "scale": 0.5}
    w = {"q": g.normal(size=(4, 3)), "k": g.normal(size=(2, 3)), "v": g.normal(size=(2, 3)), "g": np.array([[50.0, 0, 0], [-50.0, 0, 0]]), "o": np.eye(4)}
    h = np.abs(g.normal(size=(4, 3))) + 1.0
    out = plain.gated_softmax_attention(h, w, m, "")
    assert np.abs(out[:, 2:]).max() < 1e-12 and np.abs(out[:, :2]).max() > 1e-3
    # the router by hand: three groups of two, two kept; group scores are the best corrected score of a group
    z = np.log(np.array([[0.30, 0.05, 0.10, 0.20, 0.25, 0.10]]))
    corr = np.array([-0.30, 0.0, 0.0, 0.0, 0.0, 0.25])
    chosen, wts = plain.route(z, corr, 2, 3, 2, 2.0)
    # corrected: 0.00 0.05 | 0.10 0.20 | 0.25 0.35 -> groups 1 and 2 kept, experts 5 and 4 chosen, weights from 0.10 and 0.25
    assert chosen.tolist() == [[5, 4]] and np.allclose(wts, [[2.0 * 0.10 / 0.35, 2.0 * 0.25 / 0.35]])
    chosen, _ = plain.route(z, corr - 1.0, 3, 3, 1, 1.0)          # every score negative, one group kept: the third choice has nowhere to go but
    assert set(chosen[0, :2].tolist()) == {4, 5}                  # ... the kept group's two come first
    # an expert: the gate is capped from above only, the other branch on both sides
    w = {"gate": np.array([[3.0], [-3.0]]), "up": np.array([[-4.0], [4.0]]), "down": np.eye(2)}
    y = plain.clamped_expert(np.array([[1.0]]), w, "", 2.0)
    assert np.allclose(y[0], [2.0 * plain.sigmoid(1.702 * 2.0) * (-2.0 + 1.0), -3.0 * plain.sigmoid(1.702 * -3.0) * (2.0 + 1.0)])
    # identity experts give the input back: one routed expert that is an identity expert, weight = scale
    mlp = {"expert": {"ff": 2, "limit": 1.0}, "router": {"experts": 0, "top": 1, "identity": 1, "scale": 3.0}}
    hh = g.normal(size=(2, 3))
    assert np.allclose(plain.moe_ffn(hh, {"router": g.normal(size=(1, 3)), "correction": np.zeros(1)}, mlp, ""), 3.0 * hh)


def test_plain_model_is_causal_and_loops_take_the_embedding_again():
    cfg = M.CFG_A
    W = M.tensors_for(cfg, 5)
    t = M.tokens(cfg, 20, 0)
    full, runs = plain.forward(cfg, W, t, return_layers=True)
    assert np.allclose(plain.forward(cfg, W, t[:13]), full[:13], atol=1e-9)
    assert runs.shape == (8, 20, 64) and np.abs(full).max() <= 12.0
    # without the embedding's second entry the looped passes would differ: scale the table's rows and only the sum changes
    assert [a for _, a in plain.layer_order(cfg)] == [False, False, False, True, False, True, False, False]
