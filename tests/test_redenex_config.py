"""Host-side parts of the Redenex decoder: the configuration reader and its plan, the tensor names and shapes, the run
order with a looped stretch (each pass with a cache entry of its own), what the layers keep, and the plain
implementation's own mechanisms against brute force."""
import copy

import numpy as np
import pytest
import torch

import plain_redenex as plain
import redenex_models as M
from edgelm_b200.cache import CompositeEntry, SequenceCache
from edgelm_b200.config import ConfigError, config_class_for
from edgelm_b200.engine.model import DecoderModel
from edgelm_b200.parts import KVNeed, StateNeed


@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_plan_names_every_tensor_with_its_shape(name):
    cfg = M.CONFIGS[name]
    conf = config_class_for(cfg).from_dict(cfg)
    assert type(conf).__name__ == "RedenexConfig"
    W = M.tensors_for(cfg, 0)
    want = DecoderModel(conf.plan(), torch.float32).expected_weights()
    assert {k: tuple(v) for k, v in want.items()} == {k: tuple(v.shape) for k, v in W.items()}
    again = config_class_for(conf.to_dict()).from_dict(conf.to_dict())
    assert again.plan() == conf.plan()


def test_the_plan_reads_every_constant():
    plan = config_class_for(M.CFG_A).from_dict(M.CFG_A).plan()
    assert plan.embedding["scale"] == 3.0 and plan.hidden_size == 64 and plan.vocab_size == 173 and plan.residual_streams == 3
    assert [e.layer for e in plan.schedule] == [0, 1, 2, 1, 2, 1, 2, 3]
    att, att2 = plan.layers[0].mixer, plan.layers[2].mixer
    assert att.kind == "masked_attention" and att["mask"] == {"kind": "chunk", "size": 7} and att["rot_pairs"] == "half"
    assert att["rot_dims"] == 8 and att["rot_base"] == 700.0 and att["scale"] == 0.3 and att["v_head_dim"] == 24 and att["conv"] == 2
    assert att["diff"] == {"offset": 0.3, "eps": 1e-5} and att["qk_norm"] == {"eps": 1e-5} and att["num_kv_heads"] == 2
    assert att2["num_heads"] == 8 and att2["num_kv_heads"] == 1 and att2["conv"] == 4 and att2["diff"]["offset"] == 0.8
    rec = plan.layers[1].mixer
    assert rec.kind == "rglru" and rec["width"] == 96 and rec["blocks"] == 3 and rec["conv"] == 4 and rec["decay_scale"] == 8.0
    assert plan.layers[2].ffn is None and plan.layers[0].ffn["limit"] == 2.0 and plan.layers[1].ffn["intermediate_size"] == 56
    assert plan.layers[0].ffn["alpha"] == 1.702 and plan.layers[0].mixer_norm["offset"] == 1.0 and plan.layers[0].block == "hyper"
    b = config_class_for(M.CFG_B).from_dict(M.CFG_B).plan()
    assert b.residual_streams == 1 and b.layers[0].block == "hyper"         # one stream with its own weights is not the plain sum
    assert b.layers[1].mixer["rot_dims"] == 0 and b.layers[2].mixer["mask"] is None and [e.layer for e in b.schedule] == [0, 1, 2, 3]
    c = config_class_for(M.CFG_C).from_dict(M.CFG_C).plan()
    assert c.residual_streams == 1 and c.layers[0].block == "prenorm" and c.layers[0].mixer["conv"] is None
    assert [e.layer for e in c.schedule] == [0, 1, 0, 1, 2]


def test_refusals():
    for change, text in ((lambda c: c["layers"][0].update(type="conv"), "not part of this architecture"),
                         (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "kind 'moe'"),
                         (lambda c: c["layers"][0]["mixer"].pop("scale"), "'scale' is missing"),
                         (lambda c: c["layers"][0]["mixer"].pop("diff"), "'diff' is missing"),
                         (lambda c: c.pop("norm"), "'norm'"),
                         (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
                         (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "rotated dimensions"),
                         (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "chunk of 0"),
                         (lambda c: c["layers"][1]["mixer"].update(blocks=5), "5 blocks"),
                         (lambda c: c.update(streams=0), "0 residual streams"),
                         (lambda c: c.update(streams=9), "9 residual streams"),
                         (lambda c: c["loop"].update(stop=5), "loop"),
                         (lambda c: c["loop"].update(times=0), "loop")):
        cfg = copy.deepcopy(M.CFG_A)
        change(cfg)
        with pytest.raises(ConfigError, match=text):
            DecoderModel(config_class_for(cfg).from_dict(cfg).plan(), torch.float32)


def test_what_the_layer_runs_keep():
    """Every run of a looped layer has an entry of its own; a convolution of one tap keeps no input."""
    model = DecoderModel(config_class_for(M.CFG_A).from_dict(M.CFG_A).plan(), torch.bfloat16)
    needs = model.cache_needs()
    assert len(needs) == 8
    att0 = dict(needs[0].items)
    assert att0 == {"kv": KVNeed(2, 32, None, v_head_dim=24), "conv": StateNeed((1, 4 * 32 + 2 * 32 + 2 * 24))}
    for run in (1, 3, 5):
        assert dict(needs[run].items) == {"conv": StateNeed((3, 96)), "rglru": StateNeed((96,))}
    for run in (2, 4, 6):
        assert dict(needs[run].items) == {"kv": KVNeed(1, 16, None, v_head_dim=8), "conv": StateNeed((3, 8 * 16 + 16 + 8))}
    assert dict(needs[7].items) == {"rglru": StateNeed((40,))}
    no_conv = DecoderModel(config_class_for(M.CFG_C).from_dict(M.CFG_C).plan(), torch.float32).cache_needs()
    assert no_conv[0] == KVNeed(2, 48, None, v_head_dim=16) and no_conv[2] == no_conv[0]
    cache = SequenceCache(needs, max_tokens=256, max_positions=1 << 20)
    assert all(isinstance(e, CompositeEntry) for e in cache.entries[:7])
    passes = [cache.entries[run]["rglru"] for run in (1, 3, 5)]
    assert len({id(e.group) for e in passes}) == 1 and sorted(e.index for e in passes) == [0, 1, 2]     # three passes, three states
    assert sorted(cache.entries[run]["kv"].index for run in (2, 4, 6)) == [0, 1, 2]
    s = cache.open()
    cache.reserve(s, 130)
    cache.advance(s, 130)
    cache.check()
    assert all(g.n_held[s] == 3 for g in cache.kv_groups)
    cache.close(s)
    cache.check()


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
    # the recurrent unit with one block of one channel, by hand: S_0 = sqrt(1 - a^2) i u (no special first token)
    w = {"y": np.array([[0.5]]), "y.b": np.array([0.1]), "x": np.array([[2.0]]), "x.b": np.array([-0.3]), "conv": np.array([[1.0]]),
         "conv.b": np.array([0.2]), "ra": np.array([[[0.7]]]), "ra.b": np.array([[0.1]]), "ri": np.array([[[-0.4]]]), "ri.b": np.array([[0.3]]),
         "lam": np.array([-1.0]), "o": np.array([[1.5]])}
    h = np.array([[0.8], [-0.6]])
    out = plain.rglru_mixer(h, w, {"width": 1, "blocks": 1, "conv": 1}, "")
    S, want = 0.0, []
    for t in range(2):
        u_t = 2.0 * h[t, 0] - 0.3 + 0.2
        a_t = np.exp(-8.0 * plain.sigmoid(0.7 * u_t + 0.1) * np.log1p(np.exp(-1.0)))
        S = a_t * S + np.sqrt(1 - a_t * a_t) * plain.sigmoid(-0.4 * u_t + 0.3) * u_t
        want.append(1.5 * S * plain.gelu_tanh(0.5 * h[t, 0] + 0.1))
    assert np.allclose(out[:, 0], want)
    # differential attention of one head, row 5 of a chunk of 4, by hand
    d, e = 3, 2
    m = {"heads": 1, "kv_heads": 1, "dim": d, "vdim": e, "diff": 0.4, "scale": 0.6, "mask": {"size": 4}}
    w = {"q": g.normal(size=(2 * d, 5)), "k": g.normal(size=(2 * d, 5)), "v": g.normal(size=(e, 5)), "q.b": g.normal(size=2 * d),
         "k.b": g.normal(size=2 * d), "v.b": g.normal(size=e), "q.norm": g.uniform(0.5, 1.5, d), "k.norm": g.uniform(0.5, 1.5, d),
         "lq1": g.normal(size=d), "lk1": g.normal(size=d), "lq2": g.normal(size=d), "lk2": g.normal(size=d), "o": np.eye(e)}
    h = g.normal(size=(7, 5))
    out = plain.differential_attention(h, w, m, "", 1e-6)
    unit = lambda z, nw: z / np.sqrt((z * z).mean() + 1e-6) * nw
    lam = np.exp(w["lq1"] @ w["lk1"]) - np.exp(w["lq2"] @ w["lk2"]) + 0.4
    maps = []
    for j in range(2):
        qj = unit((w["q"] @ h[5] + w["q.b"])[j * d:(j + 1) * d], w["q.norm"])
        s = np.array([qj @ unit((w["k"] @ h[t] + w["k.b"])[j * d:(j + 1) * d], w["k.norm"]) * 0.6 for t in (4, 5)])
        p = np.exp(s) / np.exp(s).sum()
        maps.append(p @ np.stack([w["v"] @ h[t] + w["v.b"] for t in (4, 5)]))
    o = maps[0] - lam * maps[1]
    assert np.allclose(out[5], o / np.sqrt((o * o).mean() + 1e-6) * 0.6)
    # the feed-forward: the gate is capped from above only, the other branch on both sides
    w = {"gate": np.array([[3.0], [-3.0]]), "up": np.array([[-4.0], [4.0]]), "down": np.eye(2)}
    y = plain.clamped_glu(np.array([[1.0]]), w, {"limit": 2.0}, "")
    assert np.allclose(y[0], [2.0 * plain.sigmoid(1.702 * 2.0) * (-2.0 + 1.0), -3.0 * plain.sigmoid(1.702 * -3.0) * (2.0 + 1.0)])
    # streams: the mix matrix is [from, to]
    xs = g.normal(size=(2, 1, 3))
    w = {"in": np.array([0.5, 2.0]), "out": np.array([1.0, -1.0]), "mix": np.array([[1.0, 10.0], [0.0, 1.0]])}
    new = plain.hyper_sublayer(xs, w, "", lambda u: 2.0 * u)
    y = 2.0 * (0.5 * xs[0] + 2.0 * xs[1])
    assert np.allclose(new[0], xs[0] + y) and np.allclose(new[1], 10.0 * xs[0] + xs[1] - y)


def test_plain_model_is_causal_and_chunked():
    """A later token changes no earlier logits; with every mixer chunked attention, a token past a chunk's edge does not
    see the tokens before the edge."""
    cfg = M.CFG_A
    W = M.tensors_for(cfg, 5)
    t = M.tokens(cfg, 20, 0)
    full = plain.forward(cfg, W, t)
    assert np.allclose(plain.forward(cfg, W, t[:13]), full[:13], atol=1e-9)
    only = {"architecture": "Redenex", "vocab": 50, "width": 16, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0}, "streams": 2,
            "layers": [M.attention(2, 1, 8, 4, None, 0.5, 0.3, {"base": 10.0, "dims": 8}, 5, M.dense(8, 1.0))]}
    W = M.tensors_for(only, 6)
    a, b = M.tokens(only, 12, 1), M.tokens(only, 12, 2)
    b[10:] = a[10:]
    assert np.allclose(plain.forward(only, W, a)[10:], plain.forward(only, W, b)[10:], atol=1e-9)       # positions 10, 11: chunk 2
    b[9] = a[9]
    assert not np.allclose(plain.forward(only, W, a)[9], plain.forward(only, W, b)[9], atol=1e-6)       # position 9 sees 5 .. 8
