"""Small Radupel configurations and model folders for the tests.

Weights are drawn so that nothing hides: convolution taps of comparable size (a lost tail shows), decays from 0.3 to 1 (a
state remembers a few tokens in one head and hundreds in another), router matrices large enough for decisive scores,
corrections as large as the scores' differences (and all negative in one model, so that a masked group counted as 0 instead of
minus infinity would win), biases of order 1, gates away from one half.  The folders are written in bfloat16 (what a float32
engine widens exactly), so the plain implementation and the library compute from the same numbers.
"""
import json
import os

import numpy as np
import torch


def left(heads, kv_heads, dim, vdim, conv, rot, scale):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if conv:
        m["conv"] = conv
    if rot:
        m["rot"] = rot
    return m


def right(heads, dim, vdim, decay):
    assert len(decay) == heads
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def layer(l, r, ls, rs, mlp):
    return {"type": "parallel", "mixer": {"left": l, "right": r, "left_scale": ls, "right_scale": rs}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, limit, experts, top, identity, groups, keep, scale, shared):
    r = {"experts": experts, "top": top, "identity": identity, "scale": scale}
    if groups:
        r["groups"] = {"count": groups, "keep": keep}
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": r}
    if shared:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


# Sizes differ in everything from layer to layer and between the models: grouped, multi-query (eight query heads to a key
# head: decoding shares staged keys and splits pages) and one key head per query head; value heads wider and narrower than
# key heads in both mixers; rotation of a part of a head, of all of it, and none; 1 to 4 taps and no convolution; key sizes
# of the linear attention under, at and over a warp's 32 lanes; one to three chosen of 3 to 9 routed experts with 0 to 3
# identity experts, one group, two of three, one of three; shared expert or none; layers without a feed-forward; a loop in the
# middle run three times, a loop from the first layer, no loop; a soft cap or none; widths that are no multiple of 8.
CFG_A = {"architecture": "Radupel", "vocab": 173, "width": 64, "norm": {"eps": 1e-5}, "logit_softcap": 12.0,
         "loop": {"start": 1, "stop": 3, "times": 3}, "layers": [
    layer(left(4, 2, 16, 24, 2, {"base": 700.0, "dims": 8}, 0.3), right(2, 24, 16, (0.9, 0.998)), 1.3, 0.7, dense(40)),
    layer(left(8, 1, 8, 8, 4, {"base": 10000.0, "dims": 8}, 0.4), right(3, 40, 8, (0.3, 0.97, 1.0)), 0.8, 1.1,
          moe(24, 1.5, 6, 3, 3, 3, 2, 1.7, (32, 1.0))),
    layer(left(2, 2, 24, 8, 3, {"base": 50.0, "dims": 12}, 0.25), right(1, 32, 48, (0.95,)), 1.0, 1.0, None),
    layer(left(3, 1, 12, 20, None, None, 0.35), right(4, 8, 8, (0.5, 0.8, 0.99, 0.9)), 0.6, 1.4, moe(16, 0.8, 3, 1, 0, None, None, 1.0, None)),
]}
CFG_B = {"architecture": "Radupel", "vocab": 97, "width": 50, "norm": {"eps": 3e-4}, "layers": [
    layer(left(3, 3, 10, 14, 1, None, 0.35), right(2, 20, 30, (0.85, 0.6)), 1.1, 0.9, moe(20, 3.0, 5, 2, 1, 3, 2, 2.2, (18, 2.0))),
    layer(left(2, 1, 32, 20, 3, {"base": 90.0, "dims": 32}, 0.2), right(5, 10, 6, (0.99, 0.9, 0.7, 0.4, 0.995)), 0.9, 1.2, dense(30)),
    layer(left(6, 3, 8, 40, 2, {"base": 3000.0, "dims": 4}, 0.5), right(2, 64, 12, (0.98, 0.93)), 1.2, 0.5, dense(18)),
]}
CFG_C = {"architecture": "Radupel", "vocab": 120, "width": 48, "norm": {"eps": 1e-6}, "logit_softcap": 4.0,
         "loop": {"start": 0, "stop": 2, "times": 2}, "layers": [
    layer(left(2, 2, 24, 16, 4, {"base": 50.0, "dims": 12}, 0.25), right(3, 16, 24, (0.9, 0.99, 0.75)), 1.0, 0.8,
          moe(32, 1.2, 7, 2, 2, 3, 1, 0.9, (24, 0.7))),
    layer(left(16, 2, 8, 12, 2, {"base": 300.0, "dims": 6}, 0.45), right(2, 12, 20, (0.96, 0.88)), 0.7, 1.3, None),
    layer(left(1, 1, 40, 40, 3, None, 0.15), right(1, 72, 8, (0.97,)), 1.5, 0.6, dense(64)),
]}
# head sizes that the tensor-core kernels take (softmax attention with key = value heads of 64 and 32, in bfloat16) and that the
# chunked linear attention reads 16 bytes at a time
CFG_D = {"architecture": "Radupel", "vocab": 150, "width": 64, "norm": {"eps": 1e-5}, "logit_softcap": 20.0,
         "loop": {"start": 1, "stop": 2, "times": 2}, "layers": [
    layer(left(4, 2, 64, 64, 3, {"base": 4000.0, "dims": 16}, 0.12), right(2, 64, 64, (0.92, 0.99)), 1.1, 0.9, dense(48)),
    layer(left(2, 2, 32, 32, 2, {"base": 100.0, "dims": 32}, 0.2), right(1, 32, 64, (0.97,)), 0.9, 1.2,
          moe(16, 1.1, 4, 2, 2, 2, 1, 1.4, (16, 0.9))),
]}
CONFIGS = {"a": CFG_A, "b": CFG_B, "c": CFG_C, "d": CFG_D}
NEGATIVE_CORRECTIONS = ("c",)      # models whose corrections make every choice score negative


def tensors_for(cfg, seed, negative_corrections=False):
    g = np.random.default_rng(seed)
    D, V = cfg["width"], cfg["vocab"]
    W = {}

    def mat(name, rows, cols, gain=1.0):
        W[name] = g.normal(0.0, gain / np.sqrt(cols), size=(rows, cols))

    def vec(name, n, lo, hi):
        W[name] = g.uniform(lo, hi, size=(n,))

    def taps(name, n, k):
        W[name] = g.normal(0.0, 0.5, size=(n, k)) + (np.arange(k) == k - 1) * 0.8

    W["embed"] = g.normal(0.0, 0.7, size=(V, D))
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        vec(p + "norm1", D, 0.6, 1.4)
        l, r = m["left"], m["right"]
        H, G, d, e = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
        for s, n in (("q", H * d), ("k", G * d), ("v", G * e)):
            mat(p + "mix.left." + s, n, D, 2.0)
            if l.get("conv"):
                taps(p + "mix.left." + s + ".conv", n, l["conv"])
        mat(p + "mix.left.g", H, D, 2.0)
        mat(p + "mix.left.o", D, H * e)
        Hr, dr, er = r["heads"], r["dim"], r["vdim"]
        mat(p + "mix.right.q", Hr * dr, D, 1.5)
        mat(p + "mix.right.k", Hr * dr, D, 1.5)
        mat(p + "mix.right.v", Hr * er, D, 1.5)
        mat(p + "mix.right.g", Hr * er, D, 2.0)
        vec(p + "mix.right.norm", Hr * er, 0.5, 1.5)
        mat(p + "mix.right.o", D, Hr * er)
        mlp = L.get("mlp")
        if not mlp:
            continue
        vec(p + "norm2", D, 0.6, 1.4)
        if mlp["kind"] == "dense":
            ff = mlp["ff"]
            for s, rows, cols in (("gate", ff, D), ("up", ff, D), ("down", D, ff)):
                mat(p + "mlp." + s, rows, cols, 1.5)
                vec(p + "mlp." + s + ".b", rows, -0.7, 0.7)
            continue
        rt, ff = mlp["router"], mlp["expert"]["ff"]
        for x in range(rt["experts"]):
            mat(f"{p}mlp.e{x}.gate", ff, D, 2.5)        # (large enough for the clamps to bite on part of the channels)
            mat(f"{p}mlp.e{x}.up", ff, D, 2.5)
            mat(f"{p}mlp.e{x}.down", D, ff)
        routed = rt["experts"] + rt.get("identity", 0)
        mat(p + "mlp.router", routed, D, 3.0)
        if negative_corrections:
            vec(p + "mlp.correction", routed, -0.9, -0.6)
        else:
            vec(p + "mlp.correction", routed, -0.15, 0.15)
        if mlp.get("shared"):
            sf = mlp["shared"]["ff"]
            mat(p + "mlp.shared.gate", sf, D, 2.5)
            mat(p + "mlp.shared.up", sf, D, 2.5)
            mat(p + "mlp.shared.down", D, sf)
            mat(p + "mlp.shared.sg", 1, D, 2.0)
    vec("final.norm", D, 0.6, 1.4)
    return W


def write_dir(path, cfg, seed, overrides=None, negative_corrections=False):
    """config.json and model.safetensors (bfloat16) for `cfg`; `overrides`: name -> array put in place of the drawn one."""
    from edgelm_b200.weights import write_file
    os.makedirs(path, exist_ok=True)
    W = tensors_for(cfg, seed, negative_corrections)
    for k, v in (overrides or {}).items():
        assert k in W and np.shape(v) == W[k].shape, k
        W[k] = np.asarray(v)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_file(os.path.join(path, "model.safetensors"), {k: torch.tensor(v, dtype=torch.float32).to(torch.bfloat16) for k, v in W.items()})
    return path


def tokens(cfg, n, salt):
    return [int(t) for t in np.random.default_rng(9000 + salt).integers(0, cfg["vocab"], size=n)]
