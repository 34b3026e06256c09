"""Small Redenex configurations and model folders for the tests.

Weights are drawn so that nothing hides: decays close to 1 (a state remembers tens of tokens), convolution taps of
comparable size (a lost tail shows), stream weights far from the identity (a mix matrix read the wrong way round shows),
lambda tensors that give every layer another lambda, matrices wide enough for logits of order 1.  The folders are written in
bfloat16 (what a float32 engine widens exactly), so the plain implementation and the library compute from the same numbers.
"""
import json
import os

import numpy as np
import torch


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def rglru(width, blocks, conv, mlp):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv}, "mlp": mlp}


def attention(heads, kv_heads, dim, vdim, conv, diff, scale, rot, chunk, mlp):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff, "scale": scale}
    if conv:
        m["conv"] = conv
    if rot:
        m["rot"] = rot
    if chunk:
        m["mask"] = {"size": chunk}
    return {"type": "attention", "mixer": m, "mlp": mlp}


# Sizes differ in everything from layer to layer and between the models: grouped, multi-query (eight query heads to a key
# head: decoding shares staged keys and splits pages) and one key head per query head; value heads wider and narrower than
# a map's keys; chunks shorter than, equal to and longer than a page of 64, and none; rotation of a part of a map and of all
# of it, and none; 1 to 4 taps; recurrent widths that are no multiple of 32, one block and several; three streams, one
# stream with its own weights, and the plain residual sum; a loop in the middle run three times, a loop from the first
# layer, no loop; layers without a feed-forward; widths that are no multiple of 8.
CFG_A = {"architecture": "Redenex", "vocab": 173, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0}, "streams": 3,
         "loop": {"start": 1, "stop": 3, "times": 3}, "layers": [
    attention(4, 2, 16, 24, 2, 0.3, 0.3, {"base": 700.0, "dims": 8}, 7, dense(40, 2.0)),
    rglru(96, 3, 4, dense(56, 0.7)),
    attention(8, 1, 8, 8, 4, 0.8, 0.4, {"base": 10000.0, "dims": 8}, 70, None),
    rglru(40, 1, 1, dense(24, 1.5)),
]}
CFG_B = {"architecture": "Redenex", "vocab": 97, "width": 50, "norm": {"eps": 3e-4}, "embedding": {"scale": 0.5}, "streams": 1, "layers": [
    rglru(70, 2, 2, dense(30, 1.0)),
    attention(3, 3, 10, 14, 1, 0.5, 0.35, None, 64, dense(20, 3.0)),
    attention(2, 1, 32, 20, 3, 0.2, 0.2, {"base": 90.0, "dims": 32}, None, None),
    rglru(33, 3, 3, dense(18, 0.5)),
]}
CFG_C = {"architecture": "Redenex", "vocab": 120, "width": 48, "norm": {"eps": 1e-6}, "embedding": {"scale": 7.0},
         "loop": {"start": 0, "stop": 2, "times": 2}, "layers": [
    attention(2, 2, 24, 16, None, 0.45, 0.25, {"base": 50.0, "dims": 12}, 33, dense(64, 1.2)),
    rglru(64, 4, 3, None),
    attention(6, 3, 8, 40, 2, 0.6, 0.5, {"base": 3000.0, "dims": 4}, 128, dense(32, 0.9)),
]}
CONFIGS = {"a": CFG_A, "b": CFG_B, "c": CFG_C}


def tensors_for(cfg, seed):
    g = np.random.default_rng(seed)
    D, V, S = cfg["width"], cfg["vocab"], cfg.get("streams")
    W = {}

    def mat(name, rows, cols, gain=1.0):
        W[name] = g.normal(0.0, gain / np.sqrt(cols), size=(rows, cols))

    def vec(name, n, lo, hi):
        W[name] = g.uniform(lo, hi, size=(n,))

    def taps(name, n, k):
        W[name] = g.normal(0.0, 0.5, size=(n, k)) + (np.arange(k) == k - 1) * 0.8

    W["embed"] = g.normal(0.0, 0.7 / cfg["embedding"]["scale"], size=(V, D))
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        vec(p + "norm1", D, -0.4, 0.4)       # (the norms multiply by 1 + w)
        if L["type"] == "rglru":
            Wd, B = m["width"], m["blocks"]
            for s in ("y", "x"):
                mat(p + "mix." + s, Wd, D, 1.5)
                vec(p + "mix." + s + ".b", Wd, -0.5, 0.5)
            taps(p + "mix.conv", Wd, m["conv"])
            vec(p + "mix.conv.b", Wd, -0.3, 0.3)
            for s in ("ra", "ri"):
                W[p + "mix." + s] = g.normal(0.0, 1.5 / np.sqrt(Wd // B), size=(B, Wd // B, Wd // B))
                W[p + "mix." + s + ".b"] = g.uniform(-1.0, 1.0, size=(B, Wd // B))
            vec(p + "mix.lam", Wd, -5.0, -1.0)     # softplus: 0.007 .. 0.3, so a = exp(-8 r softplus) spans 0.1 .. 0.99
            mat(p + "mix.o", D, Wd)
        else:
            H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for s, n in (("q", H * 2 * d), ("k", G * 2 * d), ("v", G * e)):
                mat(p + "mix." + s, n, D, 2.0)
                vec(p + "mix." + s + ".b", n, -0.5, 0.5)
                if m.get("conv"):
                    taps(p + "mix." + s + ".conv", n, m["conv"])
            vec(p + "mix.q.norm", d, 0.6, 1.6)
            vec(p + "mix.k.norm", d, 0.6, 1.6)
            for s in ("lq1", "lk1", "lq2", "lk2"):
                W[p + "mix." + s] = g.normal(0.0, 0.25, size=(d,))
            mat(p + "mix.o", D, H * e)
        if L.get("mlp"):
            ff = L["mlp"]["ff"]
            vec(p + "norm2", D, -0.4, 0.4)
            mat(p + "mlp.gate", ff, D, 2.5)       # (large enough for the clamps to bite on part of the channels)
            mat(p + "mlp.up", ff, D, 2.5)
            mat(p + "mlp.down", D, ff)
        if S is not None:
            for q in ("hc1", "hc2") if L.get("mlp") else ("hc1",):
                vec(f"{p}{q}.in", S, 0.2, 0.9)
                vec(f"{p}{q}.out", S, 0.4, 1.2)
                W[f"{p}{q}.mix"] = np.eye(S) * 0.8 + g.uniform(-0.3, 0.3, size=(S, S))
    vec("final.norm", D, -0.4, 0.4)
    mat("head", V, D, 2.0)
    return W


def write_dir(path, cfg, seed, overrides=None):
    """config.json and model.safetensors (bfloat16) for `cfg`; `overrides`: name -> array put in place of the drawn one."""
    from edgelm_b200.weights import write_file
    os.makedirs(path, exist_ok=True)
    W = tensors_for(cfg, seed)
    for k, v in (overrides or {}).items():
        assert k in W and np.shape(v) == W[k].shape, k
        W[k] = np.asarray(v)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_file(os.path.join(path, "model.safetensors"), {k: torch.tensor(v, dtype=torch.float32).to(torch.bfloat16) for k, v in W.items()})
    return path


def tokens(cfg, n, salt):
    return [int(t) for t in np.random.default_rng(7000 + salt).integers(0, cfg["vocab"], size=n)]
