"""The Radupel decoder in plain NumPy (float64), one function per mechanism, whole sequences recomputed from their
first token: no cache, no state, no batches.  What the library computes is compared with this.

A model is (config, weights): `config` is the config.json dictionary, `weights` maps tensor names to arrays.
"""
import math

import numpy as np

GLU_ALPHA = 1.702       # an expert's gate is g * sigmoid(GLU_ALPHA * g)
WEIGHT_SUM_EPS = 1e-20  # added to the sum of the chosen experts' scores before dividing by it


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def rms_norm(x, eps, weight=None):
    """x / sqrt(mean(x^2) + eps) over the last axis, times `weight`."""
    y = x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return y if weight is None else y * weight


def causal_conv(u, taps):
    """u [n, channels], taps [channels, k]: y_t = sum_j taps[:, j] * u_(t - k + 1 + j), zeros before the first row."""
    n, k = u.shape[0], taps.shape[1]
    padded = np.concatenate([np.zeros((k - 1, u.shape[1])), u], axis=0)
    y = np.zeros_like(u)
    for j in range(k):
        y += padded[j:j + n] * taps[:, j]
    return y


def rotate_half_pairs(x, positions, dims, base):
    """x [n, heads, d]: dimension i of the first `dims` is paired with i + dims / 2 and turned by position * base^(-2i/dims)."""
    half = dims // 2
    f = base ** (-2.0 * np.arange(half) / dims)
    ang = positions.astype(np.float64)[:, None] * f
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return np.concatenate([a * c - b * s, b * c + a * s, x[..., dims:]], axis=-1)


def causal_softmax_attention(q, k, v, scale):
    """q [n, H, d], k [n, G, d], v [n, G, e] from position 0; query head h reads key/value head h // (H / G).  -> [n, H, e]"""
    n, H, G = q.shape[0], q.shape[1], k.shape[1]
    seen = np.arange(n)[None, :] <= np.arange(n)[:, None]
    out = np.zeros((n, H, v.shape[2]))
    for head in range(H):
        g = head // (H // G)
        s = np.where(seen, (q[:, head] @ k[:, g].T) * scale, -np.inf)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        out[:, head] = (p / p.sum(axis=1, keepdims=True)) @ v[:, g]
    return out


def gated_softmax_attention(h, w, m, pre):
    """The left mixer: projections, a short convolution on each, a partial rotation, causal softmax, a gate per head."""
    n = h.shape[0]
    H, G, d, e = m["heads"], m.get("kv_heads") or m["heads"], m["dim"], m.get("vdim") or m["dim"]
    q, k, v = (h @ w[pre + s].T for s in "qkv")
    if m.get("conv"):
        q, k, v = (causal_conv(t, w[pre + s + ".conv"]) for t, s in zip((q, k, v), "qkv"))
    q, k, v = q.reshape(n, H, d), k.reshape(n, G, d), v.reshape(n, G, e)
    rot = m.get("rot")
    if rot:
        pos = np.arange(n)
        q, k = rotate_half_pairs(q, pos, rot["dims"], rot["base"]), rotate_half_pairs(k, pos, rot["dims"], rot["base"])
    o = causal_softmax_attention(q, k, v, m["scale"])
    o = o * sigmoid(h @ w[pre + "g"].T)[:, :, None]
    return o.reshape(n, H * e) @ w[pre + "o"].T


def decayed_linear_attention(q, k, v, decay):
    """Per head S_t = decay_h S_(t-1) + k_t v_t^T and o_t = S_t^T q_t, S_0 = 0.  q, k [n, H, d], v [n, H, e] -> [n, H, e]"""
    n, H, d = q.shape
    e = v.shape[2]
    out = np.zeros((n, H, e))
    for head in range(H):
        S = np.zeros((d, e))
        for t in range(n):
            S = decay[head] * S + np.outer(k[t, head], v[t, head])
            out[t, head] = S.T @ q[t, head]
    return out


def lightning_mixer(h, w, m, pre, eps):
    """The right mixer: silu projections, the decayed outer-product recurrence, one norm over all heads, a sigmoid gate."""
    n = h.shape[0]
    H, d, e = m["heads"], m["dim"], m.get("vdim") or m["dim"]
    q, k, v = (silu(h @ w[pre + s].T) for s in "qkv")
    o = decayed_linear_attention(q.reshape(n, H, d), k.reshape(n, H, d), v.reshape(n, H, e), np.asarray(m["decay"], dtype=np.float64))
    o = rms_norm(o.reshape(n, H * e), eps, w[pre + "norm"]) * sigmoid(h @ w[pre + "g"].T)
    return o @ w[pre + "o"].T


def parallel_mixer(h, w, m, pre, eps):
    left = gated_softmax_attention(h, w, m["left"], pre + "left.")
    right = lightning_mixer(h, w, m["right"], pre + "right.", eps)
    return m["left_scale"] * left + m["right_scale"] * right


def dense_ffn(h, w, pre):
    """W_down (silu(W_gate h + b) * (W_up h + b)) + b."""
    g = h @ w[pre + "gate"].T + w[pre + "gate.b"]
    u = h @ w[pre + "up"].T + w[pre + "up.b"]
    return (silu(g) * u) @ w[pre + "down"].T + w[pre + "down.b"]


def clamped_expert(h, w, pre, limit):
    g = np.minimum(h @ w[pre + "gate"].T, limit)
    u = np.clip(h @ w[pre + "up"].T, -limit, limit)
    return (g * sigmoid(GLU_ALPHA * g) * (u + 1.0)) @ w[pre + "down"].T


def route(z, correction, top, groups, keep, scale):
    """z [n, E] router logits -> (chosen [n, top] expert numbers, weights [n, top]).  Scores are the softmax over all E; the
    choice adds `correction` and looks only at the `keep` groups of neighbours whose largest corrected score is largest; the
    weights are the chosen experts' uncorrected scores over their sum, times `scale`."""
    n, E = z.shape
    s = np.exp(z - z.max(axis=1, keepdims=True))
    s = s / s.sum(axis=1, keepdims=True)
    c = s + correction
    if groups > 1:
        size = E // groups
        best = c.reshape(n, groups, size).max(axis=2)
        kept = np.argsort(-best, axis=1, kind="stable")[:, :keep]
        allowed = np.zeros((n, groups), dtype=bool)
        np.put_along_axis(allowed, kept, True, axis=1)
        c = np.where(np.repeat(allowed, size, axis=1), c, -np.inf)
    chosen = np.argsort(-c, axis=1, kind="stable")[:, :top]
    picked = np.take_along_axis(s, chosen, axis=1)
    return chosen, picked / (picked.sum(axis=1, keepdims=True) + WEIGHT_SUM_EPS) * scale


def moe_ffn(h, w, mlp, pre):
    """Routed experts (the last `identity` of the router's outputs give back their input), plus a gated shared expert."""
    r = mlp["router"]
    real, ident = r["experts"], r.get("identity", 0)
    grp = r.get("groups") or {"count": 1, "keep": 1}
    z = h @ w[pre + "router"].T
    chosen, wts = route(z, w[pre + "correction"], r["top"], grp["count"], grp["keep"], r.get("scale", 1.0))
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t], wts[t]):
            y = clamped_expert(h[t:t + 1], w, f"{pre}e{e}.", mlp["expert"]["limit"])[0] if e < real else h[t]
            out[t] += a * y
    sh = mlp.get("shared")
    if sh:
        out += clamped_expert(h, w, pre + "shared.", sh["limit"]) * sigmoid(h @ w[pre + "shared.sg"].T)
    return out


def layer_order(cfg):
    """(layer, whether the embedding output is added first) in run order."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    order = [(i, False) for i in range(loop["start"])]
    for p in range(loop["times"]):
        order += [(i, p > 0 and i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return order + [(i, False) for i in range(loop["stop"], n)]


def forward(cfg, w, tokens, return_layers=False):
    """Logits [n, vocab] of one sequence from its first token (and the residual stream after every layer run)."""
    eps = cfg["norm"]["eps"]
    x0 = w["embed"][np.asarray(tokens)]
    x, runs = x0.copy(), []
    for i, add in layer_order(cfg):
        L, pre = cfg["layers"][i], f"l{i}."
        if add:
            x = x + x0
        y = parallel_mixer(rms_norm(x, eps, w[pre + "norm1"]), w, L["mixer"], pre + "mix.", eps)
        mlp = L.get("mlp")
        if mlp:
            h2 = rms_norm(x, eps, w[pre + "norm2"])
            y = y + (dense_ffn(h2, w, pre + "mlp.") if mlp["kind"] == "dense" else moe_ffn(h2, w, mlp, pre + "mlp."))
        x = x + y
        runs.append(x.copy())
    logits = rms_norm(x, eps, w["final.norm"]) @ w["embed"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * np.tanh(logits / cap)
    return (logits, np.stack(runs)) if return_layers else logits


def load(model_dir):
    """(config.json dictionary, name -> float64 array) of a model folder."""
    import json
    import os

    from plain_redenex import read_safetensors
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))
