"""The Redenex decoder in plain NumPy (float64), one function per mechanism, whole sequences recomputed from their
first token: no cache, no state, no batches.  What the library computes is compared with this.

A model is (config, weights): `config` is the config.json dictionary, `weights` maps tensor names to arrays.
"""
import json
import math
import os

import numpy as np


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def rms_norm(x, eps, weight=None, one_plus=False):
    """x / sqrt(mean(x^2) + eps) over the last axis, times `weight` or (1 + weight)."""
    y = x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    if weight is not None:
        y = y * ((1.0 + weight) if one_plus else weight)
    return y


def causal_conv(u, taps, bias=None):
    """u [n, channels], taps [channels, k]: y_t = sum_j taps[:, j] * u_(t - k + 1 + j), zeros before the first row."""
    n, k = u.shape[0], taps.shape[1]
    padded = np.concatenate([np.zeros((k - 1, u.shape[1])), u], axis=0)
    y = np.zeros_like(u)
    for j in range(k):
        y += padded[j:j + n] * taps[:, j]
    return y if bias is None else y + bias


def rotate_half_pairs(x, positions, dims, base):
    """x [n, ..., d]: dimension i of the first `dims` is paired with i + dims / 2 and turned by position * base^(-2i/dims)."""
    half = dims // 2
    f = base ** (-2.0 * np.arange(half) / dims)
    ang = positions.astype(np.float64)[:, None] * f
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (half,)
    c, s = np.cos(ang).reshape(shape), np.sin(ang).reshape(shape)
    a, b = x[..., :half], x[..., half:dims]
    return np.concatenate([a * c - b * s, b * c + a * s, x[..., dims:]], axis=-1)


def rglru_mixer(h, w, m, pre):
    """The recurrent block: a gelu branch and a convolved branch that feeds a gated diagonal recurrence."""
    W, blocks = m["width"], m.get("blocks", 1)
    y = gelu_tanh(h @ w[pre + "y"].T + w[pre + "y.b"])
    u = h @ w[pre + "x"].T + w[pre + "x.b"]
    u = causal_conv(u, w[pre + "conv"], w[pre + "conv.b"])
    bw = W // blocks
    ub = u.reshape(-1, blocks, bw)
    r = sigmoid(np.einsum("bok,nbk->nbo", w[pre + "ra"], ub) + w[pre + "ra.b"]).reshape(-1, W)
    i = sigmoid(np.einsum("bok,nbk->nbo", w[pre + "ri"], ub) + w[pre + "ri.b"]).reshape(-1, W)
    log_a = -8.0 * r * softplus(w[pre + "lam"])
    a = np.exp(log_a)
    b = np.sqrt(1.0 - a * a) * i * u
    S = np.zeros(W)
    out = np.zeros_like(u)
    for t in range(u.shape[0]):
        S = a[t] * S + b[t]
        out[t] = S
    return (out * y) @ w[pre + "o"].T


def chunked_softmax_attention(q, k, v, scale, chunk=None):
    """q [n, H, d], k [n, G, d], v [n, G, e] from position 0: position i sees the j <= i of its own chunk (all j <= i without
    one); query head h reads key/value head h // (H / G).  -> [n, H, e]"""
    n, H = q.shape[0], q.shape[1]
    G = k.shape[1]
    pos = np.arange(n)
    seen = pos[None, :] <= pos[:, None]
    if chunk:
        seen &= (pos[None, :] // chunk) == (pos[:, None] // chunk)
    out = np.zeros((n, H, v.shape[2]))
    for head in range(H):
        g = head // (H // G)
        s = np.where(seen, (q[:, head] @ k[:, g].T) * scale, -np.inf)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        out[:, head] = (p / p.sum(axis=1, keepdims=True)) @ v[:, g]
    return out


def map_weight(w, pre, offset):
    """lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + offset: one number per layer."""
    return math.exp(float(np.sum(w[pre + "lq1"] * w[pre + "lk1"]))) - math.exp(float(np.sum(w[pre + "lq2"] * w[pre + "lk2"]))) + offset


def combine_maps(a1, a2, lam, offset, eps):
    """o = a1 - lambda a2, divided by its root mean square over a head's values, times (1 - offset)."""
    return rms_norm(a1 - lam * a2, eps) * (1.0 - offset)


def differential_attention(h, w, m, pre, eps):
    """Two softmax maps per head over the same values, subtracted, normed per head."""
    n = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(n)
    q, k, v = (h @ w[pre + s].T + w[pre + s + ".b"] for s in "qkv")
    if m.get("conv"):
        q, k, v = (causal_conv(t, w[pre + s + ".conv"]) for t, s in zip((q, k, v), "qkv"))
    q, k, v = q.reshape(n, H, 2, d), k.reshape(n, G, 2, d), v.reshape(n, G, dv)
    q = rms_norm(q, eps, w[pre + "q.norm"])
    k = rms_norm(k, eps, w[pre + "k.norm"])
    rot = m.get("rot")
    if rot:
        q = rotate_half_pairs(q, pos, rot["dims"], rot["base"])
        k = rotate_half_pairs(k, pos, rot["dims"], rot["base"])
    size = (m.get("mask") or {}).get("size")
    a1, a2 = (chunked_softmax_attention(q[:, :, j], k[:, :, j], v, m["scale"], size) for j in range(2))
    o = combine_maps(a1, a2, map_weight(w, pre, m["diff"]), m["diff"], eps)
    return o.reshape(n, H * dv) @ w[pre + "o"].T


def clamped_glu(h, w, mlp, pre):
    g = np.minimum(h @ w[pre + "gate"].T, mlp["limit"])
    u = np.clip(h @ w[pre + "up"].T, -mlp["limit"], mlp["limit"])
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[pre + "down"].T


def mixer(h, w, layer, pre, eps):
    if layer["type"] == "rglru":
        return rglru_mixer(h, w, layer["mixer"], pre)
    if layer["type"] == "attention":
        return differential_attention(h, w, layer["mixer"], pre, eps)
    raise ValueError(layer["type"])


def schedule(config):
    """Layer indices in run order: the looped run of layers repeated in a row."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(n))
    return list(range(loop["start"])) + list(range(loop["start"], loop["stop"])) * loop["times"] + list(range(loop["stop"], n))


def hyper_sublayer(xs, w, pre, fn):
    """xs [streams, n, width]: read the sublayer's input as a weighted sum, write its output back into every stream."""
    u = np.einsum("s,snd->nd", w[pre + "in"], xs)
    y = fn(u)
    return np.einsum("st,snd->tnd", w[pre + "mix"], xs) + w[pre + "out"][:, None, None] * y[None]


def forward(config, weights, tokens, return_layers=False):
    """logits [n, vocab] (and the residual stream after every layer run, summed over the streams)."""
    w = {k: np.asarray(v, dtype=np.float64) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)] * (config.get("embedding") or {}).get("scale", 1.0)
    streams = config.get("streams")
    xs = np.repeat(x[None], streams, axis=0) if streams else None
    after = []
    for li in schedule(config):
        layer, pre = config["layers"][li], f"l{li}."
        mix = lambda u: mixer(rms_norm(u, eps, w[pre + "norm1"], True), w, layer, pre + "mix.", eps)
        ff = lambda u: clamped_glu(rms_norm(u, eps, w[pre + "norm2"], True), w, layer["mlp"], pre + "mlp.")
        if streams:
            xs = hyper_sublayer(xs, w, pre + "hc1.", mix)
            if layer.get("mlp"):
                xs = hyper_sublayer(xs, w, pre + "hc2.", ff)
            after.append(xs.sum(axis=0))
        else:
            x = x + mix(x)
            if layer.get("mlp"):
                x = x + ff(x)
            after.append(x)
    if streams:
        x = xs.sum(axis=0)
    logits = rms_norm(x, eps, w["final.norm"], True) @ w["head"].T
    return (logits, np.stack(after)) if return_layers else logits


def read_safetensors(path):
    """name -> float64 array, from the file format itself (8-byte length, JSON header, data); bfloat16, float32 and int32."""
    with open(path, "rb") as f:
        n = int.from_bytes(f.read(8), "little")
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        raw = data[a:b]
        if info["dtype"] == "BF16":
            arr = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif info["dtype"] == "F32":
            arr = np.frombuffer(raw, dtype="<f4")
        elif info["dtype"] == "I32":
            arr = np.frombuffer(raw, dtype="<i4")
        else:
            raise ValueError(info["dtype"])
        out[name] = arr.astype(np.float64).reshape(info["shape"])
    return out


def load(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))
