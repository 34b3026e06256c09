"""The kernels of the Vosulorn decoder's mechanisms, each alone against the plain implementation's function for the same
mechanism (tests/plain_vosulorn.py): the gated delta rule over several steps on scattered state rows; attention with a
key range per query (causal, chunk, window) and a sink, for steps of one token and for prompt steps, on pages in no
particular order, with one far key made so large that "seen" and "not seen" differ by much more than any tolerance;
the latent's preparation, the per-head products and attention over rows that are key and value at once; the router, the
grouping by expert, the experts' products and the weighted sum."""
import numpy as np
import pytest
import torch

import plain_vosulorn as plain
from edgelm_b200.csrc import ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PAGE = 64


def i32(a):
    return torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)


def f32(a):
    return torch.tensor(np.asarray(a), dtype=torch.float32, device=DEV).contiguous()


def packed(lengths):
    tok0 = np.concatenate([[0], np.cumsum(lengths)])
    tok_seq = np.repeat(np.arange(len(lengths)), lengths)
    return i32(tok0), i32(tok_seq)


def steps_of(total, cuts):
    n_steps = max(len(c) for c in cuts)
    at = [0] * len(total)
    out = []
    for k in range(n_steps):
        step = []
        for s, c in enumerate(cuts):
            n = c[k] if k < len(c) else 0
            step.append((at[s], n))
            at[s] += n
        out.append(step)
    assert at == list(total)
    return out


def make_tiles(lengths, pos0, tile):
    seq, tok0, ntok, p0 = [], [], [], []
    t0 = 0
    for s, (n, p) in enumerate(zip(lengths, pos0)):
        for a in range(0, n, tile):
            seq.append(s); tok0.append(t0 + a); ntok.append(min(tile, n - a)); p0.append(p + a)
        t0 += n
    return i32(seq), i32(tok0), i32(ntok), i32(p0), len(seq)


# ----------------------------------------------------------------------------- gated delta rule
@pytest.mark.parametrize("H,G,d,e,taps", [(4, 2, 16, 24, 4), (3, 3, 40, 12, 2), (2, 1, 70, 40, 1), (1, 1, 130, 33, 3), (6, 2, 8, 8, 3)])
def test_delta_rule_over_steps(H, G, d, e, taps):
    """Convolution, unit norms, step sizes and decays, and the recurrence, fed in pieces (down to one token, shorter than
    the convolution's tail) on state rows in no particular order; a slot of nobody is never touched."""
    g = np.random.default_rng(d + e)
    total, cuts, slots = [43, 6, 1, 70], [[5, 1, 37], [2, 4], [1], [1, 1, 68]], [4, 0, 2, 5]
    C = 2 * G * d + H * e
    raw = [g.normal(size=(n, C)) for n in total]                 # the projections q | k | v before the convolution
    rb, ra = [g.normal(size=(n, H)) for n in total], [g.normal(size=(n, H)) for n in total]
    conv_w = g.normal(0, 0.6, size=(C, taps))
    A_log, dt_bias = g.uniform(-4, -1, H), g.uniform(-1, 0.5, H)
    want = []
    for s in range(len(total)):
        x = plain.causal_conv_silu(raw[s], conv_w)
        q = plain.unit_vectors(x[:, :G * d].reshape(-1, G, d)) * d ** -0.5
        k = plain.unit_vectors(x[:, G * d:2 * G * d].reshape(-1, G, d))
        q, k = np.repeat(q, H // G, axis=1), np.repeat(k, H // G, axis=1)
        beta = plain.sigmoid(rb[s])
        dec = np.exp(-np.exp(A_log) * plain.softplus(ra[s] + dt_bias))
        want.append(plain.delta_recurrence(q, k, x[:, 2 * G * d:].reshape(-1, H, e), beta, dec).reshape(-1, H * e))
    state = torch.zeros(7, H, e, d, device=DEV)
    tail = torch.zeros(7, taps - 1, C, device=DEV)
    state[1].fill_(float("nan"))
    got = [np.zeros_like(w) for w in want]
    zero_b = torch.zeros(C, device=DEV)
    for step in steps_of(total, cuts):
        live = [(s, a, n) for s, (a, n) in enumerate(step) if n]
        tok0, tok_seq = packed([n for _, _, n in live])
        seqslot = i32([slots[s] for s, _, _ in live])
        u = f32(np.concatenate([np.concatenate([raw[s][a:a + n], rb[s][a:a + n], ra[s][a:a + n]], axis=1) for s, a, n in live]))
        T = u.shape[0]
        qkv = torch.full((T, C), float("nan"), device=DEV)
        ops.conv_silu(u, 0, f32(conv_w), zero_b, tail, qkv, tok_seq, tok0, seqslot, len(live), update_state=True)
        bg = torch.empty(2 * T * H, device=DEV)
        ops.delta_prepare(qkv, u, C, C + H, f32(A_log), f32(dt_bias), bg, H, G, d, e, 1e-6, d ** -0.5)
        o = torch.full((T, H * e), float("nan"), device=DEV)
        ops.delta_scan(qkv, bg, state, o, tok0, seqslot, len(live), H, G, d, e)
        o = o.cpu().numpy()
        at = 0
        for s, a, n in live:
            got[s][a:a + n] = o[at:at + n]
            at += n
    for w, o in zip(want, got):
        assert np.abs(o - w).max() < 2e-5 * max(1.0, np.abs(w).max())
    assert torch.isnan(state[1]).all()


# ----------------------------------------------------------------------------- attention with a key range and a sink
class PagedKV:
    """Keys and values of a few sequences in pages handed out in a scrambled order, the rest poisoned."""

    def __init__(self, lengths, G, dk, dv, dtype, seed, values_in_keys=False):
        g = np.random.default_rng(seed)
        self.lengths = lengths
        per = [(n + PAGE - 1) // PAGE for n in lengths]
        n_pages = sum(per) + 3
        order = g.permutation(n_pages)
        self.table = np.full((len(lengths), max(per) + 1), -1, np.int32)
        at = 0
        for s, p in enumerate(per):
            self.table[s, :p] = order[at:at + p]
            at += p
        self.k = torch.full((n_pages, G, PAGE, dk), 1e4, dtype=dtype, device=DEV)
        self.v = None if values_in_keys else torch.full((n_pages, G, PAGE, dv), float("nan"), dtype=dtype, device=DEV)

    def put(self, s, keys, values=None):
        """keys [n, G, dk] (values [n, G, dv]) of sequence s from position 0."""
        for p in range(keys.shape[0]):
            page = self.table[s, p // PAGE]
            self.k[page, :, p % PAGE] = torch.tensor(keys[p], dtype=self.k.dtype, device=DEV)
            if values is not None:
                self.v[page, :, p % PAGE] = torch.tensor(values[p], dtype=self.v.dtype, device=DEV)


def mask_args(kind, size):
    return {"causal": (ops.MASK_CAUSAL, 0), "chunk": (ops.MASK_CHUNK, size), "window": (ops.MASK_WINDOW, size)}[kind]


def plain_attention(q, k, v, scale, kind, size, sink):
    """The plain softmax attention with a key range: `chunk` is the plain implementation's own mask; a window is
    written out here."""
    if kind != "window":
        return plain.masked_softmax_attention(q, k, v, scale, chunk=size if kind == "chunk" else None, sink=sink)
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        for i in range(T):
            lo = max(0, i - size + 1)
            s = (k[lo:i + 1, h // (H // G)] @ q[i, h]) * scale
            m = max(s.max(), sink[h]) if sink is not None else s.max()
            p = np.exp(s - m)
            den = p.sum() + (np.exp(sink[h] - m) if sink is not None else 0.0)
            out[i, h] = (p / den) @ v[lo:i + 1, h // (H // G)]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dk,dv,kind,size,with_sink", [
    (6, 2, 16, 8, "chunk", 7, True), (4, 2, 32, 32, "chunk", 64, True), (3, 3, 10, 14, "chunk", 70, True), (2, 1, 24, 40, "causal", 0, True),
    (4, 4, 48, 16, "window", 33, False), (8, 1, 20, 130, "causal", 0, False), (5, 5, 72, 264, "chunk", 100, True)])
def test_attention_with_a_key_range(H, G, dk, dv, kind, size, with_sink, dtype):
    """Prompt steps (tiles) and steps of one token against the plain attention, for sequences of several pages.  In each
    sequence one early key is made 12 times larger and the queries point at it, so whether a query sees it decides its
    output: the positions just before and just after every edge of a chunk or window then show a mask that is off by one."""
    g = np.random.default_rng(dk * 7 + dv)
    lengths = [150, 67, 1, 203]
    scale = 0.9 / np.sqrt(dk)
    sink = g.uniform(-1, 2, H) if with_sink else None
    rnd = lambda a: torch.tensor(a, dtype=dtype).double().numpy()      # what the cache holds
    kv = PagedKV(lengths, G, dk, dv, dtype, seed=3)
    Q, want = [], []
    for s, n in enumerate(lengths):
        q, k, v = g.normal(size=(n, H, dk)), rnd(g.normal(size=(n, G, dk))), rnd(g.normal(size=(n, G, dv)))
        far = min(n - 1, 5 if size == 0 else size - 2)
        k[far] *= 12.0 / np.sqrt(dk)
        q += 0.4 * np.repeat(k[far], H // G, axis=0)[None]
        q = torch.tensor(q, dtype=torch.float32).double().numpy()
        kv.put(s, k, v)
        Q.append(q)
        want.append(plain_attention(q, k, v, scale, kind, size, sink))
    table = i32(kv.table)
    mk, ms = mask_args(kind, size)
    sk = f32(sink) if with_sink else None
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    # prompt steps: every sequence whole (the keys are in the cache already), then in two pieces
    for pieces in ([(0, n) for n in lengths], [(n // 3, n - n // 3) for n in lengths]):
        live = [(s, a, n) for s, (a, n) in enumerate(pieces) if n]
        tile = max(1, 32 // (H // G))
        tseq, ttok0, tntok, tpos0, count = make_tiles([n for _, _, n in live], [a for _, a, _ in live], tile)
        q = f32(np.concatenate([Q[s][a:a + n].reshape(n, H * dk) for s, a, n in live]))
        out = torch.full((q.shape[0], H * dv), float("nan"), dtype=dtype, device=DEV)
        ops.masked_attn_tiled(q, out, kv.k, kv.v, table[[s for s, _, _ in live]].contiguous(), tseq, ttok0, tntok, tpos0, count, tile, H, G, dk, dv,
                              scale, mk, ms, sk)
        got = out.float().cpu().numpy()
        ref = np.concatenate([want[s][a:a + n].reshape(n, H * dv) for s, a, n in live])
        assert np.abs(got - ref).max() < tol * max(1.0, np.abs(ref).max()), ("tiled", pieces[0])
    # steps of one token a sequence, at positions around every edge
    for back in (0, 1, 2, 3, 64, 66):
        live = [(s, n - 1 - back) for s, n in enumerate(lengths) if n - 1 - back >= 0]
        q = f32(np.stack([Q[s][p].reshape(H * dk) for s, p in live]))
        out = torch.full((len(live), H * dv), float("nan"), dtype=dtype, device=DEV)
        ops.masked_attn(q, out, kv.k, kv.v, i32([p for _, p in live]), i32(list(range(len(live)))), table[[s for s, _ in live]].contiguous(), H, G, dk, dv,
                        scale, mk, ms, sk, 1 << 30 if kind == "causal" else size)
        got = out.float().cpu().numpy()
        ref = np.stack([want[s][p].reshape(H * dv) for s, p in live])
        assert np.abs(got - ref).max() < tol * max(1.0, np.abs(ref).max()), ("single", back)
        for splits in (2, 4):       # the same kernel with a token's keys dealt to several blocks; the sink joins in the merge
            out1 = torch.full((len(live), H * dv), float("nan"), dtype=dtype, device=DEV)
            part = torch.full((len(live) * H * splits * (2 + dv),), float("nan"), device=DEV)
            ops.masked_attn(q, out1, kv.k, kv.v, i32([p for _, p in live]), i32(list(range(len(live)))), table[[s for s, _ in live]].contiguous(), H, G, dk, dv,
                            scale, mk, ms, sk, 1 << 30 if kind == "causal" else size, n_splits=splits, part=part)
            assert np.abs(out1.float().cpu().numpy() - ref).max() < tol * max(1.0, np.abs(ref).max()), ("single, keys split", back, splits)
        # the same tokens as tiles of one token, their pages dealt to 1, 3 and 5 blocks whose results a second launch merges
        for splits in (1, 3, 5):
            out2 = torch.full((len(live), H * dv), float("nan"), dtype=dtype, device=DEV)
            part = torch.full((len(live) * H * splits * (2 + dv),), float("nan"), device=DEV)
            n = len(live)
            ops.masked_attn_tiled(q, out2, kv.k, kv.v, table[[s for s, _ in live]].contiguous(), i32(list(range(n))), i32(list(range(n))), i32([1] * n),
                                  i32([p for _, p in live]), n, 1, H, G, dk, dv, scale, mk, ms, sk, n_splits=splits, part=part)
            assert np.abs(out2.float().cpu().numpy() - ref).max() < tol * max(1.0, np.abs(ref).max()), ("single, split", back, splits)


@pytest.mark.parametrize("interleaved", [True, False])
def test_rotation_bias_and_append(interleaved):
    """Bias, rotation of a part of every head with either pairing and stretched wavelengths at large positions, and the
    rows that reach the cache pages."""
    g = np.random.default_rng(9)
    H, G, dk, dv, rot = 3, 1, 20, 6, 12
    scaling = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}
    from edgelm_b200.parts.rope import rotary_frequencies
    freq = rotary_frequencies(rot, 300.0, scaling)
    assert np.allclose(freq.numpy(), plain.frequencies(rot, 300.0, scaling), rtol=1e-14)
    pos = [0, 1, 63, 64, 1000, 5000]
    T = len(pos)
    qkv, bias = g.normal(size=(T, (H + G) * dk + G * dv)), g.normal(size=((H + G) * dk + G * dv))
    kc = torch.zeros(90, G, PAGE, dk, device=DEV)
    vc = torch.zeros(90, G, PAGE, dv, device=DEV)
    table = i32(np.arange(89, -1, -1)[None])
    q_out = torch.empty(T, H * dk, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.rotate_append(f32(qkv), f32(bias), q_out, i32(pos), i32([0] * T), table, kc, vc, H, G, dk, dv, rot, interleaved, freq.to(DEV), err)
    x = qkv + bias
    f = plain.frequencies(rot, 300.0, scaling)
    qw = plain.rotate(x[:, :H * dk].reshape(T, H, dk), pos, f, interleaved)
    kw = plain.rotate(x[:, H * dk:(H + G) * dk].reshape(T, G, dk), pos, f, interleaved)
    assert np.abs(q_out.cpu().numpy().reshape(T, H, dk) - qw).max() < 3e-6
    for i, p in enumerate(pos):
        page = 89 - p // PAGE
        assert np.abs(kc[page, :, p % PAGE].cpu().numpy() - kw[i]).max() < 3e-6
        assert np.abs(vc[page, :, p % PAGE].cpu().numpy() - x[i, (H + G) * dk:].reshape(G, dv)).max() < 1e-6
    assert int(err.item()) == 0


# ----------------------------------------------------------------------------- latent attention
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,d,rd,e,r", [(4, 16, 8, 24, 32), (5, 10, 4, 6, 20), (1, 12, 4, 30, 20), (3, 24, 16, 40, 72)])
def test_latent_attention_path(H, d, rd, e, r, dtype):
    """The latent's norm, the rotation of the shared key part and of the queries' rotated part, the queries moved into the
    latent's space, attention over rows that are key and value at once, and the values expanded per head: against the
    plain mixer's way (keys and values expanded per head for every token).  Two steps: a prompt, then one token each."""
    g = np.random.default_rng(r + d)
    lengths, eps, scale, base = [70, 9, 131], 1e-5, 0.3, 300.0
    rnd = lambda a: torch.tensor(a, dtype=dtype).double().numpy()
    uk, uv, nw = rnd(g.normal(size=(H * d, r)) / np.sqrt(r)), rnd(g.normal(size=(H * e, r)) / np.sqrt(r)), g.uniform(0.6, 1.4, r)
    U = [g.normal(size=(n, H * (d + rd) + r + rd)) for n in lengths]
    kv = PagedKV(lengths, 1, r + rd, r, dtype, seed=5, values_in_keys=True)
    table = i32(kv.table)
    from edgelm_b200.parts.rope import rotary_frequencies
    freq = rotary_frequencies(rd, base).to(DEV)
    f = plain.frequencies(rd, base)
    w_ukt = torch.tensor(uk.reshape(H, d, r).transpose(0, 2, 1).copy(), dtype=dtype, device=DEV)
    w_uv = torch.tensor(uv.reshape(H, e, r), dtype=dtype, device=DEV).contiguous()
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    want = []
    for s, n in enumerate(lengths):
        u = torch.tensor(U[s], dtype=torch.float32).double().numpy()
        q = u[:, :H * (d + rd)].reshape(n, H, d + rd)
        c = plain.rmsnorm(u[:, H * (d + rd):H * (d + rd) + r], nw.astype(np.float32).astype(np.float64), eps)
        kr = plain.rotate(u[:, None, H * (d + rd) + r:], np.arange(n), f, False)[:, 0]
        c, kr = rnd(c), rnd(kr)                                   # (the cache's rounding)
        qq = np.concatenate([q[..., :d], plain.rotate(q[..., d:], np.arange(n), f, False)], -1)
        kk = np.concatenate([(c @ uk.T).reshape(n, H, d), np.broadcast_to(kr[:, None], (n, H, rd))], -1)
        want.append(plain.masked_softmax_attention(qq, kk, (c @ uv.T).reshape(n, H, e), scale).reshape(n, H * e))
    tol = 3e-5 if dtype == torch.float32 else 4e-2
    for phase in ("prompt", "single"):
        if phase == "prompt":
            live = [(s, 0, n - 1) for s, n in enumerate(lengths) if n > 1]
        else:
            live = [(s, n - 1, 1) for s, n in enumerate(lengths)]
        u = f32(np.concatenate([U[s][a:a + n] for s, a, n in live]))
        T = u.shape[0]
        pos = i32(np.concatenate([np.arange(a, a + n) for _, a, n in live]))
        _, tok_seq = packed([n for _, _, n in live])
        tb = table[[s for s, _, _ in live]].contiguous()
        qf = torch.full((T, H * (r + rd)), float("nan"), device=DEV)
        ops.latent_prepare(u, H * (d + rd), True, qf, r + rd, r, False, f32(nw), eps, pos, tok_seq, tb, kv.k, H, d, rd, r, freq, err)
        ops.head_matmul(u, d + rd, w_ukt, qf, r + rd)
        ol = torch.full((T, H * r), float("nan"), device=DEV)
        if phase == "prompt":
            tile = max(1, 32 // H)
            tseq, ttok0, tntok, tpos0, count = make_tiles([n for _, _, n in live], [a for _, a, _ in live], tile)
            ops.masked_attn_tiled(qf, ol, kv.k, None, tb, tseq, ttok0, tntok, tpos0, count, tile, H, 1, r + rd, r, scale, ops.MASK_CAUSAL, 0, None)
        else:
            ops.masked_attn(qf, ol, kv.k, None, pos, tok_seq, tb, H, 1, r + rd, r, scale, ops.MASK_CAUSAL, 0, None, 1 << 30)
        a = torch.full((T, H * e), float("nan"), dtype=dtype, device=DEV)
        ops.head_matmul(ol, r, w_uv, a, e)
        got = a.float().cpu().numpy()
        ref = np.concatenate([want[s][a0:a0 + n] for s, a0, n in live])
        assert np.abs(got - ref).max() < tol * max(1.0, np.abs(ref).max()), phase
        if phase == "prompt":
            # the same step with its own keys and values expanded per head (every sequence starts at position 0)
            q2 = torch.full((T, H * (d + rd)), float("nan"), device=DEV)
            rows = torch.full((T, r + rd), float("nan"), dtype=dtype, device=DEV)
            ops.latent_prepare(u, H * (d + rd), True, q2, d + rd, d, True, f32(nw), eps, pos, tok_seq, tb, kv.k, H, d, rd, r, freq, err, row_out=rows)
            c = rows[:, :r].float()
            kn = (c @ torch.tensor(uk, dtype=torch.float32, device=DEV).T).to(dtype).contiguous()
            vx = (c @ torch.tensor(uv, dtype=torch.float32, device=DEV).T).to(dtype).contiguous()
            kx = torch.full((T, H * (d + rd)), float("nan"), dtype=dtype, device=DEV)
            ops.latent_expand_keys(kn, rows, kx, H, d, rd, r)
            tseq, ttok0, tntok, tpos0, count = make_tiles([n for _, _, n in live], [0] * len(live), 32)
            a2 = torch.full((T, H * e), float("nan"), dtype=dtype, device=DEV)
            ops.masked_attn_tiled(q2, a2, kx, vx, None, tseq, ttok0, tntok, tpos0, count, 32, H, H, d + rd, e, scale, ops.MASK_CAUSAL, 0, None)
            assert np.abs(a2.float().cpu().numpy() - ref).max() < tol * max(1.0, np.abs(ref).max()), "own keys"
    assert int(err.item()) == 0


# ----------------------------------------------------------------------------- mixture of experts
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,D,E,top,ff", [(37, 64, 4, 2, 40), (1, 50, 2, 1, 30), (200, 48, 6, 3, 24), (9, 64, 5, 5, 16), (70, 32, 1, 1, 8)])
def test_mixture_of_experts(T, D, E, top, ff, dtype):
    """Router (float32 logits, the largest first, softmax over the chosen), grouping by expert, the experts' products and the
    weighted sum, against the plain mixture; the choice of every token is the plain one."""
    g = np.random.default_rng(T + E)
    rnd = lambda a: torch.tensor(a, dtype=dtype).double().numpy()
    W = {"router": rnd(g.normal(size=(E, D)) * 3 / np.sqrt(D)).astype(np.float32).astype(np.float64), "router.b": g.uniform(-0.5, 0.5, E).astype(np.float32).astype(np.float64)}
    for e in range(E):
        W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"] = rnd(g.normal(size=(ff, D)) / np.sqrt(D)), rnd(g.normal(size=(ff, D)) / np.sqrt(D)), rnd(g.normal(size=(D, ff)) / np.sqrt(ff))
    h = rnd(g.normal(size=(T, D)))
    mlp = {"router": {"experts": E, "top": top}}
    chosen, weights = plain.router(W, "", mlp["router"], h)
    want = plain.moe(W, "", mlp, h)
    hd = torch.tensor(h, dtype=dtype, device=DEV)
    idx = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, device=DEV)
    ops.moe_route(hd, f32(W["router"]), f32(W["router.b"]), idx, wts, top)
    z = np.sort(h @ W["router"].T + W["router.b"], axis=-1)[:, ::-1]
    clear = (z[:, top - 1] - z[:, top]) > 1e-4 if top < E else np.ones(T, bool)      # (a tie within float32 rounding may go either way)
    assert np.array_equal(idx.cpu().numpy()[clear], chosen[clear])
    assert np.abs(wts.cpu().numpy()[clear] - weights[clear]).max() < 1e-5
    flat = idx.cpu().numpy().reshape(-1)
    stack = lambda n: torch.tensor(np.stack([W[f"e{e}.{n}"] for e in range(E)]), dtype=dtype, device=DEV)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    for tensor_cores in ((False, True) if dtype == torch.bfloat16 else (False,)):     # the CUDA-core products, and the grouped tcgen05 ones
        if tensor_cores and (D % 8 or ff % 8):
            continue                                                                   # (sizes the tensor-core kernel does not take)
        rows = ops.moe_tile_rows(tensor_cores)
        max_tiles = ops.moe_max_tiles(T * top, E, rows)
        row_pair = torch.empty(max_tiles * rows, dtype=torch.int32, device=DEV)
        pair_row = torch.empty(T * top, dtype=torch.int32, device=DEV)
        tile_expert = torch.empty(max_tiles, dtype=torch.int32, device=DEV)
        ops.moe_plan(idx, E, rows, row_pair, pair_row, tile_expert)
        rp, pr, te = row_pair.cpu().numpy(), pair_row.cpu().numpy(), tile_expert.cpu().numpy()
        assert sorted(rp[rp >= 0].tolist()) == list(range(T * top))                # every pair has one row
        assert all(rp[pr[p]] == p for p in range(T * top))
        for r_, p in enumerate(rp):
            assert p < 0 or te[r_ // rows] == flat[p]                              # in a tile of its expert
        mid = torch.full((max_tiles * rows, ff), float("nan"), dtype=dtype, device=DEV)
        y = torch.full((max_tiles * rows, D), float("nan"), device=DEV)
        if tensor_cores:
            a = torch.full((max_tiles * rows, D), float("nan"), dtype=dtype, device=DEV)
            ops.moe_gather_rows(hd, a, row_pair, top)
            assert ops.gemm_tc_grouped_takes(a, stack("gate"), stack("up"))
            ops.gemm_tc_grouped(a, stack("gate"), mid, tile_expert, err, epilogue=ops.EPI_SWIGLU, w2=stack("up"))
            ops.gemm_tc_grouped(mid, stack("down"), y, tile_expert, err)
        else:
            ops.moe_gate_up(hd, stack("gate"), stack("up"), mid, row_pair, tile_expert, top)
            ops.moe_down(mid, stack("down"), y, row_pair, tile_expert, top)
        x = torch.ones(T, D, device=DEV)
        ops.moe_combine(x, y, wts, pair_row)
        got = x.cpu().numpy() - 1.0
        assert np.abs(got[clear] - want[clear]).max() < tol * max(1.0, np.abs(want).max()), tensor_cores
    assert int(err.item()) == 0
