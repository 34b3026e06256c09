"""The kernels of the Redenex decoder's mechanisms, each alone against the plain implementation's function for the same
mechanism (tests/plain_redenex.py): the gated diagonal recurrence with its convolution and block-wise gates, fed in pieces
on scattered state rows; several residual streams written and read in one pass; the clamped gated unit; per-map norm and
half-split rotation on the way into the cache pages; two attention maps per head over the same values, for steps of one
token and for prompt steps, with one key made so large that "seen" and "not seen" differ by much more than any
tolerance; the maps' combination."""
import numpy as np
import pytest
import torch

import plain_redenex as plain
from edgelm_b200.csrc import ops
from test_vosulorn_kernels_gpu import PAGE, PagedKV, f32, i32, make_tiles, packed, steps_of

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


# ----------------------------------------------------------------------------- real-gated linear recurrent unit
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,blocks,taps", [(96, 3, 4), (40, 1, 1), (70, 2, 2), (33, 3, 3), (360, 5, 4), (1030, 2, 3)])
def test_recurrent_unit_over_steps(W, blocks, taps, out_dtype):
    """Convolution with both biases, block-wise gates, decay and recurrence, fed in pieces (down to one token, shorter than
    the convolution's tail) on state rows in no particular order; a slot of nobody is never touched.  Decays close to 1:
    what a state held forty tokens ago still shows.  The last step packs the end of one sequence and the start of the next
    into one segment of the scan and runs over several segments."""
    g = np.random.default_rng(W + taps)
    total, cuts, slots = [43, 6, 1, 270], [[5, 1, 37], [2, 4], [1], [1, 1, 268]], [4, 0, 2, 5]
    bw = W // blocks
    w = {"y": np.eye(W), "y.b": g.uniform(-0.5, 0.5, W), "x": np.eye(W), "x.b": g.uniform(-0.5, 0.5, W), "conv": g.normal(0, 0.6, size=(W, taps)),
         "conv.b": g.uniform(-0.3, 0.3, W), "ra": g.normal(0, 1.5 / np.sqrt(bw), size=(blocks, bw, bw)), "ra.b": g.uniform(-1, 1, (blocks, bw)),
         "ri": g.normal(0, 1.5 / np.sqrt(bw), size=(blocks, bw, bw)), "ri.b": g.uniform(-1, 1, (blocks, bw)), "lam": g.uniform(-6, -1, W), "o": np.eye(W)}
    rnd = lambda a: torch.tensor(a, dtype=torch.float32).double().numpy()
    w = {k: rnd(v) for k, v in w.items()}
    py, px = [rnd(g.normal(size=(n, W))) for n in total], [rnd(g.normal(size=(n, W))) for n in total]      # the two projections before their biases
    want = []
    for s in range(len(total)):
        # (with identity projections the mixer's input would have to be both branches at once: run each branch's input through)
        y = plain.gelu_tanh(py[s] + w["y.b"])
        only_x = plain.rglru_mixer(px[s], {**w, "y": np.zeros((W, W)), "y.b": np.full(W, 30.0)}, {"width": W, "blocks": blocks, "conv": taps}, "")
        want.append(only_x / plain.gelu_tanh(np.full(W, 30.0)) * y)
    state = torch.zeros(7, W, device=DEV)
    tail = torch.zeros(7, taps - 1, W, device=DEV)
    state[1].fill_(float("nan"))
    decay = f32(-8.0 * plain.softplus(w["lam"]))
    got = [np.zeros_like(x) for x in want]
    for step in steps_of(total, cuts):
        live = [(s, a, n) for s, (a, n) in enumerate(step) if n]
        tok0, tok_seq = packed([n for _, _, n in live])
        seqslot = i32([slots[s] for s, _, _ in live])
        yx = f32(np.concatenate([np.concatenate([py[s][a:a + n], px[s][a:a + n]], axis=1) for s, a, n in live]))
        T = yx.shape[0]
        u = torch.full((T, W), float("nan"), device=DEV)
        ops.conv_act(yx, W, f32(w["conv"]), f32(w["conv.b"]), tail, u, tok_seq, tok0, seqslot, len(live), update_state=True, in_bias=f32(w["x.b"]), act=None)
        gates = torch.full((T, 2 * W), float("nan"), device=DEV)
        ops.rglru_gates(u, f32(w["ra"]), f32(w["ri"]), gates, blocks)
        o = torch.full((T, W), float("nan"), dtype=out_dtype, device=DEV)
        ops.rglru_scan(gates, f32(w["ra.b"].reshape(-1)), f32(w["ri.b"].reshape(-1)), u, decay, yx[:, :W], f32(w["y.b"]), state, o, tok0, seqslot,
                       len(live), all(n == 1 for _, _, n in live), tok_seq=tok_seq,
                       scratch=torch.full((ops.rglru_scratch_floats(T, len(live), W),), float("nan"), device=DEV))
        o = o.float().cpu().numpy()
        at = 0
        for s, a, n in live:
            got[s][a:a + n] = o[at:at + n]
            at += n
    tol = 2e-5 if out_dtype == torch.float32 else 1e-2
    for x, o in zip(want, got):
        assert np.abs(o - x).max() < tol * max(1.0, np.abs(x).max())
    assert torch.isnan(state[1]).all()


@pytest.mark.parametrize("w_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("W,blocks,T", [(96, 3, 37), (70, 2, 5), (33, 3, 1), (360, 5, 200), (480, 3, 131), (40, 1, 64), (384, 4, 70), (256, 2, 33),
                                       (400, 2, 65)])
def test_gate_products_are_float32(W, blocks, T, w_dtype):
    """The block-diagonal gate products keep the float32 input's low bits (rounding the input to bfloat16 would miss by a
    thousand times the tolerance), for block widths that are odd, below a tile and several tiles."""
    g = np.random.default_rng(W + T)
    bw = W // blocks
    u = torch.tensor(g.normal(size=(T, W)) * 3.0, dtype=torch.float32)
    ws = [torch.tensor(g.normal(0, 1.0, size=(blocks, bw, bw)), dtype=torch.float32).to(torch.bfloat16) for _ in range(2)]
    want = [np.einsum("bnk,tbk->tbn", w.double().numpy(), u.double().numpy().reshape(T, blocks, bw)).reshape(T, W) for w in ws]
    gates = torch.full((T, 2 * W), float("nan"), device=DEV)
    ops.rglru_gates(u.to(DEV), ws[0].to(device=DEV, dtype=w_dtype), ws[1].to(device=DEV, dtype=w_dtype), gates, blocks)
    got = gates.cpu().double().numpy()
    scale = 3.0 * np.sqrt(bw)
    tol = (1e-5 if w_dtype == torch.bfloat16 else 3e-6) * scale       # (the tensor cores' float32 sums drop the bits below the running sum's last one)
    assert np.abs(got[:, :W] - want[0]).max() < tol and np.abs(got[:, W:] - want[1]).max() < tol
    lossy = np.einsum("bnk,tbk->tbn", ws[0].double().numpy(), u.to(torch.bfloat16).double().numpy().reshape(T, blocks, bw)).reshape(T, W)
    assert np.abs(lossy - want[0]).max() > 1e-4 * scale      # (the check above can tell the two apart)


# ----------------------------------------------------------------------------- residual streams
@pytest.mark.parametrize("h_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("S,D,T", [(3, 64, 37), (1, 50, 5), (4, 208, 130), (8, 72, 3), (2, 1030, 9)])
def test_streams_write_and_read(S, D, T, h_dtype):
    g = np.random.default_rng(S * D)
    x = g.normal(size=(T, D))
    xs = torch.full((T, S, D), float("nan"), device=DEV)
    ops.streams_fill(f32(x), xs)
    assert np.array_equal(xs.cpu().numpy(), np.repeat(f32(x).cpu().numpy()[:, None], S, axis=1))
    cur = np.repeat(x[None], S, axis=0) + g.normal(size=(S, T, D))      # streams that differ
    xs = f32(cur.transpose(1, 0, 2))
    w1 = {"in": g.uniform(0.2, 0.9, S), "out": g.uniform(0.4, 1.2, S), "mix": np.eye(S) * 0.8 + g.uniform(-0.3, 0.3, (S, S))}
    w2 = {"in": g.uniform(0.2, 0.9, S), "out": g.uniform(0.4, 1.2, S), "mix": np.eye(S) * 0.8 + g.uniform(-0.3, 0.3, (S, S))}
    nw, eps = g.uniform(0.5, 1.5, D), 1e-4
    tol = 3e-6 if h_dtype == torch.float32 else 1e-2
    # a read alone, normed
    h = torch.full((T, D), float("nan"), dtype=h_dtype, device=DEV)
    ops.streams_update(xs, w_in=f32(w1["in"]), norm_w=f32(nw), eps=eps, h=h)
    u = np.einsum("s,snd->nd", w1["in"], cur)
    assert np.abs(h.float().cpu().numpy() - plain.rms_norm(u, eps, nw)).max() < tol * 4
    assert np.array_equal(xs.cpu().numpy(), f32(cur.transpose(1, 0, 2)).cpu().numpy())
    # a write and the next read in one pass; the write alone; the last write with the plain sum of the streams
    y = g.normal(size=(T, D))
    new = plain.hyper_sublayer(cur, w1, "", lambda _: y)
    ops.streams_update(xs, f32(y), f32(w1["mix"]), f32(w1["out"]), w_in=f32(w2["in"]), norm_w=f32(nw), eps=eps, h=h)
    assert np.abs(xs.cpu().numpy() - new.transpose(1, 0, 2)).max() < 1e-5
    assert np.abs(h.float().cpu().numpy() - plain.rms_norm(np.einsum("s,snd->nd", w2["in"], new), eps, nw)).max() < tol * 4
    y2 = g.normal(size=(T, D))
    new2 = plain.hyper_sublayer(new, w2, "", lambda _: y2)
    ops.streams_update(xs, f32(y2), f32(w2["mix"]), f32(w2["out"]))
    assert np.abs(xs.cpu().numpy() - new2.transpose(1, 0, 2)).max() < 2e-5
    total = torch.full((T, D), float("nan"), device=DEV)
    ops.streams_update(xs, w_in=torch.ones(S, device=DEV), h=total)
    assert np.abs(total.cpu().numpy() - new2.sum(axis=0)).max() < 3e-5


# ----------------------------------------------------------------------------- clamped gated unit
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,F,limit,alpha", [(37, 56, 0.7, 1.702), (3, 130, 2.0, 1.0), (200, 1029, 7.0, 1.702)])
def test_clamped_gated_unit(T, F, limit, alpha, dtype):
    g = np.random.default_rng(F)
    gu = torch.tensor(g.normal(0, 2.0 * limit, size=(T, 2 * F)), dtype=torch.float32)
    mid = torch.full((T, F), float("nan"), dtype=dtype, device=DEV)
    ops.clamped_glu(gu.to(DEV), mid, limit, alpha)
    a = gu.double().numpy()
    gate, up = np.minimum(a[:, :F], limit), np.clip(a[:, F:], -limit, limit)
    want = gate * plain.sigmoid(alpha * gate) * (up + 1.0)
    assert (a[:, :F] > limit).any() and (a[:, :F] < -limit).any() and (a[:, F:] < -limit).any()
    assert np.abs(mid.float().cpu().numpy() - want).max() < (3e-6 if dtype == torch.float32 else 1e-2) * max(1.0, np.abs(want).max())
    if alpha == 1.702:      # the plain function itself, with identity matrices
        w = {"gate": np.eye(F), "up": np.eye(F), "down": np.eye(F)}
        assert np.allclose(plain.clamped_glu(a[:, :F], {**w, "up": np.zeros((F, F))}, {"limit": limit}, ""), gate * plain.sigmoid(1.702 * gate))


@pytest.mark.parametrize("T,D,F,limit,alpha", [(200, 64, 130, 1.5, 1.702), (37, 48, 56, 0.7, 1.0), (300, 160, 1024, 7.0, 1.702)])
def test_clamped_gated_unit_in_the_product(T, D, F, limit, alpha):
    """The same unit as the epilogue of the tensor-core product of gate and up (prompt steps in bfloat16), against the plain
    feed-forward with an identity down projection; both clamps bite."""
    g = np.random.default_rng(T + F)
    bf = lambda a: torch.tensor(a, dtype=torch.float32).to(torch.bfloat16)
    h, wg, wu = bf(g.normal(size=(T, D))), bf(g.normal(0, 2.0 * limit / np.sqrt(D), size=(F, D))), bf(g.normal(0, 2.0 * limit / np.sqrt(D), size=(F, D)))
    w = {"gate": wg.double().numpy(), "up": wu.double().numpy(), "down": np.eye(F)}
    a = h.double().numpy()
    assert (a @ w["gate"].T > limit).any() and (a @ w["up"].T < -limit).any() and (a @ w["up"].T > limit).any()
    gate, up = np.minimum(a @ w["gate"].T, limit), np.clip(a @ w["up"].T, -limit, limit)
    want = gate * plain.sigmoid(alpha * gate) * (up + 1.0)
    if alpha == 1.702:
        assert np.allclose(want, plain.clamped_glu(a, w, {"limit": limit}, ""))
    mid = torch.full((T, F), float("nan"), dtype=torch.bfloat16, device=DEV)
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    w_gu = torch.cat([wg, wu]).to(DEV).contiguous()
    assert ops.gemm_tc_takes(h.to(DEV), w_gu[:F], mid, w_gu[F:])
    ops.gemm_tc(h.to(DEV), w_gu[:F], mid, err, epilogue=ops.EPI_SWIGLU, w2=w_gu[F:], glu=(limit, alpha, 1.0))
    assert int(err.abs().sum()) == 0
    assert np.abs(mid.float().cpu().numpy() - want).max() < 1e-2 * max(1.0, np.abs(want).max())


# ----------------------------------------------------------------------------- norm and rotation per map, into the cache
@pytest.mark.parametrize("H,G,d,dv,rot", [(3, 1, 20, 6, 12), (4, 2, 16, 24, 16), (2, 2, 10, 14, 0)])
def test_map_norm_rotation_and_append(H, G, d, dv, rot):
    """Every map of every head is normed by itself (a weight shared by all), then its first `rot` dimensions are turned
    with half-split pairs; keys go to their pages as [map 1, map 2] rows."""
    g = np.random.default_rng(d)
    from edgelm_b200.parts.rope import rotary_frequencies
    freq = rotary_frequencies(rot, 300.0, None) if rot else None
    pos = np.array([0, 1, 63, 64, 1000, 5000])
    T, kw = len(pos), 2 * d
    qkv = g.normal(size=(T, (H + G) * kw + G * dv)) * g.uniform(0.2, 5.0, size=(T, 1))
    qn, kn, eps = g.uniform(0.5, 1.5, d), g.uniform(0.5, 1.5, d), 1e-3
    kc = torch.zeros(90, G, PAGE, kw, device=DEV)
    vc = torch.zeros(90, G, PAGE, dv, device=DEV)
    table = i32(np.arange(89, -1, -1)[None])
    q_out = torch.empty(T, H * kw, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.rotate_append(f32(qkv), None, q_out, i32(pos), i32([0] * T), table, kc, vc, H, G, kw, dv, rot, False, freq.to(DEV) if rot else None, err,
                      maps=2, q_norm=f32(qn), k_norm=f32(kn), eps=eps)
    qw = plain.rms_norm(qkv[:, :H * kw].reshape(T, H, 2, d), eps, qn)
    kwant = plain.rms_norm(qkv[:, H * kw:(H + G) * kw].reshape(T, G, 2, d), eps, kn)
    if rot:
        qw, kwant = plain.rotate_half_pairs(qw, pos, rot, 300.0), plain.rotate_half_pairs(kwant, pos, rot, 300.0)
    assert np.abs(q_out.cpu().numpy().reshape(T, H, 2, d) - qw).max() < 5e-6
    for i, p in enumerate(pos):
        page = 89 - p // PAGE
        assert np.abs(kc[page, :, p % PAGE].cpu().numpy().reshape(G, 2, d) - kwant[i]).max() < 5e-6
        assert np.abs(vc[page, :, p % PAGE].cpu().numpy() - qkv[i, (H + G) * kw:].reshape(G, dv)).max() < 1e-6
    assert int(err.item()) == 0


# ----------------------------------------------------------------------------- two maps per head
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,size", [(4, 2, 16, 24, 7), (8, 1, 8, 8, 70), (3, 3, 10, 14, 64), (2, 1, 32, 20, 0), (6, 3, 8, 40, 128),
                                           (16, 2, 40, 88, 100), (4, 1, 24, 130, 33)])
def test_two_maps_over_the_same_values(H, G, d, dv, size, dtype):
    """Prompt steps (tiles) and steps of one token (a block per head, and tiles of one token with their pages dealt to
    several blocks) against the plain attention run once per map.  In each sequence one early key is made large in map 2
    only, and the queries of map 2 point at it: whether map 2 of a query sees it decides the second output, so a map read
    from the wrong half, or a chunk's edge one token off, shows at the positions just before and after the edge."""
    g = np.random.default_rng(d * 7 + dv)
    lengths = [150, 67, 1, 203]
    scale = 0.9 / np.sqrt(d)
    rnd = lambda a: torch.tensor(a, dtype=dtype).double().numpy()      # what the cache holds
    kv = PagedKV(lengths, G, 2 * d, dv, dtype, seed=3)
    Q, want = [], []
    for s, n in enumerate(lengths):
        q, k, v = g.normal(size=(n, H, 2, d)), g.normal(size=(n, G, 2, d)), rnd(g.normal(size=(n, G, dv)))
        far = min(n - 1, 5 if size == 0 else size - 2)
        k[far, :, 1] *= 12.0 / np.sqrt(d)
        k = rnd(k)
        q[:, :, 1] += 0.4 * np.repeat(k[far, :, 1], H // G, axis=0)[None]
        q = torch.tensor(q, dtype=torch.float32).double().numpy()
        kv.put(s, k.reshape(n, G, 2 * d), v)
        Q.append(q)
        maps = [plain.chunked_softmax_attention(q[:, :, j], k[:, :, j], v, scale, size or None) for j in range(2)]
        want.append(np.stack(maps, axis=2))                             # [n, H, 2, dv]
    table = i32(kv.table)
    mk, ms = (ops.MASK_CHUNK, size) if size else (ops.MASK_CAUSAL, 0)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for pieces in ([(0, n) for n in lengths], [(n // 3, n - n // 3) for n in lengths]):
        live = [(s, a, n) for s, (a, n) in enumerate(pieces) if n]
        tile = max(1, 32 // (H // G))
        tseq, ttok0, tntok, tpos0, count = make_tiles([n for _, _, n in live], [a for _, a, _ in live], tile)
        q = f32(np.concatenate([Q[s][a:a + n].reshape(n, H * 2 * d) for s, a, n in live]))
        out = torch.full((q.shape[0], H * 2 * dv), float("nan"), device=DEV)
        ops.masked_attn_tiled(q, out, kv.k, kv.v, table[[s for s, _, _ in live]].contiguous(), tseq, ttok0, tntok, tpos0, count, tile, H, G, d, dv,
                              scale, mk, ms, None, maps=2)
        ref = np.concatenate([want[s][a:a + n].reshape(n, H * 2 * dv) for s, a, n in live])
        assert np.abs(out.cpu().numpy() - ref).max() < tol * max(1.0, np.abs(ref).max()), ("tiled", pieces[0])
    for back in (0, 1, 2, 3, 64, 66):
        live = [(s, n - 1 - back) for s, n in enumerate(lengths) if n - 1 - back >= 0]
        q = f32(np.stack([Q[s][p].reshape(H * 2 * d) for s, p in live]))
        ref = np.stack([want[s][p].reshape(H * 2 * dv) for s, p in live])
        n = len(live)
        rows = table[[s for s, _ in live]].contiguous()
        out = torch.full((n, H * 2 * dv), float("nan"), device=DEV)
        ops.masked_attn(q, out, kv.k, kv.v, i32([p for _, p in live]), i32(list(range(n))), rows, H, G, d, dv, scale, mk, ms, None,
                        size if size else 1 << 30, maps=2)
        assert np.abs(out.cpu().numpy() - ref).max() < tol * max(1.0, np.abs(ref).max()), ("single", back)
        for splits in (1, 3, 5):
            out2 = torch.full((n, H * 2 * dv), float("nan"), device=DEV)
            part = torch.full((n * H * 2 * splits * (2 + dv),), float("nan"), device=DEV)
            ops.masked_attn_tiled(q, out2, kv.k, kv.v, rows, i32(list(range(n))), i32(list(range(n))), i32([1] * n), i32([p for _, p in live]), n, 1,
                                  H, G, d, dv, scale, mk, ms, None, n_splits=splits, part=part, maps=2)
            assert np.abs(out2.cpu().numpy() - ref).max() < tol * max(1.0, np.abs(ref).max()), ("single, split", back, splits)


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,dv,lam,offset", [(37, 4, 24, 0.37, 0.3), (3, 1, 130, -0.2, 0.8), (130, 16, 80, 1.4, 0.7), (5, 3, 7, 0.5, 0.5)])
def test_maps_combined(T, H, dv, lam, offset, out_dtype):
    g = np.random.default_rng(dv)
    a = torch.tensor(g.normal(size=(T, H, 2, dv)) * g.uniform(0.01, 3.0, size=(T, H, 1, 1)), dtype=torch.float32)
    out = torch.full((T, H * dv), float("nan"), dtype=out_dtype, device=DEV)
    ops.diff_combine(a.to(DEV), out, lam, 1e-5, 1.0 - offset)
    want = plain.combine_maps(a[:, :, 0].double().numpy(), a[:, :, 1].double().numpy(), lam, offset, 1e-5).reshape(T, H * dv)
    assert np.abs(out.float().cpu().numpy() - want).max() < (5e-6 if out_dtype == torch.float32 else 1e-2) * max(1.0, np.abs(want).max())
