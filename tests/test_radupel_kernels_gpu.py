"""The kernels of the Radupel decoder's mechanisms, each alone against the plain implementation's function for the same
mechanism (tests/plain_radupel.py): the decayed linear attention fed in pieces on scattered state rows; the norm over all
heads with a sigmoid gate; two norms of the same rows in one pass (with rows added first); the soft cap; the gated unit with
biases; softmax attention with a gate per head, for prompt steps and steps of one token, reading queries, keys and values
out of rows that hold more; the scoring router with corrections, groups and negative scores; identity experts, the shared
expert and the clamped experts through the grouping, the products and the weighted sum."""
import numpy as np
import pytest
import torch

import plain_radupel as plain
from edgelm_b200.csrc import ops
from test_vosulorn_kernels_gpu import PAGE, PagedKV, f32, i32, make_tiles, packed, steps_of

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


# ----------------------------------------------------------------------------- linear attention with a constant decay
@pytest.mark.parametrize("H,d,e,decay", [(2, 24, 16, (0.9, 0.998)), (3, 40, 8, (0.3, 0.97, 1.0)), (1, 32, 48, (0.95,)), (4, 8, 8, (0.5, 0.8, 0.99, 0.0)),
                                         (2, 64, 12, (0.98, 0.93)), (1, 72, 130, (0.97,)), (2, 130, 5, (0.9, 0.6)), (1, 256, 3, (0.99,))])
def test_decayed_linear_attention_over_steps(H, d, e, decay):
    """silu of the projections and the recurrence, fed in pieces (down to one token) on state rows in no particular order; a
    slot of nobody is never touched.  Decays up to 1: what a state took in at the start still shows at the end."""
    g = np.random.default_rng(d + e)
    total, cuts, slots = [43, 6, 1, 270], [[5, 1, 37], [2, 4], [1], [1, 1, 268]], [4, 0, 2, 5]
    C = 2 * H * d + H * e
    extra = 5                                                     # (columns after q | k | v that the kernels must leave alone)
    raw = [torch.tensor(g.normal(size=(n, C + extra)), dtype=torch.float32).double().numpy() for n in total]
    want = []
    for s, n in enumerate(total):
        x = plain.silu(raw[s][:, :C])
        want.append(plain.decayed_linear_attention(x[:, :H * d].reshape(n, H, d), x[:, H * d:2 * H * d].reshape(n, H, d), x[:, 2 * H * d:].reshape(n, H, e),
                                                   np.asarray(decay)).reshape(n, H * e))
    state = torch.zeros(7, H, e, d, device=DEV)
    state[1].fill_(float("nan"))
    got = [np.zeros_like(w) for w in want]
    for step in steps_of(total, cuts):
        live = [(s, a, n) for s, (a, n) in enumerate(step) if n]
        tok0, _ = packed([n for _, _, n in live])
        seqslot = i32([slots[s] for s, _, _ in live])
        u = f32(np.concatenate([raw[s][a:a + n] for s, a, n in live]))
        keep = u[:, C:].clone()
        inside = all(n == 1 for _, _, n in live)          # (steps of one token a sequence: the activation inside the walk)
        if not inside:
            ops.silu_columns(u, 0, C)
        assert torch.equal(u[:, C:], keep)
        o = torch.full((u.shape[0], H * e), float("nan"), device=DEV)
        ops.decay_scan(u, 0, H * d, 2 * H * d, f32(decay), state, o, tok0, seqslot, len(live), H, d, e, act="silu" if inside else None)
        o = o.cpu().numpy()
        at = 0
        for s, a, n in live:
            got[s][a:a + n] = o[at:at + n]
            at += n
    for w, o in zip(want, got):
        assert np.abs(o - w).max() < 2e-5 * max(1.0, np.abs(w).max())
    assert torch.isnan(state[1]).all()


@pytest.mark.parametrize("H,d,e,decay", [(2, 24, 16, (0.9, 0.998)), (3, 40, 8, (0.3, 0.97, 1.0)), (1, 32, 48, (0.95,)), (4, 8, 8, (0.5, 0.8, 0.99, 0.0)),
                                         (2, 64, 64, (0.98, 0.93)), (1, 72, 128, (0.97,)), (2, 128, 5, (0.9, 0.6)), (1, 1, 1, (0.99,))])
def test_decayed_linear_attention_chunk_by_chunk(H, d, e, decay):
    """The same recurrence in its chunked form, which prompt steps take: pieces that end inside a chunk, at a chunk's edge and
    one token past it, several sequences in a step, state rows in no particular order; then the walk goes on from the state
    that the chunks left (decoding after a prompt), and the chunks from the walk's."""
    g = np.random.default_rng(d * 3 + e)
    total, cuts, slots = [300, 64, 131, 9], [[63, 1, 130, 1, 105], [64], [65, 2, 64], [2, 7]], [4, 0, 2, 5]
    walked = [{1, 3}, set(), {1}, set()]                            # (sequence -> the steps of it that the walk takes instead)
    C = 2 * H * d + H * e
    raw = [torch.tensor(g.normal(size=(n, C + 3)), dtype=torch.float32).double().numpy() for n in total]
    want = []
    for s, n in enumerate(total):
        x = plain.silu(raw[s][:, :C])
        want.append(plain.decayed_linear_attention(x[:, :H * d].reshape(n, H, d), x[:, H * d:2 * H * d].reshape(n, H, d), x[:, 2 * H * d:].reshape(n, H, e),
                                                   np.asarray(decay)).reshape(n, H * e))
    assert ops.decay_chunked_takes(d, e)
    state = torch.zeros(7, H, e, d, device=DEV)
    state[1].fill_(float("nan"))
    got = [np.zeros_like(w) for w in want]
    for k, step in enumerate(steps_of(total, cuts)):
        for walk in (False, True):
            live = [(s, a, n) for s, (a, n) in enumerate(step) if n and ((k in walked[s]) == walk)]
            if not live:
                continue
            lengths = [n for _, _, n in live]
            tok0, _ = packed(lengths)
            seqslot = i32([slots[s] for s, _, _ in live])
            u = f32(np.concatenate([raw[s][a:a + n] for s, a, n in live]))
            o = torch.full((u.shape[0], H * e), float("nan"), device=DEV)
            if walk:
                ops.silu_columns(u, 0, C)
                ops.decay_scan(u, 0, H * d, 2 * H * d, f32(decay), state, o, tok0, seqslot, len(live), H, d, e)
            else:
                _, ttok0, tntok, _, count = make_tiles(lengths, [0] * len(live), ops.DECAY_CHUNK)
                scratch = torch.full((ops.decay_chunked_scratch_floats(count, H, d, e),), float("nan"), device=DEV)
                ops.decay_chunked(u, 0, H * d, 2 * H * d, ops.decay_powers(decay).to(DEV), state, o, tok0, seqslot, len(live), ttok0, tntok, count, H, d, e, act="silu", scratch=scratch)
            o = o.cpu().numpy()
            at = 0
            for s, a, n in live:
                got[s][a:a + n] = o[at:at + n]
                at += n
    for w, o in zip(want, got):
        assert np.abs(o - w).max() < 2e-5 * max(1.0, np.abs(w).max())
    assert torch.isnan(state[1]).all()


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_norm_over_all_heads_with_a_sigmoid_gate(out_dtype):
    g = np.random.default_rng(3)
    T, inner = 9, 88
    y, gate, w = g.normal(size=(T, inner)) * 3, g.normal(size=(T, inner + 7)), g.uniform(0.5, 1.5, inner)
    out = torch.empty(T, inner, dtype=out_dtype, device=DEV)
    ops.gated_group_norm(f32(y), f32(gate)[:, 7:], f32(w), out, 1, 1e-4, gate_first=False, gate_act="sigmoid")
    want = plain.rms_norm(y, 1e-4, w) * plain.sigmoid(gate[:, 7:])
    assert np.abs(out.float().cpu().numpy() - want).max() < (1e-5 if out_dtype == torch.float32 else 2e-2)


# ----------------------------------------------------------------------------- the layer's two norms, the soft cap, the biased unit
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D", [50, 64, 1030])
def test_two_norms_of_the_same_rows(D, out_dtype):
    g = np.random.default_rng(D)
    T = 11
    x, add, w1, w2 = g.normal(size=(T, D)) * 2, g.normal(size=(T, D)), g.uniform(0.5, 1.5, D), g.uniform(-1, 1, D)
    tol = 1e-5 if out_dtype == torch.float32 else 2e-2
    for with_add in (False, True):
        for second in (True, False):
            xd = f32(x)
            y1 = torch.empty(T, D, dtype=out_dtype, device=DEV)
            y2 = torch.empty(T, D, dtype=out_dtype, device=DEV) if second else None
            ops.rmsnorm_pair(xd, f32(w1), 1e-5, y1, f32(w2) if second else None, y2, add=f32(add) if with_add else None)
            xs = np.float32(x) + np.float32(add) if with_add else np.float32(x)
            assert np.array_equal(xd.cpu().numpy(), xs)          # x itself took the added rows, and nothing else
            assert np.abs(y1.float().cpu().numpy() - plain.rms_norm(xs.astype(np.float64), 1e-5, w1)).max() < tol * 4
            if second:
                assert np.abs(y2.float().cpu().numpy() - plain.rms_norm(xs.astype(np.float64), 1e-5, w2)).max() < tol * 4


def test_soft_cap_and_accumulating_sum():
    g = np.random.default_rng(5)
    z = g.normal(size=(7, 301)) * 40
    zd = f32(z)
    ops.softcap(zd, 12.5)
    assert np.abs(zd.cpu().numpy() - 12.5 * np.tanh(z / 12.5)).max() < 1e-5
    a, b, x = g.normal(size=(5, 33)), g.normal(size=(5, 33)), g.normal(size=(5, 33))
    xd = f32(x)
    ops.scaled_sum(f32(a), 1.3, f32(b), -0.4, xd, add=True)
    assert np.abs(xd.cpu().numpy() - (x + 1.3 * a - 0.4 * b)).max() < 1e-6
    ops.scaled_sum(f32(a), 1.3, f32(b), -0.4, xd)
    assert np.abs(xd.cpu().numpy() - (1.3 * a - 0.4 * b)).max() < 1e-6


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gated_unit_with_biases(out_dtype):
    """silu(gate + b) (up + b): the clamped unit's kernel without clamps, with slope 1 and no shift."""
    g = np.random.default_rng(8)
    T, F = 6, 70
    gu, bias = g.normal(size=(T, 2 * F)) * 2, g.uniform(-1, 1, 2 * F)
    mid = torch.empty(T, F, dtype=out_dtype, device=DEV)
    ops.clamped_glu(f32(gu), mid, 0.0, 1.0, shift=0.0, bias=f32(bias))
    want = plain.silu(gu[:, :F] + bias[:F]) * (gu[:, F:] + bias[F:])
    rel = 1e-5 if out_dtype == torch.float32 else 5e-3
    assert (np.abs(mid.float().cpu().numpy() - want) <= rel * (1.0 + np.abs(want))).all()
    # and the clamped form with a limit, a slope and the shift of 1, on the same kernel
    ops.clamped_glu(f32(gu), mid, 1.2, 1.702)
    gg, uu = np.minimum(gu[:, :F], 1.2), np.clip(gu[:, F:], -1.2, 1.2)
    want = gg * plain.sigmoid(1.702 * gg) * (uu + 1)
    assert (np.abs(mid.float().cpu().numpy() - want) <= rel * (1.0 + np.abs(want))).all()


@pytest.mark.parametrize("M,N,K", [(200, 40, 64), (17, 320, 320), (2048, 1536, 576), (130, 72, 1032)])
def test_biases_in_the_tensor_core_gated_epilogue(M, N, K):
    """silu(a Wg^T + bg) (a Wu^T + bu) as the epilogue of the tcgen05 product of both weights, for one tile, many tiles and the
    sizes that split K."""
    g = np.random.default_rng(M + N)
    bf = lambda x: torch.tensor(x, dtype=torch.bfloat16, device=DEV)
    a, wg, wu = bf(g.normal(size=(M, K))), bf(g.normal(size=(N, K)) / np.sqrt(K)), bf(g.normal(size=(N, K)) / np.sqrt(K))
    bias = f32(g.uniform(-1, 1, 2 * N))
    mid = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert ops.gemm_tc_takes(a, wg, mid, wu)
    ops.gemm_tc(a, wg, mid, err, epilogue=ops.EPI_SWIGLU, w2=wu, glu_bias=bias)
    ad, b = a.double().cpu().numpy(), bias.double().cpu().numpy()
    want = plain.silu(ad @ wg.double().cpu().numpy().T + b[:N]) * (ad @ wu.double().cpu().numpy().T + b[N:])
    assert (np.abs(mid.float().cpu().numpy() - want) <= 1e-2 * (1.0 + np.abs(want))).all()
    assert int(err.item()) == 0


# ----------------------------------------------------------------------------- softmax attention with a gate per head
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dk,dv,rot", [(4, 2, 16, 24, 8), (8, 1, 8, 8, 8), (3, 3, 10, 14, 0), (16, 2, 8, 12, 6), (2, 1, 96, 40, 24), (4, 2, 64, 64, 32),
                                           (2, 1, 96, 96, 24), (3, 3, 32, 32, 0), (2, 2, 128, 128, 64)])
def test_gated_softmax_attention(H, G, dk, dv, rot, dtype):
    """Rotation and append from rows that hold q | k | v | gate, then causal attention with each head's output times the
    sigmoid of its gate: prompt steps in tiles, steps of one token (a block per head, and pages dealt to several blocks).
    One early key is made large and the queries point at it, so a key lost or a head's gate read from another head's
    column shows."""
    g = np.random.default_rng(dk * 7 + dv)
    lengths = [150, 67, 1, 203]
    scale = 0.9 / np.sqrt(dk)
    rnd = lambda a: torch.tensor(a, dtype=dtype).double().numpy()      # what the cache holds
    kv = PagedKV(lengths, G, dk, dv, dtype, seed=3)
    kv.v.fill_(0)                                                       # (rotate_append fills both)
    from edgelm_b200.parts.rope import rotary_frequencies
    freq = rotary_frequencies(rot, 900.0, None).to(DEV) if rot else None
    d_qkv = (H + G) * dk + G * dv
    rows, want = [], []
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    table = i32(kv.table)
    for s, n in enumerate(lengths):
        q, k, v, gate = g.normal(size=(n, H, dk)), g.normal(size=(n, G, dk)), g.normal(size=(n, G, dv)), g.normal(size=(n, H)) * 2
        far = min(n - 1, 5)
        k[far] *= 12.0 / np.sqrt(dk)
        q += 0.4 * np.repeat(k[far], H // G, axis=0)[None]
        u = torch.tensor(np.concatenate([q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1), gate], axis=1), dtype=torch.float32)
        rows.append(u)
        ud = u.double().numpy()
        q, k, v, gate = ud[:, :H * dk].reshape(n, H, dk), ud[:, H * dk:(H + G) * dk].reshape(n, G, dk), ud[:, (H + G) * dk:d_qkv].reshape(n, G, dv), ud[:, d_qkv:]
        if rot:
            q, k = plain.rotate_half_pairs(q, np.arange(n), rot, 900.0), plain.rotate_half_pairs(k, np.arange(n), rot, 900.0)
        o = plain.causal_softmax_attention(q, rnd(k), rnd(v), scale) * plain.sigmoid(gate)[:, :, None]
        want.append(o.reshape(n, H * dv))
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    # the whole sequences as one prompt step: append, then attend
    u = torch.cat(rows).to(DEV)
    tok0, tok_seq = packed(lengths)
    pos = i32(np.concatenate([np.arange(n) for n in lengths]))
    qo = torch.empty(u.shape[0], H * dk, device=DEV)
    ops.rotate_append(u[:, :d_qkv], None, qo, pos, tok_seq, table, kv.k, kv.v, H, G, dk, dv, rot, False, freq, err)
    tile = max(1, 32 // (H // G))
    tseq, ttok0, tntok, tpos0, count = make_tiles(lengths, [0] * len(lengths), tile)
    out = torch.full((u.shape[0], H * dv), float("nan"), dtype=dtype, device=DEV)
    ops.masked_attn_tiled(qo, out, kv.k, kv.v, table, tseq, ttok0, tntok, tpos0, count, tile, H, G, dk, dv, scale, ops.MASK_CAUSAL, 0, None, gate=u[:, d_qkv:])
    ref = np.concatenate(want)
    assert np.abs(out.float().cpu().numpy() - ref).max() < tol * max(1.0, np.abs(ref).max())
    if ops.attn_prefill_split_takes(dtype, dk, dv):
        # the tensor-core kernel with float32 scores and weights, whole sequences and then their second halves over the first
        tseq, ttok0, tntok, tpos0, count = make_tiles(lengths, [0] * len(lengths), ops.SPLIT_PREFILL_TILE)
        out = torch.full((u.shape[0], H * dv), float("nan"), dtype=dtype, device=DEV)
        ops.attn_prefill_split(qo, out, kv.k, kv.v, table, tseq, ttok0, tntok, tpos0, count, H, G, dk, scale, gate=u[:, d_qkv:], max_keys=max(lengths))
        got = out.float().cpu().numpy()
        assert np.abs(got - ref).max() < tol * max(1.0, np.abs(ref).max())
        halves = [(n // 3, n - n // 3) for n in lengths]
        starts0 = np.concatenate([[0], np.cumsum(lengths)])
        sel = torch.tensor(np.concatenate([np.arange(starts0[s] + a, starts0[s] + a + n) for s, (a, n) in enumerate(halves)]), device=DEV)
        tseq, ttok0, tntok, tpos0, count = make_tiles([n for _, n in halves], [a for a, _ in halves], ops.SPLIT_PREFILL_TILE)
        out = torch.full((len(sel), H * dv), float("nan"), dtype=dtype, device=DEV)
        ops.attn_prefill_split(qo[sel].contiguous(), out, kv.k, kv.v, table, tseq, ttok0, tntok, tpos0, count, H, G, dk, scale,
                               gate=u[sel][:, d_qkv:], max_keys=max(lengths))
        assert np.abs(out.float().cpu().numpy() - ref[sel.cpu().numpy()]).max() < tol * max(1.0, np.abs(ref).max())
    # steps of one token a sequence at the sequences' ends and around a page border
    starts = np.concatenate([[0], np.cumsum(lengths)])
    for back in (0, 1, 64, 66):
        live = [(s, n - 1 - back) for s, n in enumerate(lengths) if n - 1 - back >= 0]
        sel = torch.tensor([int(starts[s]) + p for s, p in live], device=DEV)
        q1, g1 = qo[sel].contiguous(), u[sel][:, d_qkv:]
        ref = np.stack([want[s][p] for s, p in live])
        sub = table[[s for s, _ in live]].contiguous()
        n = len(live)
        out = torch.full((n, H * dv), float("nan"), dtype=dtype, device=DEV)
        ops.masked_attn(q1, out, kv.k, kv.v, i32([p for _, p in live]), i32(list(range(n))), sub, H, G, dk, dv, scale, ops.MASK_CAUSAL, 0, None, 1 << 30, gate=g1)
        assert np.abs(out.float().cpu().numpy() - ref).max() < tol * max(1.0, np.abs(ref).max()), ("single", back)
        for splits in (2, 5):       # the same kernel with a pair's keys dealt to several blocks (some of which get none)
            out3 = torch.full((n, H * dv), float("nan"), dtype=dtype, device=DEV)
            part = torch.full((n * H * splits * (2 + dv),), float("nan"), device=DEV)
            ops.masked_attn(q1, out3, kv.k, kv.v, i32([p for _, p in live]), i32(list(range(n))), sub, H, G, dk, dv, scale, ops.MASK_CAUSAL, 0, None, 1 << 30,
                            gate=g1, n_splits=splits, part=part)
            assert np.abs(out3.float().cpu().numpy() - ref).max() < tol * max(1.0, np.abs(ref).max()), ("single, keys split", back, splits)
        for splits in (1, 3):
            out2 = torch.full((n, H * dv), float("nan"), dtype=dtype, device=DEV)
            part = torch.full((n * H * splits * (2 + dv),), float("nan"), device=DEV)
            ops.masked_attn_tiled(q1, out2, kv.k, kv.v, sub, i32(list(range(n))), i32(list(range(n))), i32([1] * n), i32([p for _, p in live]), n, 1, H, G,
                                  dk, dv, scale, ops.MASK_CAUSAL, 0, None, n_splits=splits, part=part, gate=g1)
            assert np.abs(out2.float().cpu().numpy() - ref).max() < tol * max(1.0, np.abs(ref).max()), ("single, split", back, splits)
    assert int(err.item()) == 0


@pytest.mark.parametrize("taps", [1, 2, 4])
def test_filter_over_time_inside_rotation_and_append(taps):
    """The short causal filter on q, k and v, the rotation and the cache append in one kernel, fed in pieces (down to one token,
    shorter than the filter's tail, and steps of one token a sequence, which move the tails on themselves) on tail rows in no
    particular order: what reaches q and the cache pages is the plain filter of the whole sequence, rotated."""
    from edgelm_b200.parts.rope import rotary_frequencies
    g = np.random.default_rng(taps)
    H, G, dk, dv, rot = 3, 1, 12, 6, 8
    C = (H + G) * dk + G * dv
    total, cuts, slots = [43, 6, 1, 70], [[5, 1, 37], [2, 4], [1], [1, 1, 68]], [4, 0, 2, 5]
    raw = [torch.tensor(g.normal(size=(n, C + 2)), dtype=torch.float32).double().numpy() for n in total]     # (two more columns: rows hold more than q | k | v)
    w = torch.tensor(g.normal(0, 0.6, size=(C, taps)), dtype=torch.float32).double().numpy()
    freq = rotary_frequencies(rot, 300.0, None)
    kv = PagedKV(total, G, dk, dv, torch.float32, seed=2)
    kv.v.fill_(0)
    table = i32(kv.table)
    tails = torch.zeros(7, taps - 1, C, device=DEV)
    tails[1].fill_(float("nan"))
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    got_q = [np.zeros((n, H * dk)) for n in total]
    for step in steps_of(total, cuts):
        live = [(s, a, n) for s, (a, n) in enumerate(step) if n]
        tok0, tok_seq = packed([n for _, _, n in live])
        u = f32(np.concatenate([raw[s][a:a + n] for s, a, n in live]))
        pos = i32(np.concatenate([np.arange(a, a + n) for _, a, n in live]))
        q = torch.full((u.shape[0], H * dk), float("nan"), device=DEV)
        ops.rotate_append(u[:, :C], None, q, pos, tok_seq, table[[s for s, _, _ in live]].contiguous(), kv.k, kv.v, H, G, dk, dv, rot, False, freq.to(DEV), err,
                          conv_w=f32(w), conv_state=tails if taps > 1 else None, seq_tok0=tok0, seq_slot=i32([slots[s] for s, _, _ in live]), n_seqs=len(live))
        q = q.cpu().numpy()
        at = 0
        for s, a, n in live:
            got_q[s][a:a + n] = q[at:at + n]
            at += n
    for s, n in enumerate(total):
        y = plain.causal_conv(raw[s][:, :C], w)
        qw = plain.rotate_half_pairs(y[:, :H * dk].reshape(n, H, dk), np.arange(n), rot, 300.0)
        kw = plain.rotate_half_pairs(y[:, H * dk:(H + G) * dk].reshape(n, G, dk), np.arange(n), rot, 300.0)
        assert np.abs(got_q[s] - qw.reshape(n, H * dk)).max() < 1e-5
        for p in range(n):
            page = kv.table[s, p // PAGE]
            assert np.abs(kv.k[page, :, p % PAGE].cpu().numpy() - kw[p]).max() < 1e-5
            assert np.abs(kv.v[page, :, p % PAGE].cpu().numpy() - y[p, (H + G) * dk:].reshape(G, dv)).max() < 1e-5
    assert int(err.item()) == 0 and (taps == 1 or torch.isnan(tails[1]).all())


def test_tensor_core_attention_keeps_float32_scores_and_weights():
    """Queries so large that their rounding to bfloat16 would move the scores by a good part of 1, and values of very
    different sizes under weights of very different sizes: the kernel's output follows the float64 attention of the float32
    queries, not that of rounded queries nor that of rounded weights."""
    g = np.random.default_rng(4)
    H, G, d, n = 2, 1, 64, 200
    bf = lambda a: torch.tensor(a, dtype=torch.bfloat16).double().numpy()
    q = torch.tensor(g.normal(size=(n, H, d)) * 10.0, dtype=torch.float32).double().numpy()
    k, v = bf(g.normal(size=(n, G, d))), bf(g.normal(size=(n, G, d)) * np.exp(g.normal(size=(n, 1, 1)) * 3))
    scale = 1.0 / np.sqrt(d)
    want = plain.causal_softmax_attention(q, k, v, scale).reshape(n, H * d)
    rounded_q = plain.causal_softmax_attention(bf(q), k, v, scale).reshape(n, H * d)
    kv = PagedKV([n], G, d, d, torch.bfloat16, seed=1)
    kv.put(0, k, v)
    tseq, ttok0, tntok, tpos0, count = make_tiles([n], [0], ops.SPLIT_PREFILL_TILE)
    out = torch.full((n, H * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.attn_prefill_split(f32(q.reshape(n, H * d)), out, kv.k, kv.v, i32(kv.table), tseq, ttok0, tntok, tpos0, count, H, G, d, scale, max_keys=n)
    got = out.float().cpu().numpy()
    size = np.abs(want).max(axis=1, keepdims=True) + 1e-9
    ours, theirs = (np.abs(got - want) / size).max(), (np.abs(rounded_q - want) / size).max()
    assert ours < 6e-3 and theirs > 5 * ours, (ours, theirs)       # (6e-3: the output's own rounding to bfloat16)


# ----------------------------------------------------------------------------- the scoring router and its experts
@pytest.mark.parametrize("E,ident,top,groups,keep,negative", [(6, 3, 3, 3, 2, False), (3, 0, 1, 1, 1, False), (5, 1, 2, 2, 1, True), (7, 2, 2, 3, 1, True),
                                                              (8, 0, 4, 4, 2, False), (2, 2, 2, 1, 1, True), (12, 4, 3, 8, 2, False), (4, 2, 3, 3, 1, True)])
def test_scoring_router(E, ident, top, groups, keep, negative):
    """Scores over all routed experts (identity experts too), the choice by corrected scores inside the best groups only (a
    group left out counts as minus infinity, which shows when every corrected score is negative), the weights from the
    uncorrected scores; the extra router row gives the shared expert's gate."""
    g = np.random.default_rng(E + top)
    T, D, R = 300, 40, E + ident
    h = torch.tensor(g.normal(size=(T, D)), dtype=torch.float32).double().numpy()
    wr = torch.tensor(g.normal(size=(R + 1, D)) * 2 / np.sqrt(D), dtype=torch.float32).double().numpy()
    corr = torch.tensor(g.uniform(-0.9, -0.6, R) if negative else g.uniform(-0.2, 0.2, R), dtype=torch.float32).double().numpy()
    chosen, weights = plain.route(h @ wr[:R].T, corr, top, groups, keep, 1.7)
    idx = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, device=DEV)
    extra = torch.empty(T, 1, device=DEV)
    ops.moe_route_scored(f32(h), f32(wr), f32(corr), idx, wts, top, R, groups, keep, 1.7, extra=extra)
    # (a call closer than float32 rounding may go either way: compare where the plain choice is clear)
    z = h @ wr[:R].T
    s = np.exp(z - z.max(1, keepdims=True)); s /= s.sum(1, keepdims=True)
    c = np.sort(s + corr, axis=1)
    clear = np.diff(c, axis=1).min(axis=1) > 1e-5
    assert clear.mean() > 0.9
    if keep * (R // groups) < top:       # more choices than the kept groups hold: the rest are the left-out experts in the order of their numbers
        assert (chosen[:, keep * (R // groups):] < R).all() and (np.diff(chosen[:, keep * (R // groups):], axis=1) > 0).all()
    assert np.array_equal(idx.cpu().numpy()[clear], chosen[clear])
    assert np.abs(wts.cpu().numpy()[clear] - weights[clear]).max() < 1e-5
    assert np.abs(extra.cpu().numpy()[:, 0] - plain.sigmoid(h @ wr[R])).max() < 1e-6
    if groups > 1:      # the choice is not what it would be without groups (the test can tell)
        free, _ = plain.route(z, corr, top, 1, 1, 1.7)
        assert not np.array_equal(free, chosen)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,D,E,ident,top,ff,shared", [(37, 64, 4, 2, 2, 40, 24), (1, 50, 2, 1, 3, 30, None), (200, 48, 6, 3, 3, 24, 32), (70, 32, 1, 0, 1, 8, 16)])
def test_clamped_experts_identity_and_shared(T, D, E, ident, top, ff, shared, dtype):
    """From the router's choice to the residual sum: grouping (identity experts' pairs get no row), the clamped gated unit in
    both products' kernels, the weighted sum with the token's own input for identity experts and the gated shared term."""
    g = np.random.default_rng(T + E)
    rnd = lambda a: torch.tensor(a, dtype=dtype).double().numpy()
    R, limit = E + ident, 1.3
    W = {"router": torch.tensor(g.normal(size=(R, D)) * 3 / np.sqrt(D), dtype=torch.float32).double().numpy(),
         "correction": torch.tensor(g.uniform(-0.1, 0.1, R), dtype=torch.float32).double().numpy()}
    for e in range(E):
        W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"] = rnd(g.normal(size=(ff, D)) * 2 / np.sqrt(D)), rnd(g.normal(size=(ff, D)) * 2 / np.sqrt(D)), rnd(g.normal(size=(D, ff)) / np.sqrt(ff))
    mlp = {"expert": {"ff": ff, "limit": limit}, "router": {"experts": E, "top": top, "identity": ident, "scale": 1.9}}
    if shared:
        W["shared.gate"], W["shared.up"], W["shared.down"] = rnd(g.normal(size=(shared, D)) / np.sqrt(D)), rnd(g.normal(size=(shared, D)) / np.sqrt(D)), rnd(g.normal(size=(D, shared)) / np.sqrt(shared))
        W["shared.sg"] = torch.tensor(g.normal(size=(1, D)) / np.sqrt(D), dtype=torch.float32).double().numpy()
        mlp["shared"] = {"ff": shared, "limit": 0.9}
    h = rnd(g.normal(size=(T, D)))
    want = plain.moe_ffn(h, W, mlp, "")
    hd = torch.tensor(h, dtype=dtype, device=DEV)
    idx = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, device=DEV)
    wr = np.concatenate([W["router"], W["shared.sg"]]) if shared else W["router"]
    gate = torch.empty(T, 1, device=DEV) if shared else None
    ops.moe_route_scored(hd, f32(wr), f32(W["correction"]), idx, wts, top, R, 1, 1, 1.9, extra=gate)
    z = h @ W["router"].T
    s = np.exp(z - z.max(1, keepdims=True)); s /= s.sum(1, keepdims=True)
    c = np.sort(s + W["correction"], axis=1)
    clear = np.diff(c, axis=1).min(axis=1) > 1e-5 if R > 1 else np.ones(T, bool)
    ys = None
    if shared:      # the shared expert's output, float32 rows (its products are the library's matrix products; here the plain ones)
        ys = f32(plain.clamped_expert(h, W, "shared.", 0.9))
    stack = lambda n: torch.tensor(np.stack([W[f"e{e}.{n}"] for e in range(E)]), dtype=dtype, device=DEV)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    glu = (limit, 1.702, 1.0)
    for tensor_cores in ((False, True) if dtype == torch.bfloat16 else (False,)):
        if tensor_cores and (D % 8 or ff % 8):
            continue
        rows = ops.moe_tile_rows(tensor_cores)
        max_tiles = ops.moe_max_tiles(T * top, E, rows)
        row_pair = torch.empty(max_tiles * rows, dtype=torch.int32, device=DEV)
        pair_row = torch.empty(T * top, dtype=torch.int32, device=DEV)
        tile_expert = torch.empty(max_tiles, dtype=torch.int32, device=DEV)
        ops.moe_plan(idx, E, rows, row_pair, pair_row, tile_expert)
        flat, pr = idx.cpu().numpy().reshape(-1), pair_row.cpu().numpy()
        assert all((pr[p] < 0) == (flat[p] >= E) for p in range(T * top))          # identity experts' pairs have no row, all others one
        mid = torch.full((max_tiles * rows, ff), float("nan"), dtype=dtype, device=DEV)
        y = torch.full((max_tiles * rows, D), float("nan"), device=DEV)
        if tensor_cores:
            a = torch.full((max_tiles * rows, D), float("nan"), dtype=dtype, device=DEV)
            ops.moe_gather_rows(hd, a, row_pair, top)
            ops.gemm_tc_grouped(a, stack("gate"), mid, tile_expert, err, epilogue=ops.EPI_SWIGLU, w2=stack("up"), glu=glu)
            ops.gemm_tc_grouped(mid, stack("down"), y, tile_expert, err)
        else:
            ops.moe_gate_up(hd, stack("gate"), stack("up"), mid, row_pair, tile_expert, top, glu=glu)
            ops.moe_down(mid, stack("down"), y, row_pair, tile_expert, top)
        x = torch.ones(T, D, device=DEV)
        ops.moe_combine(x, y, wts, pair_row, idx=idx if ident else None, n_real=E, h=hd if ident else None, shared=ys, gate=gate)
        got = x.cpu().numpy() - 1.0
        assert np.abs(got[clear] - want[clear]).max() < tol * max(1.0, np.abs(want).max()), tensor_cores
    assert int(err.item()) == 0
