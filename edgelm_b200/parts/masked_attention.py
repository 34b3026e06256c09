"""Grouped-query attention whose queries see a range of keys, with an optional sink in the softmax.

q, k, v are projections of the mixer's input (one matrix product over the three weights stacked; its float32 sums are
kept), with optional biases on q, k, v and the output projection.  The first `rot_dims` dimensions of every query and key
head are rotated by position * f_i, with neighbouring pairs (2i, 2i + 1) (`rot_pairs` "interleaved") or half-split
pairs (i, i + rot_dims / 2) ("half"); the frequencies are base^(-2i / rot_dims), optionally with the long wavelengths
stretched (`parts.rope.rotary_frequencies`).  score = (q . k) * scale.  The mask (`mask`: {"kind", "size"}):

    causal   position i sees every j <= i
    window   the last `size` keys, its own included
    chunk    the j <= i of its own chunk, floor(i / size) = floor(j / size), counted from the sequence's first position

With `sink` (a tensor's name) the softmax's denominator has one more term exp(sink_h) per query head, which has no key
and no value and is not scaled.  A value head may have another size than a key head.  Angles, scores, the softmax and
the weighted values are float32 in both precisions; keys and values are kept in the compute dtype.

Options, each with its constants in the spec:
    conv      q, k and v each pass a depthwise causal filter over time straight after the projection:
              out_t[c] = sum_j taps[c, j] * in_(t - conv + 1 + j)[c], no bias, inputs from before a sequence's start
              counting as zero; the filter's memory, the previous conv - 1 projected rows, is kept per sequence as state
    qk_norm   {eps}: every query and key head (every map of it) is divided by its root mean square and multiplied by a
              weight of head_dim values that all heads share (`q_norm`, `k_norm`), before the rotation
    diff      {offset, eps}: "differential" attention.  A head has two maps, each with queries and keys of head_dim of its
              own (q and k rows laid out head by head as [map 1, map 2]) and a softmax of its own over the same values.
              With lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + offset (four tensors of head_dim, one number per layer):
              o = a_1 - lambda a_2, divided by its root mean square over the head's values (eps), times (1 - offset)
    head_gate True: one more projection of the mixer's input with one row per query head (`names["gate"]`, no bias); head h's
              output is multiplied by the sigmoid of its number before the output projection.  The rows ride in the stacked
              q, k, v product; the attention kernels multiply before they round.
"""
import torch

from ..config.base import ConfigError
from ..csrc import ops
from . import linear
from .base import KVNeed, NeedSet, Part, StateNeed, as_matrix, as_vector, nbytes
from .registry import register_mixer
from .rope import rotary_frequencies

MASKS = {"causal": ops.MASK_CAUSAL, "window": ops.MASK_WINDOW, "chunk": ops.MASK_CHUNK}


def read_mask(mask, where):
    """(kernel code, size) of a mask spec {"kind", "size"} (None: causal)."""
    if not mask:
        return ops.MASK_CAUSAL, 0
    kind = mask.get("kind", "causal")
    if kind not in MASKS:
        raise ConfigError(f"{where}: a mask of kind '{kind}' is not known ({', '.join(MASKS)})")
    size = int(mask.get("size") or 0)
    if kind != "causal" and size < 1:
        raise ConfigError(f"{where}: a {kind} of {size} positions")
    return MASKS[kind], size


def most_keys(mask, size):
    """The most keys that a token can see under the mask (a bound that does not depend on the step: the choice it
    drives is frozen into a captured graph)."""
    return size if mask != ops.MASK_CAUSAL else 1 << 30


# Steps of one token a sequence: with at least so many query heads to a key head the tiled kernel is used (a tile = one
# token, its rows = the heads that share the key head, so a key row is staged once for all of them), its pages dealt to
# several blocks; with fewer, a block per (token, head) whose warps share the keys.  Where a token may see more than
# SPLIT_KEYS_FROM keys (no mask, or a long one) and the step has too few (token, head) pairs for two blocks an SM, the walk over
# one pair's keys is what the step waits for (8 sequences of 9 heads over 2,048 keys: 72 blocks, 184 us a layer): then a pair's
# keys are dealt to several such blocks and a second launch merges them (8 sequences of 32 heads of one to a key head: 254 ->
# 143 us a layer), or, from SHARED_KEYS_LONG_GROUP heads to a key head on, the tiled kernel with its splits takes the step (9
# heads of 3 to a key head: 72 us a layer against 85 with the pairs' keys dealt out; with one head to a key head it stages
# every key for a tile of one row and loses, 254 against 183 us).
SHARED_KEYS_MIN_GROUP = 8
SPLIT_KEYS_FROM = 1024
MAX_HEAD_SPLITS = 16
BLOCKS_AN_SM = 4        # (8 sequences of 32 heads over 2,048 keys, a decode step: 0.722 ms with 2, 0.703 with 4, 0.717 with 8)
SHARED_KEYS_LONG_GROUP = 3


def head_splits(ctx, n_pairs, mask, mask_size):
    """Blocks that share a (token, head) pair's keys in the block-per-pair kernel: about BLOCKS_AN_SM blocks of four warps an SM."""
    if most_keys(mask, mask_size) <= SPLIT_KEYS_FROM:
        return 1
    return min(MAX_HEAD_SPLITS, max(1, (BLOCKS_AN_SM * ctx.n_sms + n_pairs - 1) // max(1, n_pairs)))
MAX_SPLITS = 32
_ones = {}


def single_token_tiles(ctx):
    """The tiles of a step of one token a sequence, from what the step's metadata holds already: (row of the page table,
    packed row, token count, position) per tile."""
    key = str(ctx.device)
    if key not in _ones or _ones[key].numel() < ctx.n_seqs:
        _ones[key] = torch.ones(max(256, 2 * ctx.n_seqs), dtype=torch.int32, device=ctx.device)
    return ctx.seq_index, ctx.seq_index, _ones[key][:ctx.n_seqs], ctx.tok_pos


def decode_splits(ctx, n_kv_heads, group, mask, mask_size):
    """Blocks that share a token's pages in the tiled kernel: about two blocks an SM, at most a block a page of the mask."""
    tiles = max(1, ctx.n_seqs * n_kv_heads * ((group + 31) // 32))
    splits = min(MAX_SPLITS, max(1, (2 * ctx.n_sms + tiles - 1) // tiles))
    if mask != ops.MASK_CAUSAL:
        splits = min(splits, (mask_size + 63) // 64 + 1)
    return splits


def splits_room(n_seqs, n_heads, dv):
    """Bytes of the splits' partial results for a step of `n_seqs` single tokens (sequences x splits stays under 2 SMs' worth
    of blocks plus the sequences themselves, (token, head) pairs x their splits under BLOCKS_AN_SM SMs' worth plus the pairs; 600 and
    300 cover devices of up to 300 SMs)."""
    return nbytes((((600 + n_seqs) * n_heads + BLOCKS_AN_SM * 300) * (2 + dv),), torch.float32)


@register_mixer("masked_attention")
class MaskedAttention(Part):
    graph_safe = True

    def __init__(self, spec, env):
        self.hidden = spec["hidden_size"]
        self.nh, self.nkv, self.dk = spec["num_heads"], spec["num_kv_heads"], spec["head_dim"]
        self.dv = spec.get("v_head_dim") or self.dk
        self.scale = float(spec["scale"])
        self.rot = int(spec.get("rot_dims") or 0)
        self.interleaved = spec.get("rot_pairs", "half") == "interleaved"
        self.rot_base, self.rot_scaling = float(spec.get("rot_base") or 10000.0), spec.get("rot_scaling")
        self.bias = bool(spec.get("bias", False))
        self.out_bias = bool(spec.get("output_bias", self.bias))
        self.taps = int(spec.get("conv") or 0)                    # 0: no convolution
        self.qk_norm, self.diff = spec.get("qk_norm"), spec.get("diff")
        self.head_gate = bool(spec.get("head_gate", False))
        self.maps = 2 if self.diff else 1
        self.names = dict(spec["names"])
        self.dtype = env.dtype
        if self.nh <= 0 or self.nkv <= 0 or self.nh % self.nkv:
            raise ConfigError(f"masked_attention: {self.nh} query heads are not a multiple of {self.nkv} key/value heads")
        if not (1 <= self.dk * self.maps <= 1024 and 1 <= self.dv <= 512):
            raise ConfigError(f"masked_attention: head sizes {self.dk} / {self.dv} are not taken (key rows to 1024, values to 512)")
        if self.diff and "sink" in self.names:
            raise ConfigError("masked_attention: differential maps take no sink")
        if self.diff and self.head_gate:
            raise ConfigError("masked_attention: differential maps take no gate per head")
        if self.rot % 2 or not 0 <= self.rot <= self.dk:
            raise ConfigError(f"masked_attention: {self.rot} rotated dimensions of a head of {self.dk}")
        self.mask, self.mask_size = read_mask(spec.get("mask"), "masked_attention")
        self.kw = self.dk * self.maps                                # what a head's queries and a key row hold
        self.d_qkv = (self.nh + self.nkv) * self.kw + self.nkv * self.dv
        self.d_in = self.d_qkv + (self.nh if self.head_gate else 0)     # columns of the stacked product: q | k | v | gate
        self.tile_tokens = max(1, 32 // (self.nh // self.nkv))
        self.freq = self.b_qkv = self.b_o = self.sink = self.conv_w = self.q_norm = self.k_norm = self.no_tail = None
        self.lam = 0.0
        self.out_scale = 1.0

    def input_weight(self, view=None):
        """The weight of this mixer's one product of its input (q | k | v | gate rows); with `view`, keep that tensor instead (a
        slice of a stack that the caller multiplies once for several mixers, handing the result's columns in as `pre`)."""
        if view is not None:
            self.w_qkv = view
        return self.w_qkv

    def input_weight_rows(self):
        return self.d_in

    def fold_out_scale(self, scale, ask=False):
        """Multiply this mixer's output by `scale` from now on (before its weights are loaded), if that costs nothing: the output
        is linear in the values, and with a convolution on them the values' taps take the constant.  False: it cannot."""
        can = self.taps > 0 and not self.diff and not self.out_bias
        if can and not ask:
            self.out_scale = float(scale)
        return can

    def _on_tensor_cores(self):
        """Whether prompt steps take the tensor-core kernel with float32 scores and weights (three bfloat16 terms for each
        float32 operand): a causal mask, no sink, one map a head, a bfloat16 cache, key = value head sizes that it takes."""
        return (self.mask == ops.MASK_CAUSAL and self.maps == 1 and "sink" not in self.names and
                ops.attn_prefill_split_takes(self.dtype, self.dk, self.dv))

    def tile_sizes(self):
        return (self.tile_tokens, ops.SPLIT_PREFILL_TILE) if self._on_tensor_cores() else (self.tile_tokens,)

    def sizes(self):
        out = {"heads": self.nh, "kv_heads": self.nkv, "head_dim": self.dk, "v_head_dim": self.dv, "rot_dims": self.rot,
               "mask": {v: k for k, v in MASKS.items()}[self.mask], "mask_size": self.mask_size, "sink": "sink" in self.names}
        if self.taps:
            out["conv_taps"] = self.taps
        if self.diff:
            out["diff_offset"] = float(self.diff["offset"])
        if self.qk_norm:
            out["qk_norm"] = True
        if self.head_gate:
            out["head_gate"] = True
        return out

    def flops(self, n_tokens, attended):
        proj = 2.0 * n_tokens * self.hidden * (self.d_in + self.nh * self.dv)
        if self.mask != ops.MASK_CAUSAL:
            attended = min(attended, n_tokens * self.mask_size)
        return proj + 2.0 * attended * self.nh * self.maps * (self.dk + self.dv)

    def weight_shapes(self, prefix):
        n = self.names
        rows = {"q": self.nh * self.kw, "k": self.nkv * self.kw, "v": self.nkv * self.dv}
        out = {prefix + n[k]: (r, self.hidden) for k, r in rows.items()}
        out[prefix + n["o"]] = (self.hidden, self.nh * self.dv)
        if self.head_gate:
            out[prefix + n["gate"]] = (self.nh, self.hidden)
        if self.bias:
            out.update({prefix + n[k] + n["bias"]: (r,) for k, r in rows.items()})
        if self.out_bias:
            out[prefix + n["o"] + n["bias"]] = (self.hidden,)
        if "sink" in n:
            out[prefix + n["sink"]] = (self.nh,)
        if self.taps:
            out.update({prefix + n[k] + n["conv"]: (r, self.taps) for k, r in rows.items()})
        if self.qk_norm:
            out.update({prefix + n["q_norm"]: (self.dk,), prefix + n["k_norm"]: (self.dk,)})
        if self.diff:
            out.update({prefix + n[k]: (self.dk,) for k in ("lq1", "lk1", "lq2", "lk2")})
        return out

    def load(self, tensors, prefix, device):
        n = self.names
        stacked = ("q", "k", "v", "gate") if self.head_gate else ("q", "k", "v")
        self.w_qkv = torch.cat([as_matrix(tensors[prefix + n[k]], self.dtype, device) for k in stacked], dim=0).contiguous()
        self.w_o = as_matrix(tensors[prefix + n["o"]], self.dtype, device)
        if self.bias:
            self.b_qkv = torch.cat([as_vector(tensors[prefix + n[k] + n["bias"]], device) for k in ("q", "k", "v")]).contiguous()
        if self.out_bias:
            self.b_o = as_vector(tensors[prefix + n["o"] + n["bias"]], device)
        if self.taps:
            self.conv_w = torch.cat([as_matrix(tensors[prefix + n[k] + n["conv"]], torch.float32, device) for k in ("q", "k", "v")], dim=0).contiguous()
            self.no_tail = torch.zeros((1, 0, self.d_qkv), dtype=torch.float32, device=device)      # (one tap: no earlier row is kept)
            if self.out_scale != 1.0:
                self.conv_w[(self.nh + self.nkv) * self.kw:] *= self.out_scale
        if self.qk_norm:
            self.q_norm, self.k_norm = as_vector(tensors[prefix + n["q_norm"]], device), as_vector(tensors[prefix + n["k_norm"]], device)
        if self.diff:
            l = {k: tensors[prefix + n[k]].to(torch.float64) for k in ("lq1", "lk1", "lq2", "lk2")}
            self.lam = float(torch.exp((l["lq1"] * l["lk1"]).sum()) - torch.exp((l["lq2"] * l["lk2"]).sum())) + float(self.diff["offset"])
        if "sink" in n:
            self.sink = as_vector(tensors[prefix + n["sink"]], device)
        if self.rot:
            self.freq = rotary_frequencies(self.rot, self.rot_base, self.rot_scaling).to(device).contiguous()

    def first_weights(self):
        return (self.w_qkv,)

    def cache_need(self):
        # (a window's pages could be given back as the sequence moves on, `KVNeed.window`; the kernels here read through
        # the whole table, so every page is kept)
        kv = KVNeed(self.nkv, self.kw, None, v_head_dim=self.dv)
        if self.taps > 1:
            return NeedSet.of(kv=kv, conv=StateNeed((self.taps - 1, self.d_qkv)))
        return kv

    def workspace_bytes(self, n_tokens, n_seqs):
        f32 = torch.float32
        return (nbytes((n_tokens, self.d_in), f32) + nbytes((n_tokens, self.nh * self.kw), f32) +
                nbytes((n_tokens, self.nh * self.maps * self.dv), f32 if self.diff else self.dtype) +
                (nbytes((n_tokens, self.nh * self.dv), self.dtype) if self.diff else 0) + nbytes((n_tokens, self.hidden), self.dtype) +
                splits_room(n_seqs, self.nh * self.maps, self.dv))

    def forward(self, ctx, h, x, cache, accumulate=True, pre=None):
        h = linear.as_tensor(h)
        T, ws = h.shape[0], ctx.ws
        if pre is not None:
            u = pre           # (float32 rows [T, d_in] of any pitch: the product is done)
        else:
            u = ws.alloc((T, self.d_in), torch.float32)
            with ctx.prof("qkv_proj"):
                linear.matmul(ctx, h, self.w_qkv, u, prefetch=(self.w_o,))
        qkv = u[:, :self.d_qkv]
        gate = u[:, self.d_qkv:] if self.head_gate else None
        bias = self.b_qkv
        conv = None
        if self.taps:       # (the filter over time runs inside the kernel that norms, rotates and appends)
            conv = cache.get("conv") if self.taps > 1 else None
            cache = cache["kv"] if self.taps > 1 else cache
        q = ws.alloc((T, self.nh * self.kw), torch.float32)
        table = ctx.page_table(cache.group)
        with ctx.prof("rotate_append"):
            ops.rotate_append(qkv, bias, q, ctx.tok_pos, ctx.tok_seq, table, cache.k, cache.v, self.nh, self.nkv, self.kw, self.dv,
                              self.rot, self.interleaved, self.freq, ctx.err, maps=self.maps, q_norm=self.q_norm, k_norm=self.k_norm,
                              eps=float(self.qk_norm["eps"]) if self.qk_norm else 0.0,
                              conv_w=self.conv_w if self.taps else None, conv_state=conv.state if conv is not None else None,
                              seq_tok0=ctx.seq_tok0 if self.taps else None, seq_slot=ctx.seq_slots if self.taps else None, n_seqs=ctx.n_seqs)
        a = ws.alloc((T, self.nh * self.maps * self.dv), torch.float32 if self.diff else self.dtype)
        with ctx.prof("attn_masked"):
            pairs = T * self.nh * self.maps
            long_and_few = ctx.all_single and most_keys(self.mask, self.mask_size) > SPLIT_KEYS_FROM and pairs < 2 * ctx.n_sms
            if ctx.all_single and (self.nh // self.nkv >= SHARED_KEYS_MIN_GROUP or (long_and_few and self.nh // self.nkv >= SHARED_KEYS_LONG_GROUP)):
                splits = decode_splits(ctx, self.nkv * self.maps, self.nh // self.nkv, self.mask, self.mask_size)
                part = ws.alloc((T * self.nh * self.maps * splits * (2 + self.dv),), torch.float32) if splits > 1 else None
                tseq, ttok0, tntok, tpos0 = single_token_tiles(ctx)
                ops.masked_attn_tiled(q, a, cache.k, cache.v, table, tseq, ttok0, tntok, tpos0, T, 1, self.nh, self.nkv, self.dk, self.dv,
                                      self.scale, self.mask, self.mask_size, self.sink, n_splits=splits, part=part, maps=self.maps, gate=gate)
            elif ctx.all_single:
                splits = head_splits(ctx, T * self.nh * self.maps, self.mask, self.mask_size)
                part = ws.alloc((T * self.nh * self.maps * splits * (2 + self.dv),), torch.float32) if splits > 1 else None
                ops.masked_attn(q, a, cache.k, cache.v, ctx.tok_pos, ctx.tok_seq, table, self.nh, self.nkv, self.dk, self.dv, self.scale,
                                self.mask, self.mask_size, self.sink, most_keys(self.mask, self.mask_size), maps=self.maps, gate=gate,
                                n_splits=splits, part=part)
            elif self._on_tensor_cores():
                tiles = ctx.tiles(ops.SPLIT_PREFILL_TILE)
                ops.attn_prefill_split(q, a, cache.k, cache.v, table, tiles.seq, tiles.tok0, tiles.ntok, tiles.pos0, tiles.count, self.nh, self.nkv,
                                       self.dk, self.scale, gate=gate, max_keys=max(p + n for p, n in zip(ctx.seq_first_positions, ctx.seq_lengths)))
            else:
                tiles = ctx.tiles(self.tile_tokens)
                ops.masked_attn_tiled(q, a, cache.k, cache.v, table, tiles.seq, tiles.tok0, tiles.ntok, tiles.pos0, tiles.count,
                                      self.tile_tokens, self.nh, self.nkv, self.dk, self.dv, self.scale, self.mask, self.mask_size, self.sink,
                                      maps=self.maps, gate=gate)
        if self.diff:
            o = ws.alloc((T, self.nh * self.dv), self.dtype)
            with ctx.prof("diff_combine"):
                ops.diff_combine(a.view(T, self.nh, 2, self.dv), o, self.lam, float(self.diff["eps"]), 1.0 - float(self.diff["offset"]))
            a = o
        with ctx.prof("o_proj"):
            linear.matmul(ctx, a, self.w_o, x, epilogue=linear.EPI_RESIDUAL if accumulate else linear.EPI_STORE,
                          residual=x if accumulate else None, prefetch=ctx.weights_after)
            if self.b_o is not None:
                ops.add_row_bias(x, self.b_o)
