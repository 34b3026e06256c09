"""Arrangements of one layer's parts.  "prenorm": x += mixer(norm1(x)); x += ffn(norm2(x))
(adarsh-sgh/edgelm tools/elm.py:122-153); a layer may have no feed-forward.  "sublayer_norm": x += norm1(mixer(x)); x += norm2(ffn(x)), with an
optional blend of the mixer's input with the previous token's.  "parallel_prenorm": x += mixer(norm1(x)) + ffn(norm2(x)), both
sublayers reading the same x.  "hyper": the pre-norm arrangement over several copies of the
residual stream, which every sublayer reads through learned weights and rewrites through a learned matrix."""
import torch

from ..config.base import ConfigError
from ..csrc import ops
from . import linear
from .base import NeedSet, Part, StateNeed, as_vector, nbytes
from .registry import register_block


@register_block("prenorm")
class PreNormBlock(Part):
    def __init__(self, layer_spec, env):
        self.prefix = layer_spec.prefix
        self.dtype = env.dtype
        self.mixer_norm = env.build("norm", layer_spec.mixer_norm)
        self.mixer = env.build("mixer", layer_spec.mixer)
        self.ffn_norm = env.build("norm", layer_spec.ffn_norm) if layer_spec.ffn is not None else None
        self.ffn = env.build("ffn", layer_spec.ffn) if layer_spec.ffn is not None else None
        self.parts = tuple(p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None)
        self.hidden = layer_spec.mixer_norm["dim"]

    def weight_shapes(self, prefix=None):
        out = {}
        for p in self.parts:
            out.update(p.weight_shapes(self.prefix))
        return out

    def load(self, tensors, prefix, device):
        for p in self.parts:
            p.load(tensors, self.prefix, device)

    def cache_need(self):
        return self.mixer.cache_need()

    def sizes(self):
        out = {}
        for p in (self.mixer, self.ffn, self.mixer_norm):
            if p is not None:
                out.update(p.sizes())
        return out

    def flops(self, n_tokens, attended):
        return sum(p.flops(n_tokens, attended) for p in self.parts)

    def describe(self):
        ffn = f"; {self.ffn_norm.describe()} -> {self.ffn.describe()}" if self.ffn is not None else ""
        return f"{self.kind}: {self.mixer_norm.describe()} -> {self.mixer.describe()}{ffn}"

    def tile_sizes(self):
        return tuple(self.mixer.tile_sizes())

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts)

    def workspace_bytes(self, n_tokens, n_seqs):
        return nbytes((n_tokens, self.hidden), self.dtype) + max(self.mixer.workspace_bytes(n_tokens, n_seqs),
                                                                  self.ffn.workspace_bytes(n_tokens, n_seqs) if self.ffn is not None else 0)

    def _normed(self, ctx, x, norm, part):
        """The part's input: lazily normalised if both the norm and the part can work that way
        (the part's first matrix product then computes the norm itself when the step is small)."""
        if getattr(part, "takes_normed_input", False) and getattr(norm, "fusable", False):
            return linear.NormedInput(ctx, x, norm, self.dtype)
        h = ctx.ws.alloc((x.shape[0], self.hidden), self.dtype)
        with ctx.prof("norm"):
            norm.forward(ctx, x, h)
        return h

    def first_weights(self):
        return self.mixer.first_weights()

    def forward(self, ctx, x, cache):
        # `ctx.weights_after`: what the step reads once the running part is done (a part's last product may start
        # it on its way into L2): after the mixer the feed-forward's first weights, after that whatever the caller
        # named as coming after this layer
        after_layer = ctx.weights_after
        if self.ffn is not None:
            ctx.weights_after = self.ffn.first_weights()
        with ctx.ws.frame():
            self.mixer.forward(ctx, self._normed(ctx, x, self.mixer_norm, self.mixer), x, cache)
        ctx.weights_after = after_layer
        if self.ffn is not None:
            with ctx.ws.frame():
                self.ffn.forward(ctx, self._normed(ctx, x, self.ffn_norm, self.ffn), x)


@register_block("parallel_prenorm")
class ParallelPreNormBlock(PreNormBlock):
    """Both sublayers read the same x: x += mixer(norm1(x)) + ffn(norm2(x)); a layer may have no feed-forward.  The two
    norms divide by the same root mean square, so one kernel computes it once and writes both inputs (`rmsnorm_pair`); the
    sublayers then add into x one after the other (their residual sums stay the epilogues of their last products).  Rows that
    the model hands in as `ctx.rows_to_add` join x in that same first pass."""
    takes_added_rows = True

    def __init__(self, layer_spec, env):
        super().__init__(layer_spec, env)
        for n in (self.mixer_norm, self.ffn_norm):
            if n is not None and not (getattr(n, "fusable", False) and n.eps == self.mixer_norm.eps):
                raise ConfigError(f"block 'parallel_prenorm': the norm '{n.kind}' is not one that the paired kernel computes (weight, one eps)")

        self.unused_norm = layer_spec.options.get("unused_norm") if self.ffn is None else None

    def ignorable(self):
        """A layer without a feed-forward may still come with its second norm's weight in the files."""
        return (self.prefix + self.unused_norm,) if self.unused_norm else ()

    def workspace_bytes(self, n_tokens, n_seqs):
        inner = max(self.mixer.workspace_bytes(n_tokens, n_seqs), self.ffn.workspace_bytes(n_tokens, n_seqs) if self.ffn is not None else 0)
        return 2 * nbytes((n_tokens, self.hidden), self.dtype) + inner

    def describe(self):
        ffn = f" + {self.ffn_norm.describe()} -> {self.ffn.describe()}" if self.ffn is not None else ""
        return f"{self.kind}: x += {self.mixer_norm.describe()} -> {self.mixer.describe()}{ffn}"

    def forward(self, ctx, x, cache):
        T, ws = x.shape[0], ctx.ws
        after_layer = ctx.weights_after
        add, ctx.rows_to_add = ctx.rows_to_add, None
        with ws.frame():
            h1 = ws.alloc((T, self.hidden), self.dtype)
            h2 = ws.alloc((T, self.hidden), self.dtype) if self.ffn is not None else None
            with ctx.prof("norm_pair"):
                ops.rmsnorm_pair(x, self.mixer_norm.weight, self.mixer_norm.eps, h1, self.ffn_norm.weight if self.ffn is not None else None, h2, add=add)
            if self.ffn is not None:
                ctx.weights_after = self.ffn.first_weights()
            with ws.frame():
                self.mixer.forward(ctx, h1, x, cache)
            ctx.weights_after = after_layer
            if self.ffn is not None:
                with ws.frame():
                    self.ffn.forward(ctx, h2, x)


@register_block("sublayer_norm")
class SublayerNormBlock(Part):
    """The norm on each sublayer's OUTPUT: x += norm1(mixer(h)); x += norm2(ffn(x)), the sublayers reading the
    residual stream itself.  With the option `shift` (a tensor's name) the mixer's input is first blended with the
    previous token's: h_t = x_t + (x_(t-1) - x_t) * shift, element by element, with zeros before a sequence's first
    token; the last x of every sequence is then part of its state (a float32 row of its own beside the mixer's).
    A layer may have no feed-forward.  Mixers and feed-forwards are asked to STORE their output (`accumulate=False`):
    the residual sum is the norm kernel's, which also hands the feed-forward its input in the compute dtype."""

    def __init__(self, layer_spec, env):
        self.prefix = layer_spec.prefix
        self.dtype = env.dtype
        self.mixer_norm = env.build("norm", layer_spec.mixer_norm)
        self.mixer = env.build("mixer", layer_spec.mixer)
        self.ffn = env.build("ffn", layer_spec.ffn) if layer_spec.ffn is not None else None
        self.ffn_norm = env.build("norm", layer_spec.ffn_norm) if layer_spec.ffn is not None else None
        for n in (self.mixer_norm, self.ffn_norm):
            if n is not None and not hasattr(n, "add_normed"):
                raise ConfigError(f"block 'sublayer_norm': the norm '{n.kind}' cannot be applied to a sublayer's output (no add_normed)")
        self.parts = tuple(p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None)
        self.hidden = layer_spec.mixer_norm["dim"]
        self.shift_name = layer_spec.options.get("shift")
        self.shift = None

    def weight_shapes(self, prefix=None):
        out = {}
        for p in self.parts:
            out.update(p.weight_shapes(self.prefix))
        if self.shift_name:
            out[self.prefix + self.shift_name] = (self.hidden,)
        return out

    def load(self, tensors, prefix, device):
        for p in self.parts:
            p.load(tensors, self.prefix, device)
        if self.shift_name:
            self.shift = as_vector(tensors[self.prefix + self.shift_name], device).view(1, self.hidden)

    def cache_need(self):
        return NeedSet.of(shift=StateNeed((self.hidden,)) if self.shift_name else None, mixer=self.mixer.cache_need())

    def sizes(self):
        out = {}
        for p in (self.mixer, self.ffn, self.mixer_norm):
            if p is not None:
                out.update(p.sizes())
        out["token_shift"] = bool(self.shift_name)
        return out

    def flops(self, n_tokens, attended):
        return sum(p.flops(n_tokens, attended) for p in self.parts)

    def describe(self):
        ffn = f"; x += {self.ffn_norm.describe()}({self.ffn.describe()})" if self.ffn is not None else ""
        return f"{self.kind}{' with token shift' if self.shift_name else ''}: x += {self.mixer_norm.describe()}({self.mixer.describe()}){ffn}"

    def tile_sizes(self):
        return tuple(self.mixer.tile_sizes())

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts)

    def workspace_bytes(self, n_tokens, n_seqs):
        inner = max(self.mixer.workspace_bytes(n_tokens, n_seqs), self.ffn.workspace_bytes(n_tokens, n_seqs) if self.ffn is not None else 0)
        return nbytes((n_tokens, self.hidden), self.dtype) + nbytes((n_tokens, self.hidden), torch.float32) + inner

    def first_weights(self):
        return self.mixer.first_weights()

    def forward(self, ctx, x, cache):
        T, ws = x.shape[0], ctx.ws
        after_layer = ctx.weights_after
        with ws.frame():
            h = ws.alloc((T, self.hidden), self.dtype)      # the mixer's input; later the feed-forward's
            y = ws.alloc((T, self.hidden), torch.float32)   # a sublayer's output before its norm
            if self.shift is not None:
                state = cache["shift"].state
                with ctx.prof("token_shift"):
                    ops.shift_mix(x, state, self.shift, h.view(1, T, self.hidden), ctx.tok_seq, ctx.seq_tok0, ctx.seq_slots, move_state=True)
                mixer_in = h
            elif self.dtype == torch.float32:
                mixer_in = x
            else:
                h.copy_(x)
                mixer_in = h
            ctx.weights_after = self.ffn.first_weights() if self.ffn is not None else after_layer
            with ws.frame():
                self.mixer.forward(ctx, mixer_in, y, cache.get("mixer"), accumulate=False)
            ctx.weights_after = after_layer
            feeds = self.ffn is not None and self.dtype != torch.float32
            with ctx.prof("norm_residual"):
                self.mixer_norm.add_normed(ctx, x, y, cast=h if feeds else None)
            if self.ffn is not None:
                with ws.frame():
                    self.ffn.forward(ctx, h if feeds else x, y, accumulate=False)
                with ctx.prof("norm_residual"):
                    self.ffn_norm.add_normed(ctx, x, y)


@register_block("hyper")
class HyperBlock(Part):
    """Pre-norm sublayers over S copies x_1 .. x_S of the residual stream (xs [tokens, S, hidden] float32, all equal at
    the model's start).  For sublayer q (the mixer, then the feed-forward) with its tensors `in` [S], `out` [S] and `mix`
    [S, S] (indexed [from, to]):

        u = sum_s in[s] x_s;   y = sublayer(norm(u));   x'_t = sum_s mix[s, t] x_s + out[t] y     (every x' from the streams as they were)

    One kernel does a write and the read that follows it, also the next layer's (or the sum of the streams after the last
    layer): `ctx.streams_next` names that read, `ctx.streams_h` says that this layer's first read is done already.
    Mixers and feed-forwards STORE their output (`accumulate=False`)."""

    def __init__(self, layer_spec, env):
        self.prefix = layer_spec.prefix
        self.dtype = env.dtype
        self.mixer_norm = env.build("norm", layer_spec.mixer_norm)
        self.mixer = env.build("mixer", layer_spec.mixer)
        self.ffn_norm = env.build("norm", layer_spec.ffn_norm) if layer_spec.ffn is not None else None
        self.ffn = env.build("ffn", layer_spec.ffn) if layer_spec.ffn is not None else None
        for n in (self.mixer_norm, self.ffn_norm):
            if n is not None and not getattr(n, "fusable", False):
                raise ConfigError(f"block 'hyper': the norm '{n.kind}' is not one that the streams' read-out computes (weight, eps)")
        self.parts = tuple(p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None)
        self.hidden = layer_spec.mixer_norm["dim"]
        self.streams = int(layer_spec.options["streams"])
        self.names = dict(layer_spec.options["names"])
        if not 1 <= self.streams <= 8:
            raise ConfigError(f"block 'hyper': {self.streams} residual streams are not taken (1 to 8)")
        self.hc = {}

    def _hc_names(self, q):
        n = self.names
        return {k: self.prefix + n[q] + n[k] for k in ("in", "out", "mix")}

    def weight_shapes(self, prefix=None):
        out, S = {}, self.streams
        for p in self.parts:
            out.update(p.weight_shapes(self.prefix))
        for q in ("mixer", "ffn") if self.ffn is not None else ("mixer",):
            names = self._hc_names(q)
            out.update({names["in"]: (S,), names["out"]: (S,), names["mix"]: (S, S)})
        return out

    def load(self, tensors, prefix, device):
        for p in self.parts:
            p.load(tensors, self.prefix, device)
        for q in ("mixer", "ffn") if self.ffn is not None else ("mixer",):
            self.hc[q] = {k: tensors[name].to(device=device, dtype=torch.float32).contiguous() for k, name in self._hc_names(q).items()}

    def cache_need(self):
        return self.mixer.cache_need()

    def sizes(self):
        out = {"residual_streams": self.streams}
        for p in (self.mixer, self.ffn, self.mixer_norm):
            if p is not None:
                out.update(p.sizes())
        return out

    def flops(self, n_tokens, attended):
        return sum(p.flops(n_tokens, attended) for p in self.parts)

    def describe(self):
        ffn = f"; {self.ffn_norm.describe()} -> {self.ffn.describe()}" if self.ffn is not None else ""
        return f"{self.kind} over {self.streams} streams: {self.mixer_norm.describe()} -> {self.mixer.describe()}{ffn}"

    def tile_sizes(self):
        return tuple(self.mixer.tile_sizes())

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts)

    def workspace_bytes(self, n_tokens, n_seqs):
        inner = max(self.mixer.workspace_bytes(n_tokens, n_seqs), self.ffn.workspace_bytes(n_tokens, n_seqs) if self.ffn is not None else 0)
        return nbytes((n_tokens, self.hidden), self.dtype) + nbytes((n_tokens, self.hidden), torch.float32) + inner

    def first_weights(self):
        return self.mixer.first_weights()

    def first_read(self):
        """(in-weights, norm weight, eps) of the read that this layer starts with: the layer before may do it with its last write."""
        return self.hc["mixer"]["in"], self.mixer_norm.weight, self.mixer_norm.eps

    def forward(self, ctx, xs, cache):
        T, ws = xs.shape[0], ctx.ws
        after_layer = ctx.weights_after
        nxt, ctx.streams_next = getattr(ctx, "streams_next", None), None
        with ws.frame():
            y = ws.alloc((T, self.hidden), torch.float32)      # a sublayer's output
            h = getattr(ctx, "streams_h", None)                # this layer's first read, if the layer before did it
            ctx.streams_h = None
            if h is None:
                h = ws.alloc((T, self.hidden), self.dtype)
                w_in, nw, eps = self.first_read()
                with ctx.prof("streams"):
                    ops.streams_update(xs, w_in=w_in, norm_w=nw, eps=eps, h=h)
            ctx.weights_after = self.ffn.first_weights() if self.ffn is not None else after_layer
            with ws.frame():
                self.mixer.forward(ctx, h, y, cache, accumulate=False)
            ctx.weights_after = after_layer
            last = self.hc["mixer"]
            if self.ffn is not None:
                h2 = ws.alloc((T, self.hidden), self.dtype)
                with ctx.prof("streams"):
                    ops.streams_update(xs, y, last["mix"], last["out"], w_in=self.hc["ffn"]["in"], norm_w=self.ffn_norm.weight,
                                       eps=self.ffn_norm.eps, h=h2)
                with ws.frame():
                    self.ffn.forward(ctx, h2, y, accumulate=False)
                last = self.hc["ffn"]
            with ctx.prof("streams"):
                if nxt is not None:
                    w_in, nw, eps, h_next, is_input = nxt
                    ops.streams_update(xs, y, last["mix"], last["out"], w_in=w_in, norm_w=nw, eps=eps, h=h_next)
                    ctx.streams_h = h_next if is_input else None
                else:
                    ops.streams_update(xs, y, last["mix"], last["out"])
