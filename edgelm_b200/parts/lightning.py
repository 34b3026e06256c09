"""Linear attention with a constant decay per head ("lightning attention"), a recurrent mixer with a matrix-valued state.

q = act(W_q h) and k = act(W_k h) (`heads` heads of `head_dim`), v = act(W_v h) (`heads` heads of `v_head_dim`), laid out head by
head, act = silu (`activation` "silu") or nothing ("none").  Per head, with the head's constant `decay`:

    S_t = decay S_(t-1) + k_t v_t^T;   o_t = S_t^T q_t          (S is head_dim x v_head_dim, zero at the start; no other scale)

so the read-out sees the token's own write.  The heads side by side are divided by their common root mean square (`eps`
inside the root) and multiplied by a weight (`names["norm"]`), then by sigmoid(W_g h), and projected back.  A sequence's state
is S per head.  The recurrence, its state and the norm are float32 in both precisions; the projections run in the compute
dtype and their float32 sums are kept (one stacked product: q | k | v | gate).

Steps of one token a sequence (and head sizes over 128) walk the tokens in order (`decay_scan`); prompt steps run the same
recurrence chunk by chunk (`decay_chunked`: a chunk's own tokens as a small masked attention with the decay's powers as
weights, what came before through the state at the chunk's start), which keeps the whole device busy where the walk has one
warp per value channel.
"""
import torch

from ..config.base import ConfigError
from ..csrc import ops
from . import linear
from .base import Part, StateNeed, as_matrix, as_vector, nbytes
from .registry import register_mixer


@register_mixer("decay_linear_attention")
class DecayLinearAttention(Part):
    graph_safe = True

    def __init__(self, spec, env):
        self.hidden = spec["hidden_size"]
        self.heads, self.d = spec["heads"], spec["head_dim"]
        self.e = spec.get("v_head_dim") or self.d
        self.eps = float(spec["eps"])
        self.act = spec.get("activation", "silu")
        self.decay_values = tuple(float(a) for a in spec["decay"])
        self.names = dict(spec["names"])
        self.dtype = env.dtype
        if self.heads < 1 or not 1 <= self.d <= 256 or self.e < 1:
            raise ConfigError(f"decay_linear_attention: {self.heads} heads of {self.d} x {self.e} are not taken (key size up to 256)")
        if len(self.decay_values) != self.heads or not all(0.0 <= a <= 1.0 for a in self.decay_values):
            raise ConfigError(f"decay_linear_attention: {len(self.decay_values)} decays for {self.heads} heads (one in [0, 1] each)")
        if self.act not in ("silu", "none"):
            raise ConfigError(f"decay_linear_attention: activation '{self.act}' is not known (silu, none)")
        self.out_scale = 1.0
        self.qk, self.inner = self.heads * self.d, self.heads * self.e
        self.k_off, self.v_off, self.g_off = self.qk, 2 * self.qk, 2 * self.qk + self.inner
        self.d_in = 2 * self.qk + 2 * self.inner            # q | k | v | gate

    def sizes(self):
        return {"linear_heads": self.heads, "linear_head_dim": self.d, "linear_v_head_dim": self.e, "decay": list(self.decay_values)}

    def flops(self, n_tokens, attended):
        return 2.0 * n_tokens * self.hidden * (self.d_in + self.inner) + 4.0 * n_tokens * self.inner * self.d

    def weight_shapes(self, prefix):
        n = self.names
        return {prefix + n["q"]: (self.qk, self.hidden), prefix + n["k"]: (self.qk, self.hidden), prefix + n["v"]: (self.inner, self.hidden),
                prefix + n["g"]: (self.inner, self.hidden), prefix + n["norm"]: (self.inner,), prefix + n["o"]: (self.hidden, self.inner)}

    def load(self, tensors, prefix, device):
        n = self.names
        self.w_in = torch.cat([as_matrix(tensors[prefix + n[k]], self.dtype, device) for k in ("q", "k", "v", "g")], dim=0).contiguous()
        self.norm_w = as_vector(tensors[prefix + n["norm"]], device)
        if self.out_scale != 1.0:
            self.norm_w = (self.norm_w * self.out_scale).contiguous()
        self.w_o = as_matrix(tensors[prefix + n["o"]], self.dtype, device)
        self.decay = torch.tensor(self.decay_values, dtype=torch.float64).to(device=device, dtype=torch.float32).contiguous()
        self.powers = ops.decay_powers(self.decay_values).to(device)

    def first_weights(self):
        return (self.w_in,)

    def input_weight(self, view=None):
        """The weight of this mixer's one product of its input (q | k | v | gate rows); with `view`, keep that tensor instead (a
        slice of a stack that the caller multiplies once for several mixers, handing the result's columns in as `pre`)."""
        if view is not None:
            self.w_in = view
        return self.w_in

    def input_weight_rows(self):
        return self.d_in

    def fold_out_scale(self, scale, ask=False):
        """Multiply this mixer's output by `scale` from now on (before its weights are loaded): the norm's weight takes it."""
        if not ask:
            self.out_scale = float(scale)
        return True

    def _chunked(self):
        return ops.decay_chunked_takes(self.d, self.e)

    def tile_sizes(self):
        return (ops.DECAY_CHUNK,) if self._chunked() else ()

    def cache_need(self):
        return StateNeed((self.heads, self.e, self.d))

    def workspace_bytes(self, n_tokens, n_seqs):
        f32 = torch.float32
        chunks = n_tokens // ops.DECAY_CHUNK + n_seqs
        return (nbytes((n_tokens, self.d_in), f32) + nbytes((n_tokens, self.inner), f32) + nbytes((n_tokens, self.inner), self.dtype) +
                nbytes((n_tokens, self.hidden), self.dtype) +
                (nbytes((ops.decay_chunked_scratch_floats(chunks, self.heads, self.d, self.e),), f32) if self._chunked() else 0))

    def forward(self, ctx, h, x, cache, accumulate=True, pre=None):
        h = linear.as_tensor(h)
        T, ws, f32 = h.shape[0], ctx.ws, torch.float32
        if pre is not None:
            u = pre           # (float32 rows [T, d_in] of any pitch: the product is done)
        else:
            u = ws.alloc((T, self.d_in), f32)
            with ctx.prof("linear_attn_in_proj"):
                linear.matmul(ctx, h, self.w_in, u, prefetch=(self.w_o,))
        o = ws.alloc((T, self.inner), f32)
        if not ctx.all_single and T >= 8 * ctx.n_seqs and self._chunked():
            tiles = ctx.tiles(ops.DECAY_CHUNK)
            scratch = ws.alloc((ops.decay_chunked_scratch_floats(tiles.count, self.heads, self.d, self.e),), f32)
            with ctx.prof("linear_attn_chunks"):
                ops.decay_chunked(u, 0, self.k_off, self.v_off, self.powers, cache.state, o, ctx.seq_tok0, ctx.seq_slots, ctx.n_seqs,
                                  tiles.tok0, tiles.ntok, tiles.count, self.heads, self.d, self.e,
                                  act="silu" if self.act == "silu" else None, scratch=scratch)
        else:
            in_scan = ctx.all_single         # one token a sequence: the activation inside the walk saves its launch
            if self.act == "silu" and not in_scan:
                with ctx.prof("linear_attn_act"):
                    ops.silu_columns(u, 0, self.g_off)
            with ctx.prof("linear_attn_scan"):
                ops.decay_scan(u, 0, self.k_off, self.v_off, self.decay, cache.state, o, ctx.seq_tok0, ctx.seq_slots, ctx.n_seqs,
                               self.heads, self.d, self.e, act="silu" if self.act == "silu" and in_scan else None)
        on = ws.alloc((T, self.inner), self.dtype)
        with ctx.prof("linear_attn_gate_norm"):
            ops.gated_group_norm(o, u[:, self.g_off:], self.norm_w, on, 1, self.eps, gate_first=False, gate_act="sigmoid")
        with ctx.prof("linear_attn_out_proj"):
            linear.matmul(ctx, on, self.w_o, x, epilogue=linear.EPI_RESIDUAL if accumulate else linear.EPI_STORE,
                          residual=x if accumulate else None, prefetch=ctx.weights_after)
