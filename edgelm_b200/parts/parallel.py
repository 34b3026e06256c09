"""Two mixers side by side on the same input: x (+)= left_scale * left(h) + right_scale * right(h).  Each keeps what it
keeps (the layer run's cache entry answers `entry["left"]` and `entry["right"]`)."""
import torch

from ..csrc import ops
from .base import NeedSet, Part, nbytes
from .registry import register_mixer


@register_mixer("parallel")
class ParallelMixers(Part):
    def __init__(self, spec, env):
        self.hidden = spec["hidden_size"]
        self.left, self.right = env.build("mixer", spec["left"]), env.build("mixer", spec["right"])
        self.left_scale, self.right_scale = float(spec["left_scale"]), float(spec["right_scale"])
        self.dtype = env.dtype
        self.parts = (self.left, self.right)
        # a mixer that can multiply its own output by a constant at no cost (in a weight it applies anyway) is asked to: when
        # both can, each adds into x through its last product's epilogue and the scaled sum needs no kernel
        self.folded = all(hasattr(p, "fold_out_scale") for p in self.parts) and \
            self.left.fold_out_scale(self.left_scale, ask=True) and self.right.fold_out_scale(self.right_scale, ask=True)
        if self.folded:
            self.left.fold_out_scale(self.left_scale)
            self.right.fold_out_scale(self.right_scale)
        # mixers that start with one matrix product of their input into float32 rows (`input_weight`) share one product over
        # their weights stacked, the right mixer's first (its kernels read 16 bytes at a time where rows start on such a boundary)
        self.stacked = all(hasattr(p, "input_weight") for p in self.parts)
        self.w_in = None

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts)

    def sizes(self):
        out = {"left_scale": self.left_scale, "right_scale": self.right_scale}
        for p in self.parts:
            out.update(p.sizes())
        return out

    def describe(self):
        return f"parallel({self.left_scale} * {self.left.describe()} + {self.right_scale} * {self.right.describe()})"

    def flops(self, n_tokens, attended):
        return sum(p.flops(n_tokens, attended) for p in self.parts)

    def weight_shapes(self, prefix):
        out = {}
        for p in self.parts:
            out.update(p.weight_shapes(prefix))
        return out

    def load(self, tensors, prefix, device):
        for p in self.parts:
            p.load(tensors, prefix, device)
        if self.stacked:
            wr, wl = self.right.input_weight(), self.left.input_weight()
            self.w_in = torch.cat([wr, wl], dim=0).contiguous()
            self.n_right = wr.shape[0]
            self.right.input_weight(self.w_in[:self.n_right])       # (the mixers keep views: the stacked copy is the only one)
            self.left.input_weight(self.w_in[self.n_right:])

    def first_weights(self):
        return (self.w_in,) if self.stacked else self.left.first_weights()

    def tile_sizes(self):
        return tuple(self.left.tile_sizes()) + tuple(self.right.tile_sizes())

    def cache_need(self):
        return NeedSet.of(left=self.left.cache_need(), right=self.right.cache_need())

    def workspace_bytes(self, n_tokens, n_seqs):
        both = nbytes((n_tokens, sum(p.input_weight_rows() for p in self.parts) + 8), torch.float32) if self.stacked else 0
        return 2 * nbytes((n_tokens, self.hidden), torch.float32) + both + max(p.workspace_bytes(n_tokens, n_seqs) for p in self.parts)

    def forward(self, ctx, h, x, cache, accumulate=True):
        from . import linear
        h = linear.as_tensor(h)
        T, ws = h.shape[0], ctx.ws
        pre_l = pre_r = None
        if self.stacked:
            n = self.w_in.shape[0]
            u = ws.alloc((T, (n + 7) // 8 * 8), torch.float32)[:, :n]      # (rows on 16-byte boundaries, whatever the mixers' widths add up to)
            with ctx.prof("mixers_in_proj"):
                linear.matmul(ctx, h, self.w_in, u)
            pre_r, pre_l = u[:, :self.n_right], u[:, self.n_right:]
        kw_l = {"pre": pre_l} if self.stacked else {}
        kw_r = {"pre": pre_r} if self.stacked else {}
        if self.folded:
            # the mixers scale their own outputs: the left one stores or adds as the caller asks, the right one adds to that
            after = ctx.weights_after
            ctx.weights_after = () if self.stacked else self.right.first_weights()
            with ws.frame():
                self.left.forward(ctx, h, x, cache.get("left"), accumulate=accumulate, **kw_l)
            ctx.weights_after = after
            with ws.frame():
                self.right.forward(ctx, h, x, cache.get("right"), accumulate=True, **kw_r)
            return
        y1 = ws.alloc((T, self.hidden), torch.float32)
        y2 = ws.alloc((T, self.hidden), torch.float32)
        after = ctx.weights_after
        ctx.weights_after = self.right.first_weights()
        with ws.frame():
            self.left.forward(ctx, h, y1, cache.get("left"), accumulate=False, **kw_l)
        ctx.weights_after = after
        with ws.frame():
            self.right.forward(ctx, h, y2, cache.get("right"), accumulate=False, **kw_r)
        with ctx.prof("parallel_sum"):
            ops.scaled_sum(y1, self.left_scale, y2, self.right_scale, x, add=accumulate)
