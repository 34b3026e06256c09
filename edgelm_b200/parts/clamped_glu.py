"""A gated feed-forward with clamped branches: g = min(h Wg^T, limit), v = clamp(h Wu^T, -limit, limit),
x += (g * sigmoid(alpha g) * (v + 1)) Wd^T, no bias.  `limit` and `alpha` are constants of the spec.  Prompt steps in
bfloat16 compute the unit in the epilogue of the tensor-core product of gate and up (two accumulators a tile); other steps
run one matrix product over the two weights stacked, whose float32 sums feed the activation kernel.  Either way the result
(in the compute dtype) is the down projection's input, and the residual sum is the down projection's epilogue."""
import torch

from ..config.base import ConfigError
from ..csrc import ops
from . import linear
from .base import Part, as_matrix, nbytes
from .registry import register_ffn


@register_ffn("clamped_glu")
class ClampedGLU(Part):
    graph_safe = True
    takes_normed_input = True

    def __init__(self, spec, env):
        self.hidden, self.inter = spec["hidden_size"], spec["intermediate_size"]
        self.limit, self.alpha = float(spec["limit"]), float(spec.get("alpha", 1.0))
        self.names = dict(spec["names"])
        self.dtype = env.dtype
        if self.inter < 1 or not self.limit > 0:
            raise ConfigError(f"clamped_glu: {self.inter} inner channels with limit {self.limit}")
        self.w_gu = self.w_down = None

    def sizes(self):
        return {"intermediate": self.inter, "glu_limit": self.limit, "glu_alpha": self.alpha}

    def flops(self, n_tokens, attended):
        return 6.0 * n_tokens * self.hidden * self.inter

    def weight_shapes(self, prefix):
        n = self.names
        return {prefix + n["gate"]: (self.inter, self.hidden), prefix + n["up"]: (self.inter, self.hidden),
                prefix + n["down"]: (self.hidden, self.inter)}

    def load(self, tensors, prefix, device):
        n = self.names
        self.w_gu = torch.cat([as_matrix(tensors[prefix + n[k]], self.dtype, device) for k in ("gate", "up")], dim=0).contiguous()
        self.w_down = as_matrix(tensors[prefix + n["down"]], self.dtype, device)

    def workspace_bytes(self, n_tokens, n_seqs):
        return (nbytes((n_tokens, 2 * self.inter), torch.float32) + nbytes((n_tokens, self.inter), self.dtype) +
                nbytes((n_tokens, self.hidden), self.dtype))

    def first_weights(self):
        return (self.w_gu,)

    def forward(self, ctx, h, x, accumulate=True):
        """x += feed_forward(h); with `accumulate` False, x = feed_forward(h) (float32)."""
        T, F = h.shape[0], self.inter
        mid = ctx.ws.alloc((T, F), self.dtype)
        w_gate, w_up = self.w_gu[:F], self.w_gu[F:]
        if T > linear.FEW_ROWS and self.dtype == torch.bfloat16 and ops.gemm_tc_takes(linear.as_tensor(h), w_gate, mid, w_up):
            # prompt steps in bfloat16: the gate and up products share a tile and the unit is the product's epilogue
            with ctx.prof("gate_up_clamped_glu"):
                ops.gemm_tc(linear.as_tensor(h), w_gate, mid, ctx.err, epilogue=linear.EPI_SWIGLU, w2=w_up, glu=(self.limit, self.alpha, 1.0))
        else:
            gu = ctx.ws.alloc((T, 2 * F), torch.float32)
            with ctx.prof("gate_up"):
                linear.matmul(ctx, h, self.w_gu, gu, prefetch=(self.w_down,))
            with ctx.prof("clamped_glu"):
                ops.clamped_glu(gu, mid, self.limit, self.alpha)
        with ctx.prof("down_proj_residual"):
            linear.matmul(ctx, mid, self.w_down, x, epilogue=linear.EPI_RESIDUAL if accumulate else linear.EPI_STORE,
                          residual=x if accumulate else None, prefetch=ctx.weights_after)
