"""SwiGLU feed-forward: x += (silu(h Wg^T) * (h Wu^T)) Wd^T, silu(z) = z / (1 + exp(-z)), no bias
(adarsh-sgh/edgelm src/kernels_ref.cpp:143-160, tools/elm.py:140-152).  Gate and up never reach
memory: the activation is the epilogue of their matrix product, the residual sum that of the
down projection.  With `bias` (a suffix of the tensors' names) all three projections have biases: x += Wd (silu(Wg h + bg) *
(Wu h + bu)) + bd.  Prompt steps in bfloat16 add the two biases in the same tensor-core epilogue; other steps run gate and up as one
product over the two weights stacked, whose float32 sums feed the gated unit's kernel together with the biases.  The down
projection's bias is added to the residual stream after its product."""
import torch

from ..csrc import ops
from . import linear
from .base import Part, as_matrix, as_vector, nbytes
from .registry import register_ffn


@register_ffn("swiglu")
class SwiGLU(Part):
    graph_safe = True
    takes_normed_input = True

    def __init__(self, spec, env):
        self.hidden, self.inter = spec["hidden_size"], spec["intermediate_size"]
        self.names = dict(spec["names"])
        self.bias = spec.get("bias")            # a suffix, or None
        self.dtype = env.dtype
        self.w_gate = self.w_up = self.w_down = self.w_gu = self.b_gu = self.b_down = None

    def sizes(self):
        return {"intermediate": self.inter, **({"ffn_bias": True} if self.bias else {})}

    def flops(self, n_tokens, attended):
        return 6.0 * n_tokens * self.hidden * self.inter

    def weight_shapes(self, prefix):
        n = self.names
        out = {prefix + n["gate"]: (self.inter, self.hidden), prefix + n["up"]: (self.inter, self.hidden),
               prefix + n["down"]: (self.hidden, self.inter)}
        if self.bias:
            out.update({prefix + n["gate"] + self.bias: (self.inter,), prefix + n["up"] + self.bias: (self.inter,),
                        prefix + n["down"] + self.bias: (self.hidden,)})
        return out

    def load(self, tensors, prefix, device):
        n = self.names
        self.w_down = as_matrix(tensors[prefix + n["down"]], self.dtype, device)
        if self.bias:
            self.w_gu = torch.cat([as_matrix(tensors[prefix + n[k]], self.dtype, device) for k in ("gate", "up")], dim=0).contiguous()
            self.b_gu = torch.cat([as_vector(tensors[prefix + n[k] + self.bias], device) for k in ("gate", "up")]).contiguous()
            self.b_down = as_vector(tensors[prefix + n["down"] + self.bias], device)
        else:
            self.w_gate = as_matrix(tensors[prefix + n["gate"]], self.dtype, device)
            self.w_up = as_matrix(tensors[prefix + n["up"]], self.dtype, device)

    def workspace_bytes(self, n_tokens, n_seqs):
        return (nbytes((n_tokens, self.inter), self.dtype) + nbytes((n_tokens, self.hidden), self.dtype) +
                (nbytes((n_tokens, 2 * self.inter), torch.float32) if self.bias else 0))

    def first_weights(self):
        return (self.w_gu,) if self.bias else (self.w_gate, self.w_up)

    def forward(self, ctx, h, x, accumulate=True):
        """x += feed_forward(h); with `accumulate` False, x = feed_forward(h) (float32), for an arrangement that
        norms the sublayer's output before the residual sum."""
        mid = ctx.ws.alloc((h.shape[0], self.inter), self.dtype)
        T, F = h.shape[0], self.inter
        down_bias_done = False
        w_gate, w_up = (self.w_gu[:F], self.w_gu[F:]) if self.bias else (None, None)
        if self.bias and T > linear.FEW_ROWS and self.dtype == torch.bfloat16 and ops.gemm_tc_takes(linear.as_tensor(h), w_gate, mid, w_up):
            # prompt steps in bfloat16: the two products share a tile, biases and activation are the product's epilogue
            with ctx.prof("gate_up_swiglu"):
                ops.gemm_tc(linear.as_tensor(h), w_gate, mid, ctx.err, epilogue=linear.EPI_SWIGLU, w2=w_up, glu_bias=self.b_gu)
        elif self.bias:
            gu = ctx.ws.alloc((T, 2 * F), torch.float32)
            with ctx.prof("gate_up"):
                linear.matmul(ctx, h, self.w_gu, gu, prefetch=(self.w_down,))
            with ctx.prof("swiglu_bias"):      # (with the residual sum to follow, the down projection's bias joins x here)
                ops.clamped_glu(gu, mid, 0.0, 1.0, shift=0.0, bias=self.b_gu, x=x if accumulate else None, x_bias=self.b_down if accumulate else None)
            down_bias_done = accumulate
        else:
            with ctx.prof("gate_up_swiglu"):
                linear.matmul(ctx, h, self.w_gate, mid, epilogue=linear.EPI_SWIGLU, w2=self.w_up, prefetch=(self.w_down,))
        with ctx.prof("down_proj_residual"):
            linear.matmul(ctx, mid, self.w_down, x, epilogue=linear.EPI_RESIDUAL if accumulate else linear.EPI_STORE,
                          residual=x if accumulate else None, prefetch=ctx.weights_after)
            if self.b_down is not None and not down_bias_done:
                ops.add_row_bias(x, self.b_down)
