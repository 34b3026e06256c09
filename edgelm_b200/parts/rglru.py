"""A recurrent block around a real-gated linear recurrent unit: a diagonal recurrence whose decay depends on the input.

The mixer's input h is projected twice to `width` channels.  One projection (with bias) goes through gelu_tanh and
gates the output: y.  The other (with bias) goes through a depthwise causal filter over time, u_t[c] = cb[c] + sum_j
taps[c, j] * x_(t - taps + 1 + j)[c] with x = 0 before a sequence's start and no activation.  The channels of u form
`blocks` groups of width / blocks; group b has two square matrices R_b, I_b and bias vectors of its own:

    r = sigmoid(R_b u_b + br_b),   i = sigmoid(I_b u_b + bi_b)
    log a = -decay_scale * r * softplus(lambda),   S_t = a S_(t-1) + sqrt(1 - a^2) * i * u      (S_(-1) = 0; the first token is no exception)

and the mixer returns W_o (S * y).  A sequence's state: S (float32) and the convolution's last taps - 1 inputs.  The gates'
products, the decay, the recurrence and its state are float32 in both precisions; the three projections run in the
compute dtype and their float32 sums are kept.
"""
import torch

from ..config.base import ConfigError
from ..csrc import ops
from . import linear
from .base import NeedSet, Part, StateNeed, as_matrix, as_vector, nbytes
from .registry import register_mixer


@register_mixer("rglru")
class RGLRU(Part):
    graph_safe = True

    def __init__(self, spec, env):
        self.hidden, self.width, self.blocks, self.taps = spec["hidden_size"], spec["width"], spec.get("blocks") or 1, spec.get("conv") or 1
        self.decay_scale = float(spec.get("decay_scale", 8.0))
        self.names = dict(spec["names"])
        self.dtype = env.dtype
        if self.width < 1 or self.blocks < 1 or self.width % self.blocks or self.taps < 1:
            raise ConfigError(f"rglru: {self.width} channels in {self.blocks} blocks with {self.taps} taps")
        self.bw = self.width // self.blocks

    def sizes(self):
        return {"rglru_width": self.width, "rglru_blocks": self.blocks, "conv_taps": self.taps}

    def flops(self, n_tokens, attended):
        return 2.0 * n_tokens * self.hidden * 3 * self.width + 4.0 * n_tokens * self.width * self.bw

    def weight_shapes(self, prefix):
        n, W = self.names, self.width
        return {prefix + n["y"]: (W, self.hidden), prefix + n["y"] + n["bias"]: (W,), prefix + n["x"]: (W, self.hidden),
                prefix + n["x"] + n["bias"]: (W,), prefix + n["conv"]: (W, self.taps), prefix + n["conv_bias"]: (W,),
                prefix + n["ra"]: (self.blocks, self.bw, self.bw), prefix + n["ra"] + n["bias"]: (self.blocks, self.bw),
                prefix + n["ri"]: (self.blocks, self.bw, self.bw), prefix + n["ri"] + n["bias"]: (self.blocks, self.bw),
                prefix + n["lam"]: (W,), prefix + n["o"]: (self.hidden, W)}

    def load(self, tensors, prefix, device):
        n, f32 = self.names, torch.float32
        self.w_in = torch.cat([as_matrix(tensors[prefix + n[k]], self.dtype, device) for k in ("y", "x")], dim=0).contiguous()   # y | x
        self.b_y = as_vector(tensors[prefix + n["y"] + n["bias"]], device)
        self.b_x = as_vector(tensors[prefix + n["x"] + n["bias"]], device)
        self.conv_w = as_matrix(tensors[prefix + n["conv"]], f32, device)
        self.conv_b = as_vector(tensors[prefix + n["conv_bias"]], device)
        self.no_tail = torch.zeros((1, 0, self.width), dtype=f32, device=device)      # (one tap: no earlier input is kept)
        # the gates' products are float32 sums of float32 inputs whatever the compute dtype (they are part of the recurrence);
        # the matrices are kept in the compute dtype, which holds stored bfloat16 values exactly
        self.w_ra = tensors[prefix + n["ra"]].to(device=device, dtype=self.dtype).contiguous()
        self.w_ri = tensors[prefix + n["ri"]].to(device=device, dtype=self.dtype).contiguous()
        self.b_ra = as_vector(tensors[prefix + n["ra"] + n["bias"]].reshape(-1), device)
        self.b_ri = as_vector(tensors[prefix + n["ri"] + n["bias"]].reshape(-1), device)
        lam = tensors[prefix + n["lam"]].to(torch.float64)
        self.decay = (-self.decay_scale * torch.nn.functional.softplus(lam)).to(device=device, dtype=f32).contiguous()   # log a = decay * r
        self.w_o = as_matrix(tensors[prefix + n["o"]], self.dtype, device)

    def first_weights(self):
        return (self.w_in,)

    def cache_need(self):
        return NeedSet.of(conv=StateNeed((self.taps - 1, self.width)) if self.taps > 1 else None, rglru=StateNeed((self.width,)))

    def workspace_bytes(self, n_tokens, n_seqs):
        f32, W = torch.float32, self.width
        return (nbytes((n_tokens, 2 * W), f32) * 2 + nbytes((n_tokens, W), f32) + nbytes((n_tokens, W), self.dtype) +
                nbytes((ops.rglru_scratch_floats(n_tokens, n_seqs, W),), f32) +
                nbytes((n_tokens, self.hidden), self.dtype))

    def forward(self, ctx, h, x, cache, accumulate=True):
        h = linear.as_tensor(h)
        T, ws, f32, W = h.shape[0], ctx.ws, torch.float32, self.width
        yx = ws.alloc((T, 2 * W), f32)
        with ctx.prof("rglru_in_proj"):
            linear.matmul(ctx, h, self.w_in, yx, prefetch=(self.w_o,))
        u = ws.alloc((T, W), f32)
        conv = cache.get("conv")
        with ctx.prof("rglru_conv"):
            ops.conv_act(yx, W, self.conv_w, self.conv_b, conv.state if conv is not None else self.no_tail, u,
                         ctx.tok_seq, ctx.seq_tok0, ctx.seq_slots, ctx.n_seqs, update_state=True, in_bias=self.b_x, act=None)
        gates = ws.alloc((T, 2 * W), f32)
        with ctx.prof("rglru_gates"):
            ops.rglru_gates(u, self.w_ra, self.w_ri, gates, self.blocks)
        s = ws.alloc((T, W), self.dtype)
        with ctx.prof("rglru_scan"):
            scratch = None if ctx.all_single else ws.alloc((ops.rglru_scratch_floats(T, ctx.n_seqs, W),), f32)
            ops.rglru_scan(gates, self.b_ra, self.b_ri, u, self.decay, yx[:, :W], self.b_y, cache["rglru"].state, s,
                           ctx.seq_tok0, ctx.seq_slots, ctx.n_seqs, ctx.all_single, tok_seq=ctx.tok_seq, scratch=scratch)
        with ctx.prof("rglru_out_proj"):
            linear.matmul(ctx, s, self.w_o, x, epilogue=linear.EPI_RESIDUAL if accumulate else linear.EPI_STORE,
                          residual=x if accumulate else None, prefetch=ctx.weights_after)
