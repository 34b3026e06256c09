"""A feed-forward made of experts: x += sum over the token's chosen experts of weight * W_down (silu(W_gate h) * (W_up h)).

The router's logits z = W_r h + b_r are computed in float32; the `top` experts with the largest logits are chosen (the
first of equal ones), and their weights are the softmax over the chosen logits only.  Experts have no biases.  The
step's (token, choice) pairs are grouped by expert on the device (no count ever reaches the host, so a step can be
replayed from a CUDA graph): each expert's rows start at a multiple of the products' row tile, the gate and up products
with the activation run over the grouped rows, the down product writes a float32 row per pair, and the weighted sum
into the residual stream takes a token's pairs in the order of its choices.

Options, each with its constants in the spec:
    glu       (limit, alpha, shift): an expert's unit is g sigmoid(alpha g) (v + shift) with g = min(W_gate h, limit) and
              v = clamp(W_up h, -limit, limit) (absent: silu(g) v)
    router    {"kind": "scored", ...}: scores s = softmax(z) over ALL experts; the choice takes the `top` largest of s + a
              correction per expert (a tensor, `names["correction"]`), looking only inside the `keep` of `groups` equal groups
              of neighbouring experts whose largest corrected score is largest (other experts count as minus infinity: if the
              kept groups hold fewer than `top` experts, the others follow in the order of their numbers);
              the weights are the chosen experts' s over their sum (+ 1e-20), times `scale`.  `identity`: so many router
              outputs after the experts' belong to identity experts, which have no tensors and return their input (they
              are scored, corrected, grouped and chosen like the others).  This router has no bias.
    shared    a feed-forward spec: one more expert that every token uses, added after multiplying by sigmoid(w_sg . h), one
              number per token (`names["shared_gate"]`, a [1, hidden] tensor that rides in the router's product)
"""
import torch

from ..config.base import ConfigError
from ..csrc import ops
from . import linear
from .base import Part, as_matrix, as_vector, nbytes
from .registry import register_ffn


@register_ffn("moe")
class MixtureOfExperts(Part):
    graph_safe = True

    def __init__(self, spec, env):
        self.hidden, self.inter = spec["hidden_size"], spec["intermediate_size"]
        self.n_experts, self.top = spec["experts"], spec["top"]
        self.names = dict(spec["names"])
        self.dtype = env.dtype
        self.glu = tuple(float(v) for v in spec.get("glu") or ops.GLU_SWIGLU)
        r = dict(spec.get("router") or {"kind": "top_logits"})
        self.router = r.get("kind", "top_logits")
        if self.router not in ("top_logits", "scored"):
            raise ConfigError(f"moe: a router of kind '{self.router}' is not known (top_logits, scored)")
        self.identity = int(r.get("identity") or 0) if self.router == "scored" else 0
        self.routed = self.n_experts + self.identity                 # what the router scores
        self.groups, self.keep, self.scale = int(r.get("groups") or 1), int(r.get("keep") or 1), float(r.get("scale", 1.0))
        if self.n_experts < 1 or not 1 <= self.top <= self.routed or self.routed > 1024:
            raise ConfigError(f"moe: {self.top} of {self.n_experts} experts and {self.identity} identity experts (up to 1024)")
        if self.router == "scored" and (self.groups < 1 or self.routed % self.groups or not 1 <= self.keep <= self.groups):
            raise ConfigError(f"moe: {self.routed} routed experts in {self.groups} groups of which {self.keep} are kept")
        self.shared = env.build("ffn", spec["shared"]) if spec.get("shared") is not None else None
        self.w_gate = self.w_up = self.w_down = self.w_router = self.b_router = self.correction = None

    def sizes(self):
        out = {"intermediate": self.inter, "experts": self.n_experts, "experts_per_token": self.top}
        if self.router == "scored":
            out.update({"router": "scored", "identity_experts": self.identity, "expert_groups": self.groups, "groups_kept": self.keep,
                        "router_scale": self.scale})
        if self.glu != tuple(ops.GLU_SWIGLU):
            out["expert_glu"] = list(self.glu)
        if self.shared is not None:
            out["shared_expert"] = self.shared.sizes()
        return out

    def flops(self, n_tokens, attended):
        return (2.0 * n_tokens * self.hidden * self.routed + 6.0 * n_tokens * self.top * self.hidden * self.inter +
                (self.shared.flops(n_tokens, attended) if self.shared is not None else 0.0))

    def _expert(self, e, which):
        n = self.names
        return f"{n['expert']}{e}.{n[which]}"

    def weight_shapes(self, prefix):
        n, out = self.names, {}
        for e in range(self.n_experts):
            out[prefix + self._expert(e, "gate")] = (self.inter, self.hidden)
            out[prefix + self._expert(e, "up")] = (self.inter, self.hidden)
            out[prefix + self._expert(e, "down")] = (self.hidden, self.inter)
        out[prefix + n["router"]] = (self.routed, self.hidden)
        if self.router == "scored":
            out[prefix + n["correction"]] = (self.routed,)
        else:
            out[prefix + n["router_bias"]] = (self.n_experts,)
        if self.shared is not None:
            out.update(self.shared.weight_shapes(prefix))
            out[prefix + n["shared_gate"]] = (1, self.hidden)
        return out

    def load(self, tensors, prefix, device):
        n = self.names
        stack = lambda which: torch.stack([as_matrix(tensors[prefix + self._expert(e, which)], self.dtype, device)
                                           for e in range(self.n_experts)]).contiguous()
        self.w_gate, self.w_up, self.w_down = stack("gate"), stack("up"), stack("down")
        self.w_router = as_matrix(tensors[prefix + n["router"]], torch.float32, device)
        if self.router == "scored":
            self.correction = as_vector(tensors[prefix + n["correction"]], device)
        else:
            self.b_router = as_vector(tensors[prefix + n["router_bias"]], device)
        if self.shared is not None:
            self.shared.load(tensors, prefix, device)
            self.w_router = torch.cat([self.w_router, as_matrix(tensors[prefix + n["shared_gate"]], torch.float32, device)], dim=0).contiguous()

    def _on_tensor_cores(self):
        """Whether the experts' products run as grouped tcgen05 products (bfloat16 and sizes that kernel takes)."""
        return (self.dtype == torch.bfloat16 and self.hidden % 8 == 0 and self.inter % 8 == 0 and self.w_gate is not None and
                self.w_gate.data_ptr() % 16 == 0 and self.w_up.data_ptr() % 16 == 0 and self.w_down.data_ptr() % 16 == 0)

    def _max_tiles(self, n_tokens, tile_rows):
        return ops.moe_max_tiles(n_tokens * self.top, self.n_experts, tile_rows)

    def workspace_bytes(self, n_tokens, n_seqs):
        tile_rows = ops.moe_tile_rows(self._on_tensor_cores())
        tiles = self._max_tiles(n_tokens, tile_rows)
        rows, pairs = tiles * tile_rows, n_tokens * self.top
        own = (nbytes((n_tokens, self.hidden), self.dtype) + 2 * nbytes((pairs,), torch.int32) + nbytes((pairs,), torch.float32) +
               nbytes((rows,), torch.int32) + nbytes((tiles,), torch.int32) + nbytes((rows, self.hidden), self.dtype) +
               nbytes((rows, self.inter), self.dtype) + nbytes((rows, self.hidden), torch.float32))
        if self.shared is not None:
            own += nbytes((n_tokens,), torch.float32) + nbytes((n_tokens, self.hidden), torch.float32) + self.shared.workspace_bytes(n_tokens, n_seqs)
        return own

    def first_weights(self):
        return ()

    def forward(self, ctx, h, x, accumulate=True):
        h = linear.as_tensor(h)
        T, ws = h.shape[0], ctx.ws
        tc = self._on_tensor_cores()
        tile_rows = ops.moe_tile_rows(tc)
        max_tiles = self._max_tiles(T, tile_rows)
        rows = max_tiles * tile_rows
        idx = ws.alloc((T, self.top), torch.int32)
        wts = ws.alloc((T, self.top), torch.float32)
        row_pair = ws.alloc((rows,), torch.int32)
        pair_row = ws.alloc((T * self.top,), torch.int32)
        tile_expert = ws.alloc((max_tiles,), torch.int32)
        gate = ws.alloc((T, 1), torch.float32) if self.shared is not None else None
        with ctx.prof("moe_route"):
            if self.router == "scored":
                ops.moe_route_scored(h, self.w_router, self.correction, idx, wts, self.top, self.routed, self.groups, self.keep, self.scale, extra=gate)
            else:
                ops.moe_route(h, self.w_router, self.b_router, idx, wts, self.top)
            ops.moe_plan(idx, self.n_experts, tile_rows, row_pair, pair_row, tile_expert)     # (an identity expert's pair gets no row)
        mid = ws.alloc((rows, self.inter), self.dtype)
        y = ws.alloc((rows, self.hidden), torch.float32)
        if tc:
            a = ws.alloc((rows, self.hidden), self.dtype)
            with ctx.prof("moe_gather"):
                ops.moe_gather_rows(h, a, row_pair, self.top)
            with ctx.prof("moe_gate_up"):
                ops.gemm_tc_grouped(a, self.w_gate, mid, tile_expert, ctx.err, epilogue=linear.EPI_SWIGLU, w2=self.w_up, glu=self.glu)
            with ctx.prof("moe_down"):
                ops.gemm_tc_grouped(mid, self.w_down, y, tile_expert, ctx.err)
        else:
            with ctx.prof("moe_gate_up"):
                ops.moe_gate_up(h, self.w_gate, self.w_up, mid, row_pair, tile_expert, self.top, glu=self.glu)
            with ctx.prof("moe_down"):
                ops.moe_down(mid, self.w_down, y, row_pair, tile_expert, self.top)
        ys = None
        if self.shared is not None:
            ys = ws.alloc((T, self.hidden), torch.float32)
            with ws.frame():
                self.shared.forward(ctx, h, ys, accumulate=False)
        with ctx.prof("moe_combine"):
            if not accumulate:
                x.zero_()
            ops.moe_combine(x, y, wts, pair_row, idx=idx if self.identity else None, n_real=self.n_experts, h=h if self.identity else None,
                            shared=ys, gate=gate)
