"""RMSNorm: y = x * (1 / sqrt(mean(x^2) + eps)) * w, statistics in float32
(adarsh-sgh/edgelm src/kernels_ref.cpp:48-56).  The weight is used as stored, or with `offset` (a constant of
the spec, default 0) added to it: a weight kept around zero that multiplies as 1 + w has offset 1."""
from ..csrc import ops
from .base import Part, as_vector
from .registry import register_norm


@register_norm("rmsnorm")
class RMSNorm(Part):
    graph_safe = True
    fusable = True  # a few-rows matrix product can compute this norm in its prologue (weight, eps)

    def __init__(self, spec, env):
        self.dim, self.eps, self.name = spec["dim"], float(spec["eps"]), spec["name"]
        self.offset = float(spec.get("offset") or 0.0)
        self.weight = None

    def sizes(self):
        return {"rms_norm_eps": self.eps, **({"norm_weight_offset": self.offset} if self.offset else {})}

    def weight_shapes(self, prefix):
        return {prefix + self.name: (self.dim,)}

    def load(self, tensors, prefix, device):
        self.weight = as_vector(tensors[prefix + self.name], device)
        if self.offset:
            self.weight = (self.weight + self.offset).contiguous()     # (float32: what the kernels multiply by)

    def forward(self, ctx, x, out, rows=None):
        ops.rmsnorm(x, self.weight, self.eps, out, rows_idx=rows)

    def add_normed(self, ctx, x, y, cast=None, a=1.0, y2=None, b=0.0):
        """x += norm(a y + b y2): the norm on a sublayer's OUTPUT, with the residual sum in the same kernel.  x, y, y2
        float32; `cast` (optional) receives the new x in the compute dtype, for the matrix product that reads it next."""
        ops.rmsnorm_add(x, y, self.weight, self.eps, a=a, y2=y2, b=b, cast=cast)
