"""The Radupel decoder's configuration, from its own config.json keys.

config.json: `architecture` "Radupel", `vocab`, `width`, `norm.eps`, `logit_softcap` (absent: none), `loop` {start, stop, times}
(the stretch of layers from `start` up to but not including `stop` runs `times` times in a row with the same weights, every
pass with pages and states of its own, and every pass but the first takes the embedding's output into the residual stream
again right before its first layer; absent: every layer once) and `layers`, one entry per layer: `type` ("parallel"), `mixer`
(its sizes and constants) and `mlp` (a dense or a mixture-of-experts feed-forward, or null for none).  Optional:
`max_positions`.  Tensors: `embed` (also the output head), `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.left.*`, `l<i>.mix.right.*`,
`l<i>.mlp.*`, `final.norm`.

A layer is x += mixer(norm1(x)) + mlp(norm2(x)), both sublayers reading the same x (block "parallel_prenorm").  The mixer is two
mixers on one input, left_scale * left + right_scale * right (`parts/parallel.py`):
  left    grouped softmax attention, causal: `heads`, `kv_heads`, `dim`, `vdim`, `conv` (taps of the short convolution that q, k
          and v pass straight after their projections), `rot` {dims, base} (half-split pairs over the first `dims` dimensions),
          `scale`, and a sigmoid gate per head on the output (`parts/masked_attention.py` with its options)
  right   linear attention with a constant decay per head (`parts/lightning.py`): `heads`, `dim`, `vdim`, `decay` (one per head)
The feed-forward: {"kind": "dense", "ff"}: SwiGLU with biases on all three projections (`parts/swiglu.py`);
{"kind": "moe", "expert": {ff, limit}, "router": {experts, top, identity, groups: {count, keep}, scale}, "shared": {ff, limit}}: a
mixture of clamped gated units with a scoring router, identity experts and a gated shared expert (`parts/moe.py`).
"""
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .base import ConfigError, LayerSpec, ModelPlan, PartSpec, ScheduleEntry, optional, require
from .registry import register_architecture

DEFAULT_MAX_POSITIONS = 1 << 20
GLU_ALPHA = 1.702          # an expert's gate is g * sigmoid(GLU_ALPHA * g)
GLU_SHIFT = 1.0            # ... times (u + GLU_SHIFT)


def _sub(d, key, where, needed=True):
    v = d.get(key)
    if v is None and not needed:
        return None
    if not isinstance(v, Mapping):
        raise ConfigError(f"{where}: key '{key}' should be an object, found {v!r}")
    return v


@register_architecture("Radupel", model_type="radupel")
@dataclass(frozen=True)
class RadupelConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[Mapping[str, Any], ...]
    logit_softcap: Optional[float] = None
    loop: Optional[Tuple[int, int, int]] = None
    max_positions: int = DEFAULT_MAX_POSITIONS

    architecture = "Radupel"

    @classmethod
    def from_dict(cls, d):
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' should be a non-empty list")
        loop = _sub(d, "loop", "config.json", needed=False)
        if loop is not None:
            loop = tuple(require(loop, k, int, "config.json loop") for k in ("start", "stop", "times"))
        cfg = cls(vocab=require(d, "vocab", int), width=require(d, "width", int),
                  eps=require(_sub(d, "norm", "config.json"), "eps", float, "config.json norm"), layers=tuple(layers),
                  logit_softcap=optional(d, "logit_softcap", float, None), loop=loop,
                  max_positions=optional(d, "max_positions", int, DEFAULT_MAX_POSITIONS))
        if cfg.vocab <= 0 or cfg.width <= 0 or cfg.max_positions <= 0 or not cfg.eps > 0:
            raise ConfigError("config.json: vocab, width, max_positions and norm.eps must be positive")
        if cfg.logit_softcap is not None and not cfg.logit_softcap > 0:
            raise ConfigError(f"config.json: a logit_softcap of {cfg.logit_softcap}")
        if loop is not None and not (0 <= loop[0] <= loop[1] <= len(layers) and loop[2] >= 1):
            raise ConfigError(f"config.json loop: layers {loop[0]} .. {loop[1]} - 1, {loop[2]} times, of {len(layers)} layers")
        cfg.plan()     # every layer's keys are read and checked here
        return cfg

    def to_dict(self):
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
               "layers": [dict(l) for l in self.layers]}
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        if self.loop is not None:
            out["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out

    # ------------------------------------------------------------------ mixers
    def _left(self, m, where):
        heads, dim = require(m, "heads", int, where), require(m, "dim", int, where)
        rot = _sub(m, "rot", where, needed=False)
        return PartSpec("masked_attention", {
            "hidden_size": self.width, "num_heads": heads, "num_kv_heads": optional(m, "kv_heads", int, None, where) or heads,
            "head_dim": dim, "v_head_dim": optional(m, "vdim", int, None, where) or dim, "scale": require(m, "scale", float, where),
            "rot_dims": require(rot, "dims", int, where + " rot") if rot is not None else 0,
            "rot_base": require(rot, "base", float, where + " rot") if rot is not None else None, "rot_scaling": None,
            "rot_pairs": "half", "bias": False, "output_bias": False, "conv": optional(m, "conv", int, None, where),
            "head_gate": True, "mask": None,
            "names": {"q": "mix.left.q", "k": "mix.left.k", "v": "mix.left.v", "o": "mix.left.o", "gate": "mix.left.g", "conv": ".conv"}})

    def _right(self, m, where):
        heads = require(m, "heads", int, where)
        decay = m.get("decay")
        if not isinstance(decay, (list, tuple)) or len(decay) != heads or not all(isinstance(a, (int, float)) and not isinstance(a, bool) for a in decay):
            raise ConfigError(f"{where}: key 'decay' should list one number per head ({heads})")
        dim = require(m, "dim", int, where)
        return PartSpec("decay_linear_attention", {
            "hidden_size": self.width, "heads": heads, "head_dim": dim, "v_head_dim": optional(m, "vdim", int, None, where) or dim,
            "decay": tuple(float(a) for a in decay), "activation": "silu", "eps": self.eps,
            "names": {"q": "mix.right.q", "k": "mix.right.k", "v": "mix.right.v", "g": "mix.right.g", "norm": "mix.right.norm", "o": "mix.right.o"}})

    def _mixer(self, m, where):
        return PartSpec("parallel", {
            "hidden_size": self.width, "left": self._left(_sub(m, "left", where), where + " left"),
            "right": self._right(_sub(m, "right", where), where + " right"),
            "left_scale": require(m, "left_scale", float, where), "right_scale": require(m, "right_scale", float, where)})

    # ------------------------------------------------------------------ feed-forwards
    def _expert(self, e, where, names):
        return PartSpec("clamped_glu", {"hidden_size": self.width, "intermediate_size": require(e, "ff", int, where),
                                        "limit": require(e, "limit", float, where), "alpha": GLU_ALPHA, "names": names})

    def _mlp(self, mlp, where):
        kind = require(mlp, "kind", str, where)
        if kind == "dense":
            return PartSpec("swiglu", {"hidden_size": self.width, "intermediate_size": require(mlp, "ff", int, where), "bias": ".b",
                                       "names": {"gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"}})
        if kind != "moe":
            raise ConfigError(f"{where}: kind '{kind}' is not part of this architecture (dense, moe)")
        e, r = _sub(mlp, "expert", where), _sub(mlp, "router", where)
        groups = _sub(r, "groups", where + " router", needed=False)
        shared = _sub(mlp, "shared", where, needed=False)
        limit = require(e, "limit", float, where + " expert")
        if not limit > 0:
            raise ConfigError(f"{where} expert: a limit of {limit}")
        return PartSpec("moe", {
            "hidden_size": self.width, "intermediate_size": require(e, "ff", int, where + " expert"),
            "experts": require(r, "experts", int, where + " router"), "top": require(r, "top", int, where + " router"),
            "glu": (limit, GLU_ALPHA, GLU_SHIFT),
            "router": {"kind": "scored", "identity": optional(r, "identity", int, 0, where + " router"),
                       "groups": require(groups, "count", int, where + " router groups") if groups is not None else 1,
                       "keep": require(groups, "keep", int, where + " router groups") if groups is not None else 1,
                       "scale": optional(r, "scale", float, 1.0, where + " router")},
            "shared": self._expert(shared, where + " shared", {"gate": "mlp.shared.gate", "up": "mlp.shared.up", "down": "mlp.shared.down"})
                      if shared is not None else None,
            "names": {"expert": "mlp.e", "gate": "gate", "up": "up", "down": "down", "router": "mlp.router", "correction": "mlp.correction",
                      "shared_gate": "mlp.shared.sg"}})

    def _layer(self, i, layer):
        where = f"config.json layers[{i}]"
        if not isinstance(layer, Mapping):
            raise ConfigError(f"{where} should be an object")
        kind = require(layer, "type", str, where)
        if kind != "parallel":
            raise ConfigError(f"{where}: a layer of type '{kind}' is not part of this architecture (parallel)")
        norm = {"dim": self.width, "eps": self.eps}
        mlp, ffn, ffn_norm = layer.get("mlp"), None, None
        if mlp is not None:
            if not isinstance(mlp, Mapping):
                raise ConfigError(f"{where}: key 'mlp' should be an object or null")
            ffn = self._mlp(mlp, where + " mlp")
            ffn_norm = PartSpec("rmsnorm", {**norm, "name": "norm2"})
        return LayerSpec(prefix=f"l{i}.", block="parallel_prenorm", mixer=self._mixer(_sub(layer, "mixer", where), where + " mixer"),
                         mixer_norm=PartSpec("rmsnorm", {**norm, "name": "norm1"}), ffn=ffn, ffn_norm=ffn_norm,
                         options={"unused_norm": "norm2"} if ffn is None else {})

    def order(self):
        """(layer, whether the embedding's output is added right before it) in run order."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, False) for i in range(n)]
        start, stop, times = self.loop
        out = [(i, False) for i in range(start)]
        for p in range(times):
            out += [(i, p > 0 and i == start) for i in range(start, stop)]
        return out + [(i, False) for i in range(stop, n)]

    def plan(self) -> ModelPlan:
        norm = {"dim": self.width, "eps": self.eps}
        return ModelPlan(
            hidden_size=self.width, vocab_size=self.vocab, max_positions=self.max_positions,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab, "dim": self.width, "name": "embed"}),
            layers=tuple(self._layer(i, l) for i, l in enumerate(self.layers)),
            schedule=tuple(ScheduleEntry(i, add_embedding=add) for i, add in self.order()),   # (every run has a cache entry of its own)
            final_norm=PartSpec("rmsnorm", {**norm, "name": "final.norm"}),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "dim": self.width, "tied_to": "embed", "name": "head",
                                      "softcap": self.logit_softcap}),
            stop_token_ids=(), bos_token_id=None,
        ).validate()
