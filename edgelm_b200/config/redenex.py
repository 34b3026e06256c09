"""The Redenex decoder's configuration, from its own config.json keys.

config.json: `architecture` "Redenex", `vocab`, `width`, `norm.eps`, `embedding.scale`, `streams` (how many copies of the
residual stream the layers keep; absent: one plain stream), `loop` {start, stop, times} (the stretch of layers from
`start` up to but not including `stop` is repeated `times` times before the layers after it, the weights shared and every
repetition with pages and states of its own; absent: every layer once) and `layers`,
one entry per layer: `type` ("rglru" or "attention"), `mixer` (its sizes and constants) and `mlp` ({"kind": "dense", "ff",
"limit"} or null for a layer without a feed-forward).  Optional: `max_positions`.  Tensors: `embed`, `l<i>.norm1`,
`l<i>.norm2`, `l<i>.mix.*`, `l<i>.mlp.{gate,up,down}`, `l<i>.hc<q>.{in,out,mix}` (with `streams`), `final.norm`, `head`.

Every norm multiplies by 1 + its stored weight.  The mixers:
  rglru       a recurrent block around a real-gated linear recurrent unit (`parts/rglru.py`): `width`, `blocks`, `conv`
  attention   grouped heads with biases whose queries and keys pass a short convolution, a per-head norm and a half-split
              rotation, two attention maps per head combined into one ("differential"), a chunked mask `mask.size`
              (absent: causal): `heads`, `kv_heads`, `dim`, `vdim`, `conv`, `rot` {dims, base}, `scale`, `diff`
              (`parts/masked_attention.py` with its options)
The feed-forward is a clamped gated unit (`parts/clamped_glu.py`).
"""
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .base import ConfigError, LayerSpec, ModelPlan, PartSpec, ScheduleEntry, optional, require
from .registry import register_architecture

DEFAULT_MAX_POSITIONS = 1 << 20
GLU_ALPHA = 1.702          # the feed-forward's gate is g * sigmoid(GLU_ALPHA * g)
DECAY_SCALE = 8.0          # log a = -DECAY_SCALE * r * softplus(lambda) in the recurrent unit


def _sub(d, key, where):
    v = d.get(key)
    if not isinstance(v, Mapping):
        raise ConfigError(f"{where}: key '{key}' should be an object, found {v!r}")
    return v


@register_architecture("Redenex", model_type="redenex")
@dataclass(frozen=True)
class RedenexConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    layers: Tuple[Mapping[str, Any], ...]
    streams: Optional[int] = None
    loop: Optional[Tuple[int, int, int]] = None
    max_positions: int = DEFAULT_MAX_POSITIONS

    architecture = "Redenex"

    @classmethod
    def from_dict(cls, d):
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' should be a non-empty list")
        emb = d.get("embedding")
        loop = d.get("loop")
        if loop is not None:
            if not isinstance(loop, Mapping):
                raise ConfigError("config.json: key 'loop' should be an object")
            loop = tuple(require(loop, k, int, "config.json loop") for k in ("start", "stop", "times"))
        cfg = cls(vocab=require(d, "vocab", int), width=require(d, "width", int),
                  eps=require(_sub(d, "norm", "config.json"), "eps", float, "config.json norm"),
                  embedding_scale=optional(emb, "scale", float, 1.0, "config.json embedding") if isinstance(emb, Mapping) else 1.0,
                  layers=tuple(layers), streams=optional(d, "streams", int, None), loop=loop,
                  max_positions=optional(d, "max_positions", int, DEFAULT_MAX_POSITIONS))
        if cfg.vocab <= 0 or cfg.width <= 0 or cfg.max_positions <= 0 or not cfg.eps > 0:
            raise ConfigError("config.json: vocab, width, max_positions and norm.eps must be positive")
        if cfg.streams is not None and cfg.streams < 1:
            raise ConfigError(f"config.json: {cfg.streams} residual streams")
        if loop is not None and not (0 <= loop[0] <= loop[1] <= len(layers) and loop[2] >= 1):
            raise ConfigError(f"config.json loop: layers {loop[0]} .. {loop[1]} - 1, {loop[2]} times, of {len(layers)} layers")
        cfg.plan()     # every layer's keys are read and checked here
        return cfg

    def to_dict(self):
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
               "embedding": {"scale": self.embedding_scale}, "layers": [dict(l) for l in self.layers]}
        if self.streams is not None:
            out["streams"] = self.streams
        if self.loop is not None:
            out["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out

    # ------------------------------------------------------------------ mixers
    def _rglru(self, m, where):
        return PartSpec("rglru", {
            "hidden_size": self.width, "width": require(m, "width", int, where), "blocks": optional(m, "blocks", int, 1, where),
            "conv": optional(m, "conv", int, 1, where), "decay_scale": DECAY_SCALE,
            "names": {"y": "mix.y", "x": "mix.x", "bias": ".b", "conv": "mix.conv", "conv_bias": "mix.conv.b", "ra": "mix.ra", "ri": "mix.ri",
                      "lam": "mix.lam", "o": "mix.o"}})

    def _attention(self, m, where):
        heads, dim = require(m, "heads", int, where), require(m, "dim", int, where)
        rot = m.get("rot")
        if rot is not None and not isinstance(rot, Mapping):
            raise ConfigError(f"{where}: key 'rot' should be an object")
        mask = m.get("mask")
        if mask is not None and not isinstance(mask, Mapping):
            raise ConfigError(f"{where}: key 'mask' should be an object")
        return PartSpec("masked_attention", {
            "hidden_size": self.width, "num_heads": heads, "num_kv_heads": optional(m, "kv_heads", int, None, where) or heads,
            "head_dim": dim, "v_head_dim": optional(m, "vdim", int, None, where) or dim, "scale": require(m, "scale", float, where),
            "rot_dims": require(rot, "dims", int, where + " rot") if rot is not None else 0,
            "rot_base": require(rot, "base", float, where + " rot") if rot is not None else None, "rot_scaling": None,
            "rot_pairs": "half", "bias": True, "output_bias": False, "conv": optional(m, "conv", int, None, where),
            "qk_norm": {"eps": self.eps}, "diff": {"offset": require(m, "diff", float, where), "eps": self.eps},
            "mask": {"kind": "chunk", "size": require(mask, "size", int, where + " mask")} if mask is not None else None,
            "names": {"q": "mix.q", "k": "mix.k", "v": "mix.v", "o": "mix.o", "bias": ".b", "conv": ".conv", "q_norm": "mix.q.norm",
                      "k_norm": "mix.k.norm", "lq1": "mix.lq1", "lk1": "mix.lk1", "lq2": "mix.lq2", "lk2": "mix.lk2"}})

    def _layer(self, i, layer):
        where = f"config.json layers[{i}]"
        if not isinstance(layer, Mapping):
            raise ConfigError(f"{where} should be an object")
        kind = require(layer, "type", str, where)
        m = _sub(layer, "mixer", where)
        if kind == "rglru":
            mixer = self._rglru(m, where + " mixer")
        elif kind == "attention":
            mixer = self._attention(m, where + " mixer")
        else:
            raise ConfigError(f"{where}: a layer of type '{kind}' is not part of this architecture (rglru, attention)")
        norm = {"dim": self.width, "eps": self.eps, "offset": 1.0}
        mlp, ffn, ffn_norm = layer.get("mlp"), None, None
        if mlp is not None:
            if not isinstance(mlp, Mapping):
                raise ConfigError(f"{where}: key 'mlp' should be an object or null")
            mk = require(mlp, "kind", str, where + " mlp")
            if mk != "dense":
                raise ConfigError(f"{where} mlp: kind '{mk}' is not part of this architecture (dense)")
            ffn = PartSpec("clamped_glu", {"hidden_size": self.width, "intermediate_size": require(mlp, "ff", int, where + " mlp"),
                                           "limit": require(mlp, "limit", float, where + " mlp"), "alpha": GLU_ALPHA,
                                           "names": {"gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"}})
            ffn_norm = PartSpec("rmsnorm", {**norm, "name": "norm2"})
        options = {}
        if self.streams is not None:
            options = {"streams": self.streams, "names": {"mixer": "hc1", "ffn": "hc2", "in": ".in", "out": ".out", "mix": ".mix"}}
        return LayerSpec(prefix=f"l{i}.", block="hyper" if self.streams is not None else "prenorm", mixer=mixer,
                         mixer_norm=PartSpec("rmsnorm", {**norm, "name": "norm1"}), ffn=ffn, ffn_norm=ffn_norm, options=options)

    def order(self):
        """The layers' indices in the order they run."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        start, stop, times = self.loop
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))

    def plan(self) -> ModelPlan:
        norm = {"dim": self.width, "eps": self.eps, "offset": 1.0}
        return ModelPlan(
            hidden_size=self.width, vocab_size=self.vocab, max_positions=self.max_positions,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab, "dim": self.width, "name": "embed", "scale": self.embedding_scale}),
            layers=tuple(self._layer(i, l) for i, l in enumerate(self.layers)),
            schedule=tuple(ScheduleEntry(i) for i in self.order()),     # (a second run of a layer has a cache entry of its own)
            final_norm=PartSpec("rmsnorm", {**norm, "name": "final.norm"}),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "dim": self.width, "tied_to": None, "name": "head"}),
            stop_token_ids=(), bos_token_id=None, residual_streams=self.streams or 1,
        ).validate()
