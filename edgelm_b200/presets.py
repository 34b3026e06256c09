"""config.json contents of the model shapes the benchmarks and the command line can build with
random weights (no checkpoint is needed or read).  These are data, handed to the same
configuration reader as any config.json; no size here is known to model code."""

def _llama(vocab, hidden, inter, layers, heads, kv_heads, head_dim, max_pos, theta, eps, tied):
    return {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": vocab, "hidden_size": hidden,
            "intermediate_size": inter, "num_hidden_layers": layers, "num_attention_heads": heads,
            "num_key_value_heads": kv_heads, "head_dim": head_dim, "max_position_embeddings": max_pos,
            "rope_theta": theta, "rms_norm_eps": eps, "tie_word_embeddings": tied, "bos_token_id": 0, "eos_token_id": 0}


def _sagizen(vocab, width, ff, groups_of_layers, ssm_heads, ssm_state, heads, kv_heads, window, pool):
    """A Sagizen-shaped model: per group three state-space layers and one layer of attention beside a time mix, heads of
    64 everywhere, the state-space mixer twice as wide inside as the model (the usual expansion)."""
    dense = {"kind": "dense", "ff": ff}
    ssm = {"type": "mamba2", "mlp": dense,
           "mixer": {"heads": ssm_heads, "vdim": 64, "state": ssm_state, "groups": 1, "conv": 4, "norm_groups": 1}}
    par = {"type": "parallel", "mlp": dense, "decay_rank": 64, "mixer": {
        "left": {"heads": heads, "kv_heads": kv_heads, "dim": 64, "vdim": 64, "mask": {"size": window, "pool": pool},
                 "rot": {"base": 500000.0, "dims": 64, "scaling": {"factor": 1.0}}, "scale": 0.125},
        "left_scale": 1.0, "right": {"heads": heads, "dim": 64}, "right_scale": 1.0}}
    return {"architecture": "Sagizen", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "max_positions": 8192,
            "layers": [ssm, ssm, ssm, par] * groups_of_layers}


def _vosulorn(vocab, width, ff, groups_of_layers, heads, kv_heads, kv_rank, rot_dim, chunk, experts, top):
    """A Vosulorn-shaped model: per group a delta-rule layer, a latent-attention layer, a second delta-rule layer and a
    layer of chunked attention with a sink, heads of 64 everywhere, every layer with a mixture of `experts` experts of which
    a token uses `top` (so `top * ff` is the feed-forward width a token sees)."""
    moe = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    delta = {"type": "delta", "mlp": moe, "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": 64, "vdim": 64, "conv": 4}}
    latent = {"type": "latent_attention", "mlp": moe, "mixer": {
        "heads": heads, "dim": 64, "rot_dim": rot_dim, "vdim": 64, "kv_rank": kv_rank, "scale": (64 + rot_dim) ** -0.5,
        "rot": {"base": 1000000.0, "dims": rot_dim}}}
    attn = {"type": "attention", "mlp": moe, "mixer": {
        "heads": heads, "kv_heads": kv_heads, "dim": 64, "vdim": 64, "scale": 0.125, "mask": {"size": chunk},
        "rot": {"base": 250000.0, "dims": 64, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 2048}}}}
    return {"architecture": "Vosulorn", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
            "max_positions": 8192, "layers": [delta, latent, delta, attn] * groups_of_layers}


def _redenex(vocab, width, ff, pattern, rec_width, rec_blocks, heads, kv_heads, dim, chunk, streams):
    """A Redenex-shaped model: recurrent ("r") and attention ("a") layers in the order of `pattern`, each with a clamped
    gated feed-forward; an attention head has two maps of `dim` and values of 2 * dim (so heads * 2 * dim query rows, as many
    as a plain decoder of the same width has), the recurrent mixer is `rec_width` wide in `rec_blocks` blocks; `streams` copies
    of the residual stream."""
    dense = {"kind": "dense", "ff": ff, "limit": 7.0}
    rec = {"type": "rglru", "mlp": dense, "mixer": {"width": rec_width, "blocks": rec_blocks, "conv": 4}}
    att = {"type": "attention", "mlp": dense, "mixer": {
        "heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": 2 * dim, "conv": 3, "diff": 0.8, "scale": dim ** -0.5,
        "mask": {"size": chunk}, "rot": {"base": 500000.0, "dims": dim}}}
    return {"architecture": "Redenex", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
            "streams": streams, "max_positions": 8192, "layers": [rec if c == "r" else att for c in pattern]}


def _radupel(vocab, width, ff, pattern, loop, heads, kv_heads, lin_heads, experts, expert_ff, shared_ff):
    """A Radupel-shaped model: every layer a softmax attention (heads of 64, half of each rotated, a convolution of 4 taps on
    q, k and v, a gate per head) beside a linear attention with a constant decay per head (heads of 64 x 64), with a dense
    feed-forward ("d") or a mixture of `experts` clamped experts plus four identity experts in three groups, two chosen out of
    the two better groups, and a shared expert ("m"), in the order of `pattern`; `loop` (start, stop, times) or None."""
    decay = [round(1.0 - 2.0 ** -(3.0 + 6.0 * h / max(1, lin_heads - 1)), 6) for h in range(lin_heads)]
    mixer = {"left": {"heads": heads, "kv_heads": kv_heads, "dim": 64, "vdim": 64, "conv": 4, "scale": 0.125,
                      "rot": {"base": 1000000.0, "dims": 32}},
             "left_scale": 1.0, "right": {"heads": lin_heads, "dim": 64, "vdim": 64, "decay": decay}, "right_scale": 1.0}
    dense = {"kind": "dense", "ff": ff}
    moe = {"kind": "moe", "expert": {"ff": expert_ff, "limit": 7.0},
           "router": {"experts": experts, "top": 2, "identity": 4, "groups": {"count": 3, "keep": 2}, "scale": 2.0},
           "shared": {"ff": shared_ff, "limit": 7.0}}
    out = {"architecture": "Radupel", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "logit_softcap": 50.0, "max_positions": 8192,
           "layers": [{"type": "parallel", "mixer": mixer, "mlp": dense if c == "d" else moe} for c in pattern]}
    if loop:
        out["loop"] = dict(zip(("start", "stop", "times"), loop))
    return out


PRESETS = {
    # the layer sizes of smollm2-135m and smollm2-1.7b (width, feed-forward, as many query, key and output rows, vocabulary)
    # in the Radupel design: dense and expert feed-forwards in turn, the first layers run twice (8 and 4 layer runs)
    "radupel-576": _radupel(49152, 576, 1536, "dmdmdm", (0, 2, 2), 9, 3, 9, 8, 768, 768),
    "radupel-2048": _radupel(49152, 2048, 8192, "dmd", (0, 1, 2), 32, 32, 32, 8, 4096, 4096),
    # the layer sizes of smollm2-135m and smollm2-1.7b (width, feed-forward, as many query, key and output rows, vocabulary)
    # in the Redenex design: two recurrent layers to one of attention, four residual streams
    "redenex-576": _redenex(49152, 576, 1536, "rrarrarr", 768, 12, 9, 3, 32, 1024, 4),
    "redenex-2048": _redenex(49152, 2048, 8192, "rrar", 2560, 16, 16, 16, 64, 1024, 4),
    # the layer sizes of smollm2-135m and smollm2-1.7b (width, heads of 64, vocabulary; a token's two experts together as
    # wide as the dense feed-forward) in the Vosulorn design
    "vosulorn-576": _vosulorn(49152, 576, 768, 2, 9, 3, 128, 32, 1024, 8, 2),
    "vosulorn-2048": _vosulorn(49152, 2048, 4096, 1, 32, 32, 512, 64, 1024, 8, 2),
    # the layer sizes of smollm2-135m and smollm2-1.7b (width, feed-forward, heads of 64, vocabulary) in the Sagizen design
    "sagizen-576": _sagizen(49152, 576, 1536, 2, 18, 128, 9, 3, 512, 64),
    "sagizen-2048": _sagizen(49152, 2048, 8192, 1, 64, 128, 32, 32, 1024, 64),
    "tiny-a": _llama(256, 64, 128, 2, 4, 2, 16, 128, 10000.0, 1e-5, True),
    "tiny-b": _llama(397, 96, 200, 3, 3, 1, 32, 256, 100000.0, 1e-6, False),
    "smollm2-135m": _llama(49152, 576, 1536, 30, 9, 3, 64, 8192, 100000.0, 1e-5, True),
    "smollm2-360m": _llama(49152, 960, 2560, 32, 15, 5, 64, 8192, 100000.0, 1e-5, True),
    "smollm2-1.7b": _llama(49152, 2048, 8192, 24, 32, 32, 64, 8192, 130000.0, 1e-5, True),
}


def preset_config(name):
    from .config import config_class_for
    if name not in PRESETS:
        raise KeyError(f"unknown preset '{name}'; there are: {', '.join(sorted(PRESETS))}")
    d = PRESETS[name]
    return config_class_for(d).from_dict(d)


def random_model(config, seed=0, sigma=0.02, dtype="bfloat16", device="cuda:0", layers=None):
    """A DecoderModel of `config` with random weights made on the device (matrices N(0, sigma),
    norm weights 1 + N(0, sigma)); `layers` keeps only the plan's first so many layer runs (the configuration
    object stays whole: it is the plan that is cut)."""
    import torch

    from .engine.engine import DTYPES
    from .engine.model import DecoderModel
    from .weights import random_tensors
    plan = config.plan()
    if layers is not None and int(layers) != len(plan.schedule):
        plan = plan.first_runs(layers)
    torch_dtype = DTYPES[dtype] if isinstance(dtype, str) else dtype
    model = DecoderModel(plan, torch_dtype)
    tensors = random_tensors(model.expected_weights(), seed, sigma, torch_dtype, device=device)
    model.load(tensors, device)
    model.config = config
    return model
