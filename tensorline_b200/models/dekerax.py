"""The Dekerax decoder as a `ModelSpec`.

The embedded tokens pass the model's norm (`embed.norm`); every layer is a block whose sub-blocks are normalised before
and after (`norm1`, `norm1b`, `norm2`, `norm2b`: plain RMS norms in float32) with one of three mixers: grouped-query
attention without rotation over a sliding window, attention through a latent (a normalised latent and one rotated key part
a token in the cache) over a sliding window, or the gated delta rule (a matrix memory per head behind short
convolutions).  The feed-forward, where a layer has one, is dense (the tanh form of gelu) or a mixture of gated silu
experts chosen by sigmoid scores that weigh the experts' inputs, beside a shared expert with a sigmoid gate.  `loop` runs a
range of layers several times with the same weights, every pass with caches of its own and a learned vector
(`loop.step[pass]`) added to the stream in front of it.  Tensor names: `embed`, `embed.norm`, `loop.step`, `l<i>.norm1`
..., `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`, each tensor under its own name.
"""
from __future__ import annotations

from ..config.dekerax import DekeraxConfig, DenseSizes
from ..parts import PartSpec
from .spec import LayerSpec, ModelSpec, RunEntry

_QKVO = {"q": "q", "k": "k", "v": "v", "o": "o"}


def describe_dekerax(cfg: DekeraxConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    norm = PartSpec("rms_norm", {"dim": W, "eps": eps, "tensor": "", "cast_first": False})
    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if layer.type == "attention":
            position = PartSpec("none") if m.rot is None else PartSpec("rotary_half", {"theta": m.rot.base, "rotary_dim": m.rot.dims})
            mixer = PartSpec("paged_attention", {
                "hidden": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "v_head_dim": m.vdim,
                "qkv_bias": False, "scale": m.scale, "window": m.window, "names": _QKVO, "position": position})
        elif layer.type == "latent_attention":
            mixer = PartSpec("latent_attention", {
                "hidden": W, "num_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "v_head_dim": m.vdim,
                "q_rank": m.q_rank, "kv_rank": m.kv_rank, "scale": m.scale, "norm_eps": eps, "window": m.window,
                "position": PartSpec("rotary_half", {"theta": m.rot.base, "rotary_dim": m.rot.dims})})
        else:
            mixer = PartSpec("gated_delta", {"hidden": W, "num_heads": m.heads, "num_qk_heads": m.kv_heads, "head_dim": m.dim,
                                             "v_head_dim": m.vdim, "taps": m.conv, "norm_eps": eps})
        ff = None
        if isinstance(layer.mlp, DenseSizes):
            ff = PartSpec("gated_mlp", {"hidden": W, "intermediate": layer.mlp.ff, "activation": "gelu_tanh",
                                        "names": {"gate": "gate", "up": "up", "down": "down"}})
        elif layer.mlp is not None:
            ff = PartSpec("routed_experts", {"hidden": W, "inner": layer.mlp.ff, "experts": layer.mlp.experts, "top": layer.mlp.top,
                                             "activation": "silu", "gated": True, "router_bias": False, "scoring": "sigmoid",
                                             "weight_on": "input", "shared_inner": layer.mlp.shared_ff})
        block = PartSpec("sandwich_norm", {"mixer": mixer, "feed_forward": ff, "norm1": norm, "norm2": norm, "post_norm1": norm,
                                           "post_norm2": norm,
                                           "names": {"norm1": "norm1", "mixer": "mix", "norm2": "norm2", "feed_forward": "mlp"}})
        layers.append(LayerSpec(block, f"l{i}"))
    run = tuple(RunEntry(i, add_row=p) for i, p in cfg.run_order())
    return ModelSpec(
        vocab_size=cfg.vocab, hidden_size=W, layers=tuple(layers), run=run, final_norm=norm, tie_word_embeddings=False,
        embedding_prefix="embed", final_norm_prefix="final.norm", head_prefix="head",
        embedding=PartSpec("token_table", {"tensor": ""}), head=PartSpec("linear", {"tensor": ""}),
        embedding_norm=norm, embedding_norm_prefix="embed.norm",
        stream_rows=cfg.loop.times if cfg.loop is not None else 0,       # the table exists whenever the file names a loop
        stream_rows_name="loop.step", stream_rows_eps=eps)
