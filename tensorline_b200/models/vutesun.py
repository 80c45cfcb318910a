"""The Vutesun decoder as a `ModelSpec`.

Every layer is a pre-norm block whose sub-blocks count `residual_mult` times in the residual sum; its norms are
RMS norms in float32 with a weight stored around zero (x / rms(x) * (1 + w)).  A layer's mixer is either the
matrix memory of the xLSTM (`mlstm`) or a pair of mixers side by side (`parallel`): grouped-query attention with
biases, interleaved rotary pairs, a scale of its own and a learned sink per head, beside a retention layer with
rotate-half pairs; each output is RMS-normalised over the width and the two are averaged.  The feed-forward,
where a layer has one, is a mixture of experts with relu^2 experts and a softmax over the chosen logits.  The
model's norm and an untied head follow.  Tensor names: `embed`, `l<i>.norm1`, `l<i>.mix.*`, `l<i>.norm2`,
`l<i>.mlp.*`, `final.norm`, `head`, each tensor under its own name (no `.weight` suffix), biases with `.b`.
"""
from __future__ import annotations

from ..config.vutesun import VutesunConfig
from ..parts import PartSpec
from .spec import LayerSpec, ModelSpec, RunEntry

_ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "sink": "sink"}


def describe_vutesun(cfg: VutesunConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    norm = PartSpec("rms_norm", {"dim": W, "eps": eps, "tensor": "", "one_plus": True, "cast_first": False})
    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if layer.type == "mlstm":
            mixer = PartSpec("mlstm", {"hidden": W, "num_heads": m.heads, "head_dim": m.dim, "v_head_dim": m.vdim,
                                       "gate_cap": m.gate_cap, "norm_eps": eps})
        else:
            a, b = m.left, m.right
            left = PartSpec("paged_attention", {
                "hidden": W, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim, "v_head_dim": a.vdim,
                "qkv_bias": True, "scale": a.scale, "sink": True, "names": _ATTENTION_NAMES,
                "position": PartSpec("rotary_interleaved", {"theta": a.rot.base, "rotary_dim": a.rot.dims})})
            right = PartSpec("retention", {
                "hidden": W, "num_heads": b.heads, "head_dim": b.dim, "v_head_dim": b.vdim, "decay": b.decay, "norm_eps": eps,
                "position": PartSpec("rotary_half", {"theta": b.rot.base, "rotary_dim": b.rot.dims})})
            mixer = PartSpec("parallel_pair", {"hidden": W, "left": left, "right": right, "norm_eps": eps, "scale": 0.5})
        ff = None
        if layer.mlp is not None:
            ff = PartSpec("routed_experts", {"hidden": W, "inner": layer.mlp.ff, "experts": layer.mlp.experts,
                                             "top": layer.mlp.top, "activation": "relu_squared"})
        block = PartSpec("pre_norm", {"mixer": mixer, "feed_forward": ff, "norm1": norm, "norm2": norm,
                                      "residual_scale": cfg.residual_mult,
                                      "names": {"norm1": "norm1", "mixer": "mix", "norm2": "norm2", "feed_forward": "mlp"}})
        layers.append(LayerSpec(block, f"l{i}"))
    return ModelSpec(
        vocab_size=cfg.vocab, hidden_size=W, layers=tuple(layers), run=tuple(RunEntry(i) for i in range(len(layers))),
        final_norm=norm, tie_word_embeddings=False, embedding_prefix="embed", final_norm_prefix="final.norm",
        head_prefix="head", embedding=PartSpec("token_table", {"tensor": ""}), head=PartSpec("linear", {"tensor": ""}))
