"""The Dobelix decoder as an arrangement of parts.

    x = table[token] * embedding_scale
    every layer:  x += norm1(mixer(x + conv(x)));  x += norm2(ffn(x))  (if it has a feed-forward)
    logits = head(norm(x)) * logit_scale

Layer i's tensors are named ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.canon1`` (the convolution in
front of the mixer), ``l<i>.mix.*`` and ``l<i>.mlp.*``; model level: ``embed``, ``final.norm``,
``head``.
"""
from __future__ import annotations

from ..config.dobelix import DobelixConfig
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec


def dobelix_spec(cfg: DobelixConfig) -> ModelSpec:
    norm = PartSpec("rms_norm", width=cfg.width, eps=cfg.eps)
    conv = PartSpec("causal_depthwise", width=cfg.width, taps=cfg.taps)
    block = PartSpec("output_norm", width=cfg.width)
    layers = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        names = {"mixer_norm.weight": p + "norm1", "mixer_conv.weight": p + "canon1"}
        if layer.type == "lightning":
            mixer = PartSpec("decay_linear_attention", width=cfg.width, heads=m.heads, key_dim=m.dim, value_dim=m.vdim,
                             decay=tuple(m.decay), activation="silu", eps=cfg.eps)
            names.update({f"mixer.{k}": p + "mix." + k for k in ("q", "k", "v", "g", "o", "norm")})
        else:
            position = PartSpec("rotary", head_dim=m.dim, rope_dim=m.rot_dims, theta=m.rot_base, scaling=None, pairing="half")
            mixer = PartSpec("sigmoid_attention", width=cfg.width, heads=m.heads, kv_heads=m.kv_heads, head_dim=m.dim,
                             position=position, scale=m.scale, chunk=m.chunk, window=None, qk_norm_eps=cfg.eps,
                             values="keys", gate=True, head_temperature=True, head_bias=True)
            names.update({"mixer.q": p + "mix.q", "mixer.k": p + "mix.k", "mixer.g": p + "mix.g", "mixer.o": p + "mix.o",
                          "mixer.q_norm": p + "mix.q.norm", "mixer.k_norm": p + "mix.k.norm",
                          "mixer.temp": p + "mix.temp", "mixer.bias": p + "mix.pb"})
        parts = {"mixer": ("mixer", mixer), "mixer_norm": ("norm", norm), "mixer_conv": ("conv", conv)}
        if layer.mlp is not None:
            parts["ffn"] = ("feed_forward", PartSpec("gated", width=cfg.width, inner=layer.mlp.ff, activation="gelu_tanh"))
            parts["ffn_norm"] = ("norm", norm)
            names.update({"ffn.gate": p + "mlp.gate", "ffn.up": p + "mlp.up", "ffn.down": p + "mlp.down",
                          "ffn_norm.weight": p + "norm2"})
        layers.append(LayerSpec(block, parts, names))
    return ModelSpec(
        width=cfg.width, vocab=cfg.vocab,
        embedding=PartSpec("token", vocab=cfg.vocab, width=cfg.width, scale=cfg.embedding_scale),
        layers=tuple(layers), schedule=ModelSpec.sequential(len(layers)), final_norm=norm,
        head=PartSpec("linear", vocab=cfg.vocab, width=cfg.width, tied=False, scale=cfg.logit_scale),
        names={"embedding.table": "embed", "final_norm.weight": "final.norm", "head.weight": "head"},
        max_positions=cfg.max_positions)


register_architecture("Dobelix", DobelixConfig.from_dict, dobelix_spec)
