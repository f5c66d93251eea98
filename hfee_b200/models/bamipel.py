"""The Bamipel decoder as an arrangement of parts.

    x = table[token]
    every layer:  x += norm1b(mixer(norm1(x)));  x += norm2b(ffn(norm2(x)))  (if it has a feed-forward)
    logits = head(norm(x))

Layer i's tensors are named ``l<i>.norm1``, ``l<i>.norm1b``, ``l<i>.norm2``, ``l<i>.norm2b``, ``l<i>.mix.*`` and
``l<i>.mlp.*``; model level: ``embed``, ``final.norm``, ``head``.  A layer with ``weights_of`` has no tensors: the
schedule runs the named layer once more with a cache of its own.
"""
from __future__ import annotations

from ..config.bamipel import BamipelConfig
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunSpec


def _mixer(cfg: BamipelConfig, layer, p: str):
    m = layer.mixer
    if layer.type == "attention":
        position = PartSpec("rotary", head_dim=m.dim, rope_dim=m.rot.dims, theta=m.rot.base, scaling=m.rot.scaling, pairing="half")
        spec = PartSpec("gated_attention", width=cfg.width, heads=m.heads, kv_heads=m.kv_heads, head_dim=m.dim,
                        value_dim=m.vdim, position=position, scale=m.scale, window=m.window, qk_unit_norm_eps=cfg.eps,
                        gate="head")
        keys = ("q", "k", "v", "g", "o")
    elif layer.type == "latent_attention":
        position = PartSpec("rotary", head_dim=m.rot_dim, rope_dim=m.rot.dims, theta=m.rot.base, scaling=m.rot.scaling,
                            pairing="half")
        spec = PartSpec("latent_attention", width=cfg.width, heads=m.heads, head_dim=m.dim, rope_dim=m.rot_dim,
                        value_dim=m.vdim, q_rank=m.q_rank, kv_rank=m.kv_rank, position=position, scale=m.scale,
                        window=m.window, eps=cfg.eps, gate="head")
        keys = ("dq", "dq_norm", "uq", "dkv", "dkv_norm", "uk", "uv", "g", "o")
    else:
        spec = PartSpec("gated_delta_rule", width=cfg.width, heads=m.heads, qk_heads=m.kv_heads, key_dim=m.dim,
                        value_dim=m.vdim, taps=m.taps, eps=cfg.eps)
        keys = ("q", "k", "v", "q_conv", "k_conv", "v_conv", "b", "a", "A_log", "dt_bias", "norm", "g", "o")
    stored = {"dq_norm": "dq.norm", "dkv_norm": "dkv.norm", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv"}
    return spec, {f"mixer.{k}": p + "mix." + stored.get(k, k) for k in keys}


def bamipel_spec(cfg: BamipelConfig) -> ModelSpec:
    norm = PartSpec("rms_norm", width=cfg.width, eps=cfg.eps)
    block = PartSpec("sandwich_norm", width=cfg.width)
    layers, index_of = [], {}
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is not None:
            continue
        p = f"l{i}."
        mixer, names = _mixer(cfg, layer, p)
        names.update({"mixer_norm.weight": p + "norm1", "mixer_out_norm.weight": p + "norm1b"})
        parts = {"mixer": ("mixer", mixer), "mixer_norm": ("norm", norm), "mixer_out_norm": ("norm", norm)}
        if layer.mlp is not None:
            parts["ffn"] = ("feed_forward", PartSpec("dense", width=cfg.width, inner=layer.mlp.ff, activation="relu2"))
            parts["ffn_norm"] = ("norm", norm)
            parts["ffn_out_norm"] = ("norm", norm)
            names.update({"ffn.up": p + "mlp.up", "ffn.down": p + "mlp.down", "ffn_norm.weight": p + "norm2",
                          "ffn_out_norm.weight": p + "norm2b"})
        index_of[i] = len(layers)
        layers.append(LayerSpec(block, parts, names))
    # every entry of the configuration runs once, in order, with a cache of its own
    schedule = tuple(RunSpec(layer=index_of[i if layer.weights_of is None else layer.weights_of], cache=i)
                     for i, layer in enumerate(cfg.layers))
    return ModelSpec(
        width=cfg.width, vocab=cfg.vocab,
        embedding=PartSpec("token", vocab=cfg.vocab, width=cfg.width),
        layers=tuple(layers), schedule=schedule, final_norm=norm,
        head=PartSpec("linear", vocab=cfg.vocab, width=cfg.width, tied=False),
        names={"embedding.table": "embed", "final_norm.weight": "final.norm", "head.weight": "head"},
        max_positions=cfg.max_positions)


register_architecture("Bamipel", BamipelConfig.from_dict, bamipel_spec)
