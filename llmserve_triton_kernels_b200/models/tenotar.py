"""Tenotar as data: which parts each layer has, from a :class:`TenotarConfig`.

Every layer is a pre-norm block with RMS norms (``l<i>.norm1``, ``l<i>.norm2``); a layer whose ``mlp`` is null has no
feed-forward.  The mixers are parts with parameters of their own:

* ``latent_attention`` (parts/latent_attention.py) with a latent for the queries, the half layout of the rotated lanes,
  a sliding window and one gate a head;
* ``attention`` = ``softmax_attention`` (parts/softmax_attention.py) with biases on q, k, v and o, per-head norms,
  interleaved rotation and a window that keeps the first tokens;
* ``attention_2`` = ``softmax_attention`` with a short convolution behind q, k and v, capped scores, a distance bias of
  slope ``2^(-8 (h+1) / heads)`` and keys of the query's own block of positions.

The first layer with ``v_mix`` is the source of the values that every later such layer mixes into its own.  The
feed-forward is ``gated_mlp`` with biases or ``routed_gated_mlp`` (parts/feed_forward.py).  The logits are the output
matrix's product times ``logit_scale``.  Tensor names: ``embed``, ``head``, ``final.norm``, and per layer ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""

from __future__ import annotations

from ..config.registry import register_architecture
from ..config.tenotar import TenotarConfig
from ..parts.base import PartSpec
from .plan import LayerRun, LayerSpec, ModelPlan

DISTANCE_BIAS = 8.0  # the design fixes it: head h's scores lose 2^(-8 (h+1) / heads) per position of distance


def _value_mix(index: int, m: dict, source: int | None) -> str | None:
    if not m.get("v_mix"):
        return None
    return "source" if index == source else "mixed"


def _mixer(cfg: TenotarConfig, index: int, layer, prefix: str) -> PartSpec:
    m, source = layer.mixer, cfg.value_mix_source()
    if layer.type == "latent_attention":
        return PartSpec("latent_attention", {
            "hidden_size": cfg.width, "num_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"], "value_dim": m["vdim"],
            "rank": m["kv_rank"], "scale": float(m["scale"]), "rotary_base": float(m["rot"].get("base", 10000.0)),
            "rotary_dims": m["rot"]["dims"], "norm_eps": cfg.norm_eps, "output_gate": True, "gate_per_head": True,
            "query_rank": m["q_rank"], "rotary_layout": "half", "window": m["mask"]["size"],
        }, prefix)
    common = {
        "hidden_size": cfg.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"], "value_dim": m["vdim"],
        "scale": float(m["scale"]), "value_mix": _value_mix(index, m, source),
    }
    if layer.type == "attention":
        return PartSpec("softmax_attention", {
            **common, "bias": True, "out_bias": True, "qk_norm_eps": cfg.norm_eps, "rotary": m.get("rot"), "rotary_layout": "interleaved",
            "window": m["mask"]["size"], "keep_first": m["mask"].get("keep_first"),
        }, prefix)
    return PartSpec("softmax_attention", {
        **common, "conv": m["conv"], "softcap": m.get("softcap"), "distance_bias": DISTANCE_BIAS, "chunk": m["mask"]["size"],
    }, prefix)


def _feed_forward(cfg: TenotarConfig, mlp: dict, prefix: str) -> PartSpec:
    if mlp["kind"] == "dense":
        names = {"gate": "gate", "up": "up", "down": "down", "gate_bias": "gate.b", "up_bias": "up.b", "down_bias": "down.b"}
        return PartSpec("gated_mlp", {"hidden_size": cfg.width, "intermediate_size": mlp["ff"], "bias": True, "tensor_names": names}, prefix)
    shared = mlp.get("shared")
    return PartSpec("routed_gated_mlp", {
        "hidden_size": cfg.width, "experts": mlp["router"]["experts"], "top": mlp["router"]["top"], "expert_size": mlp["expert"]["ff"],
        "shared_size": shared["ff"] if shared else None,
    }, prefix)


def tenotar_plan(cfg: TenotarConfig) -> ModelPlan:
    norm = {"size": cfg.width, "eps": cfg.norm_eps}
    layers, ignored = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        parts = {"mixer_norm": PartSpec("rms_norm", {**norm, "weight_name": "norm1"}, p), "mixer": _mixer(cfg, i, layer, p + "mix.")}
        if layer.type != "latent_attention" and not layer.mixer.get("v_mix"):
            ignored.append(p + "mix.vmix")  # a checkpoint may carry the mixing weight of a layer that does not mix
        if layer.mlp is None:
            kind = "pre_norm_mixer_only"
            ignored.append(p + "norm2")  # no feed-forward: no use for the norm in front of one
        else:
            kind = "pre_norm"
            parts["ff_norm"] = PartSpec("rms_norm", {**norm, "weight_name": "norm2"}, p)
            parts["feed_forward"] = _feed_forward(cfg, layer.mlp, p + "mlp.")
        layers.append(LayerSpec(PartSpec(kind, {}, p), parts))
    return ModelPlan(
        hidden_size=cfg.width,
        vocab_size=cfg.vocab_size,
        max_positions=cfg.max_positions,
        embedding="embed",
        layers=tuple(layers),
        schedule=tuple(LayerRun(i) for i in range(len(layers))),
        final_norm=PartSpec("rms_norm", {**norm, "weight_name": "norm"}, "final."),
        head="head",
        ignored=tuple(ignored),
        logit_scale=cfg.logit_scale,
    )


register_architecture("Tenotar", TenotarConfig, tenotar_plan)
