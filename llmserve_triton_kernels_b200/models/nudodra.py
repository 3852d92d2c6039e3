"""Nudodra as data: which parts each layer has, from a :class:`NudodraConfig`.

Every layer is a pre-norm block with RMS norms (``l<i>.norm1``, ``l<i>.norm2``).  With ``streams`` the residual stream
is kept in that many copies and the block is the hyper-connection one (parts/block.py: ``l<i>.hc1.*`` around the mixer,
``l<i>.hc2.*`` around the feed-forward); without, the plain pre-norm block.  A layer of type ``attention`` has the
``softmax_attention`` mixer (parts/softmax_attention.py) with biases, the queries' factor ``q_temp`` and an output gate;
with ``kv_from: j`` it has no key and value projections and its entry of the order reads the pages of layer j's entry.
A layer of type ``parallel`` has the ``parallel`` mixer (parts/parallel.py) without output norms: ``left`` =
``softmax_attention`` whose values are its keys, with per-head norms, partly rotated heads and sinks; ``right`` =
``gated_linear_attention`` (parts/recurrent.py); they meet as ``left_scale * left + right_scale * right``.  The
feed-forward is ``table_routed_mlp`` (parts/feed_forward.py), or absent.  Tensor names: ``embed``, ``head``,
``final.norm``, and per layer ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.hc1.*``, ``l<i>.hc2.*``.
"""

from __future__ import annotations

from ..config.nudodra import NudodraConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from .plan import LayerRun, LayerSpec, ModelPlan

EXPERT_SLOPE = 1.702  # the design fixes it: an expert's activation is g * sigmoid(1.702 g) * (u + 1)


def _attention(cfg: NudodraConfig, m: dict, prefix: str) -> PartSpec:
    return PartSpec("softmax_attention", {
        "hidden_size": cfg.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"], "value_dim": m["vdim"],
        "scale": float(m["scale"]), "bias": True, "q_temp": m.get("q_temp"), "gate": True, "own_kv": m.get("kv_from") is None,
        "window": m.get("window"),
    }, prefix)


def _parallel(cfg: NudodraConfig, m: dict, prefix: str) -> PartSpec:
    left, right = m["left"], m["right"]
    attention = PartSpec("softmax_attention", {
        "hidden_size": cfg.width, "num_heads": left["heads"], "num_kv_heads": left["kv_heads"], "head_dim": left["dim"],
        "value_dim": left["vdim"], "scale": float(left["scale"]), "bias": True, "qk_norm_eps": cfg.norm_eps, "rotary": left.get("rot"),
        "sink": True, "values_are_keys": True, "window": left.get("window"),
    })
    recurrence = PartSpec("gated_linear_attention", {
        "hidden_size": cfg.width, "num_heads": right["heads"], "head_dim": right["dim"], "value_dim": right["vdim"],
        "tau": float(right["tau"]), "norm_eps": cfg.norm_eps, "decay_rank": right.get("rank"),
    })
    params = {"hidden_size": cfg.width, "branches": {"left": attention, "right": recurrence}, "norm_eps": cfg.norm_eps,
              "branch_norm": False, "scales": [float(m["left_scale"]), float(m["right_scale"])]}
    return PartSpec("parallel", params, prefix)


def _feed_forward(cfg: NudodraConfig, mlp: dict, prefix: str) -> PartSpec:
    shared = mlp.get("shared")
    return PartSpec("table_routed_mlp", {
        "hidden_size": cfg.width, "vocab_size": cfg.vocab_size, "experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
        "expert_size": mlp["expert"]["ff"], "limit": float(mlp["expert"]["limit"]), "shared_size": shared["ff"] if shared else None,
        "shared_limit": float(shared["limit"]) if shared else None, "slope": EXPERT_SLOPE,
    }, prefix)


def nudodra_plan(cfg: NudodraConfig) -> ModelPlan:
    norm = {"size": cfg.width, "eps": cfg.norm_eps}
    hyper = cfg.streams is not None
    layers, schedule, ignored = [], [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        mixer = _attention(cfg, layer.mixer, p + "mix.") if layer.type == "attention" else _parallel(cfg, layer.mixer, p + "mix.")
        parts = {"mixer_norm": PartSpec("rms_norm", {**norm, "weight_name": "norm1"}, p), "mixer": mixer}
        if layer.mlp is None:
            kind = "hyper_connection_mixer_only" if hyper else "pre_norm_mixer_only"
            ignored += [p + "norm2"] + [f"{p}hc2.{k}" for k in ("in", "out", "mix")]  # no feed-forward: no use for what surrounds one
        else:
            kind = "hyper_connection" if hyper else "pre_norm"
            parts["ff_norm"] = PartSpec("rms_norm", {**norm, "weight_name": "norm2"}, p)
            parts["feed_forward"] = _feed_forward(cfg, layer.mlp, p + "mlp.")
        layers.append(LayerSpec(PartSpec(kind, {"streams": cfg.streams} if hyper else {}, p), parts))
        # layers run once, in order: entry i of the order is layer i, and so is the entry whose pages ``kv_from`` names
        schedule.append(LayerRun(i, cache_of=layer.mixer.get("kv_from") if layer.type == "attention" else None))
    return ModelPlan(
        hidden_size=cfg.width,
        vocab_size=cfg.vocab_size,
        max_positions=cfg.max_positions,
        embedding="embed",
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=PartSpec("rms_norm", {**norm, "weight_name": "norm"}, "final."),
        head="head",
        ignored=tuple(ignored),
        streams=cfg.streams,
    )


register_architecture("Nudodra", NudodraConfig, nudodra_plan)
