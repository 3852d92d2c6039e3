"""Typed configuration of the Tenotar design, read from its own config.json keys.

A Tenotar model is a list of pre-norm layers.  A layer's mixer is one of three kinds of softmax attention:
``latent_attention`` (queries, keys and values through low-rank latents, a rotated key part shared by the heads, a sliding
window, a sigmoid gate per head), ``attention`` (grouped-query attention with biases, per-head norms of q and k,
neighbouring lanes rotated, a sliding window that also keeps the first tokens) and ``attention_2`` (grouped-query
attention whose q, k and v pass a short causal convolution, with capped scores, a distance bias per head and keys of the
query's own block of positions only).  Layers with ``v_mix`` take up the values that the first such layer computed for
the same token.  The feed-forward is dense (gated, with biases) or a mixture of gated experts under a router with a
bias, with an optional shared expert, or absent.  Every size and every constant that can differ between models comes
from the dictionary: ``vocab``, ``width``, ``norm.eps``, ``logit_scale``, ``layers[].type / mixer / mlp``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass

from .llama import ConfigError
from .nurolorn import _need, _positive_int

MIXER_TYPES = ("latent_attention", "attention", "attention_2")
MLP_KINDS = ("dense", "moe")


def _rot(rot, most: int, where: str) -> None:
    if rot is None:
        return
    dims = _need(rot, "dims", where)
    if isinstance(dims, bool) or not isinstance(dims, int) or dims % 2 or not 0 <= dims <= most:
        raise ConfigError(f"config.json: {where}.dims {dims!r} must be even and at most {most}")
    if dims:
        _need(rot, "base", where)


def _mask(m: dict, where: str) -> None:
    mask = _need(m, "mask", where)
    _positive_int(_need(mask, "size", f"{where}.mask"), f"{where}.mask.size")
    keep = mask.get("keep_first")
    if keep is not None and (isinstance(keep, bool) or not isinstance(keep, int) or keep < 0):
        raise ConfigError(f"config.json: {where}.mask.keep_first {keep!r} must be a count of tokens")


def _mixer(kind: str, m: dict, where: str) -> None:
    for key in ("heads", "dim", "vdim"):
        _positive_int(_need(m, key, where), f"{where}.{key}")
    _need(m, "scale", where)
    _mask(m, where)
    if kind == "latent_attention":
        for key in ("kv_rank", "rot_dim", "q_rank"):
            _positive_int(_need(m, key, where), f"{where}.{key}")
        _rot(_need(m, "rot", where), m["rot_dim"], f"{where}.rot")
        return
    _positive_int(_need(m, "kv_heads", where), f"{where}.kv_heads")
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"config.json: {where}.heads {m['heads']} is not a multiple of kv_heads {m['kv_heads']}")
    if kind == "attention":
        _rot(m.get("rot"), m["dim"], f"{where}.rot")
    else:
        taps = _positive_int(_need(m, "conv", where), f"{where}.conv")
        if taps > 16:
            raise ConfigError(f"config.json: {where}.conv {taps}: convolutions of up to 16 taps are built")
        if m.get("softcap") is not None and not float(m["softcap"]) > 0:
            raise ConfigError(f"config.json: {where}.softcap must be positive")


def _mlp(mlp: dict, where: str) -> None:
    kind = _need(mlp, "kind", where)
    if kind not in MLP_KINDS:
        raise ConfigError(f"config.json: {where}.kind {kind!r} is not built; known: {list(MLP_KINDS)}")
    if kind == "dense":
        _positive_int(_need(mlp, "ff", where), f"{where}.ff")
        return
    router = _need(mlp, "router", where)
    experts = _positive_int(_need(router, "experts", f"{where}.router"), f"{where}.router.experts")
    top = _positive_int(_need(router, "top", f"{where}.router"), f"{where}.router.top")
    if top > experts:
        raise ConfigError(f"config.json: {where}.router.top {top} exceeds the {experts} experts")
    for name in ("expert",) + (("shared",) if mlp.get("shared") else ()):
        _positive_int(_need(_need(mlp, name, where), "ff", f"{where}.{name}"), f"{where}.{name}.ff")


@dataclass(frozen=True)
class TenotarLayer:
    type: str  # one of MIXER_TYPES
    mixer: dict  # the mixer's sizes and constants, as config.json gives them
    mlp: dict | None  # {"kind": "dense", "ff"} | {"kind": "moe", "router", "expert", "shared"} | None


@dataclass(frozen=True)
class TenotarConfig:
    vocab_size: int  # [vocab]
    width: int  # [width]
    layers: tuple[TenotarLayer, ...]  # [layers]
    norm_eps: float  # [norm.eps]
    logit_scale: float  # [logit_scale]
    max_positions: int | None = None  # not a key of the design: an engine may bound a request's length with it

    architecture = "Tenotar"

    def __post_init__(self) -> None:
        _positive_int(self.vocab_size, "vocab")
        _positive_int(self.width, "width")
        if not self.norm_eps >= 0:
            raise ConfigError("config.json: norm.eps must not be negative")
        if not self.layers:
            raise ConfigError("config.json: layers is empty")
        shared_values = None
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if layer.type not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}.type {layer.type!r} is not a mixer of this design; known: {list(MIXER_TYPES)}")
            _mixer(layer.type, layer.mixer, f"{where}.mixer")
            if layer.mlp is not None:
                _mlp(layer.mlp, f"{where}.mlp")
            if layer.mixer.get("v_mix"):
                if layer.type == "latent_attention":
                    raise ConfigError(f"config.json: {where}.mixer.v_mix: a layer whose values come from a latent has none to mix")
                size = layer.mixer["kv_heads"] * layer.mixer["vdim"]
                if shared_values is not None and size != shared_values:
                    raise ConfigError(f"config.json: {where}.mixer: kv_heads * vdim = {size} differs from the {shared_values} of the first layer with v_mix")
                shared_values = size

    def value_mix_source(self) -> int | None:
        """The first layer with ``v_mix``: the one whose values the others take up."""
        return next((i for i, layer in enumerate(self.layers) if layer.mixer.get("v_mix")), None)

    @classmethod
    def from_dict(cls, d: dict) -> "TenotarConfig":
        layers = []
        for i, entry in enumerate(_need(d, "layers", "the configuration")):
            where = f"layers[{i}]"
            mlp = entry.get("mlp") if isinstance(entry, dict) else None
            layers.append(TenotarLayer(_need(entry, "type", where), copy.deepcopy(_need(entry, "mixer", where)), copy.deepcopy(mlp) if mlp else None))
        limit = d.get("max_positions")
        return cls(
            vocab_size=_need(d, "vocab", "the configuration"),
            width=_need(d, "width", "the configuration"),
            layers=tuple(layers),
            norm_eps=float(_need(_need(d, "norm", "the configuration"), "eps", "norm")),
            logit_scale=float(d.get("logit_scale", 1.0)),
            max_positions=None if limit is None else int(limit),
        )

    def to_dict(self) -> dict:
        """The config.json this configuration is read back from."""
        d = {
            "architecture": self.architecture,
            "layers": [{"type": x.type, "mixer": copy.deepcopy(x.mixer), "mlp": copy.deepcopy(x.mlp)} for x in self.layers],
            "logit_scale": self.logit_scale,
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab_size,
            "width": self.width,
        }
        if self.max_positions is not None:
            d["max_positions"] = self.max_positions
        return d
