"""Typed configuration of the Nudodra design, read from its own config.json keys.

A Nudodra model is a list of pre-norm layers over a residual stream that may be kept in several copies
(``streams``: hyper-connections).  A layer's mixer is of type ``attention`` (grouped-query softmax attention without
rotation, with biases, a factor on the queries that grows with the position (``q_temp``), a sigmoid gate on its output,
and optionally the keys and values of an earlier layer: ``kv_from``) or of type ``parallel`` (``left``: softmax attention
whose values are its keys as projected, with per-head norms of q and k, partly rotated heads and a sink per head;
``right``: linear attention whose state decays per key channel as every token chooses; the two meet as
``left_scale * left + right_scale * right``).  The feed-forward is a mixture of gated experts that a table assigns to
token ids, with an optional shared expert, or absent.  Every size and every constant that can differ between models comes
from the dictionary: ``vocab``, ``width``, ``streams``, ``norm.eps``, ``layers[].type / mixer / mlp``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass

from .llama import ConfigError
from .nurolorn import _need, _positive_int

MIXER_TYPES = ("attention", "parallel")
MLP_KINDS = ("moe",)


def _heads(m: dict, where: str, grouped: bool) -> None:
    for key in ("heads", "dim", "vdim") + (("kv_heads",) if grouped else ()):
        _positive_int(_need(m, key, where), f"{where}.{key}")
    if grouped and m["heads"] % m["kv_heads"]:
        raise ConfigError(f"config.json: {where}.heads {m['heads']} is not a multiple of kv_heads {m['kv_heads']}")


def _rot(rot, head: int, where: str) -> None:
    if rot is None:
        return
    dims = _need(rot, "dims", where)
    if isinstance(dims, bool) or not isinstance(dims, int) or dims % 2 or not 0 <= dims <= head:
        raise ConfigError(f"config.json: {where}.dims {dims!r} must be even and at most the head size {head}")
    if dims:
        _need(rot, "base", where)


def _attention(m: dict, where: str, index: int, layers) -> None:
    _heads(m, where, grouped=True)
    _need(m, "scale", where)
    if m.get("q_temp") is not None:
        _need(m["q_temp"], "coef", f"{where}.q_temp")
        _positive_int(_need(m["q_temp"], "every", f"{where}.q_temp"), f"{where}.q_temp.every")
    src = m.get("kv_from")
    if src is None:
        return
    if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < index:
        raise ConfigError(f"config.json: {where}.kv_from {src!r} must name an earlier layer")
    other = layers[src]
    if other.type != "attention" or other.mixer.get("kv_from") is not None:
        raise ConfigError(f"config.json: {where}.kv_from names layer {src}, which has no keys and values of its own kind")
    for key in ("kv_heads", "dim", "vdim"):
        if other.mixer.get(key) != m[key]:
            raise ConfigError(f"config.json: {where}.{key} {m[key]} differs from that of layer {src}, whose keys and values it reads")


def _parallel(m: dict, where: str) -> None:
    left, right = _need(m, "left", where), _need(m, "right", where)
    _heads(left, f"{where}.left", grouped=True)
    if left["vdim"] != left["dim"]:
        raise ConfigError(f"config.json: {where}.left.vdim {left['vdim']}: the values are the keys, so their size is dim {left['dim']}")
    _need(left, "scale", f"{where}.left")
    _rot(left.get("rot"), left["dim"], f"{where}.left.rot")
    _heads(right, f"{where}.right", grouped=False)
    if not float(_need(right, "tau", f"{where}.right")) > 0:
        raise ConfigError(f"config.json: {where}.right.tau must be positive")
    if right.get("rank") is not None:
        _positive_int(right["rank"], f"{where}.right.rank")
    for key in ("left_scale", "right_scale"):
        _need(m, key, where)


def _mlp(mlp: dict, where: str) -> None:
    kind = _need(mlp, "kind", where)
    if kind not in MLP_KINDS:
        raise ConfigError(f"config.json: {where}.kind {kind!r} is not built; known: {list(MLP_KINDS)}")
    router = _need(mlp, "router", where)
    experts = _positive_int(_need(router, "experts", f"{where}.router"), f"{where}.router.experts")
    top = _positive_int(_need(router, "top", f"{where}.router"), f"{where}.router.top")
    if top > experts:
        raise ConfigError(f"config.json: {where}.router.top {top} exceeds the {experts} experts")
    for name in ("expert",) + (("shared",) if mlp.get("shared") else ()):
        part = _need(mlp, name, where)
        _positive_int(_need(part, "ff", f"{where}.{name}"), f"{where}.{name}.ff")
        if not float(_need(part, "limit", f"{where}.{name}")) > 0:
            raise ConfigError(f"config.json: {where}.{name}.limit must be positive")


@dataclass(frozen=True)
class NudodraLayer:
    type: str  # one of MIXER_TYPES
    mixer: dict  # the mixer's sizes and constants, as config.json gives them
    mlp: dict | None  # {"kind": "moe", "router", "expert", "shared"} | None


@dataclass(frozen=True)
class NudodraConfig:
    vocab_size: int  # [vocab]
    width: int  # [width]
    layers: tuple[NudodraLayer, ...]  # [layers]
    norm_eps: float  # [norm.eps]
    streams: int | None  # [streams]: copies of the residual stream; None (the key is absent): one plain stream
    max_positions: int | None = None  # not a key of the design: an engine may bound a request's length with it

    architecture = "Nudodra"

    def __post_init__(self) -> None:
        _positive_int(self.vocab_size, "vocab")
        _positive_int(self.width, "width")
        if self.streams is not None and _positive_int(self.streams, "streams") > 8:
            raise ConfigError(f"config.json: streams {self.streams}: at most eight copies of the stream are built")
        if not self.norm_eps >= 0:
            raise ConfigError("config.json: norm.eps must not be negative")
        if not self.layers:
            raise ConfigError("config.json: layers is empty")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if layer.type not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}.type {layer.type!r} is not a mixer of this design; known: {list(MIXER_TYPES)}")
            if layer.type == "attention":
                _attention(layer.mixer, f"{where}.mixer", i, self.layers)
            else:
                _parallel(layer.mixer, f"{where}.mixer")
            if layer.mlp is not None:
                _mlp(layer.mlp, f"{where}.mlp")

    @classmethod
    def from_dict(cls, d: dict) -> "NudodraConfig":
        layers = []
        for i, entry in enumerate(_need(d, "layers", "the configuration")):
            where = f"layers[{i}]"
            mlp = entry.get("mlp") if isinstance(entry, dict) else None
            layers.append(NudodraLayer(_need(entry, "type", where), copy.deepcopy(_need(entry, "mixer", where)), copy.deepcopy(mlp) if mlp else None))
        limit = d.get("max_positions")
        return cls(
            vocab_size=_need(d, "vocab", "the configuration"),
            width=_need(d, "width", "the configuration"),
            layers=tuple(layers),
            norm_eps=float(_need(_need(d, "norm", "the configuration"), "eps", "norm")),
            streams=d.get("streams"),
            max_positions=None if limit is None else int(limit),
        )

    def to_dict(self) -> dict:
        """The config.json this configuration is read back from."""
        d = {
            "architecture": self.architecture,
            "layers": [{"type": x.type, "mixer": copy.deepcopy(x.mixer), "mlp": copy.deepcopy(x.mlp)} for x in self.layers],
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab_size,
            "width": self.width,
        }
        if self.streams is not None:
            d["streams"] = self.streams
        if self.max_positions is not None:
            d["max_positions"] = self.max_positions
        return d
