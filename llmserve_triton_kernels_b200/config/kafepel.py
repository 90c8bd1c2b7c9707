"""Typed configuration of the Kafepel design, read from its own config.json keys.

A Kafepel model is a list of pre-norm layers.  Every layer's mixer is of type ``parallel``: an attention branch
(``left``: grouped-query attention with sigmoid weights, a norm over the whole query and key projections, rotary
positions with optional frequency scaling, a capped score, a bias per head and mixed heads) beside a retention branch
(``right``: a decaying matrix of state per head), their outputs RMS-normed and averaged.  The feed-forward is dense
and gated (``kind: dense``), a mixture of experts with an optional shared expert (``kind: moe``), or absent.  Every
size and every constant that can differ between models comes from the dictionary: ``vocab``, ``width``,
``embedding.scale``, ``norm.eps``, ``layers[].type / mixer / mlp``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass

from .llama import ConfigError
from .nurolorn import _need, _positive_int

MIXER_TYPES = ("parallel",)
MLP_KINDS = ("dense", "moe")


def _rot(rot, head: int, where: str) -> None:
    if rot is None:
        return
    dims = _need(rot, "dims", where)
    if isinstance(dims, bool) or not isinstance(dims, int) or dims % 2 or not 0 <= dims <= head:
        raise ConfigError(f"config.json: {where}.dims {dims!r} must be even and at most the head size {head}")
    if dims:
        _need(rot, "base", where)
    scaling = rot.get("scaling")
    if scaling:
        for key in ("factor", "low", "high", "original"):
            _need(scaling, key, f"{where}.scaling")


@dataclass(frozen=True)
class KafepelLayer:
    type: str  # one of MIXER_TYPES
    mixer: dict  # {"left": {...}, "right": {...}} as config.json gives them
    mlp: dict | None  # {"kind": "dense", "ff"} | {"kind": "moe", "expert", "router", "shared"} | None


@dataclass(frozen=True)
class KafepelConfig:
    vocab_size: int  # [vocab]
    width: int  # [width]
    layers: tuple[KafepelLayer, ...]  # [layers]
    norm_eps: float  # [norm.eps]
    embedding_scale: float  # [embedding.scale]
    max_positions: int | None = None  # not a key of the design: an engine may bound a request's length with it

    architecture = "Kafepel"

    def __post_init__(self) -> None:
        _positive_int(self.vocab_size, "vocab")
        _positive_int(self.width, "width")
        if not self.norm_eps >= 0:
            raise ConfigError("config.json: norm.eps must not be negative")
        if not self.layers:
            raise ConfigError("config.json: layers is empty")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if layer.type not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}.type {layer.type!r} is not a mixer of this design; known: {list(MIXER_TYPES)}")
            left, right = _need(layer.mixer, "left", f"{where}.mixer"), _need(layer.mixer, "right", f"{where}.mixer")
            for key in ("heads", "kv_heads", "dim", "vdim"):
                _positive_int(_need(left, key, f"{where}.mixer.left"), f"{where}.mixer.left.{key}")
            if left["heads"] % left["kv_heads"]:
                raise ConfigError(f"config.json: {where}.mixer.left.heads {left['heads']} is not a multiple of kv_heads {left['kv_heads']}")
            _need(left, "scale", f"{where}.mixer.left")
            _rot(left.get("rot"), left["dim"], f"{where}.mixer.left.rot")
            for key in ("heads", "dim", "vdim"):
                _positive_int(_need(right, key, f"{where}.mixer.right"), f"{where}.mixer.right.{key}")
            decay = _need(right, "decay", f"{where}.mixer.right")
            if not isinstance(decay, (list, tuple)) or len(decay) != right["heads"]:
                raise ConfigError(f"config.json: {where}.mixer.right.decay must list one decay for each of the {right['heads']} heads")
            _rot(right.get("rot"), right["dim"], f"{where}.mixer.right.rot")
            mlp = layer.mlp
            if mlp is None:
                continue
            kind = _need(mlp, "kind", f"{where}.mlp")
            if kind not in MLP_KINDS:
                raise ConfigError(f"config.json: {where}.mlp.kind {kind!r} is not built; known: {list(MLP_KINDS)}")
            if kind == "dense":
                _positive_int(_need(mlp, "ff", f"{where}.mlp"), f"{where}.mlp.ff")
            else:
                router = _need(mlp, "router", f"{where}.mlp")
                experts = _positive_int(_need(router, "experts", f"{where}.mlp.router"), f"{where}.mlp.router.experts")
                top = _positive_int(_need(router, "top", f"{where}.mlp.router"), f"{where}.mlp.router.top")
                if top > experts:
                    raise ConfigError(f"config.json: {where}.mlp.router.top {top} exceeds the {experts} experts")
                _positive_int(_need(_need(mlp, "expert", f"{where}.mlp"), "ff", f"{where}.mlp.expert"), f"{where}.mlp.expert.ff")
                if mlp.get("shared"):
                    _positive_int(_need(mlp["shared"], "ff", f"{where}.mlp.shared"), f"{where}.mlp.shared.ff")

    @classmethod
    def from_dict(cls, d: dict) -> "KafepelConfig":
        layers = []
        for i, entry in enumerate(_need(d, "layers", "the configuration")):
            where = f"layers[{i}]"
            mlp = entry.get("mlp") if isinstance(entry, dict) else None
            layers.append(KafepelLayer(_need(entry, "type", where), copy.deepcopy(_need(entry, "mixer", where)), copy.deepcopy(mlp) if mlp else None))
        norm = _need(d, "norm", "the configuration")
        limit = d.get("max_positions")
        return cls(
            vocab_size=_need(d, "vocab", "the configuration"),
            width=_need(d, "width", "the configuration"),
            layers=tuple(layers),
            norm_eps=float(_need(norm, "eps", "norm")),
            embedding_scale=float((d.get("embedding") or {}).get("scale", 1.0)),
            max_positions=None if limit is None else int(limit),
        )

    def to_dict(self) -> dict:
        """The config.json this configuration is read back from."""
        d = {
            "architecture": self.architecture,
            "embedding": {"scale": self.embedding_scale},
            "layers": [{"type": x.type, "mixer": copy.deepcopy(x.mixer), "mlp": copy.deepcopy(x.mlp)} for x in self.layers],
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab_size,
            "width": self.width,
        }
        if self.max_positions is not None:
            d["max_positions"] = self.max_positions
        return d
