"""Typed configuration of the Nurolorn design, read from its own config.json keys.

A Nurolorn model is a list of pre-norm layers, each with one of three mixers (attention through a low-rank latent,
a minGRU recurrence, sliding-window attention with a distance bias) and an optional dense feed-forward; a stretch of
the layers may run several times with the same weights.  Every size and every constant that can differ between
models of the design comes from the dictionary: ``vocab``, ``width``, ``layers`` (``type``, ``mixer``, ``mlp``),
``loop`` (``start``, ``stop``, ``times``), ``norm`` (``eps``, ``groups``), ``residual_mult``, ``logit_scale``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass

from .llama import ConfigError

MIXERS = {
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot"),
    "mingru": ("width",),
    "attention": ("heads", "kv_heads", "dim", "vdim", "scale", "mask"),
}


def _need(d: dict, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config.json: {where} is missing the key {key!r}")
    return d[key]


def _positive_int(value, what: str) -> int:
    if isinstance(value, bool) or not isinstance(value, int) or value < 1:
        raise ConfigError(f"config.json: {what} must be a positive integer, got {value!r}")
    return value


@dataclass(frozen=True)
class NurolornLayer:
    type: str  # one of MIXERS
    mixer: dict  # the mixer's sizes and constants, as config.json gives them
    mlp: dict | None  # {"kind": "dense", "ff": ...} or None: no feed-forward


@dataclass(frozen=True)
class NurolornConfig:
    vocab_size: int  # [vocab]
    width: int  # [width]
    layers: tuple[NurolornLayer, ...]  # [layers]
    loop: tuple[int, int, int] | None  # [loop]: (start, stop, times); None: every layer runs once
    norm_eps: float  # [norm.eps]
    norm_groups: int  # [norm.groups]
    residual_mult: float  # [residual_mult]
    logit_scale: float  # [logit_scale]
    max_positions: int | None = None  # not a key of the design: an engine may bound a request's length with it

    architecture = "Nurolorn"

    def __post_init__(self) -> None:
        _positive_int(self.vocab_size, "vocab")
        _positive_int(self.width, "width")
        _positive_int(self.norm_groups, "norm.groups")
        if self.width % self.norm_groups:
            raise ConfigError(f"config.json: width {self.width} does not split into norm.groups = {self.norm_groups} equal parts")
        if not self.norm_eps >= 0:
            raise ConfigError("config.json: norm.eps must not be negative")
        if not self.layers:
            raise ConfigError("config.json: layers is empty")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if layer.type not in MIXERS:
                raise ConfigError(f"config.json: {where}.type {layer.type!r} is not a mixer of this design; known: {sorted(MIXERS)}")
            for key in MIXERS[layer.type]:
                _need(layer.mixer, key, f"{where}.mixer")
            if layer.mlp is not None:
                if _need(layer.mlp, "kind", f"{where}.mlp") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind {layer.mlp['kind']!r} is not built (dense)")
                _positive_int(_need(layer.mlp, "ff", f"{where}.mlp"), f"{where}.mlp.ff")
            m = layer.mixer
            if layer.type == "mingru":
                _positive_int(m["width"], f"{where}.mixer.width")
                continue
            for key in ("heads", "dim", "vdim"):
                _positive_int(m[key], f"{where}.mixer.{key}")
            if layer.type == "attention":
                _positive_int(m["kv_heads"], f"{where}.mixer.kv_heads")
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"config.json: {where}.mixer.heads {m['heads']} is not a multiple of kv_heads {m['kv_heads']}")
                _positive_int(_need(m["mask"], "size", f"{where}.mixer.mask"), f"{where}.mixer.mask.size")
            else:
                _positive_int(m["kv_rank"], f"{where}.mixer.kv_rank")
                _positive_int(m["rot_dim"], f"{where}.mixer.rot_dim")
                dims = _need(m["rot"], "dims", f"{where}.mixer.rot")
                _need(m["rot"], "base", f"{where}.mixer.rot")
                if isinstance(dims, bool) or not isinstance(dims, int) or dims % 2 or not 0 <= dims <= m["rot_dim"]:
                    raise ConfigError(f"config.json: {where}.mixer.rot.dims {dims!r} must be even and at most rot_dim {m['rot_dim']}")
        if self.loop is not None:
            start, stop, times = self.loop
            if not (0 <= start < stop <= len(self.layers)) or times < 1:
                raise ConfigError(f"config.json: loop {self.loop} does not name a stretch of the {len(self.layers)} layers run at least once")

    @classmethod
    def from_dict(cls, d: dict) -> "NurolornConfig":
        layers = []
        for i, entry in enumerate(_need(d, "layers", "the configuration")):
            where = f"layers[{i}]"
            mlp = entry.get("mlp") if isinstance(entry, dict) else None
            layers.append(NurolornLayer(_need(entry, "type", where), copy.deepcopy(_need(entry, "mixer", where)), copy.deepcopy(mlp) if mlp else None))
        loop = d.get("loop")
        if loop:
            for key in ("start", "stop", "times"):
                value = _need(loop, key, "loop")
                if isinstance(value, bool) or not isinstance(value, int):
                    raise ConfigError(f"config.json: loop.{key} must be an integer, got {value!r}")
            loop = (loop["start"], loop["stop"], loop["times"])
        norm = _need(d, "norm", "the configuration")
        limit = d.get("max_positions")
        return cls(
            vocab_size=_need(d, "vocab", "the configuration"),
            width=_need(d, "width", "the configuration"),
            layers=tuple(layers),
            loop=loop or None,
            norm_eps=float(_need(norm, "eps", "norm")),
            norm_groups=int(norm.get("groups", 1)),
            residual_mult=float(d.get("residual_mult", 1.0)),
            logit_scale=float(d.get("logit_scale", 1.0)),
            max_positions=None if limit is None else int(limit),
        )

    def to_dict(self) -> dict:
        """The config.json this configuration is read back from."""
        d = {
            "architecture": self.architecture,
            "vocab": self.vocab_size,
            "width": self.width,
            "layers": [{"type": x.type, "mixer": copy.deepcopy(x.mixer), "mlp": copy.deepcopy(x.mlp)} for x in self.layers],
            "norm": {"eps": self.norm_eps, "groups": self.norm_groups},
            "residual_mult": self.residual_mult,
            "logit_scale": self.logit_scale,
        }
        if self.loop is not None:
            d["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        if self.max_positions is not None:
            d["max_positions"] = self.max_positions
        return d
