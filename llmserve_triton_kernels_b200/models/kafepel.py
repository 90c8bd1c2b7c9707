"""Kafepel as data: which parts each layer has, from a :class:`KafepelConfig`.

Every layer is a pre-norm block with RMS norms.  Its mixer is the ``parallel`` one (parts/parallel.py) with two
branches: ``left`` = ``sigmoid_attention`` (parts/sigmoid_attention.py), ``right`` = ``retention``
(parts/recurrent.py); the branches' outputs are RMS-normed with the weights ``left.out`` / ``right.out`` and averaged.
The feed-forward is the gated dense one with SiLU (``gate``, ``up``, ``down``), the routed one (parts/feed_forward.py:
softmax scores, a correction added for the choice only, weights ``router.scale * score`` not renormalised, experts
with the squared relu, a shared expert behind a sigmoid gate), or absent.  The stream starts as the token
embeddings times ``embedding.scale``.  Tensor names: ``embed``, ``head``, ``final.norm``, and per layer ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.mix.left.*``, ``l<i>.mix.right.*``, ``l<i>.mlp.*``.
"""

from __future__ import annotations

from ..config.kafepel import KafepelConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from .plan import LayerRun, LayerSpec, ModelPlan

EXPERT_ACTIVATION = "relu2"  # the design fixes it: the square of relu


def _mixer(cfg: KafepelConfig, layer, prefix: str) -> PartSpec:
    left, right = layer.mixer["left"], layer.mixer["right"]
    attention = PartSpec("sigmoid_attention", {
        "hidden_size": cfg.width, "num_heads": left["heads"], "num_kv_heads": left["kv_heads"], "head_dim": left["dim"],
        "value_dim": left["vdim"], "scale": float(left["scale"]), "softcap": left.get("softcap"), "rotary": left.get("rot"),
        "qk_norm_eps": cfg.norm_eps, "head_bias": True, "head_mix": True,
    })
    retention = PartSpec("retention", {
        "hidden_size": cfg.width, "num_heads": right["heads"], "head_dim": right["dim"], "value_dim": right["vdim"],
        "decay": list(right["decay"]), "norm_eps": cfg.norm_eps, "rotary": right.get("rot"), "gate": "silu",
    })
    params = {"hidden_size": cfg.width, "branches": {"left": attention, "right": retention}, "norm_eps": cfg.norm_eps}
    return PartSpec("parallel", params, prefix)


def _feed_forward(cfg: KafepelConfig, mlp: dict, prefix: str) -> PartSpec:
    if mlp["kind"] == "dense":
        names = {"gate": "gate", "up": "up", "down": "down"}
        return PartSpec("gated_mlp", {"hidden_size": cfg.width, "intermediate_size": mlp["ff"], "activation": "silu", "tensor_names": names}, prefix)
    router, shared = mlp["router"], mlp.get("shared")
    params = {
        "hidden_size": cfg.width, "experts": router["experts"], "top": router["top"], "expert_size": mlp["expert"]["ff"],
        "activation": EXPERT_ACTIVATION, "router_scale": float(router.get("scale", 1.0)), "correction": True, "renormalize": False,
        "shared_size": shared["ff"] if shared else None, "shared_gate": True,
    }
    return PartSpec("routed_mlp", params, prefix)


def kafepel_plan(cfg: KafepelConfig) -> ModelPlan:
    norm = {"size": cfg.width, "eps": cfg.norm_eps}
    layers, ignored = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        parts = {
            "mixer_norm": PartSpec("rms_norm", {**norm, "weight_name": "norm1"}, p),
            "mixer": _mixer(cfg, layer, p + "mix."),
        }
        if layer.mlp is None:
            block = PartSpec("pre_norm_mixer_only", {})
            ignored.append(p + "norm2")  # a layer without a feed-forward has no use for a second norm
        else:
            block = PartSpec("pre_norm", {})
            parts["ff_norm"] = PartSpec("rms_norm", {**norm, "weight_name": "norm2"}, p)
            parts["feed_forward"] = _feed_forward(cfg, layer.mlp, p + "mlp.")
        layers.append(LayerSpec(block, parts))
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
        embedding_scale=cfg.embedding_scale,
    )


register_architecture("Kafepel", KafepelConfig, kafepel_plan)
