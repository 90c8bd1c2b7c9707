"""Nurolorn as data: which parts each layer has and in which order the layers run, from a :class:`NurolornConfig`.

Every layer is a pre-norm block whose parts' contributions enter the residual stream times ``residual_mult``; its
norms are RMS norms in ``norm.groups`` groups.  The mixers are parts with parameters of their own: ``latent_attention``
(parts/latent_attention.py), ``mingru`` (parts/recurrent.py) and ``attention`` (parts/attention.py with unit-RMS
queries and keys, a distance bias of slope ``2^(-8 (h+1) / heads)`` and a sliding window); the feed-forward is the
dense one with the squared relu.  Layers ``loop.start .. loop.stop-1`` run ``loop.times`` times in a row: the order
lists them that often (each entry keeps a cache of its own), and before every pass the stream takes up row t of
``loop.step``, before every pass but the first also the token embeddings once more.  The logits are the output
matrix's product times ``logit_scale``.  Tensor names: ``embed``, ``head``, ``final.norm``, ``loop.step``, and per layer
``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""

from __future__ import annotations

from ..config.nurolorn import NurolornConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from .plan import Injection, LayerRun, LayerSpec, ModelPlan

DISTANCE_BIAS = 8.0  # slope of head h: 2^(-8 (h+1) / heads)


def _mixer(cfg: NurolornConfig, layer, prefix: str) -> PartSpec:
    m = layer.mixer
    if layer.type == "latent_attention":
        params = {
            "hidden_size": cfg.width, "num_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"],
            "value_dim": m["vdim"], "rank": m["kv_rank"], "scale": float(m["scale"]), "rotary_base": float(m["rot"]["base"]),
            "rotary_dims": m["rot"]["dims"], "norm_eps": cfg.norm_eps, "output_gate": True,
        }
        return PartSpec("latent_attention", params, prefix)
    if layer.type == "mingru":
        return PartSpec("mingru", {"hidden_size": cfg.width, "width": m["width"], "bias": True}, prefix)
    params = {
        "hidden_size": cfg.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
        "value_dim": m["vdim"], "scale": float(m["scale"]), "window": m["mask"]["size"], "qk_norm_eps": cfg.norm_eps,
        "distance_bias": DISTANCE_BIAS, "tensor_names": {"q": "q", "k": "k", "v": "v", "o": "o"},
    }
    return PartSpec("attention", params, prefix)


def nurolorn_plan(cfg: NurolornConfig) -> ModelPlan:
    norm = {"size": cfg.width, "eps": cfg.norm_eps, "groups": cfg.norm_groups}
    layers, ignored = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        parts = {
            "mixer_norm": PartSpec("rms_norm", {**norm, "weight_name": "norm1"}, p),
            "mixer": _mixer(cfg, layer, p + "mix."),
        }
        if layer.mlp is None:
            block = PartSpec("pre_norm_mixer_only", {"residual_scale": cfg.residual_mult})
            ignored.append(p + "norm2")  # a layer without a feed-forward has no use for its second norm
        else:
            block = PartSpec("pre_norm", {"residual_scale": cfg.residual_mult})
            parts["ff_norm"] = PartSpec("rms_norm", {**norm, "weight_name": "norm2"}, p)
            parts["feed_forward"] = PartSpec(
                "dense_mlp", {"hidden_size": cfg.width, "intermediate_size": layer.mlp["ff"], "activation": "relu2"}, p + "mlp."
            )
        layers.append(LayerSpec(block, parts))
    count = len(cfg.layers)
    order, injections, extra = [], [], ()
    if cfg.loop is None:
        order = [LayerRun(i) for i in range(count)]
    else:
        start, stop, times = cfg.loop
        order = [LayerRun(i) for i in range(start)]
        for t in range(times):
            injections.append(Injection(before=len(order), add_embedding=t > 0, vector="loop.step", row=t))
            order += [LayerRun(i) for i in range(start, stop)]
        order += [LayerRun(i) for i in range(stop, count)]
        extra = (("loop.step", (times, cfg.width)),)
    return ModelPlan(
        hidden_size=cfg.width,
        vocab_size=cfg.vocab_size,
        max_positions=cfg.max_positions,
        embedding="embed",
        layers=tuple(layers),
        schedule=tuple(order),
        final_norm=PartSpec("rms_norm", {**norm, "weight_name": "norm"}, "final."),
        head="head",
        ignored=tuple(ignored),
        injections=tuple(injections),
        extra_tensors=extra,
        logit_scale=cfg.logit_scale,
    )


register_architecture("Nurolorn", NurolornConfig, nurolorn_plan)
