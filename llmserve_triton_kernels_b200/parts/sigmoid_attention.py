"""Grouped-query attention whose weights are sigmoids, not a softmax, with the heads' weights mixed.

    q = W_q x, k = W_k x, v = W_v x                       (one stacked product)
    q, k: each whole projection RMS-normed as one vector and weighted (``qk_norm_eps``; before rotation)
    q, k: lanes i and i + rot/2 of every head turned by position * f_i   (``rotary``: dims, base, optional scaling)
    s_g(i, j) = softcap * tanh(scale * q_g(i) . k(j) / softcap)
    p_g(i, j) = sigmoid(s_g(i, j) + head_bias[g])         for j <= i; nothing is normalised over j
    w_h(i, j) = sum_g head_mix[h, g] p_g(i, j)            head h applies w_h to the values of its own key/value head
    out = W_o [heads side by side]

Keys (rotated) and values live in pages of the cache manager like those of softmax attention.  The norms, the angles,
the scores, the weights and the sums over keys are 32-bit in both compute types.  ``rotary["scaling"]`` (``factor``,
``low``, ``high``, ``original``) stretches long wavelengths: with wavelength ``l = 2 pi / f`` a frequency stays where
``l < original / high``, becomes ``f / factor`` where ``l > original / low``, and in between is
``(1 - t) f / factor + t f`` with ``t = (original / l - low) / (high - low)``.
"""

from __future__ import annotations

import math

import torch

from .. import ops
from .base import Mixer, PagedKVSpec, TensorSpec, register_part

_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "bias": "pb", "mix": "talk"}


def rotary_frequencies(dims: int, base: float, scaling: dict | None = None) -> torch.Tensor:
    """``f_i = base^(-2i / dims)`` for ``i < dims / 2`` (float64 on the host, rounded to float32 once), with long
    wavelengths stretched as ``scaling`` says."""
    if dims % 2:
        raise ValueError(f"rotated lanes come in pairs, got {dims}")
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = float(base) ** (-2.0 * i / max(dims, 1))
    if scaling:
        factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        wavelength = 2.0 * math.pi / f
        t = (original / wavelength - low) / (high - low) if high != low else torch.ones_like(f)
        between = (1.0 - t) * f / factor + t * f
        f = torch.where(wavelength < original / high, f, torch.where(wavelength > original / low, f / factor, between))
    return f.to(torch.float32)


class SigmoidAttention(Mixer):
    graph_safe = True
    accepts_sink = True
    takes_projection = True  # a mixer that runs this one beside others may run the input product itself (``forward(proj=)``)

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int, scale: float,
                 softcap: float | None = None, rotary: dict | None = None, qk_norm_eps: float | None = None,
                 head_bias: bool = True, head_mix: bool = True, window: int | None = None,
                 tensor_names: dict[str, str] | None = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        if not (1 <= int(head_dim) and 1 <= int(value_dim) <= 256):
            raise ValueError(f"head_dim {head_dim} / value_dim {value_dim}: the kernels take values of up to 256 lanes")
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.head_dim, self.value_dim, self.scale = int(head_dim), int(value_dim), float(scale)
        self.softcap = float(softcap) if softcap else None
        self.rotary = dict(rotary) if rotary and rotary.get("dims") else None
        if self.rotary and not 0 < self.rotary["dims"] <= self.head_dim:
            raise ValueError(f"rotary dims {self.rotary['dims']} do not fit a head of {self.head_dim}")
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        self.has_bias, self.has_mix = bool(head_bias), bool(head_mix)
        self.window = None if window is None else int(window)
        self.names = {**_NAMES, **(tensor_names or {})}
        self.w_in = self.w_out = self.q_weight = self.k_weight = self.bias = self.mix = self.freq = None

    def tensors(self) -> dict[str, TensorSpec]:
        n, H, KV, D, V = self.names, self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim
        specs = {n["q"]: TensorSpec((H * D, self.hidden_size)), n["k"]: TensorSpec((KV * D, self.hidden_size)),
                 n["v"]: TensorSpec((KV * V, self.hidden_size)), n["o"]: TensorSpec((self.hidden_size, H * V))}
        if self.qk_norm_eps is not None:
            specs[n["q_norm"]] = TensorSpec((H * D,), init="ones_plus_normal")
            specs[n["k_norm"]] = TensorSpec((KV * D,), init="ones_plus_normal")
        if self.has_bias:
            specs[n["bias"]] = TensorSpec((H,))
        if self.has_mix:
            specs[n["mix"]] = TensorSpec((H, H))
        return specs

    def bind(self, tensors, dtype, device) -> None:
        n = self.names
        self.w_in = torch.cat([tensors[n[k]].to(dtype) for k in ("q", "k", "v")], dim=0).to(device).contiguous()
        self.w_out = tensors[n["o"]].to(device=device, dtype=dtype).contiguous()
        f32 = lambda t: t.to(device=device, dtype=torch.float32).contiguous()  # noqa: E731
        if self.qk_norm_eps is not None:
            self.q_weight, self.k_weight = f32(tensors[n["q_norm"]]), f32(tensors[n["k_norm"]])
        if self.has_bias:
            self.bias = f32(tensors[n["bias"]])
        if self.has_mix:
            self.mix = f32(tensors[n["mix"]])
        if self.rotary:
            self.freq = rotary_frequencies(self.rotary["dims"], self.rotary["base"], self.rotary.get("scaling")).to(device)

    def cache_spec(self) -> PagedKVSpec:
        return PagedKVSpec(self.num_kv_heads, max(self.head_dim, self.value_dim), self.window)

    def forward(self, x, ctx, cache, sink=None, proj=None):
        """``proj``: the stacked projections ``[N, q | k | v]`` (32-bit, rows may have a pitch) where the caller ran the product."""
        H, KV, D, V = self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim
        # the projections leave their product in 32-bit: the norm over the whole projection reads them as they are
        if proj is None:
            proj = ops.linear(x, self.w_in, out_dtype=torch.float32)
        q = ops.qk_prepare(proj, ctx.positions, heads=H, kv_heads=KV, dim=D, value_dim=V, freq=self.freq, q_weight=self.q_weight,
                           k_weight=self.k_weight, eps=self.qk_norm_eps or 0.0, pool=cache.pool, slot_map=cache.slot_map)
        out = ops.sigmoid_attention(q, cache.pool, cache.page_table, ctx, num_heads=H, num_kv_heads=KV, key_dim=D, value_dim=V,
                                    scale=self.scale, softcap=self.softcap, head_bias=self.bias, head_mix=self.mix, window=self.window)
        if sink is not None:
            handed_on = sink.linear(out, self.w_out)
            if handed_on is not None:
                return handed_on
        return ops.linear(out, self.w_out, out_dtype=torch.float32)


register_part("mixer", "sigmoid_attention", SigmoidAttention)
