"""A plain, slow implementation of the Nurolorn design: whole sequences, no cache, one function per mechanism.

It shares no code with the engine.  Everything is computed in the precision of the tensors it is given (the tests
pass float64 or float32), so it is the oracle that the engine's 32-bit and bfloat16 paths are compared with.
``config`` is the dictionary of a config.json, ``tensors`` maps checkpoint names to tensors.
"""

from __future__ import annotations

import math

import torch


def grouped_rms_norm(x, weight, groups: int, eps: float):
    """Each of ``groups`` equal consecutive parts of a row is divided by its own root mean square; then the weight."""
    n, d = x.shape
    parts = x.reshape(n, groups, d // groups)
    parts = parts / torch.sqrt(parts.pow(2).mean(-1, keepdim=True) + eps)
    return parts.reshape(n, d) * weight


def unit_rms(x, eps: float):
    """A vector divided by its root mean square (a norm without a weight), over the last dimension."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def rotate_pairs(x, positions, base: float, dims: int):
    """Rotary positions in the interleaved layout on the first ``dims`` lanes of the last dimension: lanes (2i, 2i+1)
    turn by the angle ``position * base**(-2i/dims)``.  ``x [tokens, ..., lanes]``, ``positions [tokens]``."""
    i = torch.arange(dims // 2, dtype=x.dtype)
    freq = base ** (-2.0 * i / dims)
    angle = positions.to(x.dtype)[:, None] * freq  # [tokens, dims/2]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = angle.cos().reshape(shape), angle.sin().reshape(shape)
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def latent_attention(h, t, prefix: str, p: dict, eps: float):
    """Attention through a low-rank latent: keys and values of every head are products of one latent vector per token;
    one rotated key part is shared by all heads; an output gate reads the mixer's input."""
    n = h.shape[0]
    H, dim, rot, vdim, rank = p["heads"], p["dim"], p["rot_dim"], p["vdim"], p["kv_rank"]
    pos = torch.arange(n)
    q = (h @ t[prefix + "q"].T).reshape(n, H, dim + rot)
    q_plain, q_rot = q[..., :dim], q[..., dim:]
    dkv = h @ t[prefix + "dkv"].T
    latent = unit_rms(dkv[:, :rank], eps) * t[prefix + "dkv.norm"]
    k_rot = dkv[:, rank:]
    q_rot = rotate_pairs(q_rot, pos, p["rot"]["base"], p["rot"]["dims"])
    k_rot = rotate_pairs(k_rot, pos, p["rot"]["base"], p["rot"]["dims"])
    k_plain = (latent @ t[prefix + "uk"].T).reshape(n, H, dim)
    v = (latent @ t[prefix + "uv"].T).reshape(n, H, vdim)
    scores = torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)
    scores = scores * p["scale"]
    visible = pos[None, :] <= pos[:, None]
    scores = scores.masked_fill(~visible, -math.inf)
    weights = torch.softmax(scores, dim=-1)
    heads = torch.einsum("hij,jhd->ihd", weights, v).reshape(n, H * vdim)
    heads = heads * torch.sigmoid(h @ t[prefix + "g"].T)
    return heads @ t[prefix + "o"].T


def mingru(h, t, prefix: str, p: dict, state=None):
    """A gated recurrence whose gate and candidate read only the current token; returns (output, last state)."""
    z = torch.sigmoid(h @ t[prefix + "z"].T + t[prefix + "z.b"])
    u = h @ t[prefix + "x"].T + t[prefix + "x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    s = torch.zeros(p["width"], dtype=h.dtype) if state is None else state
    states = []
    for i in range(h.shape[0]):
        s = (1 - z[i]) * s + z[i] * cand[i]
        states.append(s)
    states = torch.stack(states)
    gate = h @ t[prefix + "g"].T
    return (states * (gate * torch.sigmoid(gate))) @ t[prefix + "o"].T, s


def window_attention(h, t, prefix: str, p: dict, eps: float):
    """Grouped-query attention without rotation: unit-RMS queries and keys, a distance bias per head, a sliding window."""
    n = h.shape[0]
    H, G, dim, vdim = p["heads"], p["kv_heads"], p["dim"], p["vdim"]
    pos = torch.arange(n)
    q = unit_rms((h @ t[prefix + "q"].T).reshape(n, H, dim), eps)
    k = unit_rms((h @ t[prefix + "k"].T).reshape(n, G, dim), eps)
    v = (h @ t[prefix + "v"].T).reshape(n, G, vdim)
    k = k.repeat_interleave(H // G, dim=1)
    v = v.repeat_interleave(H // G, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * p["scale"]
    slopes = torch.tensor([2.0 ** (-8.0 * (x + 1) / H) for x in range(H)], dtype=h.dtype)
    distance = (pos[:, None] - pos[None, :]).to(h.dtype)
    scores = scores - slopes[:, None, None] * distance
    visible = (pos[None, :] <= pos[:, None]) & (pos[:, None] - pos[None, :] < p["mask"]["size"])
    scores = scores.masked_fill(~visible, -math.inf)
    weights = torch.softmax(scores, dim=-1)
    heads = torch.einsum("hij,jhd->ihd", weights, v).reshape(n, H * vdim)
    return heads @ t[prefix + "o"].T


def dense_mlp(h, t, prefix: str):
    return torch.relu(h @ t[prefix + "up"].T).pow(2) @ t[prefix + "down"].T


def layer_order(config: dict):
    """``[(layer index, pass number or None, first of its pass)]`` in execution order."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop or loop["stop"] <= loop["start"]:
        return [(i, None, False) for i in range(n)]
    order = [(i, None, False) for i in range(loop["start"])]
    for t in range(loop["times"]):
        order += [(i, t, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    order += [(i, None, False) for i in range(loop["stop"], n)]
    return order


def forward(config: dict, tensors: dict, tokens, dtype=torch.float64, return_layers: bool = False):
    """Logits ``[tokens, vocab]`` of one whole sequence (and, if asked, the residual stream after every layer run)."""
    t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps, groups, m = config["norm"]["eps"], config["norm"]["groups"], config["residual_mult"]
    x = t["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    embedded = x.clone()
    after = []
    for i, loop_pass, first in layer_order(config):
        if first:
            if loop_pass > 0:
                x = x + embedded
            x = x + t["loop.step"][loop_pass]
        spec, pre = config["layers"][i], f"l{i}."
        h = grouped_rms_norm(x, t[pre + "norm1"], groups, eps)
        kind = spec["type"]
        if kind == "latent_attention":
            y = latent_attention(h, t, pre + "mix.", spec["mixer"], eps)
        elif kind == "mingru":
            y, _ = mingru(h, t, pre + "mix.", spec["mixer"])
        elif kind == "attention":
            y = window_attention(h, t, pre + "mix.", spec["mixer"], eps)
        else:
            raise ValueError(f"unknown mixer {kind!r}")
        x = x + m * y
        if spec.get("mlp"):
            x = x + m * dense_mlp(grouped_rms_norm(x, t[pre + "norm2"], groups, eps), t, pre + "mlp.")
        after.append(x.clone())
    x = grouped_rms_norm(x, t["final.norm"], groups, eps)
    logits = (x @ t["head"].T) * config["logit_scale"]
    return (logits, torch.stack(after)) if return_layers else logits
