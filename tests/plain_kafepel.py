"""The Kafepel design stated plainly: whole sequences, float64, no cache, no batching, one function per mechanism.
It shares no code with the package; the tests compare the engine's logits with :func:`forward`.

Notation: ``x [T, width]`` is the residual stream of one sequence whose tokens stand at positions ``0..T-1``;
``W[name]`` a tensor of the checkpoint; linear weights are ``[out, in]``.
"""

from __future__ import annotations

import math

import torch

DT = torch.float64


def rms(x, eps, weight=None):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def frequencies(rot):
    dims = rot["dims"]
    i = torch.arange(dims // 2, dtype=DT)
    f = float(rot["base"]) ** (-2 * i / dims)
    sc = rot.get("scaling")
    if sc:
        factor, low, high, original = (float(sc[k]) for k in ("factor", "low", "high", "original"))
        wavelength = 2 * math.pi / f
        t = (original / wavelength - low) / (high - low)
        f = torch.where(wavelength < original / high, f, torch.where(wavelength > original / low, f / factor, (1 - t) * f / factor + t * f))
    return f


def rotate(x, rot):
    """x [T, heads, D]: lanes i and i + dims/2 of the first ``dims`` lanes turn by position * f_i."""
    if not rot or not rot.get("dims"):
        return x
    dims = rot["dims"]
    angle = torch.arange(x.shape[0], dtype=DT)[:, None] * frequencies(rot)[None, :]
    c, s = angle.cos()[:, None, :], angle.sin()[:, None, :]
    u, v = x[..., : dims // 2], x[..., dims // 2 : dims]
    return torch.cat((u * c - v * s, v * c + u * s, x[..., dims:]), dim=-1)


def sigmoid_attention(h, W, p, m, eps):
    T, H, G, D, V = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms(h @ W[p + "q"].T, eps, W[p + "q.norm"])
    k = rms(h @ W[p + "k"].T, eps, W[p + "k.norm"])
    v = (h @ W[p + "v"].T).view(T, G, V)
    q, k = rotate(q.view(T, H, D), m.get("rot")), rotate(k.view(T, G, D), m.get("rot"))
    kv_of = torch.arange(H) // (H // G)
    s = torch.einsum("ihd,jhd->hij", q, k[:, kv_of]) * m["scale"]
    if m.get("softcap"):
        s = m["softcap"] * torch.tanh(s / m["softcap"])
    w = torch.sigmoid(s + W[p + "pb"][:, None, None]) * torch.tril(torch.ones(T, T, dtype=DT))
    w = torch.einsum("hg,gij->hij", W[p + "talk"], w)
    return torch.einsum("hij,jhd->ihd", w, v[:, kv_of]).reshape(T, H * V) @ W[p + "o"].T


def retention(h, W, p, m, eps):
    T, H, D, V = h.shape[0], m["heads"], m["dim"], m["vdim"]
    q = rotate((h @ W[p + "q"].T).view(T, H, D), m.get("rot"))
    k = rotate((h @ W[p + "k"].T).view(T, H, D), m.get("rot")) * D ** -0.5
    v = (h @ W[p + "v"].T).view(T, H, V)
    decay = torch.tensor(m["decay"], dtype=DT)[:, None, None]
    S = torch.zeros(H, D, V, dtype=DT)
    o = torch.zeros(T, H, V, dtype=DT)
    for t in range(T):
        S = decay * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    g = h @ W[p + "g"].T
    return (rms(o, eps).reshape(T, H * V) * g * torch.sigmoid(g)) @ W[p + "o"].T


def parallel_mixer(h, W, p, m, eps):
    left = rms(sigmoid_attention(h, W, p + "left.", m["left"], eps), eps, W[p + "left.out"])
    right = rms(retention(h, W, p + "right.", m["right"], eps), eps, W[p + "right.out"])
    return 0.5 * (left + right)


def dense_mlp(h, W, p):
    g = h @ W[p + "gate"].T
    return (g * torch.sigmoid(g) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def expert(h, W, p):
    return torch.relu(h @ W[p + "up"].T) ** 2 @ W[p + "down"].T


def routed_mlp(h, W, p, c):
    r = c["router"]
    s = torch.softmax(h @ W[p + "router"].T, dim=-1)
    chosen = (s + W[p + "correction"]).topk(r["top"], dim=-1).indices
    out = torch.zeros_like(h)
    for e in range(r["experts"]):
        mine = (chosen == e).any(-1).to(DT)
        out = out + (mine * s[:, e] * r.get("scale", 1.0))[:, None] * expert(h, W, f"{p}e{e}.")
    if c.get("shared"):
        out = out + torch.sigmoid(h @ W[p + "shared.sg"].T) * expert(h, W, p + "shared.")
    return out


def forward(cfg, tensors, tokens, return_layers=False):
    W = {k: (v.to(DT) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.tensor(tokens)] * cfg.get("embedding", {}).get("scale", 1.0)
    layers = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        x = x + parallel_mixer(rms(x, eps, W[p + "norm1"]), W, p + "mix.", layer["mixer"], eps)
        mlp = layer.get("mlp")
        if mlp:
            h = rms(x, eps, W[p + "norm2"])
            x = x + (dense_mlp(h, W, p + "mlp.") if mlp["kind"] == "dense" else routed_mlp(h, W, p + "mlp.", mlp))
        layers.append(x)
    logits = rms(x, eps, W["final.norm"]) @ W["head"].T
    return (logits, torch.stack(layers)) if return_layers else logits
