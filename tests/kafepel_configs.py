"""Small Kafepel configurations for the tests, as config.json dictionaries.  They differ from one another in every
size and option: values that are often equal are unequal here (key and value sizes, heads of the two branches, rotated
lanes and the head size), and options are exercised at 1 and at their ends (one head, one expert, every expert chosen,
no cap, no scaling, no shared expert, no feed-forward) as well as away from them."""

from __future__ import annotations


def left(heads, kv_heads, dim, vdim, scale, dims=None, base=10000.0, softcap=None, scaling=None):
    rot = {"base": base, "dims": dim if dims is None else dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot}
    if softcap:
        m["softcap"] = softcap
    return m


def right(heads, dim, vdim, decay, dims=None, base=10000.0):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay), "rot": {"base": base, "dims": dim if dims is None else dims}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, scale=1.0, shared=None):
    d = {"kind": "moe", "router": {"experts": experts, "top": top, "scale": scale}, "expert": {"ff": ff}}
    if shared:
        d["shared"] = {"ff": shared}
    return d


def layer(l, r, mlp=None):
    return {"type": "parallel", "mixer": {"left": l, "right": r}, "mlp": mlp}


def config(layers, vocab=97, width=40, eps=1e-5, embed_scale=3.0):
    return {"architecture": "Kafepel", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps}, "embedding": {"scale": embed_scale}}


# odd sizes everywhere: three query heads on one key/value head, fewer rotated lanes than the head has, scaled
# frequencies whose three bands are all met, a layer without a feed-forward, five experts of which two are chosen
ODD = config([
    layer(left(3, 1, 10, 6, 0.4, dims=6, base=40.0, softcap=4.0, scaling=(3.0, 1.0, 4.0, 24)), right(2, 6, 10, (0.9, 0.97), dims=2, base=30.0), dense(24)),
    layer(left(4, 2, 6, 14, 0.5, dims=4, base=100.0, softcap=9.0), right(3, 10, 4, (0.8, 0.95, 0.99), dims=10, base=200.0), moe(5, 2, 12, 1.7, shared=20)),
    layer(left(2, 2, 12, 12, 0.3, base=1000.0), right(1, 4, 20, (0.93,), dims=4)),
])
# everything at one or at its end: one head in both branches, every expert chosen, one expert, no cap, no rotation in
# the recurrent branch, an embedding scale of 1, sizes that tensor-core kernels take (multiples of 16)
ONES = config([
    layer(left(1, 1, 16, 16, 0.25), right(1, 16, 16, (1.0,), dims=0), moe(3, 3, 16)),
    layer(left(4, 4, 32, 16, 0.2, dims=16, softcap=30.0), right(2, 32, 16, (0.5, 0.999)), moe(1, 1, 32, 0.5, shared=16)),
    layer(left(4, 1, 16, 32, 0.2), right(4, 16, 32, (0.9, 0.9, 0.9, 0.9)), dense(64)),
], vocab=61, width=64, eps=1e-6, embed_scale=1.0)
# more heads than a warp has lanes' worth of rows to spare, many experts, values wider than keys
WIDE = config([
    layer(left(12, 4, 8, 40, 0.35, dims=8, softcap=15.0, scaling=(8.0, 1.0, 2.0, 16)), right(6, 20, 36, (0.7, 0.8, 0.9, 0.95, 0.98, 0.995), dims=12), moe(37, 4, 6, 2.0, shared=10)),
    layer(left(6, 3, 20, 10, 0.22, dims=10), right(2, 40, 70, (0.96, 0.99), dims=40), dense(50)),
], vocab=128, width=96, eps=1e-5, embed_scale=7.5)

ALL = {"odd": ODD, "ones": ONES, "wide": WIDE}
