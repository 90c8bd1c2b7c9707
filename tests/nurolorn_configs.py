"""Small Nurolorn configurations for the tests, as config.json dictionaries.  They differ from one another in every
size and option: values that are often equal are unequal here (key and value sizes, rotated lanes and the rotated
part, heads and key/value heads), and options are exercised at 1 (one norm group, a factor of 1, one pass, a window
of one key) as well as away from it."""

from __future__ import annotations


def latent(heads, dim, rot_dim, vdim, rank, scale, base=10000.0, dims=None, ff=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
             "rot": {"base": base, "dims": rot_dim if dims is None else dims}}
    return {"type": "latent_attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def mingru(width, ff=None):
    return {"type": "mingru", "mixer": {"width": width}, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def window(heads, kv_heads, dim, vdim, size, scale, ff=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": size}}
    return {"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(layers, vocab=97, width=64, groups=4, eps=1e-5, mult=0.5, logit_scale=1.5, loop=None):
    d = {"architecture": "Nurolorn", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps, "groups": groups},
         "residual_mult": mult, "logit_scale": logit_scale}
    if loop is not None:
        d["loop"] = dict(zip(("start", "stop", "times"), loop))
    return d


# odd sizes everywhere, a loop in the middle that runs three times, a layer without a feed-forward, fewer rotated
# lanes than the rotated part has
ODD = config(
    [mingru(40, ff=72), latent(3, 8, 8, 12, 20, 0.3, base=100.0, dims=4), window(4, 1, 10, 6, 5, 0.4, ff=48),
     latent(2, 12, 4, 8, 24, 0.25, base=5000.0, ff=56)],
    loop=(1, 3, 3),
)
# everything at one: one norm group, factor 1, no loop, logit scale 1, as many key/value heads as heads; sizes that
# the tensor-core kernels take (multiples of 16)
ONES = config(
    [window(2, 2, 16, 16, 17, 0.25, ff=128), mingru(64, ff=128), latent(4, 16, 16, 16, 32, 0.2, ff=128)],
    vocab=61, width=64, groups=1, eps=1e-6, mult=1.0, logit_scale=1.0,
)
# a loop over all layers that runs once; a window of one key; key and value sizes of the tensor-core kernels that differ
WHOLE_LOOP = config(
    [latent(2, 32, 16, 48, 64, 0.15, base=250.0, ff=96), window(4, 2, 32, 16, 1, 0.2), window(6, 3, 16, 32, 33, 0.3, ff=64), mingru(24)],
    vocab=128, width=96, groups=2, mult=0.8, logit_scale=0.7, loop=(0, 4, 1),
)
# a loop at the start, run twice, and layers behind it
HEAD_LOOP = config(
    [latent(4, 16, 16, 32, 48, 0.2, ff=80), mingru(48, ff=80), window(4, 2, 32, 32, 24, 0.18, ff=80), latent(2, 32, 32, 32, 64, 0.12)],
    vocab=200, width=128, groups=2, mult=0.7, logit_scale=2.0, loop=(0, 3, 2),
)

# the smallest of everything: one head, keys of two lanes, values of one, a state of one channel, norm parts of five
# elements, a loop over one layer that runs four times
SMALLEST = config(
    [latent(1, 2, 2, 1, 4, 0.7, base=3.0), mingru(1, ff=8), window(3, 3, 4, 2, 2, 0.6), latent(2, 6, 4, 3, 8, 0.5, dims=2, ff=12)],
    vocab=23, width=40, groups=8, mult=1.3, logit_scale=3.0, loop=(1, 2, 4),
)

ALL = {"smallest": SMALLEST, "odd": ODD, "ones": ONES, "whole_loop": WHOLE_LOOP, "head_loop": HEAD_LOOP}
