"""Small Tenotar configurations for the tests, as config.json dictionaries.  They differ from one another in every size
and option: values that are often equal are unequal here (key and value sizes, heads and key/value heads, rotated lanes
and the head size, the query latent and the key latent), and options are exercised at 1 and at their ends (one head, one
expert, every expert chosen, one tap, no kept tokens, more kept tokens than the window is wide, a window of one, no cap,
no shared expert, no feed-forward, a logit scale of one) as well as away from them."""

from __future__ import annotations


def windowed(heads, kv_heads, dim, vdim, scale, size, keep_first=None, dims=None, base=10000.0, v_mix=False):
    """The ``attention`` mixer: biases, per-head norms, neighbouring lanes rotated, a window that keeps the first tokens."""
    mask = {"size": size}
    if keep_first is not None:
        mask["keep_first"] = keep_first
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": mask,
         "rot": {"base": base, "dims": dim if dims is None else dims}}
    if v_mix:
        m["v_mix"] = True
    return {"type": "attention", "mixer": m}


def blocked(heads, kv_heads, dim, vdim, scale, size, taps, softcap=None, v_mix=False):
    """The ``attention_2`` mixer: a short convolution, capped scores, a distance bias, blocks of positions."""
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": size}, "conv": taps}
    if softcap is not None:
        m["softcap"] = softcap
    if v_mix:
        m["v_mix"] = True
    return {"type": "attention_2", "mixer": m}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, size, dims=None, base=10000.0):
    return {"type": "latent_attention", "mixer": {
        "heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
        "mask": {"size": size}, "rot": {"base": base, "dims": rot_dim if dims is None else dims}}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    d = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        d["shared"] = {"ff": shared}
    return d


def layer(mixer, mlp=None):
    return {**mixer, "mlp": mlp}


def config(layers, vocab=97, width=40, eps=1e-5, logit_scale=1.5):
    return {"architecture": "Tenotar", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps}, "logit_scale": logit_scale}


# odd sizes everywhere: three query heads on one key/value head, fewer rotated lanes than the head has, values wider than
# keys, windows and blocks that end inside pages, the first layer with mixed values of the convolution kind, a layer
# without mixed values between two with, a layer without a feed-forward, five experts of which two are chosen
ODD = config([
    layer(blocked(3, 1, 10, 14, 0.4, 7, 3, softcap=5.0, v_mix=True), moe(5, 2, 12, shared=20)),
    layer(latent(3, 6, 4, 10, 12, 9, 0.35, 11, dims=2, base=40.0), dense(28)),
    layer(windowed(2, 1, 6, 14, 0.5, 9, keep_first=3, dims=4, base=100.0, v_mix=True)),
    layer(windowed(4, 2, 6, 7, 0.5, 5, keep_first=6), moe(3, 1, 8)),
    layer(blocked(2, 1, 8, 14, 0.6, 13, 5, v_mix=True), dense(12)),
])
# everything at one or at its end: one head, one tap (no state), one expert, every expert chosen, a window of one, no
# kept tokens (the key absent, and zero), blocks of one position, a logit scale of one, sizes that tensor-core kernels take
ONES = config([
    layer(windowed(1, 1, 16, 16, 0.25, 1, v_mix=True), moe(3, 3, 16)),
    layer(blocked(1, 1, 16, 16, 0.25, 1, 1, v_mix=True), moe(1, 1, 32, shared=16)),
    layer(latent(1, 16, 16, 16, 16, 16, 0.2, 1), dense(16)),
    layer(windowed(4, 4, 32, 16, 0.2, 40, keep_first=0, dims=16), moe(2, 1, 16)),
    layer(blocked(4, 1, 16, 32, 0.2, 64, 2, softcap=1.0), moe(3, 2, 16, shared=32)),
], vocab=61, width=64, eps=1e-6, logit_scale=1.0)
# more heads, many experts, keys wider than values, heads of 48 and 80 lanes on the tensor cores, more kept tokens than
# the window is wide, windows longer than the requests, a convolution of eight taps
WIDE = config([
    layer(windowed(12, 4, 48, 16, 0.15, 6, keep_first=17, v_mix=True), moe(37, 4, 6, shared=10)),
    layer(latent(5, 32, 16, 48, 80, 24, 0.12, 20), moe(6, 3, 10)),
    layer(blocked(6, 2, 80, 32, 0.1, 16, 8, softcap=30.0, v_mix=True), dense(72)),
    layer(latent(2, 16, 32, 16, 32, 48, 0.15, 500, dims=16, base=500.0)),
    layer(windowed(4, 4, 16, 16, 0.2, 500, keep_first=2, v_mix=True), moe(2, 2, 24)),
], vocab=128, width=96, eps=1e-5, logit_scale=0.7)

ALL = {"odd": ODD, "ones": ONES, "wide": WIDE}
