"""Small Nudodra configurations for the tests, as config.json dictionaries.  They differ from one another in every size
and option: values that are often equal are unequal here (key and value sizes, heads of the two branches, rotated lanes
and the head size, the experts' and the shared expert's bounds), and options are exercised at 1 and at their ends (one
copy of the stream, one head, one expert, every expert chosen, no shared expert, no feed-forward, no ``streams`` key at
all) as well as away from them."""

from __future__ import annotations


def attention(heads, kv_heads, dim, vdim, scale, coef=None, every=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if coef is not None:
        m["q_temp"] = {"coef": coef, "every": every}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def left(heads, kv_heads, dim, scale, dims=None, base=10000.0):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale, "rot": {"base": base, "dims": dim if dims is None else dims}}


def right(heads, dim, vdim, tau, rank=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}
    if rank is not None:
        m["rank"] = rank  # the inner size of the decay's products, for random weights; a checkpoint's tensors say it themselves
    return m


def moe(experts, top, ff, limit, shared=None, shared_limit=None):
    d = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared:
        d["shared"] = {"ff": shared, "limit": shared_limit}
    return d


def attention_layer(m, mlp=None):
    return {"type": "attention", "mixer": m, "mlp": mlp}


def parallel_layer(l, r, left_scale, right_scale, mlp=None):
    return {"type": "parallel", "mixer": {"left": l, "right": r, "left_scale": left_scale, "right_scale": right_scale}, "mlp": mlp}


def config(layers, vocab=97, width=40, eps=1e-5, streams=2):
    d = {"architecture": "Nudodra", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps}}
    if streams is not None:
        d["streams"] = streams
    return d


# odd sizes everywhere: three copies of the stream, three query heads on one key/value head, fewer rotated lanes than the
# head has, values wider than keys, a layer that reads the pages of the layer in front and one that reads them two layers
# on, a layer without a feed-forward, five experts of which two are chosen, bounds that differ
ODD = config([
    parallel_layer(left(3, 1, 10, 0.4, dims=6, base=40.0), right(2, 6, 10, 7.0, rank=3), 0.7, 1.3, moe(5, 2, 12, 0.9, shared=20, shared_limit=0.4)),
    attention_layer(attention(4, 2, 6, 14, 0.5, coef=0.7, every=5), moe(3, 1, 8, 2.0)),
    attention_layer(attention(6, 2, 6, 14, 0.3, coef=1.5, every=3, kv_from=1)),
    parallel_layer(left(2, 2, 12, 0.3, base=1000.0), right(1, 4, 20, 2.5), 1.1, 0.4, moe(5, 2, 12, 0.9, shared=6, shared_limit=3.0)),
    attention_layer(attention(2, 2, 6, 14, 0.8, kv_from=1), moe(4, 4, 6, 1.2)),
], streams=3)
# everything at one or at its end: one copy of the stream, one head in every mixer, every expert chosen, one expert, the
# whole head rotated, a factor on the queries that changes at every position, sizes that tensor-core kernels take
ONES = config([
    attention_layer(attention(1, 1, 16, 16, 0.25, coef=0.3, every=1), moe(3, 3, 16, 1.0)),
    parallel_layer(left(1, 1, 16, 0.25), right(1, 16, 16, 1.0, rank=1), 1.0, 1.0, moe(1, 1, 32, 1.5, shared=16, shared_limit=1.5)),
    parallel_layer(left(4, 4, 32, 0.2, dims=16), right(2, 32, 16, 30.0), 0.5, 2.0, moe(2, 1, 16, 0.7)),
    attention_layer(attention(4, 1, 16, 16, 0.2, coef=0.4, every=64, kv_from=0), moe(3, 2, 16, 1.0, shared=32, shared_limit=0.5)),
], vocab=61, width=64, eps=1e-6, streams=1)
# more heads, many experts, four copies, keys wider than values, a head of 48 lanes on the tensor cores
WIDE = config([
    attention_layer(attention(12, 4, 48, 16, 0.15, coef=0.35, every=16), moe(37, 4, 6, 1.1, shared=10, shared_limit=2.0)),
    parallel_layer(left(6, 3, 20, 0.22, dims=10), right(3, 40, 70, 12.0, rank=5), 0.55, 0.45, moe(6, 3, 10, 0.8)),
    attention_layer(attention(4, 4, 48, 16, 0.2, coef=0.2, every=7, kv_from=0), moe(2, 2, 24, 1.0)),
], vocab=128, width=96, eps=1e-5, streams=4)
# no ``streams`` key: one plain residual stream, the contributions are simply added
PLAIN = config([
    parallel_layer(left(2, 1, 8, 0.35, dims=4), right(2, 8, 4, 4.0, rank=2), 0.9, 0.8, moe(4, 2, 8, 1.0, shared=8, shared_limit=1.0)),
    attention_layer(attention(2, 1, 8, 4, 0.35, coef=0.6, every=4)),
    attention_layer(attention(4, 1, 8, 4, 0.35, coef=0.6, every=4, kv_from=1), moe(4, 2, 8, 1.0)),
], vocab=50, width=24, streams=None)

ALL = {"odd": ODD, "ones": ONES, "wide": WIDE, "plain": PLAIN}
