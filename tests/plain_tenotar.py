"""The Tenotar design stated plainly: whole sequences, float64, no cache, no batching, one function per mechanism.
It shares no code with the package; the tests compare the engine's logits with :func:`forward`.

Notation: ``x [T, width]`` is the residual stream of one sequence whose tokens stand at positions ``0..T-1``;
``h [T, width]`` the normed input of a part; ``W[name]`` a tensor of the checkpoint; linear weights are ``[out, in]``;
``p`` the prefix of a part's tensor names and ``m`` its dictionary of the configuration.
"""

from __future__ import annotations

import math

import torch

DT = torch.float64
BIAS_STEEPNESS = 8.0  # the distance bias of head h has the slope 2^(-8 (h + 1) / heads)


def rms(x, eps, weight=None):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def linear(h, W, name):
    y = h @ W[name].T
    return y + W[name + ".b"] if name + ".b" in W else y


def angles(T, rot):
    dims = rot["dims"]
    f = float(rot["base"]) ** (-2 * torch.arange(dims // 2, dtype=DT) / dims)
    a = torch.arange(T, dtype=DT)[:, None] * f[None, :]
    return a.cos()[:, None, :], a.sin()[:, None, :]


def rotate_halves(x, rot):
    """x [T, heads, D]: lanes i and i + dims/2 of the first ``dims`` lanes turn by position * base^(-2i/dims)."""
    if not rot or not rot.get("dims"):
        return x
    dims = rot["dims"]
    c, s = angles(x.shape[0], rot)
    u, v = x[..., : dims // 2], x[..., dims // 2 : dims]
    return torch.cat((u * c - v * s, v * c + u * s, x[..., dims:]), dim=-1)


def rotate_neighbours(x, rot):
    """x [T, heads, D]: lanes 2i and 2i + 1 of the first ``dims`` lanes turn by position * base^(-2i/dims)."""
    if not rot or not rot.get("dims"):
        return x
    dims = rot["dims"]
    c, s = angles(x.shape[0], rot)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    turned = torch.stack((u * c - v * s, v * c + u * s), dim=-1).flatten(-2)
    return torch.cat((turned, x[..., dims:]), dim=-1)


def visible(T, mask, kind):
    """[T, T] booleans: may the query at position i (row) see the key at position j (column)?
    ``window``: 0 <= i - j < size; ``window_keep``: that, or j < keep_first (and j <= i); ``chunk``: j <= i in the same
    block of ``size`` positions counted from 0."""
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    causal = j <= i
    size = mask["size"]
    if kind == "window":
        return causal & (i - j < size)
    if kind == "window_keep":
        return causal & ((i - j < size) | (j < mask.get("keep_first", 0)))
    if kind == "chunk":
        return causal & (torch.div(i, size, rounding_mode="floor") == torch.div(j, size, rounding_mode="floor"))
    raise ValueError(kind)


def softmax_masked(s, see):
    """s [H, T, T] scores; rows are normalised over the keys that ``see [T, T]`` allows."""
    s = s.masked_fill(~see[None], -math.inf)
    return torch.softmax(s, dim=-1)


def short_convolution(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] * u_(t - taps + 1 + j), zeros before the sequence's start."""
    T, taps = u.shape[0], w.shape[1]
    padded = torch.cat((torch.zeros(taps - 1, u.shape[1], dtype=u.dtype), u), dim=0)
    return sum(w[:, j][None, :] * padded[j : j + T] for j in range(taps))


def mix_values(v, W, p, m, shared):
    """The values of a layer with ``v_mix``: the first such layer of the model hands its values on as they are; every
    later one takes (1 - lambda) v + lambda v_first, lambda its scalar ``vmix``."""
    if not m.get("v_mix"):
        return v
    if "v_first" not in shared:
        shared["v_first"] = v
        return v
    lam = W[p + "vmix"].to(DT).reshape(())
    return (1 - lam) * v + lam * shared["v_first"]


def grouped(x, heads):
    """[T, kv_heads, D] -> [T, heads, D]: query head h reads key/value head floor(h / (heads / kv_heads))."""
    return x.repeat_interleave(heads // x.shape[1], dim=1)


def attention(h, W, p, m, eps, shared):
    """Grouped-query attention with biases, per-head norms of q and k, neighbouring lanes rotated, a sliding window
    that also keeps the first tokens, and an output projection with a bias."""
    T, H, G, D, V = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = linear(h, W, p + "q").view(T, H, D)
    k = linear(h, W, p + "k").view(T, G, D)
    v = linear(h, W, p + "v").view(T, G, V)
    q, k = rms(q, eps, W[p + "q.norm"]), rms(k, eps, W[p + "k.norm"])
    q, k = rotate_neighbours(q, m.get("rot")), rotate_neighbours(k, m.get("rot"))
    v = mix_values(v.reshape(T, G * V), W, p, m, shared).view(T, G, V)
    s = torch.einsum("ihd,jhd->hij", q, grouped(k, H)) * float(m["scale"])
    a = softmax_masked(s, visible(T, m["mask"], "window_keep"))
    o = torch.einsum("hij,jhd->ihd", a, grouped(v, H)).reshape(T, H * V)
    return linear(o, W, p + "o")


def attention_2(h, W, p, m, eps, shared):
    """Grouped-query attention without biases and without rotation: a short causal convolution on every channel of q,
    k and v, capped scores, a distance bias per head, keys of the query's own block of positions only."""
    T, H, G, D, V = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_convolution(h @ W[p + "q"].T, W[p + "q.conv"]).view(T, H, D)
    k = short_convolution(h @ W[p + "k"].T, W[p + "k.conv"]).view(T, G, D)
    v = short_convolution(h @ W[p + "v"].T, W[p + "v.conv"])
    v = mix_values(v, W, p, m, shared).view(T, G, V)
    s = torch.einsum("ihd,jhd->hij", q, grouped(k, H)) * float(m["scale"])
    cap = m.get("softcap")
    if cap:
        s = float(cap) * torch.tanh(s / float(cap))
    slopes = 2.0 ** (-BIAS_STEEPNESS * torch.arange(1, H + 1, dtype=DT) / H)
    distance = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).to(DT)
    s = s - slopes[:, None, None] * distance[None]
    a = softmax_masked(s, visible(T, m["mask"], "chunk"))
    o = torch.einsum("hij,jhd->ihd", a, grouped(v, H)).reshape(T, H * V)
    return o @ W[p + "o"].T


def latent_attention(h, W, p, m, eps, shared=None):
    """Attention whose queries, keys and values come through low-rank latents; a rotated key part shared by the heads;
    a sliding window; every head's output times the sigmoid of one number per head and token."""
    T, H, D, R, V, rank = h.shape[0], m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms(h @ W[p + "dq"].T, eps, W[p + "dq.norm"])
    q = (cq @ W[p + "uq"].T).view(T, H, D + R)
    down = h @ W[p + "dkv"].T
    c = rms(down[:, :rank], eps, W[p + "dkv.norm"])
    rot = m["rot"]  # its ``dims`` lanes (those of the rotated part, unless the configuration says fewer) turn
    k_rot = rotate_halves(down[:, None, rank:], rot)  # [T, 1, R]
    q_rot = rotate_halves(q[..., D:], rot)
    k = (c @ W[p + "uk"].T).view(T, H, D)
    v = (c @ W[p + "uv"].T).view(T, H, V)
    s = (torch.einsum("ihd,jhd->hij", q[..., :D], k) + torch.einsum("ihd,jd->hij", q_rot, k_rot[:, 0])) * float(m["scale"])
    a = softmax_masked(s, visible(T, m["mask"], "window"))
    o = torch.einsum("hij,jhd->ihd", a, v)
    o = o * torch.sigmoid(h @ W[p + "g"].T)[:, :, None]
    return o.reshape(T, H * V) @ W[p + "o"].T


def gated_unit(h, W, p):
    """down(silu(gate h) * (up h)), with biases where the checkpoint has them."""
    g = linear(h, W, p + "gate")
    return linear(g * torch.sigmoid(g) * linear(h, W, p + "up"), W, p + "down")


def routed(h, W, p, mlp):
    """A mixture of gated units: the ``top`` largest router logits choose, their softmax (over the chosen only) weighs;
    a shared unit runs for every token."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = linear(h, W, p + "router")
    chosen = torch.topk(z, top, dim=-1)
    weights = torch.softmax(chosen.values, dim=-1)
    out = torch.zeros_like(h)
    for e in range(E):
        share = (weights * (chosen.indices == e)).sum(-1, keepdim=True)
        out = out + share * gated_unit(h, W, f"{p}e{e}.")
    if mlp.get("shared"):
        out = out + gated_unit(h, W, p + "shared.")
    return out


def feed_forward(h, W, p, mlp):
    return gated_unit(h, W, p) if mlp["kind"] == "dense" else routed(h, W, p, mlp)


MIXERS = {"attention": attention, "attention_2": attention_2, "latent_attention": latent_attention}


def forward(cfg, tensors, tokens, return_layers=False):
    """Logits ``[T, vocab]`` (float64) of one whole sequence; with ``return_layers`` also the stream after every layer."""
    W = {k: (v.to(DT) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = float(cfg["norm"]["eps"])
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    shared, seen = {}, []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        x = x + MIXERS[layer["type"]](rms(x, eps, W[p + "norm1"]), W, p + "mix.", layer["mixer"], eps, shared)
        if layer.get("mlp"):
            x = x + feed_forward(rms(x, eps, W[p + "norm2"]), W, p + "mlp.", layer["mlp"])
        seen.append(x)
    logits = (rms(x, eps, W["final.norm"]) @ W["head"].T) * float(cfg.get("logit_scale", 1.0))
    return (logits, seen) if return_layers else logits
