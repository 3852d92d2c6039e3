"""The Nudodra design stated plainly: whole sequences, float64, no cache, no batching, one function per mechanism.
It shares no code with the package; the tests compare the engine's logits with :func:`forward`.

Notation: ``X [S, T, width]`` are the S copies of the residual stream of one sequence whose tokens stand at positions
``0..T-1``; ``h [T, width]`` the normed input of a part; ``W[name]`` a tensor of the checkpoint; linear weights are
``[out, in]``; ``p`` the prefix of a part's tensor names and ``m`` its dictionary of the configuration.
"""

from __future__ import annotations

import math

import torch

DT = torch.float64
SWISH_SLOPE = 1.702  # the experts' activation is g * sigmoid(1.702 g)


def rms(x, eps, weight=None):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def linear(h, W, name):
    y = h @ W[name].T
    return y + W[name + ".b"] if name + ".b" in W else y


def rotate(x, rot):
    """x [T, heads, D]: lanes i and i + dims/2 of the first ``dims`` lanes turn by position * base^(-2i/dims)."""
    if not rot or not rot.get("dims"):
        return x
    dims = rot["dims"]
    f = float(rot["base"]) ** (-2 * torch.arange(dims // 2, dtype=DT) / dims)
    angle = torch.arange(x.shape[0], dtype=DT)[:, None] * f[None, :]
    c, s = angle.cos()[:, None, :], angle.sin()[:, None, :]
    u, v = x[..., : dims // 2], x[..., dims // 2 : dims]
    return torch.cat((u * c - v * s, v * c + u * s, x[..., dims:]), dim=-1)


def query_temperature(T, qt):
    """The factor on the query at every position: 1 + coef * ln(floor((p + 1) / every) + 1)."""
    p = torch.arange(T, dtype=DT)
    return 1.0 + float(qt["coef"]) * torch.log(torch.floor((p + 1) / qt["every"]) + 1.0)


def softmax_rows(s, sink=None):
    """s [H, T, T] scores (already scaled), causal; ``sink [H]``: one more term exp(sink) in every denominator."""
    T = s.shape[-1]
    s = s.masked_fill(~torch.tril(torch.ones(T, T, dtype=torch.bool)), -math.inf)
    top = s.max(-1, keepdim=True).values
    if sink is not None:
        top = torch.maximum(top, sink[:, None, None])
    e = torch.exp(s - top)
    denominator = e.sum(-1, keepdim=True)
    if sink is not None:
        denominator = denominator + torch.exp(sink[:, None, None] - top)
    return e / denominator


def attention(h, W, p, m, eps, shared=None):
    """The mixer of type ``attention``.  ``shared``: (keys, values) of the layer that ``kv_from`` names.  Returns the
    output and the (keys, values) this layer holds."""
    T, H, G, D, V = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = linear(h, W, p + "q").view(T, H, D)
    if shared is None:
        k, v = linear(h, W, p + "k").view(T, G, D), linear(h, W, p + "v").view(T, G, V)
    else:
        k, v = shared
    if m.get("q_temp"):
        q = q * query_temperature(T, m["q_temp"])[:, None, None]
    kv_of = torch.arange(H) // (H // G)
    w = softmax_rows(torch.einsum("ihd,jhd->hij", q, k[:, kv_of]) * m["scale"])
    o = torch.einsum("hij,jhd->ihd", w, v[:, kv_of]).reshape(T, H * V)
    o = o * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T, (k, v)


def sink_attention(h, W, p, m, eps):
    """The left half of the side-by-side mixer: the values are the keys as projected, q and k are normed per head and
    partly rotated, and every head's softmax has one more term in its denominator."""
    T, H, G, D = h.shape[0], m["heads"], m["kv_heads"], m["dim"]
    q, k = linear(h, W, p + "q").view(T, H, D), linear(h, W, p + "k").view(T, G, D)
    v = k
    q, k = rms(q, eps, W[p + "q.norm"]), rms(k, eps, W[p + "k.norm"])
    q, k = rotate(q, m.get("rot")), rotate(k, m.get("rot"))
    kv_of = torch.arange(H) // (H // G)
    w = softmax_rows(torch.einsum("ihd,jhd->hij", q, k[:, kv_of]) * m["scale"], W[p + "sink"])
    return torch.einsum("hij,jhd->ihd", w, v[:, kv_of]).reshape(T, H * D) @ W[p + "o"].T


def gated_linear_attention(h, W, p, m, eps):
    """The right half: a matrix of state per head whose rows (key channels) each decay by a factor of their own that
    the token chooses."""
    T, H, D, V = h.shape[0], m["heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).view(T, H, D) * D ** -0.5
    k = (h @ W[p + "k"].T).view(T, H, D)
    v = (h @ W[p + "v"].T).view(T, H, V)
    z = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "a2.b"]
    alpha = torch.sigmoid(z).pow(1.0 / float(m["tau"])).view(T, H, D)
    S = torch.zeros(H, D, V, dtype=DT)
    o = torch.zeros(T, H, V, dtype=DT)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms(o, eps, W[p + "norm"]).reshape(T, H * V)
    return (o * torch.nn.functional.silu(h @ W[p + "g"].T)) @ W[p + "o"].T


def parallel_mixer(h, W, p, m, eps):
    left = sink_attention(h, W, p + "left.", m["left"], eps)
    right = gated_linear_attention(h, W, p + "right.", m["right"], eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def expert(h, W, p, limit):
    g = torch.clamp(h @ W[p + "gate"].T, max=limit)
    u = torch.clamp(h @ W[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(SWISH_SLOPE * g) * (u + 1.0)) @ W[p + "down"].T


def table_routed_mlp(h, W, p, c, tokens):
    """Every token id has its experts in a table; each counts 1 / top; a shared expert is added for every token."""
    top = c["router"]["top"]
    out = torch.zeros_like(h)
    for t, token in enumerate(tokens):
        for e in W[p + "table"][token].tolist():
            out[t] += expert(h[t : t + 1], W, f"{p}e{int(e)}.", float(c["expert"]["limit"]))[0] / top
    if c.get("shared"):
        out = out + expert(h, W, p + "shared.", float(c["shared"]["limit"]))
    return out


def hyper_sublayer(X, W, p, norm_weight, eps, part):
    """One part between hyper-connections: read the S copies in, run the part, mix the copies and write out."""
    u = torch.einsum("s,stw->tw", W[p + "in"], X)
    y = part(rms(u, eps, norm_weight))
    return torch.einsum("st,snw->tnw", W[p + "mix"], X) + W[p + "out"][:, None, None] * y[None]


def forward(cfg, tensors, tokens, return_layers=False):
    """Logits ``[T, vocab]`` of one sequence (and, with ``return_layers``, the sum of the stream's copies after every layer)."""
    W = {k: (v.to(DT) if v.is_floating_point() else v.long()) for k, v in tensors.items()}
    eps = float(cfg["norm"]["eps"])
    S = cfg.get("streams")
    x = W["embed"][torch.tensor(tokens)]
    X = x[None].repeat(S or 1, 1, 1)
    held, layers = {}, []
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        if layer["type"] == "attention":
            def mixer(h, i=i, p=p, m=m):
                out, held[i] = attention(h, W, p + "mix.", m, eps, held[m["kv_from"]] if m.get("kv_from") is not None else None)
                return out
        elif layer["type"] == "parallel":
            def mixer(h, p=p, m=m):
                return parallel_mixer(h, W, p + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        parts = [(p + "hc1.", W[p + "norm1"], mixer)]
        if layer.get("mlp"):
            parts.append((p + "hc2.", W[p + "norm2"], lambda h, p=p, c=layer["mlp"]: table_routed_mlp(h, W, p + "mlp.", c, tokens)))
        for hc, weight, part in parts:
            if S:
                X = hyper_sublayer(X, W, hc, weight, eps, part)
            else:
                X = X + part(rms(X[0], eps, weight))[None]
        layers.append(X.sum(0))
    logits = rms(X.sum(0), eps, W["final.norm"]) @ W["head"].T
    return (logits, torch.stack(layers)) if return_layers else logits
