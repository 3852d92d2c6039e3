"""Grouped-query softmax attention over a paged cache, with the options that designs put around it.

    q = W_q x (+ b_q), k = W_k x (+ b_k), v = W_v x (+ b_v)           (one stacked product, result kept 32-bit)
    values_are_keys: no W_v; a key head's value is that head as projected (bias included), before norm and rotation
    conv:            every channel of q, k and v passes a short causal convolution over time directly behind the projection,
                     y_t = sum_j w[:, j] u_(t - taps + 1 + j) with weights ``<name>.conv`` [channels, taps]; a request's last
                     taps - 1 projected rows are kept in a state slot beside its pages
    qk_norm_eps:     every query head and every key head RMS-normed over its lanes, weights ``q.norm`` / ``k.norm`` [dim]
                     shared by the heads, before rotation
    rotary:          lanes i and i + dims/2 of the first ``dims`` lanes of every head turn by position * base^(-2i/dims)
                     (``rotary_layout = "interleaved"``: lanes 2i and 2i + 1)
    value_mix:       "source": the values as projected (bias included, behind the convolution) are handed to later layers of
                     the same pass; "mixed": v <- (1 - vmix) v + vmix v_source, v_source the source layer's values of the same
                     token and ``vmix`` a number of the checkpoint; what is cached is the mixed value
    q_temp:          queries times 1 + coef * ln(floor((position + 1) / every) + 1)
    score(i, j) = scale * q_i . k_j   for j <= i (within ``window`` if there is one); softmax over the visible keys
    softcap:         score <- softcap * tanh(score / softcap)
    distance_bias b: the score then loses slope_h * (i - j), slope_h = 2^(-b (h + 1) / heads)
    keep_first:      with a window, the keys at positions below it stay visible
    chunk:           only the keys of the query's own block of ``chunk`` positions (counted from 0) are visible
    sink:            the softmax's denominator also holds exp(sink_h), a number per head with no key and no value
    gate:            the heads side by side times sigmoid(W_g x), before the output projection
    out = W_o [heads side by side] (+ b_o)

With ``own_kv=False`` the layer has no key and value projections and reads the pages that an earlier entry of the order
wrote (``LayerRun.cache_of``), with queries, mask and everything else of its own.  Keys (normed, rotated) and values live
in pages of the cache manager; biases, norms, angles, the queries' factor, scores, the softmax and the gate are 32-bit in
both compute types.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import CompositeSpec, Mixer, PagedKVSpec, StateSpec, TensorSpec, register_part
from .sigmoid_attention import rotary_frequencies

_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "g": "g", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "q_norm": "q.norm",
          "k_norm": "k.norm", "sink": "sink", "o_bias": "o.b", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "value_mix": "vmix"}


class SoftmaxAttention(Mixer):
    graph_safe = True
    accepts_sink = True
    takes_projection = True  # a mixer that runs this one beside others may run the input product itself (``forward(proj=)``)

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int, scale: float,
                 bias: bool = False, qk_norm_eps: float | None = None, rotary: dict | None = None, q_temp: dict | None = None,
                 sink: bool = False, gate: bool = False, values_are_keys: bool = False, own_kv: bool = True,
                 window: int | None = None, tensor_names: dict[str, str] | None = None, out_bias: bool = False,
                 rotary_layout: str = "half", keep_first: int | None = None, chunk: int | None = None, softcap: float | None = None,
                 distance_bias: float | None = None, conv: int | None = None, value_mix: str | None = None,
                 value_mix_key: str = "first_values"):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        if not (1 <= int(head_dim) <= 640 and 1 <= int(value_dim) <= 512):
            raise ValueError(f"head_dim {head_dim} / value_dim {value_dim}: the kernels take keys of up to 640 and values of up to 512 lanes")
        if values_are_keys and int(value_dim) != int(head_dim):
            raise ValueError(f"values that are the keys have the keys' size {head_dim}, not {value_dim}")
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.head_dim, self.value_dim, self.scale = int(head_dim), int(value_dim), float(scale)
        self.bias, self.has_sink, self.has_gate = bool(bias), bool(sink), bool(gate)
        self.values_are_keys, self.own_kv = bool(values_are_keys), bool(own_kv)
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        self.rotary = dict(rotary) if rotary and rotary.get("dims") else None
        if self.rotary and (self.rotary["dims"] % 2 or not 0 < self.rotary["dims"] <= self.head_dim):
            raise ValueError(f"rotary dims {self.rotary['dims']} must be even and fit a head of {self.head_dim}")
        self.q_temp = (float(q_temp["coef"]), int(q_temp["every"])) if q_temp else None
        if self.q_temp and self.q_temp[1] < 1:
            raise ValueError(f"q_temp.every must be positive, got {self.q_temp[1]}")
        self.window = None if window is None else int(window)
        self.out_bias = bool(out_bias)
        if rotary_layout not in ("half", "interleaved"):
            raise ValueError(f"rotated lanes pair as 'half' or 'interleaved', not {rotary_layout!r}")
        self.rotary_layout = rotary_layout
        self.keep_first = int(keep_first) if keep_first else None
        self.chunk = int(chunk) if chunk else None
        self.softcap = float(softcap) if softcap else None
        self.distance_bias = None if distance_bias is None else float(distance_bias)
        for what, value in (("window", self.window), ("keep_first", self.keep_first), ("chunk", self.chunk)):
            if value is not None and value < 1:
                raise ValueError(f"{what} must be positive or None, got {value}")
        if self.keep_first and not self.window:
            raise ValueError("kept first keys go with a window")
        self.conv = int(conv) if conv else None
        if self.conv is not None and (not 1 <= self.conv <= 16 or not self.own_kv or self.values_are_keys or self.bias):
            raise ValueError("a short convolution has 1 to 16 taps and stands behind q, k and v projections without biases")
        if value_mix not in (None, "source", "mixed") or (value_mix and (not self.own_kv or self.values_are_keys)):
            raise ValueError(f"value_mix is None, 'source' or 'mixed' for a layer with values of its own, got {value_mix!r}")
        self.value_mix, self.value_mix_key = value_mix, value_mix_key
        self.names = {**_NAMES, **(tensor_names or {})}
        self.w_in = self.w_out = self.b_in = self.q_weight = self.k_weight = self.sink = self.freq = None
        self.b_out = self.w_conv = self.slopes = None
        self.mix = 0.0
        self.dtype: torch.dtype | None = None

    def _stacked(self) -> list[str]:
        """The roles whose matrices make the input product, in the order of its columns (the gate last)."""
        roles = ["q"]
        if self.own_kv:
            roles += ["k"] if self.values_are_keys else ["k", "v"]
        return roles

    def tensors(self) -> dict[str, TensorSpec]:
        n, H, KV, D, V, hid = self.names, self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim, self.hidden_size
        rows = {"q": H * D, "k": KV * D, "v": KV * V}
        specs = {}
        for role in self._stacked():
            specs[n[role]] = TensorSpec((rows[role], hid))
            if self.bias:
                specs[n[role + "_bias"]] = TensorSpec((rows[role],))
        if self.has_gate:
            specs[n["g"]] = TensorSpec((H * V, hid))
        specs[n["o"]] = TensorSpec((hid, H * V))
        if self.qk_norm_eps is not None:
            specs[n["q_norm"]] = TensorSpec((D,), init="ones_plus_normal")
            if self.own_kv:
                specs[n["k_norm"]] = TensorSpec((D,), init="ones_plus_normal")
        if self.has_sink:
            specs[n["sink"]] = TensorSpec((H,))
        if self.out_bias:
            specs[n["o_bias"]] = TensorSpec((hid,))
        if self.conv:
            for role in ("q", "k", "v"):
                specs[n[role + "_conv"]] = TensorSpec((rows[role], self.conv), init="mean_plus_normal")
        if self.value_mix:
            specs[n["value_mix"]] = TensorSpec((), init="half_plus_normal")  # the source layer has one too and does not read it
        return specs

    def bind(self, tensors, dtype, device) -> None:
        n = self.names
        roles = self._stacked()
        mats = [tensors[n[r]].to(dtype) for r in roles] + ([tensors[n["g"]].to(dtype)] if self.has_gate else [])
        self.w_in = torch.cat(mats, dim=0).to(device).contiguous()
        self.w_out = tensors[n["o"]].to(device=device, dtype=dtype).contiguous()
        f32 = lambda t: t.to(device=device, dtype=torch.float32).contiguous()  # noqa: E731
        if self.bias:
            self.b_in = f32(torch.cat([tensors[n[r + "_bias"]].float() for r in roles]))
        if self.qk_norm_eps is not None:
            self.q_weight = f32(tensors[n["q_norm"]])
            self.k_weight = f32(tensors[n["k_norm"]]) if self.own_kv else None
        if self.has_sink:
            self.sink = f32(tensors[n["sink"]])
        if self.rotary:
            self.freq = rotary_frequencies(self.rotary["dims"], self.rotary["base"]).to(device)
        if self.out_bias:
            self.b_out = f32(tensors[n["o_bias"]])
        if self.conv:
            self.w_conv = f32(torch.cat([tensors[n[r + "_conv"]].float() for r in ("q", "k", "v")], dim=0))
        if self.value_mix == "mixed":
            self.mix = float(tensors[n["value_mix"]].float().reshape(()))
        if self.distance_bias is not None:
            heads = torch.arange(1, self.num_heads + 1, dtype=torch.float64)
            self.slopes = torch.pow(2.0, -self.distance_bias * heads / self.num_heads).to(torch.float32).to(device)
        self.dtype = dtype

    def _channels(self) -> int:
        """Columns of the input product that are queries, keys and values."""
        return (self.num_heads + self.num_kv_heads) * self.head_dim + self.num_kv_heads * self.value_dim

    def cache_spec(self):
        pages = PagedKVSpec(self.num_kv_heads, max(self.head_dim, self.value_dim), self.window, self.keep_first, self.chunk)
        if self.conv and self.conv > 1:  # the rows that the convolution still reads when the next step begins
            return CompositeSpec((pages, StateSpec((self.conv - 1, self._channels()), torch.float32)))
        return pages

    def forward(self, x, ctx, cache, sink=None, proj=None):
        """``proj``: the stacked projections (32-bit, rows may have a pitch) where the caller ran the product."""
        H, KV, D, V = self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim
        if proj is None:
            proj = ops.linear(x, self.w_in, out_dtype=torch.float32)
        kv = KV if self.own_kv else 0
        if self.conv:
            tail = None
            if self.conv > 1:
                cache, tail = cache.parts
            proj = ops.short_conv(proj, self.w_conv, None if tail is None else tail.states, ctx.state_slots if tail is None else tail.slots,
                                  ctx, channels=self._channels())
        keep = first = None
        if self.value_mix == "source":  # later layers of this pass mix these values into their own
            keep = ctx.shared[self.value_mix_key] = torch.empty((proj.shape[0], KV * V), dtype=torch.float32, device=proj.device)
        elif self.value_mix == "mixed":
            first = ctx.shared[self.value_mix_key]
        q = ops.head_prepare(proj, ctx.positions, heads=H, kv_heads=kv, dim=D, value_dim=V, bias=self.b_in, q_weight=self.q_weight,
                             k_weight=self.k_weight, eps=self.qk_norm_eps or 0.0, freq=self.freq, warm=self.q_temp,
                             values_are_keys=self.values_are_keys, pool=cache.pool, slot_map=cache.slot_map, out_dtype=self.dtype,
                             interleaved=self.rotary_layout == "interleaved", values_out=keep, values_first=first, values_lambda=self.mix)
        gate = None
        if self.has_gate:
            start = (H + kv) * D + (0 if self.values_are_keys else kv * V)
            gate = proj[:, start : start + H * V]
        out = ops.paged_softmax_attention(q, cache.pool, cache.page_table, ctx, num_heads=H, num_kv_heads=KV, key_dim=D, value_dim=V,
                                          scale=self.scale, window=self.window, sinks=self.sink, gate=gate, keep_first=self.keep_first,
                                          chunk=self.chunk, softcap=self.softcap, slopes=self.slopes)
        if self.b_out is not None:
            return ops.add_bias(ops.linear(out, self.w_out, out_dtype=torch.float32), self.b_out)
        if sink is not None:
            handed_on = sink.linear(out, self.w_out)
            if handed_on is not None:
                return handed_on
        return ops.linear(out, self.w_out, out_dtype=torch.float32)


register_part("mixer", "softmax_attention", SoftmaxAttention)
