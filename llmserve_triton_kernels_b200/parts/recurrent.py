"""Recurrences with a fixed-size state per request: an element-wise gated one (minGRU), one whose state is a matrix per
head that decays by a fixed factor (retention), and one whose matrix decays row by row as each token chooses (gated linear
attention).

minGRU: the update gate and the candidate read only the current token,

    z_t = sigmoid(W_z x_t + b_z)        u_t = W_x x_t + b_x
    c_t = u_t + 1/2  where u_t >= 0,    sigmoid(u_t)  elsewhere
    S_t = (1 - z_t) S_(t-1) + z_t c_t   out_t = W_o (S_t * silu(W_g x_t))

The state starts at zero, is 32-bit and lives in the request's slot of the cache manager's state tensor; the three
projections are one stacked product whose result stays 32-bit, so that everything that enters the recurrence is.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Mixer, StateSpec, TensorSpec, register_part

_NAMES = {"z": "z", "z_bias": "z.b", "x": "x", "x_bias": "x.b", "gate": "g", "out": "o"}


class MinGRU(Mixer):
    graph_safe = True
    accepts_sink = True

    def __init__(self, hidden_size: int, width: int, bias: bool = True, tensor_names: dict[str, str] | None = None):
        self.hidden_size, self.width, self.bias = int(hidden_size), int(width), bool(bias)
        self.names = {**_NAMES, **(tensor_names or {})}
        self.w_in = self.w_out = self.b_z = self.b_x = None
        self.dtype: torch.dtype | None = None

    def tensors(self) -> dict[str, TensorSpec]:
        n, w, h = self.names, self.width, self.hidden_size
        specs = {n["z"]: TensorSpec((w, h)), n["x"]: TensorSpec((w, h)), n["gate"]: TensorSpec((w, h)), n["out"]: TensorSpec((h, w))}
        if self.bias:
            specs[n["z_bias"]] = TensorSpec((w,))
            specs[n["x_bias"]] = TensorSpec((w,))
        return specs

    def bind(self, tensors, dtype, device) -> None:
        n = self.names
        self.w_in = torch.cat([tensors[n[k]].to(dtype) for k in ("z", "x", "gate")], dim=0).to(device).contiguous()
        self.w_out = tensors[n["out"]].to(device=device, dtype=dtype).contiguous()
        if self.bias:
            self.b_z = tensors[n["z_bias"]].to(device=device, dtype=torch.float32).contiguous()
            self.b_x = tensors[n["x_bias"]].to(device=device, dtype=torch.float32).contiguous()
        self.dtype = dtype

    def cache_spec(self) -> StateSpec:
        return StateSpec((self.width,), torch.float32)

    def forward(self, x, ctx, cache, sink=None):
        proj = ops.linear(x, self.w_in, out_dtype=torch.float32)  # [N, z | x | gate], 32-bit
        out = ops.mingru_scan(proj, self.b_z, self.b_x, cache.states, cache.slots, ctx.cu_tokens, ctx.num_requests, self.width, self.dtype, ctx.max_query_len)
        if sink is not None:
            handed_on = sink.linear(out, self.w_out)
            if handed_on is not None:
                return handed_on
        return ops.linear(out, self.w_out, out_dtype=torch.float32)


register_part("mixer", "mingru", MinGRU)


class Retention(Mixer):
    """Linear attention with one fixed decay per head, no softmax and no denominator:

        q = W_q x, k = W_k x (heads x dim), v = W_v x (heads x value_dim), g = W_g x
        q, k: lanes i and i + rot/2 of every head turned by position * base^(-2i / rot); k then times dim^(-1/2)
        S_t = decay_h S_(t-1) + k_t v_t^T        o_t = S_t^T q_t
        out = W_o (unit_rms_per_head(o_t) * silu(g))

    S ``[heads, dim, value_dim]`` starts at zero, is 32-bit and lives in the request's slot of the cache manager's
    state tensor.  The four projections are one stacked product whose result stays 32-bit, so that what enters the
    recurrence (rotated queries and keys, values) is; the norm of each head's o has no weight."""

    graph_safe = True
    accepts_sink = True
    takes_projection = True  # a mixer that runs this one beside others may run the input product itself (``forward(proj=)``)

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, decay: list[float], norm_eps: float,
                 rotary: dict | None = None, gate: str = "silu", tensor_names: dict[str, str] | None = None):
        if len(decay) != num_heads:
            raise ValueError(f"{len(decay)} decays for {num_heads} heads")
        if not 1 <= int(head_dim) <= 256:
            raise ValueError(f"head_dim {head_dim}: the recurrence's kernel takes keys of up to 256 lanes")
        self.hidden_size, self.num_heads, self.head_dim, self.value_dim = int(hidden_size), int(num_heads), int(head_dim), int(value_dim)
        self.decay_values, self.norm_eps, self.gate = [float(d) for d in decay], float(norm_eps), gate
        self.rotary = dict(rotary) if rotary and rotary.get("dims") else None
        if self.rotary and not 0 < self.rotary["dims"] <= self.head_dim:
            raise ValueError(f"rotary dims {self.rotary['dims']} do not fit a head of {self.head_dim}")
        self.names = {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o", **(tensor_names or {})}
        self.w_in = self.w_out = self.decay = self.freq = None
        self.dtype: torch.dtype | None = None

    def tensors(self) -> dict[str, TensorSpec]:
        n, h, qk, vv = self.names, self.hidden_size, self.num_heads * self.head_dim, self.num_heads * self.value_dim
        return {n["q"]: TensorSpec((qk, h)), n["k"]: TensorSpec((qk, h)), n["v"]: TensorSpec((vv, h)),
                n["gate"]: TensorSpec((vv, h)), n["out"]: TensorSpec((h, vv))}

    def bind(self, tensors, dtype, device) -> None:
        from .sigmoid_attention import rotary_frequencies

        n = self.names
        self.w_in = torch.cat([tensors[n[k]].to(dtype) for k in ("q", "k", "v", "gate")], dim=0).to(device).contiguous()
        self.w_out = tensors[n["out"]].to(device=device, dtype=dtype).contiguous()
        self.decay = torch.tensor(self.decay_values, dtype=torch.float64).to(torch.float32).to(device)
        if self.rotary:
            self.freq = rotary_frequencies(self.rotary["dims"], self.rotary["base"], self.rotary.get("scaling")).to(device)
        self.dtype = dtype

    def cache_spec(self) -> StateSpec:
        return StateSpec((self.num_heads, self.head_dim, self.value_dim), torch.float32)

    def forward(self, x, ctx, cache, sink=None, proj=None):
        H, D, V = self.num_heads, self.head_dim, self.value_dim
        if proj is None:
            proj = ops.linear(x, self.w_in, out_dtype=torch.float32)  # [N, q | k | v | gate], 32-bit
        q, k = ops.qk_prepare(proj, ctx.positions, heads=H, kv_heads=H, dim=D, freq=self.freq, k_scale=D ** -0.5, out_dtype=torch.float32)
        o = ops.retention_scan(q, k, proj[:, 2 * H * D : 2 * H * D + H * V], self.decay, cache.states, cache.slots, ctx.cu_tokens,
                               ctx.num_requests, H, D, V, ctx.max_query_len)
        out = ops.head_norm_gate(o, proj[:, 2 * H * D + H * V :], self.norm_eps, self.gate, out_dtype=self.dtype)
        if sink is not None:
            handed_on = sink.linear(out, self.w_out)
            if handed_on is not None:
                return handed_on
        return ops.linear(out, self.w_out, out_dtype=torch.float32)


register_part("mixer", "retention", Retention)


class GatedLinearAttention(Mixer):
    """Linear attention whose state decays row by row, by factors that every token chooses through a low-rank product:

        q = W_q x * dim^(-1/2), k = W_k x (heads x dim), v = W_v x (heads x value_dim), g = W_g x
        alpha = sigmoid(W_a2 (W_a1 x) + b_a2) ^ (1 / tau)                    (heads x dim: one decay per key channel)
        S_t = diag(alpha_t) S_(t-1) + k_t v_t^T        o_t = S_t^T q_t       per head
        out = W_o (rmsnorm_per_head(o_t) * w_norm * silu(g))                 (w_norm [value_dim], shared by the heads)

    S ``[heads, dim, value_dim]`` starts at zero, is 32-bit and lives in the request's slot of the cache manager's state
    tensor.  The five input projections are one stacked product whose result stays 32-bit; the second product of the
    decay reads its 32-bit input as it is; the decays (through the logarithm of the sigmoid), the recurrence and the norm
    are 32-bit."""

    graph_safe = True
    accepts_sink = True
    takes_projection = True  # a mixer that runs this one beside others may run the input product itself (``forward(proj=)``)

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, tau: float, norm_eps: float,
                 decay_rank: int | None = None, gate: str = "silu", tensor_names: dict[str, str] | None = None):
        """``decay_rank``: the inner size of the decay's two products (``a1 [rank, hidden]``, ``a2 [heads * dim, rank]``);
        None: whatever the checkpoint's tensors have (a random model then takes a quarter of ``head_dim``, at least 1)."""
        if not 1 <= int(head_dim) <= 256:
            raise ValueError(f"head_dim {head_dim}: the recurrence's kernel takes keys of up to 256 lanes")
        if not float(tau) > 0:
            raise ValueError(f"tau must be positive, got {tau}")
        if decay_rank is not None and int(decay_rank) < 1:
            raise ValueError(f"decay_rank must be positive, got {decay_rank}")
        self.hidden_size, self.num_heads, self.head_dim, self.value_dim = int(hidden_size), int(num_heads), int(head_dim), int(value_dim)
        self.tau, self.norm_eps, self.gate = float(tau), float(norm_eps), gate
        self.decay_rank = None if decay_rank is None else int(decay_rank)
        self.names = {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o", "norm": "norm", "a1": "a1", "a2": "a2", "a2_bias": "a2.b",
                      **(tensor_names or {})}
        self.w_in = self.w_out = self.w_a2 = self.b_a2 = self.norm_weight = None
        self.dtype: torch.dtype | None = None

    def tensors(self) -> dict[str, TensorSpec]:
        n, h, qk, vv = self.names, self.hidden_size, self.num_heads * self.head_dim, self.num_heads * self.value_dim
        r, stand_in = (-1 if self.decay_rank is None else self.decay_rank), max(1, self.head_dim // 4)
        return {n["q"]: TensorSpec((qk, h)), n["k"]: TensorSpec((qk, h)), n["v"]: TensorSpec((vv, h)), n["gate"]: TensorSpec((vv, h)),
                n["out"]: TensorSpec((h, vv)), n["norm"]: TensorSpec((self.value_dim,), init="ones_plus_normal"),
                n["a1"]: TensorSpec((r, h), free_size=stand_in), n["a2"]: TensorSpec((qk, r), free_size=stand_in), n["a2_bias"]: TensorSpec((qk,))}

    def bind(self, tensors, dtype, device) -> None:
        n = self.names
        rank = tensors[n["a1"]].shape[0]
        if tensors[n["a2"]].shape[1] != rank or (self.decay_rank is not None and rank != self.decay_rank):
            raise ValueError(f"the decay's two matrices disagree on their inner size: {tuple(tensors[n['a1']].shape)} and {tuple(tensors[n['a2']].shape)}")
        self.rank = rank
        self.w_in = torch.cat([tensors[n[k]].to(dtype) for k in ("q", "k", "v", "gate", "a1")], dim=0).to(device).contiguous()
        self.w_out = tensors[n["out"]].to(device=device, dtype=dtype).contiguous()
        self.w_a2 = tensors[n["a2"]].to(device=device, dtype=dtype).contiguous()
        self.b_a2 = tensors[n["a2_bias"]].to(device=device, dtype=torch.float32).contiguous()
        self.norm_weight = tensors[n["norm"]].to(device=device, dtype=torch.float32).contiguous()
        self.dtype = dtype

    def cache_spec(self) -> StateSpec:
        return StateSpec((self.num_heads, self.head_dim, self.value_dim), torch.float32)

    def forward(self, x, ctx, cache, sink=None, proj=None):
        H, D, V = self.num_heads, self.head_dim, self.value_dim
        if proj is None:
            proj = ops.linear(x, self.w_in, out_dtype=torch.float32)  # [N, q | k | v | gate | a1], 32-bit
        qk, vv = H * D, H * V
        z = ops.linear32(proj[:, 2 * qk + 2 * vv : 2 * qk + 2 * vv + self.rank], self.w_a2)
        o = ops.gated_scan(proj[:, :qk], proj[:, qk : 2 * qk], proj[:, 2 * qk : 2 * qk + vv], z, self.b_a2, 1.0 / self.tau, D ** -0.5,
                           cache.states, cache.slots, ctx.cu_tokens, ctx.num_requests, H, D, V, ctx.max_query_len)
        out = ops.head_norm_gate(o, proj[:, 2 * qk + vv : 2 * qk + 2 * vv], self.norm_eps, self.gate, out_dtype=self.dtype, weight=self.norm_weight)
        if sink is not None:
            handed_on = sink.linear(out, self.w_out)
            if handed_on is not None:
                return handed_on
        return ops.linear(out, self.w_out, out_dtype=torch.float32)


register_part("mixer", "gated_linear_attention", GatedLinearAttention)
