"""Dense gated feed-forward: ``down(act(gate(x)) * up(x))`` without biases.

Parity: src/llmserve/model/llama.py:112-120, where the activation is SiLU
(``z * sigmoid(z)``); the gate and up matrices are stacked at load so that one matrix product
feeds the activation kernel.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, TensorSpec, register_part

_ACTIVATIONS = ("silu",)


class GatedMLP(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "silu", bias: bool = False,
                 tensor_names: dict[str, str] | None = None):
        """``tensor_names``: local names of the three matrices (default ``gate_proj.weight`` and so on) and, with
        ``bias``, of their bias vectors (``gate_bias`` and so on; default ``gate_proj.bias`` ...)."""
        self.names = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight", "gate_bias": "gate_proj.bias",
                      "up_bias": "up_proj.bias", "down_bias": "down_proj.bias", **(tensor_names or {})}
        if activation not in _ACTIVATIONS:
            raise ValueError(f"activation {activation!r} is not built; known: {_ACTIVATIONS}")
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.activation = activation
        self.bias = bool(bias)  # ``*_proj.bias`` vectors (none in Llama): products and bias sums as kernels of their own
        self.b_gate_up: torch.Tensor | None = None
        self.b_down: torch.Tensor | None = None
        self.w_gate_up: torch.Tensor | None = None  # [2 I, hidden]: gate rows, then up rows
        self.w_down: torch.Tensor | None = None  # [hidden, I]

    def tensors(self) -> dict[str, TensorSpec]:
        i, h = self.intermediate_size, self.hidden_size
        specs = {
            self.names["gate"]: TensorSpec((i, h)),
            self.names["up"]: TensorSpec((i, h)),
            self.names["down"]: TensorSpec((h, i)),
        }
        if self.bias:
            specs.update({self.names["gate_bias"]: TensorSpec((i,)), self.names["up_bias"]: TensorSpec((i,)), self.names["down_bias"]: TensorSpec((h,))})
        return specs

    def bind(self, tensors, dtype, device) -> None:
        fused = torch.cat([tensors[self.names["gate"]].to(dtype), tensors[self.names["up"]].to(dtype)], dim=0)
        self.w_gate_up = fused.to(device).contiguous()
        self.w_down = tensors[self.names["down"]].to(device=device, dtype=dtype).contiguous()
        if self.bias:
            self.b_gate_up = torch.cat([tensors[self.names["gate_bias"]].to(dtype), tensors[self.names["up_bias"]].to(dtype)]).to(device).contiguous()
            self.b_down = tensors[self.names["down_bias"]].to(device=device, dtype=dtype).contiguous()

    accepts_sink = True

    def forward(self, x, ctx, sink=None):
        if self.bias:
            act = ops.swiglu(ops.linear(x, self.w_gate_up), self.b_gate_up)  # the bias joins in the activation's kernel
            return ops.add_bias(ops.linear(act, self.w_down, out_dtype=torch.float32), self.b_down.float())
        act = ops.linear_swiglu(x, self.w_gate_up)
        if sink is not None:
            handed_on = sink.linear(act, self.w_down)
            if handed_on is not None:
                return handed_on
        # the contribution to the 32-bit residual stream leaves the product in 32-bit: it is the sum's largest addend
        return ops.linear(act, self.w_down, out_dtype=torch.float32)


register_part("feed_forward", "gated_mlp", GatedMLP)


class DenseMLP(FeedForward):
    """``down(act(up(x)))`` without biases; ``act`` one of ``relu2`` (the square of relu), ``gelu_tanh``, ``silu``.
    ``tensor_names``: local names of the two matrices (default ``up`` and ``down``)."""

    graph_safe = True
    accepts_sink = True
    activations = ("relu2", "gelu_tanh", "silu")

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "relu2", tensor_names: dict[str, str] | None = None):
        if activation not in self.activations:
            raise ValueError(f"activation {activation!r} is not built; known: {self.activations}")
        self.hidden_size, self.intermediate_size, self.activation = int(hidden_size), int(intermediate_size), activation
        self.names = {"up": "up", "down": "down", **(tensor_names or {})}
        self.w_up: torch.Tensor | None = None  # [I, hidden]
        self.w_down: torch.Tensor | None = None  # [hidden, I]

    def tensors(self) -> dict[str, TensorSpec]:
        i, h = self.intermediate_size, self.hidden_size
        return {self.names["up"]: TensorSpec((i, h)), self.names["down"]: TensorSpec((h, i))}

    def bind(self, tensors, dtype, device) -> None:
        self.w_up = tensors[self.names["up"]].to(device=device, dtype=dtype).contiguous()
        self.w_down = tensors[self.names["down"]].to(device=device, dtype=dtype).contiguous()

    def forward(self, x, ctx, sink=None):
        act = ops.linear_act(x, self.w_up, self.activation)
        if sink is not None:
            handed_on = sink.linear(act, self.w_down)
            if handed_on is not None:
                return handed_on
        return ops.linear(act, self.w_down, out_dtype=torch.float32)


register_part("feed_forward", "dense_mlp", DenseMLP)


class RoutedMLP(FeedForward):
    """A mixture of small feed-forward layers ``down_e(act(up_e(x)))`` without biases, of which each token uses ``top``:

        z = W_router x (32-bit), s = softmax(z) over all experts
        chosen: the ``top`` experts with the largest s + correction (``correction``: a tensor of the checkpoint)
        weights: router_scale * s of the chosen ones (divided by their sum only with ``renormalize``)
        out = sum over the chosen e of weight_e * expert_e(x)  +  sigmoid(w_sg . x) * shared(x)

    ``shared_size``: the inner size of an expert that every token uses (None: none); ``shared_gate``: whether it is
    multiplied by a sigmoid of one number per token.  Tensors: ``router``, ``correction``, ``e<i>.up``, ``e<i>.down``,
    ``shared.up``, ``shared.down``, ``shared.sg``.

    All experts' up matrices are stacked (the shared expert's last), so are the down matrices side by side: a step is
    one kernel for the router (its 32-bit product and the choice) and two matrix products over every expert with, between
    them, one kernel that applies the activation and the token's
    weight of each expert's block of columns (0 for an expert the token did not choose, the gate for the shared one).
    The second product then sums over the experts by itself.  Every weight matrix is read once a step whatever the
    tokens chose, which is what a decode step of several requests costs anyway; a prompt pays the products of the
    experts its tokens did not choose."""

    graph_safe = True
    accepts_sink = True

    def __init__(self, hidden_size: int, experts: int, top: int, expert_size: int, activation: str = "relu2",
                 router_scale: float = 1.0, correction: bool = True, renormalize: bool = False, shared_size: int | None = None,
                 shared_gate: bool = True):
        if activation not in DenseMLP.activations:
            raise ValueError(f"activation {activation!r} is not built; known: {DenseMLP.activations}")
        if not 1 <= int(top) <= int(experts):
            raise ValueError(f"a token uses {top} of {experts} experts")
        self.hidden_size, self.experts, self.top, self.expert_size = int(hidden_size), int(experts), int(top), int(expert_size)
        self.activation, self.router_scale = activation, float(router_scale)
        self.has_correction, self.renormalize = bool(correction), bool(renormalize)
        self.shared_size = int(shared_size) if shared_size else 0
        self.shared_gate = bool(shared_gate) and self.shared_size > 0
        self.w_router = self.correction = self.w_up = self.w_down = None

    def tensors(self) -> dict[str, TensorSpec]:
        h, f = self.hidden_size, self.expert_size
        specs = {"router": TensorSpec((self.experts, h))}
        if self.has_correction:
            specs["correction"] = TensorSpec((self.experts,))
        for e in range(self.experts):
            specs[f"e{e}.up"] = TensorSpec((f, h))
            specs[f"e{e}.down"] = TensorSpec((h, f))
        if self.shared_size:
            specs["shared.up"] = TensorSpec((self.shared_size, h))
            specs["shared.down"] = TensorSpec((h, self.shared_size))
            if self.shared_gate:
                specs["shared.sg"] = TensorSpec((1, h))
        return specs

    def bind(self, tensors, dtype, device) -> None:
        ups = [tensors[f"e{e}.up"] for e in range(self.experts)] + ([tensors["shared.up"]] if self.shared_size else [])
        downs = [tensors[f"e{e}.down"] for e in range(self.experts)] + ([tensors["shared.down"]] if self.shared_size else [])
        self.w_up = torch.cat([t.to(dtype) for t in ups], dim=0).to(device).contiguous()  # [E ff + shared, hidden]
        self.w_down = torch.cat([t.to(dtype) for t in downs], dim=1).to(device).contiguous()  # [hidden, E ff + shared]
        # the router (and the shared expert's gate as its last row) is a 32-bit product of its own
        rows = [tensors["router"].float()] + ([tensors["shared.sg"].float().reshape(1, -1)] if self.shared_gate else [])
        self.w_router = torch.cat(rows, dim=0).to(device).contiguous()
        if self.has_correction:
            self.correction = tensors["correction"].to(device=device, dtype=torch.float32).contiguous()

    def forward(self, x, ctx, sink=None):
        xt = x.materialize() if isinstance(x, ops.NormedInput) else x
        weights = ops.route(xt, self.w_router, self.correction, self.experts, self.top, self.router_scale, self.renormalize, self.shared_gate)
        if self.shared_size and not self.shared_gate:
            weights = torch.cat((weights, torch.ones_like(weights[:, :1])), dim=1)
        act = ops.expert_act_scale(ops.linear(xt, self.w_up), weights, self.experts, self.expert_size, self.activation)
        if sink is not None:
            handed_on = sink.linear(act, self.w_down)
            if handed_on is not None:
                return handed_on
        return ops.linear(act, self.w_down, out_dtype=torch.float32)


register_part("feed_forward", "routed_mlp", RoutedMLP)


class TableRoutedMLP(FeedForward):
    """A mixture of small gated feed-forward layers without a router: a table gives every token id its ``top`` experts
    (the entries of a row differ), each with weight ``1 / top``; a shared expert of the same form may run for every token.

        expert(x):  g = min(W_gate x, limit)     u = clamp(W_up x, -limit, limit)
                    W_down (g * sigmoid(slope * g) * (u + 1))
        out = (1 / top) * sum over table[token id] of expert_e(x)  +  shared(x)

    Tensors: ``table [vocab, top]`` (integers), ``e<i>.gate``, ``e<i>.up``, ``e<i>.down``, ``shared.gate``, ``shared.up``,
    ``shared.down``.  As in :class:`RoutedMLP` all experts' gate and up matrices are stacked (the shared expert's last)
    and so are the down matrices side by side: a step is one product over every expert, one kernel that applies the
    bounds, the activation and the token's weight of each expert's block of columns (0 for an expert the table does not
    give the token, whose columns are then not even read), and one product that sums over the experts by itself."""

    graph_safe = True
    accepts_sink = True

    def __init__(self, hidden_size: int, vocab_size: int, experts: int, top: int, expert_size: int, limit: float,
                 shared_size: int | None = None, shared_limit: float | None = None, slope: float = 1.702):
        if not 1 <= int(top) <= int(experts):
            raise ValueError(f"a token uses {top} of {experts} experts")
        self.hidden_size, self.vocab_size, self.experts, self.top = int(hidden_size), int(vocab_size), int(experts), int(top)
        self.expert_size, self.limit, self.slope = int(expert_size), float(limit), float(slope)
        self.shared_size = int(shared_size) if shared_size else 0
        self.shared_limit = float(shared_limit) if shared_limit is not None else self.limit
        self.table = self.w_up = self.w_down = None

    def tensors(self) -> dict[str, TensorSpec]:
        h, f = self.hidden_size, self.expert_size
        specs = {"table": TensorSpec((self.vocab_size, self.top), init=f"distinct:{self.experts}")}
        for e in range(self.experts):
            specs[f"e{e}.gate"] = TensorSpec((f, h))
            specs[f"e{e}.up"] = TensorSpec((f, h))
            specs[f"e{e}.down"] = TensorSpec((h, f))
        if self.shared_size:
            specs["shared.gate"] = TensorSpec((self.shared_size, h))
            specs["shared.up"] = TensorSpec((self.shared_size, h))
            specs["shared.down"] = TensorSpec((h, self.shared_size))
        return specs

    def bind(self, tensors, dtype, device) -> None:
        names = [f"e{e}." for e in range(self.experts)] + (["shared."] if self.shared_size else [])
        ups = [tensors[p + k] for p in names for k in ("gate", "up")]
        self.w_up = torch.cat([t.to(dtype) for t in ups], dim=0).to(device).contiguous()  # [E 2 ff + 2 shared, hidden]
        self.w_down = torch.cat([tensors[p + "down"].to(dtype) for p in names], dim=1).to(device).contiguous()  # [hidden, E ff + shared]
        table = tensors["table"]
        if table.is_floating_point() or int(table.min()) < 0 or int(table.max()) >= self.experts:
            raise ValueError("the experts' table must hold integers below the number of experts")
        self.table = table.to(device=device, dtype=torch.int32).contiguous()

    def forward(self, x, ctx, sink=None):
        xt = x.materialize() if isinstance(x, ops.NormedInput) else x
        act = ops.expert_gated_act(ops.linear(xt, self.w_up), self.experts, self.expert_size, self.shared_size, self.limit,
                                   self.shared_limit, self.slope, ids=ctx.token_ids, table=self.table)
        if sink is not None:
            handed_on = sink.linear(act, self.w_down)
            if handed_on is not None:
                return handed_on
        return ops.linear(act, self.w_down, out_dtype=torch.float32)


register_part("feed_forward", "table_routed_mlp", TableRoutedMLP)


class RoutedGatedMLP(FeedForward):
    """A mixture of small gated feed-forward layers ``down_e(silu(gate_e x) * up_e x)`` without biases, of which each token
    uses ``top``, chosen by a router with a bias:

        z = W_router x + b_router (32-bit)
        chosen: the ``top`` experts with the largest z; weights: the softmax over the chosen logits alone
        out = sum over the chosen e of weight_e * expert_e(x)  +  shared(x)

    ``shared_size``: the inner size of an expert of the same form that every token uses with weight one (None: none).
    Tensors: ``router``, ``router.b``, ``e<i>.gate``, ``e<i>.up``, ``e<i>.down``, ``shared.gate``, ``shared.up``, ``shared.down``.
    As in :class:`TableRoutedMLP` all experts' gate and up matrices are stacked (the shared expert's last) and the down
    matrices stand side by side: a step is one kernel for the router (its 32-bit product, the choice and the weights), one
    product over every expert, one kernel for the activation times the token's weight of each expert's block of columns
    (0, and nothing read, for an expert the token did not choose), and one product that sums over the experts by itself."""

    graph_safe = True
    accepts_sink = True
    takes_factored = False  # the router reads the normed rows themselves: the norm in front runs as its own kernel

    def __init__(self, hidden_size: int, experts: int, top: int, expert_size: int, shared_size: int | None = None, router_bias: bool = True):
        if not 1 <= int(top) <= int(experts):
            raise ValueError(f"a token uses {top} of {experts} experts")
        self.hidden_size, self.experts, self.top, self.expert_size = int(hidden_size), int(experts), int(top), int(expert_size)
        self.shared_size = int(shared_size) if shared_size else 0
        self.router_bias = bool(router_bias)
        self.w_router = self.b_router = self.w_up = self.w_down = None

    def tensors(self) -> dict[str, TensorSpec]:
        h, f = self.hidden_size, self.expert_size
        specs = {"router": TensorSpec((self.experts, h))}
        if self.router_bias:
            specs["router.b"] = TensorSpec((self.experts,))
        for e in range(self.experts):
            specs[f"e{e}.gate"] = TensorSpec((f, h))
            specs[f"e{e}.up"] = TensorSpec((f, h))
            specs[f"e{e}.down"] = TensorSpec((h, f))
        if self.shared_size:
            specs["shared.gate"] = TensorSpec((self.shared_size, h))
            specs["shared.up"] = TensorSpec((self.shared_size, h))
            specs["shared.down"] = TensorSpec((h, self.shared_size))
        return specs

    def bind(self, tensors, dtype, device) -> None:
        names = [f"e{e}." for e in range(self.experts)] + (["shared."] if self.shared_size else [])
        ups = [tensors[p + k] for p in names for k in ("gate", "up")]
        self.w_up = torch.cat([t.to(dtype) for t in ups], dim=0).to(device).contiguous()  # [E 2 ff + 2 shared, hidden]
        self.w_down = torch.cat([tensors[p + "down"].to(dtype) for p in names], dim=1).to(device).contiguous()  # [hidden, E ff + shared]
        self.w_router = tensors["router"].to(device=device, dtype=torch.float32).contiguous()
        if self.router_bias:
            self.b_router = tensors["router.b"].to(device=device, dtype=torch.float32).contiguous()

    def forward(self, x, ctx, sink=None):
        xt = x.materialize() if isinstance(x, ops.NormedInput) else x
        weights = ops.route(xt, self.w_router, None, self.experts, self.top, 1.0, True, False, bias=self.b_router, shared_one=self.shared_size > 0)
        act = ops.expert_gated_act(ops.linear(xt, self.w_up), self.experts, self.expert_size, self.shared_size, float("inf"), float("inf"), 1.0,
                                   weights=weights, up_shift=0.0)
        if sink is not None:
            handed_on = sink.linear(act, self.w_down)
            if handed_on is not None:
                return handed_on
        return ops.linear(act, self.w_down, out_dtype=torch.float32)


register_part("feed_forward", "routed_gated_mlp", RoutedGatedMLP)
