"""Mixers side by side: every branch reads the same input, and their outputs meet as

    factor * sum_b  rmsnorm(branch_b(x)) * w_b            (factor = 1 / branches: the mean)

each output RMS-normed over the model width by itself (``eps`` inside the root) with a weight of its own; or, with
``branch_norm=False``, as the plain weighted sum ``sum_b scales[b] * branch_b(x)`` without norms and weights.  A branch is
any registered mixer; what it keeps per request (pages, a state slot) is its own: the cache manager holds every
branch's as a part of a ``CompositeSpec``.  The branches' products leave their results in 32-bit, the norms and the
sum are 32-bit, and the result is a contribution to the residual stream.

Branches that start with a stacked input product of their own (an attribute ``w_in`` and ``takes_projection = True``)
hand their matrices over: the mixer stacks them once more, runs ONE product for all branches and gives each its
columns of the result (``forward(..., proj=...)``).  The input may arrive in factored normalised form
(``ops.NormedInput``) when every branch starts with a product that takes it.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import CompositeSpec, Mixer, PartSpec, TensorSpec, build_part, register_part


class ParallelMixer(Mixer):
    def __init__(self, hidden_size: int, branches: dict[str, PartSpec], norm_eps: float, factor: float | None = None,
                 weight_name: str = "out", branch_norm: bool = True, scales: list[float] | None = None):
        """``branches``: name -> the mixer's spec; the name, with a dot, is the prefix of the branch's tensors, and
        ``<name>.<weight_name>`` the weight of its output norm.  ``branch_norm=False``: the outputs are not normed and
        have no weights; branch b enters the sum times ``scales[b]`` (default 1)."""
        if not 1 <= len(branches) <= 4:
            raise ValueError(f"one to four branches run side by side, got {len(branches)}")
        self.hidden_size, self.norm_eps, self.weight_name = int(hidden_size), float(norm_eps), weight_name
        self.branch_norm = bool(branch_norm)
        self.scales = [1.0] * len(branches) if scales is None else [float(v) for v in scales]
        if len(self.scales) != len(branches) or (self.branch_norm and scales is not None):
            raise ValueError("scales: one for each branch, for branches that meet as a plain weighted sum")
        self.factor = 1.0 / len(branches) if factor is None else float(factor)
        self.branch_names = tuple(branches)
        for name, spec in branches.items():
            setattr(self, f"branch_{name}", build_part("mixer", spec))
        self.out_weights: list[torch.Tensor] = []
        self.w_in: torch.Tensor | None = None  # the branches' input matrices stacked, where all of them hand theirs over
        self._columns: list[tuple[int, int]] = []
        # the stream in factored form is welcome if every branch's first step is a product that takes it
        self.accepts_sink = all(getattr(b, "accepts_sink", False) for b in self.branches)

    @property
    def branches(self) -> list[Mixer]:
        return [getattr(self, f"branch_{name}") for name in self.branch_names]

    @property
    def graph_safe(self) -> bool:
        return all(b.graph_safe for b in self.branches)

    def tensors(self) -> dict[str, TensorSpec]:
        specs = {}
        for name, branch in zip(self.branch_names, self.branches):
            for local, spec in branch.tensors().items():
                specs[f"{name}.{local}"] = spec
            if self.branch_norm:
                specs[f"{name}.{self.weight_name}"] = TensorSpec((self.hidden_size,), init="ones_plus_normal")
        return specs

    def bind(self, tensors, dtype, device) -> None:
        self.out_weights = []
        for name, branch in zip(self.branch_names, self.branches):
            branch.bind({local: tensors[f"{name}.{local}"] for local in branch.tensors()}, dtype, device)
            if self.branch_norm:
                self.out_weights.append(tensors[f"{name}.{self.weight_name}"].to(device=device, dtype=torch.float32).contiguous())
        if len(self.branches) > 1 and all(getattr(b, "takes_projection", False) and getattr(b, "w_in", None) is not None for b in self.branches):
            self.w_in = torch.cat([b.w_in for b in self.branches], dim=0).contiguous()
            start = 0
            for b in self.branches:
                self._columns.append((start, start + b.w_in.shape[0]))
                start += b.w_in.shape[0]
                b.w_in = None  # held here from now on: the branch is given its columns of the product

    def cache_spec(self) -> CompositeSpec:
        return CompositeSpec(tuple(b.cache_spec() for b in self.branches))

    def forward(self, x, ctx, cache, sink=None):
        """``sink`` is not used: what leaves this mixer is a sum of normed outputs, not a product."""
        outs = []
        proj = ops.linear(x, self.w_in, out_dtype=torch.float32) if self.w_in is not None else None
        for i, (branch, view) in enumerate(zip(self.branches, cache.parts)):
            if proj is not None:
                a, b = self._columns[i]
                out = branch.forward(None, ctx, view, proj=proj[:, a:b])
            else:
                out = branch.forward(x, ctx, view)
            outs.append(out if out.dtype == torch.float32 else out.float())
        if not self.branch_norm:  # still a list: whoever takes the sum up may read the branches in a kernel of its own
            return ops.WeightedSum(outs, self.scales)
        # still a list of branches: the norm behind this mixer may do the meeting, the sum into the stream and itself in one kernel
        return ops.BranchSum(outs, self.out_weights, self.norm_eps, self.factor)


register_part("mixer", "parallel", ParallelMixer)
