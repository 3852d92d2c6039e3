"""RMS normalisation with the residual sum fused in.

Parity: src/llmserve/model/llama.py:18-28 — mean of squares, ``+ eps`` and rsqrt in 32-bit,
then the weight multiply.  Here the residual stream itself is 32-bit and the result is rounded
once, after the weight multiply.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Norm, TensorSpec, register_part


class RMSNorm(Norm):
    """``groups`` > 1: the row is split into that many equal consecutive parts and each is divided by its own root
    mean square (eps inside the root); the weight spans the whole row.  ``weight_name``: the local name of the
    weight tensor (checkpoints that call a norm's weight by the norm's own name pass that name with an empty prefix
    in front)."""

    graph_safe = True

    def __init__(self, size: int, eps: float, groups: int = 1, weight_name: str = "weight"):
        self.size = int(size)
        self.eps = float(eps)
        self.groups = int(groups)
        if self.groups < 1 or self.size % self.groups:
            raise ValueError(f"a row of {self.size} does not split into {groups} equal parts")
        self.weight_name = weight_name
        self.weight: torch.Tensor | None = None
        self.out_dtype: torch.dtype | None = None

    def tensors(self) -> dict[str, TensorSpec]:
        return {self.weight_name: TensorSpec((self.size,), init="ones_plus_normal")}

    def bind(self, tensors, dtype, device) -> None:
        self.weight = tensors[self.weight_name].to(device=device, dtype=torch.float32).contiguous()
        self.out_dtype = dtype

    def fused_params(self):
        """``(weight, eps)``: what a product needs to fold this norm into its ends; a norm in groups cannot be
        folded (its scale is not one number per row) and says ``(None, eps)``."""
        return (self.weight if self.groups == 1 else None), self.eps

    def forward(self, x, rows=None):
        return self.add_forward(x, None, rows)

    def add_branches(self, resid, pending):
        """``resid += pending`` for a contribution that is still a list of branch outputs (``ops.BranchSum``), then the
        norm, in one kernel where the norm is a plain RMS norm; None: the caller adds the contribution as a tensor."""
        if self.groups != 1:
            return None
        return ops.branch_sum_rmsnorm(pending, resid, self.weight, self.eps, self.out_dtype)

    def add_streams(self, streams, update, read_in, rows=None):
        """For a residual stream kept in several copies (``streams [S, N, size]``): the copies take up ``update`` (an
        ``ops.StreamUpdate`` or None) in place, are read in with the weights ``read_in [S]`` (None: summed) and the result
        is normed, all in one kernel.  With ``rows`` only those rows are produced and the copies stay as they were."""
        if self.groups != 1:
            raise NotImplementedError("a norm in groups behind a stream kept in copies is not built")
        return ops.hyper_mix_norm(streams, update, read_in, self.weight, self.eps, rows=rows, out_dtype=self.out_dtype)

    def add_forward(self, resid, delta, rows=None, alpha: float = 1.0):
        if self.groups == 1 and alpha == 1.0:
            return ops.rmsnorm(resid, self.weight, self.eps, delta=delta, rows=rows, out_dtype=self.out_dtype)
        return ops.group_rmsnorm(resid, self.weight, self.eps, self.groups, delta=delta, alpha=alpha, rows=rows, out_dtype=self.out_dtype)


register_part("norm", "rms_norm", RMSNorm)
