"""Attention through a low-rank latent, over a paged cache of one row per token.

A token's keys and values of all heads are products of one latent vector ``c`` (``rank`` lanes): the key of head h
is ``[W_uk[h] c | k_rot]`` with a rotated part ``k_rot`` (``rot_dim`` lanes) that all heads share, its value is
``W_uv[h] c``.  Only ``[c | k_rot]`` is cached.  The products with ``W_uk`` and ``W_uv`` are moved to the query side:

    score(i, j, h) = (W_uk[h]^T q_plain[i, h]) . c[j] + q_rot[i, h] . k_rot[j]
    out(i, h)      = W_uv[h] (sum_j weight(i, j, h) c[j])

so that attention runs over the cached rows themselves: every head reads the same row as its key (all
``rank + rot_dim`` lanes) and as its value (the first ``rank``).  The latent is RMS-normed (a weight of its own)
before it is cached; rotary positions use the interleaved layout (lanes 2i and 2i+1 form a pair) with angles
computed in 32-bit from the position.  In a bfloat16 step in which a request brings many tokens the softmax is taken in
two parts that a last kernel joins: the rows cached before the step as above, and the step's own tokens with keys and
values per head (``W_uk c``, ``W_uv c``: one product for all new tokens), which takes a third of the arithmetic of
attention over the latents; a step whose requests all start at position 0 (``ctx.fresh_requests``) has no cached rows and
runs the second part alone.  The concatenated heads are multiplied by ``sigmoid(W_g x)`` before the output
projection.  Sizes, the softmax scale, the rotary base and the names of the tensors are parameters.

Options: ``query_rank`` r: the queries come through a latent of their own, ``q = W_uq rmsnorm(W_dq x) * w_dq`` with
``W_dq [r, hidden]``, a norm weight ``[r]`` and ``W_uq [H (dim + rot), r]`` in place of ``W_q``; ``rotary_layout =
"half"``: the rotated lanes pair as ``(i, i + dims/2)`` instead of ``(2i, 2i + 1)``; ``gate_per_head``: the gate is one
number a head and token, ``W_g [H, hidden]``.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Mixer, PagedRowSpec, TensorSpec, register_part

_NAMES = {"q": "q", "down": "dkv", "latent_norm": "dkv.norm", "up_k": "uk", "up_v": "uv", "gate": "g", "out": "o",
          "q_down": "dq", "q_norm": "dq.norm", "q_up": "uq"}


class LatentAttention(Mixer):
    graph_safe = True
    accepts_sink = True

    def __init__(
        self,
        hidden_size: int,
        num_heads: int,
        head_dim: int,
        rot_dim: int,
        value_dim: int,
        rank: int,
        scale: float,
        rotary_base: float,
        rotary_dims: int | None = None,
        norm_eps: float = 1e-6,
        output_gate: bool = True,
        window: int | None = None,
        tensor_names: dict[str, str] | None = None,
        query_rank: int | None = None,
        rotary_layout: str = "interleaved",
        gate_per_head: bool = False,
    ):
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.head_dim, self.rot_dim, self.value_dim, self.rank = int(head_dim), int(rot_dim), int(value_dim), int(rank)
        self.scale, self.rotary_base, self.norm_eps = float(scale), float(rotary_base), float(norm_eps)
        self.rotary_dims = self.rot_dim if rotary_dims is None else int(rotary_dims)
        if self.rotary_dims % 2 or not 0 <= self.rotary_dims <= self.rot_dim:
            raise ValueError(f"{rotary_dims} rotated lanes do not fit a rotated part of {rot_dim}")
        if self.rank + self.rot_dim > 640 or self.rank > 512:
            raise ValueError(f"a cached row of {rank} + {rot_dim} lanes is not supported: the attention kernels take rows up to 640 with a latent up to 512")
        self.output_gate = bool(output_gate)
        self.query_rank = int(query_rank) if query_rank else None
        if rotary_layout not in ("half", "interleaved"):
            raise ValueError(f"rotated lanes pair as 'half' or 'interleaved', not {rotary_layout!r}")
        self.rotary_layout = rotary_layout
        self.gate_per_head = bool(gate_per_head) and self.output_gate
        self.w_uq = self.q_weight = None
        self.window = None if window is None else int(window)
        self.names = {**_NAMES, **(tensor_names or {})}
        self.w_in = self.w_uk_t = self.w_uv = self.w_up = self.w_out = self.latent_weight = self.freq = None

    def tensors(self) -> dict[str, TensorSpec]:
        H, n = self.num_heads, self.names
        if self.query_rank:
            queries = {
                n["q_down"]: TensorSpec((self.query_rank, self.hidden_size)),
                n["q_norm"]: TensorSpec((self.query_rank,), init="ones_plus_normal"),
                n["q_up"]: TensorSpec((H * (self.head_dim + self.rot_dim), self.query_rank)),
            }
        else:
            queries = {n["q"]: TensorSpec((H * (self.head_dim + self.rot_dim), self.hidden_size))}
        specs = {
            **queries,
            n["down"]: TensorSpec((self.rank + self.rot_dim, self.hidden_size)),
            n["latent_norm"]: TensorSpec((self.rank,), init="ones_plus_normal"),
            n["up_k"]: TensorSpec((H * self.head_dim, self.rank)),
            n["up_v"]: TensorSpec((H * self.value_dim, self.rank)),
            n["out"]: TensorSpec((self.hidden_size, H * self.value_dim)),
        }
        if self.output_gate:
            specs[n["gate"]] = TensorSpec((H if self.gate_per_head else H * self.value_dim, self.hidden_size))
        return specs

    def bind(self, tensors, dtype, device) -> None:
        H, n = self.num_heads, self.names
        stacked = [tensors[n["q_down" if self.query_rank else "q"]], tensors[n["down"]]] + ([tensors[n["gate"]]] if self.output_gate else [])
        if self.query_rank:
            self.w_uq = tensors[n["q_up"]].to(device=device, dtype=dtype).contiguous()
            self.q_weight = tensors[n["q_norm"]].to(device=device, dtype=torch.float32).contiguous()
        self.w_in = torch.cat([t.to(dtype) for t in stacked], dim=0).to(device).contiguous()
        # W_uk per head, turned so that it multiplies the query: [H, rank, head_dim]
        self.w_uk_t = tensors[n["up_k"]].to(dtype).view(H, self.head_dim, self.rank).transpose(1, 2).contiguous().to(device)
        self.w_uv = tensors[n["up_v"]].to(dtype).view(H, self.value_dim, self.rank).contiguous().to(device)
        # both up matrices stacked, for the keys and values of a step's own tokens: [H dim | H vdim, rank]
        self.w_up = torch.cat([tensors[n["up_k"]].to(dtype), tensors[n["up_v"]].to(dtype)], dim=0).to(device).contiguous()
        self.w_out = tensors[n["out"]].to(device=device, dtype=dtype).contiguous()
        self.latent_weight = tensors[n["latent_norm"]].to(device=device, dtype=torch.float32).contiguous()
        pairs = torch.arange(self.rotary_dims // 2, dtype=torch.float64)
        self.freq = (self.rotary_base ** (-2.0 * pairs / max(self.rotary_dims, 1))).to(torch.float32).to(device)

    def cache_spec(self) -> PagedRowSpec:
        return PagedRowSpec(self.rank + self.rot_dim, self.window)

    def forward(self, x, ctx, cache, sink=None):
        H, dim, rot, rank = self.num_heads, self.head_dim, self.rot_dim, self.rank
        proj = ops.linear(x, self.w_in)  # [N, H (dim | rot) | rank | rot | gate], or [N, query rank | rank | rot | gate]
        two_parts = ops.latent_two_parts(ctx, proj.dtype, dim, rot, rank, self.value_dim)
        halves = self.rotary_layout == "half"
        if self.query_rank:
            # the queries' latent is normed (32-bit statistics) and expanded: a product of its own behind the stacked one
            q_all = ops.linear(ops.row_rmsnorm(proj[:, : self.query_rank], self.q_weight, self.norm_eps), self.w_uq)
            gate_col = self.query_rank + rank + rot
            prepared = ops.latent_prepare(
                proj, ctx.positions, cache.slot_map, cache.pool, self.latent_weight, self.freq, self.norm_eps, H, dim, rot, rank,
                fresh=two_parts, queries=q_all, kv_col=self.query_rank, halves=halves,
            )
        else:
            q_all, gate_col = proj, H * (dim + rot) + rank + rot
            prepared = ops.latent_prepare(
                proj, ctx.positions, cache.slot_map, cache.pool, self.latent_weight, self.freq, self.norm_eps, H, dim, rot, rank,
                fresh=two_parts, halves=halves,
            )
        q_rot, fresh = prepared if two_parts else (prepared, None)
        q_plain = q_all.as_strided((q_all.shape[0], H, dim), (q_all.stride(0), dim + rot, 1), q_all.storage_offset())
        if two_parts:
            kv = ops.linear(fresh[:, :rank], self.w_up)  # keys and values of the step's own tokens, head by head
            alone = bool(getattr(ctx, "fresh_requests", False))  # every request starts with this step: no cached rows
            own = ops.fresh_latent_attention(
                q_plain, q_rot, kv, fresh, cache.page_table, ctx, dim=dim, value_dim=self.value_dim, rank=rank, scale=self.scale,
                window=self.window, want_stats=not alone,
            )
            if alone:
                heads = own
            else:
                own, own_stats = own
                q_lat = ops.head_linear(q_plain, self.w_uk_t)  # [N, H, rank]
                cached, cached_stats = ops.latent_paged_attention(
                    q_lat, q_rot, cache.pool, cache.page_table, ctx, rank=rank, scale=self.scale, window=self.window, cached_only=True
                )
                heads = ops.merge_two_parts(own, own_stats, ops.head_linear(cached, self.w_uv), cached_stats)
        else:
            q_lat = ops.head_linear(q_plain, self.w_uk_t)  # [N, H, rank]
            mixed = ops.latent_paged_attention(
                q_lat, q_rot, cache.pool, cache.page_table, ctx, rank=rank, scale=self.scale, window=self.window,
                leave_parts=ctx.num_tokens <= 16,
            )
            if isinstance(mixed, ops.AttentionParts):
                # few rows, keys cut over several CTAs: their merge, W_uv and the gate are one kernel
                if self.gate_per_head:
                    out = ops.merge_project_gate(mixed, self.w_uv, proj[:, gate_col : gate_col + H], per_head=True)
                else:
                    out = ops.merge_project_gate(mixed, self.w_uv, proj[:, gate_col:] if self.output_gate else None)
                return self._project_out(out, sink)
            heads = ops.head_linear(mixed, self.w_uv)  # [N, H, vdim]
        if self.gate_per_head:
            out = ops.gate_mul(heads, proj[:, gate_col : gate_col + H], "sigmoid", per_head=True)
        elif self.output_gate:
            out = ops.gate_mul(heads, proj[:, gate_col:], "sigmoid")
        else:
            out = heads.reshape(proj.shape[0], H * self.value_dim)
        return self._project_out(out, sink)

    def _project_out(self, out, sink):
        if sink is not None:
            handed_on = sink.linear(out, self.w_out)
            if handed_on is not None:
                return handed_on
        return ops.linear(out, self.w_out, out_dtype=torch.float32)


register_part("mixer", "latent_attention", LatentAttention)
