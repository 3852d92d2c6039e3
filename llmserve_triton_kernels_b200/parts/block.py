"""The arrangement of a layer's parts around the residual stream.

Parity: src/llmserve/model/llama.py:131-135 — ``x += mixer(norm(x)); x += ff(norm(x))``.
The residual stream is a 32-bit tensor that the norms update in place: each part returns its
contribution, and the next norm adds it before normalising (one pass over the row instead of
three).  In bfloat16 the last product of a part adds into the stream itself (see ``ops.ResidualSink``): a
small step's product also hands the stream on already normalised for the next norm, so a decode step has
no norm launches of its own; a large step's product leaves a norm kernel that only reads the stream.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Block, FeedForward, Mixer, Norm, register_part


def _takes_factored(part) -> bool:
    """Whether a part reads its input in factored form (``ops.NormedInput``): by default every part that takes a sink for its
    last product does; one whose first kernel wants the normed rows themselves says ``takes_factored = False`` and gets them
    from the norm's own kernel."""
    return bool(getattr(part, "takes_factored", getattr(part, "accepts_sink", False)))


class PreNormBlock(Block):
    roles = {"mixer_norm": "norm", "mixer": "mixer", "ff_norm": "norm", "feed_forward": "feed_forward"}

    def __init__(self, mixer_norm: Norm, mixer: Mixer, ff_norm: Norm, feed_forward: FeedForward, residual_scale: float = 1.0):
        self.mixer_norm = mixer_norm
        self.mixer = mixer
        self.ff_norm = ff_norm
        self.feed_forward = feed_forward
        self.residual_scale = float(residual_scale)  # x += residual_scale * part(norm(x))
        # whether the part behind each norm takes the stream in factored form (ops.NormedInput); where it does not, the
        # product in front of the norm is not asked for that form (it would only be multiplied out again)
        mixer_norm.feeds_factored = _takes_factored(mixer)
        ff_norm.feeds_factored = _takes_factored(feed_forward)

    @property
    def graph_safe(self) -> bool:
        return all(p.graph_safe for p in (self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward))

    def forward(self, resid, pending, ctx, cache, next_norm=None):
        x = self._normed(self.mixer_norm, resid, pending, self.mixer)
        sink = self._sink(self.mixer, self.ff_norm, resid, ctx)
        pending = self.mixer.forward(x, ctx, cache, sink=sink) if sink else self.mixer.forward(x, ctx, cache)
        x = self._normed(self.ff_norm, resid, self._scaled(pending), self.feed_forward)
        sink = self._sink(self.feed_forward, next_norm, resid, ctx)
        return self._scaled(self.feed_forward.forward(x, ctx, sink=sink) if sink else self.feed_forward.forward(x, ctx))

    def _scaled(self, pending):
        """A part's contribution as the stream is to take it: times this block's ``residual_scale``."""
        if self.residual_scale != 1.0 and isinstance(pending, torch.Tensor):
            return ops.Scaled(pending, self.residual_scale)
        return pending

    @staticmethod
    def _normed(norm, resid, pending, consumer):
        """``pending`` is a contribution still to be added (a tensor, or one with its factor), or the stream already
        summed and normalised for ``norm`` by the part before (a fused decode kernel did both).  A consumer
        that does not say it takes the factored form gets a plain tensor."""
        if isinstance(pending, ops.NormedInput):
            if pending.norm is not norm:
                raise RuntimeError("a part handed the residual stream on normalised for another norm")
            return pending if _takes_factored(consumer) else pending.materialize()
        if isinstance(pending, ops.BranchSum) and hasattr(norm, "add_branches"):
            x = norm.add_branches(resid, pending)  # the branches' meeting, the sum into the stream and the norm as one kernel
            if x is not None:
                return x
        delta, alpha = ops.split_pending(pending)
        if alpha != 1.0:
            return norm.add_forward(resid, delta, alpha=alpha)
        return norm.add_forward(resid, delta)

    def _sink(self, part, norm, resid, ctx):
        """A sink for the part's last product, if the part takes one and another norm follows (the last part of the
        last layer keeps its contribution: only the rows whose logits are wanted are summed).  Where that norm is an
        RMS norm its weight goes along, so that a small step's product can hand the stream on normalised."""
        if norm is None or not getattr(part, "accepts_sink", False):
            return None
        if not ops.ResidualSink.usable(ctx.num_tokens, getattr(norm, "out_dtype", None)):
            return None
        fused = getattr(norm, "fused_params", None)
        weight, eps = fused() if fused is not None else (None, 0.0)
        if self.residual_scale != 1.0:
            weight = None  # the product that also normalises adds its result unscaled
        if not getattr(norm, "feeds_factored", True):
            weight = None  # whoever reads that norm wants a plain tensor: the product only adds, the norm runs as a kernel
        return ops.ResidualSink(resid, weight, eps, norm, alpha=self.residual_scale)


class MixerOnlyBlock(PreNormBlock):
    """A layer without a feed-forward: ``x += residual_scale * mixer(norm(x))``."""

    roles = {"mixer_norm": "norm", "mixer": "mixer"}

    def __init__(self, mixer_norm: Norm, mixer: Mixer, residual_scale: float = 1.0):
        self.mixer_norm = mixer_norm
        self.mixer = mixer
        self.residual_scale = float(residual_scale)
        mixer_norm.feeds_factored = _takes_factored(mixer)

    @property
    def graph_safe(self) -> bool:
        return all(p.graph_safe for p in (self.mixer_norm, self.mixer))

    def forward(self, resid, pending, ctx, cache, next_norm=None):
        x = self._normed(self.mixer_norm, resid, pending, self.mixer)
        sink = self._sink(self.mixer, next_norm, resid, ctx)
        return self._scaled(self.mixer.forward(x, ctx, cache, sink=sink) if sink else self.mixer.forward(x, ctx, cache))


class HyperConnectionBlock(Block):
    """A pre-norm layer over a residual stream kept in S copies ``x_1 .. x_S`` (hyper-connections).  For each of its parts
    q (1: the mixer, 2: the feed-forward) it owns ``hc<q>.in [S]``, ``hc<q>.out [S]`` and ``hc<q>.mix [S, S]``:

        u = sum_s in[s] x_s        y = part(norm(u))        x_t <- sum_s mix[s, t] x_s + out[t] * y     (all t at once)

    ``resid`` is ``[S, N, hidden]`` (``ModelPlan.streams``).  What a part returns travels as an ``ops.StreamUpdate``; the
    copies take it up in the same kernel that reads them in and norms for the next part (``Norm.add_streams``), so a
    part costs one pass over the copies.  ``feed_forward`` may be absent (None): the layer then has no second part."""

    roles = {"mixer_norm": "norm", "mixer": "mixer", "ff_norm": "norm", "feed_forward": "feed_forward"}

    def __init__(self, mixer_norm: Norm, mixer: Mixer, ff_norm: Norm | None = None, feed_forward: FeedForward | None = None,
                 streams: int = 1, names: tuple[str, str] = ("hc1", "hc2")):
        if not 1 <= int(streams) <= 8:
            raise ValueError(f"a residual stream is kept in one to eight copies, got {streams}")
        self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward = mixer_norm, mixer, ff_norm, feed_forward
        self.streams, self.names = int(streams), tuple(names)
        self.hc: list[tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = []  # per part: (in, mix, out), 32-bit

    def owned_parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward) if p is not None]

    @property
    def graph_safe(self) -> bool:
        return all(p.graph_safe for p in self.owned_parts())

    def _parts(self) -> int:
        return 1 if self.feed_forward is None else 2

    def tensors(self):
        from .base import TensorSpec

        S, specs = self.streams, {}
        for name in self.names[: self._parts()]:
            specs[f"{name}.in"] = TensorSpec((S,), init="ones_plus_normal")
            specs[f"{name}.out"] = TensorSpec((S,), init="ones_plus_normal")
            specs[f"{name}.mix"] = TensorSpec((S, S), init="eye_plus_normal")
        return specs

    def bind(self, tensors, dtype, device) -> None:
        f32 = lambda t: t.to(device=device, dtype=torch.float32).contiguous()  # noqa: E731
        self.hc = [(f32(tensors[f"{n}.in"]), f32(tensors[f"{n}.mix"]), f32(tensors[f"{n}.out"])) for n in self.names[: self._parts()]]

    def forward(self, resid, pending, ctx, cache, next_norm=None):
        if resid.dim() != 3 or resid.shape[0] != self.streams:
            raise RuntimeError(f"this block reads a residual stream in {self.streams} copies, got a tensor of shape {tuple(resid.shape)}")
        if pending is not None and not isinstance(pending, ops.StreamUpdate):
            raise RuntimeError("a stream kept in copies takes up what a part returned together with that part's mixing weights")
        read_in, mix, take = self.hc[0]
        x = self.mixer_norm.add_streams(resid, pending, read_in)
        pending = ops.StreamUpdate(self.mixer.forward(x, ctx, cache), mix, take)
        if self.feed_forward is None:
            return pending
        read_in, mix, take = self.hc[1]
        x = self.ff_norm.add_streams(resid, pending, read_in)
        return ops.StreamUpdate(self.feed_forward.forward(x, ctx), mix, take)


class HyperConnectionMixerOnlyBlock(HyperConnectionBlock):
    """The same without a feed-forward: one part a layer."""

    roles = {"mixer_norm": "norm", "mixer": "mixer"}

    def __init__(self, mixer_norm: Norm, mixer: Mixer, streams: int = 1, names: tuple[str, str] = ("hc1", "hc2")):
        super().__init__(mixer_norm, mixer, None, None, streams=streams, names=names)


register_part("block", "hyper_connection", HyperConnectionBlock)
register_part("block", "hyper_connection_mixer_only", HyperConnectionMixerOnlyBlock)
register_part("block", "pre_norm", PreNormBlock)
register_part("block", "pre_norm_mixer_only", MixerOnlyBlock)
