"""Block arrangements: how two norms, a mixer and a feed-forward are wired around the residual
stream.  The stream is float32; a part's output ("delta") is added to it inside the next norm's
kernel, so a block hands its last delta on instead of adding it itself."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .registry import register


class DeltaSum:
    """Several sublayer outputs that are still to be added to the stream, each with a factor: what a block whose
    sublayers run side by side hands on.  A norm adds them inside its own kernel (``RMSNorm.add_forward``)."""

    def __init__(self, deltas, scales) -> None:
        self.deltas = list(deltas)
        self.scales = [float(s) for s in scales]

    def add_into(self, stream: torch.Tensor, weight_like: torch.Tensor) -> None:
        """``stream += sum_i scale_i * delta_i`` with no norm behind it (``weight_like``: any float32 tensor)."""
        ops.rmsnorm_residual_sum(stream, self.deltas, self.scales, weight_like, None, 0.0)


class NormedDelta:
    """A sublayer output that is still to go through a norm of its own and be added to the stream: what a block with a norm
    behind each sublayer hands on, so that the next block's first norm can do all of it in one kernel.  Whoever gets one and
    cannot fuse it calls ``settle(stream)``."""

    def __init__(self, delta: torch.Tensor, norm) -> None:
        self.delta = delta
        self.norm = norm

    def settle(self, stream: torch.Tensor) -> None:
        self.norm.add_after(stream, self.delta, None)


def settle_pending(stream: torch.Tensor, pending) -> None:
    """Add what the block before left to be added (nothing, one delta, several scaled ones, one behind a norm)."""
    if pending is None:
        return
    if isinstance(pending, NormedDelta):
        pending.settle(stream)
    elif isinstance(pending, DeltaSum):
        pending.add_into(stream, stream)
    else:
        stream.add_(pending)


@register("arrangement", "pre_norm")
class PreNormBlock:
    """``h = x + mixer(norm1(x))``; ``out = h + ffn(norm2(h))`` (pygguf_engine/model.py:1025-1042)."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    def __init__(self, spec, parts, runtime) -> None:
        self.runtime = runtime
        self.mixer_norm = parts["mixer_norm"]
        self.mixer = parts["mixer"]
        self.ffn_norm = parts["ffn_norm"]
        self.ffn = parts["ffn"]
        self.name = spec.name

    def forward(self, stream: torch.Tensor, pending: Optional[torch.Tensor], ctx, view, writes_cache: bool = True):
        """``stream``: float32 residual ``[N, hidden]``, updated in place; ``pending``: the previous
        block's delta that is not added yet (or None).  Returns this block's own pending delta."""
        rt = self.runtime
        if isinstance(pending, NormedDelta):
            pending.settle(stream)
            pending = None
        normed = ctx.buffer("block.normed", tuple(stream.shape), rt.dtype)
        self.mixer_norm.add_forward(stream, pending, normed)
        if writes_cache:
            mixed = self.mixer.forward(normed, ctx, view)
        else:
            mixed = self.mixer.forward(normed, ctx, view, writes_cache=False)
        self.ffn_norm.add_forward(stream, mixed, normed)
        return self.ffn.forward(normed, ctx)


@register("arrangement", "post_norm")
class PostNormBlock:
    """Norm on what a sublayer returns, not on what it reads: ``x += norm1(mixer(x))``; ``x += norm2(ffn(x))`` if the
    block has a feed-forward; ``x += side_norm(side(x))`` if it has a token side input.  Parts by name:
    ``mixer_norm, mixer`` and optionally ``ffn_norm, ffn`` and ``side_norm, side``.  The sublayers read the stream
    itself: in a float32 run directly, otherwise through a copy in the run dtype that every add leaves behind."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    def __init__(self, spec, parts, runtime) -> None:
        self.runtime = runtime
        self.name = spec.name
        self.steps = [(parts["mixer"], parts["mixer_norm"], True)]
        if "ffn" in parts:
            self.steps.append((parts["ffn"], parts["ffn_norm"], False))
        if "side" in parts:
            self.steps.append((parts["side"], parts["side_norm"], False))

    def forward(self, stream: torch.Tensor, pending: Optional[torch.Tensor], ctx, view, writes_cache: bool = True):
        rt = self.runtime
        if pending is not None:       # a block before this one left its last delta to be added
            settle_pending(stream, pending)
            ctx.stream_copy = None
        same = rt.dtype == torch.float32
        x = stream
        if not same:
            x = getattr(ctx, "stream_copy", None)
            if x is None:
                x = ctx.buffer("block.x", tuple(stream.shape), rt.dtype)
                x.copy_(stream)
        cast = None if same else ctx.buffer("block.x", tuple(stream.shape), rt.dtype)
        for part, norm, is_mixer in self.steps:
            if is_mixer:
                delta = part.forward(x, ctx, view) if writes_cache else part.forward(x, ctx, view, writes_cache=False)
            else:
                delta = part.forward(x, ctx)
            norm.add_after(stream, delta, cast)
            x = stream if same else cast
        ctx.stream_copy = None if same else cast
        return None


@register("arrangement", "parallel")
class ParallelBlock:
    """One norm feeds every sublayer, and their outputs are added together: ``h = norm(x)``;
    ``x += mult * (sum_i weight_i * mixer_i(h) + ffn(h))``.  Parts by name: ``norm``, any number of mixers (in the
    order the plan lists them), optionally ``ffn``.  ``BlockSpec.params``: ``mult`` (default 1) and ``mixer_weights``
    (mixer name -> factor, default 1).  The sum is taken in float32 inside the next norm's kernel, so the block hands
    its outputs on as a ``DeltaSum``."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    def __init__(self, spec, parts, runtime) -> None:
        self.runtime = runtime
        self.name = spec.name
        self.norm = parts["norm"]
        self.mixer_names = list(spec.mixer_names())
        self.mixers = [parts[n] for n in self.mixer_names]
        self.ffn = parts.get("ffn")
        mult = float(spec.params.get("mult", 1.0))
        weights = spec.params.get("mixer_weights") or {}
        self.scales = [mult * float(weights.get(n, 1.0)) for n in self.mixer_names]
        self.ffn_scale = mult
        if len(self.mixers) + (1 if self.ffn is not None else 0) > 4:
            raise ValueError("a parallel block adds at most four sublayer outputs")

    def forward(self, stream: torch.Tensor, pending, ctx, view, writes_cache: bool = True):
        rt = self.runtime
        if isinstance(pending, NormedDelta):
            pending.settle(stream)
            pending = None
        normed = ctx.buffer("block.normed", tuple(stream.shape), rt.dtype)
        self.norm.add_forward(stream, pending, normed)
        deltas = []
        for i, (name, mixer) in enumerate(zip(self.mixer_names, self.mixers)):
            v = view[name] if isinstance(view, dict) else view
            delta = mixer.forward(normed, ctx, v) if writes_cache else mixer.forward(normed, ctx, v, writes_cache=False)
            if any(type(m) is type(mixer) for m in self.mixers[i + 1:]):
                # a part's delta lies in a buffer that the next part of its class uses again
                keep = ctx.buffer(f"block.delta{i}", tuple(delta.shape), delta.dtype)
                keep.copy_(delta)
                delta = keep
            deltas.append(delta)
        scales = list(self.scales)
        if self.ffn is not None:
            deltas.append(self.ffn.forward(normed, ctx))
            scales.append(self.ffn_scale)
        return DeltaSum(deltas, scales)


@register("arrangement", "sandwich_depth")
class SandwichDepthBlock:
    """A norm before and after each sublayer, a token shift on what the mixer reads, and an average over depth behind
    the block:

        y = x + post_mixer_norm(mixer(shift(mixer_norm(x))))
        y = y + post_ffn_norm(ffn(ffn_norm(y)))                    (if the block has a feed-forward)
        X_(i+1) = y ;   hand on  sum_{j <= i+1} coeff[j] X_j       (X_0: the embedding's output)

    Parts by name: ``mixer_norm, shift, mixer, post_mixer_norm``, optionally ``ffn_norm, ffn, post_ffn_norm``, and
    ``average``.  ``BlockSpec.params``: ``index`` (the block's number i) and ``depth`` (the number of blocks).  The
    results X_j live in one float32 buffer of the step, ``[depth + 1, N, hidden]``; the block works in place on its own
    row of it, and the averaging kernel writes the sum both to the stream and to the next block's row."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    def __init__(self, spec, parts, runtime) -> None:
        self.runtime = runtime
        self.name = spec.name
        self.index = int(spec.params["index"])
        self.depth = int(spec.params["depth"])
        self.mixer_norm, self.shift, self.mixer = parts["mixer_norm"], parts["shift"], parts["mixer"]
        self.post_mixer_norm = parts["post_mixer_norm"]
        self.ffn = parts.get("ffn")
        self.ffn_norm, self.post_ffn_norm = parts.get("ffn_norm"), parts.get("post_ffn_norm")
        self.average = parts["average"]

    def forward(self, stream: torch.Tensor, pending, ctx, view, writes_cache: bool = True):
        rt = self.runtime
        settle_pending(stream, pending)  # a block of another arrangement before this one left its last delta to be added
        n, hidden = stream.shape
        results = ctx.buffer("depth.results", (self.depth + 1, n, hidden), torch.float32)
        work = results[self.index + 1]
        if self.index == 0 or getattr(ctx, "depth_rows_ready", None) != self.index + 1:
            # the first block of a step (or one that follows a block of another arrangement) starts the rows itself
            if self.index == 0:
                results[0].copy_(stream)
            work.copy_(stream)
        normed = ctx.buffer("block.normed", (n, hidden), rt.dtype)
        self.shift.norm_forward(work, self.mixer_norm, normed, ctx, view["shift"])
        mview = view["mixer"]
        mixed = self.mixer.forward(normed, ctx, mview) if writes_cache else self.mixer.forward(normed, ctx, mview, writes_cache=False)
        self.post_mixer_norm.add_after(work, mixed, None)
        if self.ffn is not None:
            self.ffn_norm.add_forward(work, None, normed)
            self.post_ffn_norm.add_after(work, self.ffn.forward(normed, ctx), None)
        last = self.index + 1 >= self.depth
        self.average.forward(results, stream, None if last else results[self.index + 2])
        ctx.depth_rows_ready = None if last else self.index + 2
        ctx.stream_copy = None
        return None


@register("arrangement", "sandwich")
class SandwichBlock:
    """A norm before and after each sublayer:

        x = x + post_mixer_norm(mixer(mixer_norm(x)))
        x = x + post_ffn_norm(ffn(ffn_norm(x)))                   (if the block has a feed-forward)

    Parts by name: ``mixer_norm, post_mixer_norm``, one mixer (``mixer``) or two that read the same input (any two names of
    role "mixer", with ``combine``, a part that makes one output of the two), optionally ``ffn_norm, ffn, post_ffn_norm``, and
    optionally ``inject``: a part of role "stream" that rewrites the stream in front of the block (``inject.forward(stream,
    ctx)``).  Where the post norm offers it (``add_after(..., then=)``), the add behind a sublayer and the norm in front of
    the next one are one pass; that holds across blocks too: the block hands its last sublayer's output on as a
    ``NormedDelta``, and the next block's first norm (or the model's final norm) takes it from there."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    def __init__(self, spec, parts, runtime) -> None:
        self.runtime = runtime
        self.name = spec.name
        self.mixer_norm, self.post_mixer_norm = parts["mixer_norm"], parts["post_mixer_norm"]
        self.mixer_names = list(spec.mixer_names())
        self.mixers = [parts[n] for n in self.mixer_names]
        if len(self.mixers) not in (1, 2):
            raise ValueError("a sandwich block has one mixer, or two with a 'combine' part")
        self.combine = parts.get("combine")
        if len(self.mixers) == 2 and self.combine is None:
            raise ValueError("a sandwich block with two mixers needs a 'combine' part")
        self.ffn = parts.get("ffn")
        self.ffn_norm, self.post_ffn_norm = parts.get("ffn_norm"), parts.get("post_ffn_norm")
        self.inject = parts.get("inject")

    def forward(self, stream: torch.Tensor, pending, ctx, view, writes_cache: bool = True):
        rt = self.runtime
        normed = ctx.buffer("block.normed", tuple(stream.shape), rt.dtype)
        if isinstance(pending, NormedDelta) and self.inject is None and self.fuses(pending.norm, self.mixer_norm):
            # the last add of the block before and this block's first norm in one pass
            pending.norm.add_after(stream, pending.delta, normed, then=self.mixer_norm)
        else:
            settle_pending(stream, pending)
            if self.inject is not None:
                self.inject.forward(stream, ctx)
            self.mixer_norm.add_forward(stream, None, normed)
        outs = []
        for i, (name, mixer) in enumerate(zip(self.mixer_names, self.mixers)):
            v = view[name] if isinstance(view, dict) else view
            out = mixer.forward(normed, ctx, v) if writes_cache else mixer.forward(normed, ctx, v, writes_cache=False)
            if any(type(m) is type(mixer) for m in self.mixers[i + 1:]):
                # a part's delta lies in a buffer that the next part of its class uses again
                keep = ctx.buffer(f"block.delta{i}", tuple(out.shape), out.dtype)
                keep.copy_(out)
                out = keep
            outs.append(out)
        mixed = outs[0]
        if len(outs) == 2:
            if getattr(self.post_mixer_norm, "tanh_norm", False) and hasattr(self.combine, "add_after_tanh_norm") and (
                    self.ffn is None or getattr(self.ffn_norm, "tanh_norm", False)):
                # the two outputs' mix, the norm on it, the add and the feed-forward's norm in one kernel
                self.combine.add_after_tanh_norm(outs[0], outs[1], stream, self.post_mixer_norm, self.ffn_norm,
                                                 None if self.ffn is None else normed)
                ctx.stream_copy = None
                return None if self.ffn is None else NormedDelta(self.ffn.forward(normed, ctx), self.post_ffn_norm)
            mixed = self.combine.forward(outs[0], outs[1], ctx.buffer("block.mixed", tuple(outs[0].shape), outs[0].dtype))
        ctx.stream_copy = None
        if self.ffn is None:
            if len(outs) == 2:        # (the mix lies in a buffer of this block's: add it here)
                self.post_mixer_norm.add_after(stream, mixed, None)
                return None
            return NormedDelta(mixed, self.post_mixer_norm)
        if self.fuses(self.post_mixer_norm, self.ffn_norm):
            self.post_mixer_norm.add_after(stream, mixed, normed, then=self.ffn_norm)
        else:
            self.post_mixer_norm.add_after(stream, mixed, None)
            self.ffn_norm.add_forward(stream, None, normed)
        return NormedDelta(self.ffn.forward(normed, ctx), self.post_ffn_norm)

    @staticmethod
    def fuses(post_norm, next_norm) -> bool:
        import inspect
        return type(post_norm) is type(next_norm) and "then" in inspect.signature(post_norm.add_after).parameters
