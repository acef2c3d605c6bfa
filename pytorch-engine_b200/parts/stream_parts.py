"""Parts that an arrangement applies to the stream itself or to what a sublayer reads (role "stream"; the kernels:
csrc/stream_parts.cu).

``token_shift``: what a mixer reads moves towards what the previous token's mixer would have read,

    h[t] <- h[t] + (h[t-1] - h[t]) * mix          (h[t-1]: the unmoved row; zeros before a sequence's first token)

and the sequence keeps its last unmoved row for the next step: a fixed-size state entry of the cache, float32, zero when a
slot is taken.  It runs fused with the norm that produces ``h``, in float32, and writes the run dtype.

``depth_average``: what a block hands on is a weighted sum of the embedding's output and of every block's result so far,

    x <- sum_{j = 0 .. i + 1} coeff[j] * X_j      (X_0: the embedding's output, X_(j+1): block j's result)

with the results kept for the length of a step in one float32 buffer.

``input_mix``: the stream is replaced by a learned mix of itself and the embedding's output, ``x <- W [x ; x0]`` (a block that
runs several times over takes the model's input in again in front of every pass).

``normed_mean``: two sublayer outputs side by side become one, ``(unit(a) * w_a + unit(b) * w_b) / 2``, each divided by its own
root mean square over the row first.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from .registry import register
from .spec import CacheRequest, WeightDecl


@register("stream", "token_shift")
class TokenShift:
    """params: ``dim``.  weights: ``mix [dim]``."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    @classmethod
    def weight_decls(cls, params) -> Dict[str, WeightDecl]:
        return {"mix": WeightDecl((int(params["dim"]),), "unit")}

    @classmethod
    def cache_request(cls, params) -> Optional[CacheRequest]:
        return CacheRequest(kind="state", state_shapes=(("prev", (int(params["dim"]),), "float32"),))

    def __init__(self, params, weights, runtime) -> None:
        self.runtime = runtime
        self.dim = int(params["dim"])
        self.mix = runtime.adopt(weights["mix"], torch.float32)

    def norm_forward(self, stream: torch.Tensor, norm, out: torch.Tensor, ctx, view) -> torch.Tensor:
        """``out`` = the rows of ``norm(stream)`` moved towards their predecessors; ``norm``: an RMS norm part."""
        ops.norm_token_shift(stream, norm.weight, norm.eps, self.mix, view.state("prev"), ctx.token_seq, ctx.seq_slot,
                             ctx.seq_qstart, out, self.runtime.status)
        return out


@register("stream", "depth_average")
class DepthAverage:
    """params: ``terms`` (how many results the sum runs over: the block's number + 2).  weights: ``coeff [terms]``."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    @classmethod
    def weight_decls(cls, params) -> Dict[str, WeightDecl]:
        return {"coeff": WeightDecl((int(params["terms"]),), "unit")}

    def __init__(self, params, weights, runtime) -> None:
        self.runtime = runtime
        self.terms = int(params["terms"])
        self.coeff = runtime.adopt(weights["coeff"], torch.float32)

    def forward(self, results: torch.Tensor, out: torch.Tensor, copy: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``results [>= terms, N, width]`` float32; ``out [N, width]`` gets the sum, and so does ``copy`` if given."""
        ops.depth_average(results, self.coeff, self.terms, out, copy)
        return out


@register("stream", "input_mix")
class InputMix:
    """``x <- W [x ; x0]`` with ``x0`` the embedding's output of this step (``ctx.embedding_output``; the plan sets
    ``keep_embedding_output``).  params: ``dim``.  weights: ``weight [dim, 2 * dim]`` (the stream's half first).  The result is
    the new float32 stream, so its inputs are not cut to the run dtype's 8 bits: in a bfloat16 run ``[x ; x0]`` goes into the
    product as two bfloat16 terms (its rounding, and the rounding of what that left over) stacked as rows of one product, whose
    float32 halves are added."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    @classmethod
    def weight_decls(cls, params) -> Dict[str, WeightDecl]:
        dim = int(params["dim"])
        return {"weight": WeightDecl((dim, 2 * dim))}

    def __init__(self, params, weights, runtime) -> None:
        self.runtime = runtime
        self.dim = int(params["dim"])
        self.weight = runtime.adopt(weights["weight"])

    def forward(self, stream: torch.Tensor, ctx) -> torch.Tensor:
        rt = self.runtime
        x0 = getattr(ctx, "embedding_output", None)
        if x0 is None:
            raise ValueError("input_mix needs the embedding's output of the step (ModelPlan.keep_embedding_output)")
        n, dim = stream.shape
        if rt.dtype == torch.float32:
            both = ctx.buffer("input_mix.both", (n, 2 * dim), rt.dtype)
            ops.concat_split(stream, x0, both, None)
            mixed = ctx.buffer("input_mix.mixed", (n, dim), torch.float32)
            y = rt.linear(both, self.weight, out=mixed)
            stream.copy_(y)
            return stream
        both = ctx.buffer("input_mix.both", (2 * n, 2 * dim), rt.dtype)
        ops.concat_split(stream, x0, both[:n], both[n:])
        mixed = ctx.buffer("input_mix.mixed", (2 * n, dim), torch.float32)
        y = rt.linear(both, self.weight, out=mixed, out_dtype=torch.float32)
        torch.add(y[:n], y[n:], out=stream)
        return stream


@register("stream", "normed_mean")
class NormedMean:
    """``out = scale * (unit(a) * w_a + unit(b) * w_b)`` (csrc/dyt.cu).  params: ``dim``, ``eps``, ``scale`` (default one half).
    weights: ``weight_a [dim]``, ``weight_b [dim]``."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    @classmethod
    def weight_decls(cls, params) -> Dict[str, WeightDecl]:
        dim = int(params["dim"])
        return {"weight_a": WeightDecl((dim,), "norm"), "weight_b": WeightDecl((dim,), "norm")}

    def __init__(self, params, weights, runtime) -> None:
        self.runtime = runtime
        self.eps = float(params["eps"])
        self.scale = float(params.get("scale", 0.5))
        self.weight_a = runtime.adopt(weights["weight_a"], torch.float32)
        self.weight_b = runtime.adopt(weights["weight_b"], torch.float32)

    def forward(self, a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        ops.rmsnorm_pair_mix(a, b, self.weight_a, self.weight_b, self.eps, self.scale, self.scale, out)
        return out

    def add_after_tanh_norm(self, a: torch.Tensor, b: torch.Tensor, stream: torch.Tensor, post, then=None,
                            out: Optional[torch.Tensor] = None) -> None:
        """The mix, the Dynamic Tanh norm ``post`` on it, the add into ``stream`` and (``then`` with ``out``) the norm in front
        of the next sublayer, in one kernel; ``post`` and ``then`` are ``DynamicTanh`` parts."""
        nxt = None if then is None or out is None else (then.weight, then.bias, then.alpha)
        ops.rmsnorm_pair_mix_dyt_add(a, b, self.weight_a, self.weight_b, self.eps, self.scale, self.scale, stream,
                                     (post.weight, post.bias, post.alpha), nxt, out if nxt else None)
