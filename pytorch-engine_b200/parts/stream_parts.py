"""Parts that an arrangement applies to the stream itself or to what a sublayer reads (role "stream"; the kernels:
csrc/stream_parts.cu).

``token_shift``: what a mixer reads moves towards what the previous token's mixer would have read,

    h[t] <- h[t] + (h[t-1] - h[t]) * mix          (h[t-1]: the unmoved row; zeros before a sequence's first token)

and the sequence keeps its last unmoved row for the next step: a fixed-size state entry of the cache, float32, zero when a
slot is taken.  It runs fused with the norm that produces ``h``, in float32, and writes the run dtype.

``depth_average``: what a block hands on is a weighted sum of the embedding's output and of every block's result so far,

    x <- sum_{j = 0 .. i + 1} coeff[j] * X_j      (X_0: the embedding's output, X_(j+1): block j's result)

with the results kept for the length of a step in one float32 buffer.
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
