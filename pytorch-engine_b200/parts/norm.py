"""RMSNorm and Dynamic Tanh.  RMSNorm's formula: ``x * rsqrt(mean(x^2) + eps) * w`` in float32
(pygguf_engine/quant_kernels.py:831-833, 1548; fused with the residual add 1595-1596)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from .registry import register
from .spec import WeightDecl


@register("norm", "rmsnorm")
class RMSNorm:
    """params: ``dim``, ``eps``, optionally ``offset`` (the stored weight is the distance from it: the norm multiplies by
    ``offset + weight``; random weights then lie around zero).  weights: ``weight [dim]`` (kept in float32)."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    @classmethod
    def weight_decls(cls, params) -> Dict[str, WeightDecl]:
        return {"weight": WeightDecl((int(params["dim"]),), "matrix" if params.get("offset") else "norm")}

    def __init__(self, params, weights, runtime) -> None:
        self.dim = int(params["dim"])
        self.eps = float(params["eps"])
        self.runtime = runtime
        self.weight = runtime.adopt(weights["weight"], torch.float32)
        if params.get("offset"):
            self.weight = (self.weight + float(params["offset"])).contiguous()

    def add_forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], out: torch.Tensor,
                    rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        if hasattr(delta, "settle"):      # an output that goes through a norm of its own before it is added
            delta.settle(residual)
            delta = None
        if hasattr(delta, "deltas"):      # several scaled outputs of a block whose sublayers run side by side
            ops.rmsnorm_residual_sum(residual, delta.deltas, delta.scales, self.weight, out, self.eps, rows)
            return out
        ops.rmsnorm_residual(residual, delta, self.weight, out, self.eps, rows)
        return out

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        out = torch.empty_like(x) if out is None else out
        ops.rmsnorm(x, self.weight, out, self.eps)
        return out

    def add_after(self, stream: torch.Tensor, delta: torch.Tensor, cast: Optional[torch.Tensor] = None) -> None:
        """The norm on what is added: ``stream += rmsnorm(delta) * w``; ``cast`` gets the new rows in the run dtype."""
        ops.rmsnorm_add(stream, delta, self.weight, self.eps, cast)


@register("norm", "dynamic_tanh")
class DynamicTanh:
    """A norm that computes no statistics: ``y = tanh(alpha * x) * weight + bias`` with one number ``alpha``, in float32
    (csrc/dyt.cu).  params: ``dim``.  weights: ``weight [dim]``, ``bias [dim]``, ``alpha []``."""

    graph_safe = True  # launches only; nothing in forward() waits for the device
    tanh_norm = True   # other parts may take (weight, bias, alpha) into a kernel of their own

    @classmethod
    def weight_decls(cls, params) -> Dict[str, WeightDecl]:
        dim = int(params["dim"])
        return {"weight": WeightDecl((dim,), "norm"), "bias": WeightDecl((dim,)), "alpha": WeightDecl((), "unit")}

    def __init__(self, params, weights, runtime) -> None:
        self.dim = int(params["dim"])
        self.runtime = runtime
        self.weight = runtime.adopt(weights["weight"], torch.float32)
        self.bias = runtime.adopt(weights["bias"], torch.float32)
        self.alpha = float(weights["alpha"].to(torch.float32).reshape(-1)[0].item())   # read once, when the model is built

    def add_forward(self, residual: torch.Tensor, delta, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        if delta is not None:
            if hasattr(delta, "settle"):
                if rows is None and type(delta.norm) is type(self):
                    delta.norm.add_after(residual, delta.delta, out, then=self)     # its norm, the add and this norm in one pass
                    return out
                delta.settle(residual)
            elif hasattr(delta, "deltas"):
                delta.add_into(residual, self.weight)
            else:
                residual.add_(delta)
        ops.dyt(residual, self.weight, self.bias, self.alpha, out, rows)
        return out

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        out = torch.empty_like(x) if out is None else out
        ops.dyt(x, self.weight, self.bias, self.alpha, out)
        return out

    def add_after(self, stream: torch.Tensor, delta: torch.Tensor, cast: Optional[torch.Tensor] = None, then=None) -> None:
        """The norm on what is added: ``stream += dyt(delta)``.  ``then`` (another norm of this kind) with ``cast``: ``cast``
        gets ``then``'s norm of the new rows, in the same pass over them."""
        if then is not None and cast is not None:
            ops.dyt_add(stream, delta, self.weight, self.bias, self.alpha, (then.weight, then.bias, then.alpha), cast)
            return
        ops.dyt_add(stream, delta, self.weight, self.bias, self.alpha)
        if cast is not None:
            cast.copy_(stream)
