"""A feed-forward of two products with an activation between them, ``down(act(up(x)))``.

Activations: ``polynorm`` (a N(z) + b N(z^2) + c N(z^3) + e over a token's row of ``intermediate`` values, powers taken
element by element, N the division by the row's root mean square with ``eps`` inside the root; the four numbers are a
weight), in float32 arithmetic on what the up product wrote.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops
from .registry import register
from .spec import WeightDecl


@register("feed_forward", "dense_act")
class DenseActFf:
    """params: ``hidden``, ``intermediate``, ``activation`` ("polynorm"), ``eps``.  weights: ``up_proj [I, H]``,
    ``down_proj [H, I]``, ``act [4]``."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    @classmethod
    def weight_decls(cls, params) -> Dict[str, WeightDecl]:
        h, i = int(params["hidden"]), int(params["intermediate"])
        return {"up_proj": WeightDecl((i, h)), "down_proj": WeightDecl((h, i)), "act": WeightDecl((4,), "unit")}

    def __init__(self, params, weights, runtime) -> None:
        self.runtime = runtime
        self.hidden = int(params["hidden"])
        self.intermediate = int(params["intermediate"])
        self.activation = str(params.get("activation") or "polynorm")
        if self.activation != "polynorm":
            raise ValueError(f"activation {self.activation!r} is not built ('polynorm' is)")
        self.eps = float(params["eps"])
        self.up = runtime.adopt(weights["up_proj"])
        self.down = runtime.adopt(weights["down_proj"])
        self.coeff = runtime.adopt(weights["act"], torch.float32)

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        rt = self.runtime
        n = x.shape[0]
        z = ctx.buffer("dense_ff.up", (n, self.intermediate), rt.dtype)
        rt.linear(x, self.up, out=z)
        act = ctx.buffer("dense_ff.act", (n, self.intermediate), rt.dtype)
        ops.polynorm(z, self.coeff, self.eps, act)
        delta = ctx.buffer("dense_ff.delta", (n, self.hidden), rt.dtype)
        rt.linear(act, self.down, out=delta)
        return delta
