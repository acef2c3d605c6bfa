"""Routed experts: a router picks a few small gated feed-forwards per token, optionally among them "identity experts"
that return their input, optionally with a shared expert that every token passes (the kernels: csrc/moe.cu).

    z = R h (float32) ;  s = softmax(z) over all router outputs
    chosen = the ``top`` largest of s + correction ;  their weights are s itself, not renormalised
    y = sum_chosen s_e * expert_e(h)  (+ shared(h)) ;  expert_e(h) = h for e >= n_experts (identity experts)
    expert(h) = D act(G h, U h)  with the activations of ``parts/swiglu.py``

With ``choice = "top_logits"`` the router instead takes the ``top`` largest of ``z + bias`` and weights them by a softmax
over the chosen ones alone (no correction).  With ``choice = "sigmoid_groups"`` the scores are ``s = sigmoid(z)``; the
experts form ``groups`` equal groups of neighbours, a group scores the sum of its two largest ``s``, and only experts of the
``keep_groups`` best groups can be chosen: the ``top`` largest ``s`` among them, weighted with ``s`` itself (no weights beside
the router's matrix).

The (token, choice) pairs are grouped by expert on the device and every expert's rows go through its matrices in one
launch per product, so nothing is read back to the host and a decode step stays recordable.  A handful of pairs (a
decode step) and every float32 run use the package's own kernel, which streams an expert's weights once per eight
rows; many bfloat16 rows go through the library's product over row groups (``torch._grouped_mm`` with the groups' ends
on the device), as the other many-row products of this package that no kernel of its own takes go to the library.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops
from .registry import register
from .spec import WeightDecl
from .swiglu import SwiGLU


# (token, choice) pairs up to which the package's own row-group kernel runs (it streams an expert's weights once per
# eight rows); beyond it, in bfloat16, the library's product over row groups
LIBRARY_ROWS = 64


@register("feed_forward", "routed_experts")
class RoutedExperts:
    """params: ``hidden``, ``n_experts``, ``n_identity`` (router outputs beyond the real experts), ``top``, ``intermediate``,
    ``activation`` / ``limit`` / ``alpha`` (of every expert), ``shared`` (None, or the params of a ``swiglu`` part).
    ``choice`` ("softmax_all", the default: softmax over every output, the choice moved by ``correction``, weights not
    renormalised; "top_logits": the largest of ``z + router_bias``, softmax over the chosen).
    weights: ``router [n_experts + n_identity, hidden]``, ``correction [n_experts + n_identity]`` (softmax_all) or
    ``router_bias [n_experts + n_identity]`` (top_logits), ``e<i>.gate, e<i>.up
    [I, H]``, ``e<i>.down [H, I]``, and ``shared.gate, shared.up, shared.down`` with a shared expert."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    @classmethod
    def weight_decls(cls, params) -> Dict[str, WeightDecl]:
        h, n, extra, inter = (int(params[k]) for k in ("hidden", "n_experts", "n_identity", "intermediate"))
        decls = {"router": WeightDecl((n + extra, h))}
        if params.get("choice") != "sigmoid_groups":
            decls["router_bias" if params.get("choice") == "top_logits" else "correction"] = WeightDecl((n + extra,))
        for e in range(n):
            decls[f"e{e}.gate"] = WeightDecl((inter, h))
            decls[f"e{e}.up"] = WeightDecl((inter, h))
            decls[f"e{e}.down"] = WeightDecl((h, inter))
        if params.get("shared"):
            si = int(params["shared"]["intermediate"])
            decls.update({"shared.gate": WeightDecl((si, h)), "shared.up": WeightDecl((si, h)), "shared.down": WeightDecl((h, si))})
        return decls

    def __init__(self, params, weights, runtime) -> None:
        self.runtime = runtime
        self.hidden = int(params["hidden"])
        self.n_experts = int(params["n_experts"])
        self.n_identity = int(params["n_identity"])
        self.top = int(params["top"])
        self.intermediate = int(params["intermediate"])
        if not 1 <= self.top <= self.n_experts + self.n_identity:
            raise ValueError(f"top = {self.top} experts of {self.n_experts + self.n_identity}")
        self.activation = str(params.get("activation") or "silu")
        self.glu = ops.GLU_KINDS[self.activation]
        self.limit = float(params.get("limit") or 0.0)
        self.alpha = float(params.get("alpha") or 1.0)
        dev, dt = runtime.device, runtime.dtype
        self.router = runtime.adopt(weights["router"])
        self.choice = str(params.get("choice") or "softmax_all")
        if self.choice not in ("softmax_all", "top_logits", "sigmoid_groups"):
            raise ValueError(f"router choice {self.choice!r} is not built ('softmax_all', 'top_logits' and 'sigmoid_groups' are)")
        self.correction = self.router_bias = None
        self.groups = int(params.get("groups") or 1)
        self.keep_groups = int(params.get("keep_groups") or self.groups)
        if self.choice == "sigmoid_groups":
            n_all = self.n_experts + self.n_identity
            if n_all % self.groups or not 1 <= self.keep_groups <= self.groups or self.top > self.keep_groups * (n_all // self.groups):
                raise ValueError(f"{n_all} experts in {self.groups} groups of which {self.keep_groups} are kept cannot give {self.top} choices")
        elif self.choice == "top_logits":
            self.router_bias = runtime.adopt(weights["router_bias"], torch.float32)
        else:
            self.correction = runtime.adopt(weights["correction"], torch.float32)
        if self.n_experts:
            self.gate_up = torch.stack([torch.cat([weights[f"e{e}.gate"], weights[f"e{e}.up"]]).to(device=dev, dtype=dt)
                                        for e in range(self.n_experts)]).contiguous()
            self.down = torch.stack([weights[f"e{e}.down"].to(device=dev, dtype=dt) for e in range(self.n_experts)]).contiguous()
        # the library's product over row groups takes bfloat16 rows that start on 16-byte boundaries
        self.library_product = (runtime.dtype == torch.bfloat16 and hasattr(torch, "_grouped_mm") and self.hidden % 8 == 0
                                and self.intermediate % 8 == 0)
        self.shared = None
        if params.get("shared"):
            sp = dict(params["shared"])
            sp["hidden"] = self.hidden
            self.shared = SwiGLU(sp, {"gate_proj": weights["shared.gate"], "up_proj": weights["shared.up"],
                                      "down_proj": weights["shared.down"]}, runtime)

    def runs_every_expert(self, x: torch.Tensor, n: int) -> bool:
        """A handful of rows (a decode step): what a step costs is the weights it streams, and the weight-streaming
        product reads a matrix at six times the rate of the row-group kernel; so unless the pairs are far fewer than the
        experts, every expert runs on every row (all experts' gate|up rows as one stacked matrix, the down products as
        one grouped launch), and the sum takes the chosen ones."""
        rt = self.runtime
        if not (self.n_experts and rt.dtype == torch.bfloat16 and rt.gemm_backend is None and rt.own_small_gemm
                and n <= rt.small_gemm_rows and 6 * n * self.top >= self.n_experts):
            return False
        return (self.hidden % 16 == 0 and self.intermediate % 8 == 0
                and ops.gemm_smallm_supported(x, self.gate_up.view(-1, self.hidden)))

    def route(self, logits, chosen, weight, dense_rows=None, n_real: int = 0) -> None:
        if self.choice == "sigmoid_groups":
            ops.moe_route_sigmoid_groups(logits, self.top, self.groups, self.keep_groups, chosen, weight, dense_rows, n_real)
        elif self.choice == "top_logits":
            ops.moe_route_logits(logits, self.router_bias, self.top, chosen, weight, dense_rows, n_real)
        else:
            ops.moe_route(logits, self.correction, self.top, chosen, weight, dense_rows, n_real)

    def forward_every_expert(self, x, ctx, logits, chosen, weight) -> torch.Tensor:
        rt = self.runtime
        n, E, ff = x.shape[0], self.n_experts, self.intermediate
        pair_row = ctx.buffer("moe.pair_row", (n, self.top), torch.int32)
        self.route(logits, chosen, weight, pair_row, E)
        gu = ctx.buffer("moe.every_gu", (n, E * 2 * ff), rt.dtype)
        ops.gemm_smallm(x, self.gate_up.view(E * 2 * ff, self.hidden), gu)
        act = ctx.buffer("moe.every_act", (n * E, ff), rt.dtype)
        ops.glu_act(gu.view(n * E, 2 * ff), act, self.activation, self.limit, self.alpha)
        rows = ctx.buffer("moe.every_rows", (n, E * self.hidden), rt.dtype)
        ops.gemm_smallm_grouped(act.view(n, E, ff).transpose(0, 1), self.down.view(E * self.hidden, ff), rows, self.hidden)
        shared = self.shared.forward(x, ctx) if self.shared is not None else None
        delta = ctx.buffer("moe.delta", (n, self.hidden), rt.dtype)
        ops.moe_combine(rows.view(n * E, self.hidden), x, shared, pair_row, weight, self.top, delta)
        return delta

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        rt = self.runtime
        n, top = x.shape[0], self.top
        n_all = self.n_experts + self.n_identity
        logits = ctx.buffer("moe.logits", (n, n_all), torch.float32)
        y = rt.linear(x, self.router, out=logits, out_dtype=torch.float32)
        if y.data_ptr() != logits.data_ptr():
            logits.copy_(y)
        chosen = ctx.buffer("moe.chosen", (n, top), torch.int32)
        weight = ctx.buffer("moe.weight", (n, top), torch.float32)
        if self.runs_every_expert(x, n):
            return self.forward_every_expert(x, ctx, logits, chosen, weight)
        self.route(logits, chosen, weight)
        offsets = ctx.buffer("moe.offsets", (self.n_experts + 1,), torch.int32)
        row_token = ctx.buffer("moe.row_token", (n * top,), torch.int32)
        pair_row = ctx.buffer("moe.pair_row", (n, top), torch.int32)
        ops.moe_group(chosen, n, top, self.n_experts, offsets, row_token, pair_row)
        rows = ctx.buffer("moe.rows", (n * top, self.hidden), rt.dtype)
        if self.n_experts and self.library_product and n * top > LIBRARY_ROWS and rt.gemm_backend is None:
            # many rows: the rows in expert order, then the library's product over row groups (bfloat16, float32 sums)
            xs = ctx.buffer("moe.xs", (n * top, self.hidden), rt.dtype)
            ops.moe_gather_rows(x, row_token, offsets, self.n_experts, xs)
            ends = offsets[1:]
            gu = torch._grouped_mm(xs, self.gate_up.transpose(1, 2), offs=ends, out_dtype=rt.dtype)
            act = ctx.buffer("moe.act", (n * top, self.intermediate), rt.dtype)
            ops.glu_act(gu, act, self.activation, self.limit, self.alpha)
            rows = torch._grouped_mm(act, self.down.transpose(1, 2), offs=ends, out_dtype=rt.dtype)
        elif self.n_experts:
            act = ctx.buffer("moe.act", (n * top, self.intermediate), rt.dtype)
            ops.moe_rows_gemm(x, row_token, offsets, self.n_experts, n * top, self.gate_up, act, self.glu, self.limit, self.alpha)
            ops.moe_rows_gemm(act, None, offsets, self.n_experts, n * top, self.down, rows)
        shared = self.shared.forward(x, ctx) if self.shared is not None else None
        delta = ctx.buffer("moe.delta", (n, self.hidden), rt.dtype)
        ops.moe_combine(rows, x, shared, pair_row, weight, top, delta)
        return delta
