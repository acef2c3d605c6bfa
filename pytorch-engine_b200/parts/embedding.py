"""Token embedding and output head."""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops
from .registry import register
from .spec import CacheRequest, WeightDecl


@register("embedding", "token_embedding")
class TokenEmbedding:
    """params: ``vocab``, ``hidden``, optionally ``scale`` (a factor on every row).  weights: ``weight [vocab, hidden]``.
    Output: the float32 residual stream (pygguf_engine/model.py:2237, pygguf_engine/quant_kernels.py:1846-1847)."""

    graph_safe = True  # launches only; nothing in forward() waits for the device
    writes_copy = True  # forward() can leave a second copy of its rows

    @classmethod
    def weight_decls(cls, params) -> Dict[str, WeightDecl]:
        return {"weight": WeightDecl((int(params["vocab"]), int(params["hidden"])), "embedding")}

    def __init__(self, params, weights, runtime) -> None:
        self.runtime = runtime
        self.vocab = int(params["vocab"])
        self.hidden = int(params["hidden"])
        self.scale = float(params.get("scale", 1.0) or 1.0)
        self.weight = runtime.adopt(weights["weight"])

    def forward(self, token_ids: torch.Tensor, out: torch.Tensor, copy=None) -> torch.Tensor:
        ops.embed_gather(self.weight, token_ids, out, self.runtime.status, self.scale, copy)
        return out


@register("embedding", "token_pair_embedding")
class TokenPairEmbedding:
    """A token embedding plus an embedding of the pair (previous token, token), hashed into a table:
    ``x = E[tok] + B[(prev * mul_prev + tok * mul_cur) mod buckets]``, and ``B[buckets]`` (the table's last row) for a
    sequence's first token.  params: ``vocab``, ``hidden``, ``buckets``, ``mul_prev``, ``mul_cur``.  weights: ``weight
    [vocab, hidden]``, ``pairs [buckets + 1, hidden]``.  What a sequence keeps between steps is its last token (a
    "state" entry of the cache: one int32)."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    @classmethod
    def weight_decls(cls, params) -> Dict[str, WeightDecl]:
        h = int(params["hidden"])
        return {"weight": WeightDecl((int(params["vocab"]), h), "embedding"),
                "pairs": WeightDecl((int(params["buckets"]) + 1, h), "embedding")}

    @classmethod
    def cache_request(cls, params) -> CacheRequest:
        return CacheRequest(kind="state", state_shapes=(("last_token", (1,), "int32"),))

    def __init__(self, params, weights, runtime) -> None:
        self.runtime = runtime
        self.vocab = int(params["vocab"])
        self.hidden = int(params["hidden"])
        self.buckets = int(params["buckets"])
        self.mul_prev = int(params["mul_prev"])
        self.mul_cur = int(params["mul_cur"])
        self.weight = runtime.adopt(weights["weight"])
        self.pairs = runtime.adopt(weights["pairs"])

    def forward(self, token_ids: torch.Tensor, out: torch.Tensor, ctx, view) -> torch.Tensor:
        last = view.state("last_token").view(-1)
        ops.embed_pair_gather(self.weight, self.pairs, token_ids, ctx.token_seq, ctx.token_pos, ctx.seq_slot, ctx.seq_qstart,
                              last, out, self.buckets, self.mul_prev, self.mul_cur, self.runtime.status)
        return out


@register("head", "linear_head")
class LinearHead:
    """params: ``vocab``, ``hidden``.  weights: ``weight [vocab, hidden]``; a tied head names the
    embedding's tensor and shares its storage (pygguf_engine/model.py:1678-1683, 2206-2214).
    ``scale`` (optional): a factor on the logits.  Output: float32 logits."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    @classmethod
    def weight_decls(cls, params) -> Dict[str, WeightDecl]:
        return {"weight": WeightDecl((int(params["vocab"]), int(params["hidden"])), "embedding")}

    def __init__(self, params, weights, runtime) -> None:
        self.runtime = runtime
        self.vocab = int(params["vocab"])
        self.weight = runtime.adopt(weights["weight"])
        self.scale = float(params.get("scale", 1.0) or 1.0)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        logits = self.runtime.linear(x, self.weight, out_dtype=torch.float32)
        if self.scale != 1.0:
            logits.mul_(self.scale)
        return logits
