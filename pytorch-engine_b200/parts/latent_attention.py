"""Latent attention: keys and values of every head are expansions of one cached low-rank row per position.

For a token with input ``h`` at position p (W stored [out, in]):

    q     = W_q h                       heads x (d + dr): per head d features without position, dr rotated ones
    low   = W_dkv h                     rank + dr
    c     = low[:rank] / rms(low[:rank]) * w_c            the latent row           } what the cache keeps per
    kr    = turn(low[rank:], p)                            one rotated key part     } position: [c | kr]
    k_h   = [W_uk,h c | kr] ,  v_h = W_uv,h c
    o_h   = softmax_j(scale * q_h . k_h(j)) v_h(j)   over j <= p
    out   = W_o (gate * o),   gate = sigmoid(W_g h): one number a head, or one a feature

Only ``[c | kr]`` is cached, so the products with W_uk and W_uv are moved to the query's side ("absorbed"):
``q_h . W_uk,h c = (W_uk,h^T q_h) . c`` and ``sum_j p_j W_uv,h c_j = W_uv,h (sum_j p_j c_j)``.  A step computes, per head, the
absorbed query ``[W_uk,h^T q_h | turn(q_h[d:], p)]`` of ``rank + dr`` features, attends with it over the cached rows as one
kv head shared by all query heads whose values are the rows' leading ``rank`` features, and expands the result with
W_uv,h.  Norm, rotation, scores and softmax are float32 in every run dtype; the products run in the run dtype.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from .attention import SPLIT_KEYS
from .linear import fuse_rows
from .registry import register
from .spec import CacheRequest, WeightDecl


# Keys per partial result of the tensor-core decode kernel while one wave of blocks holds them.  Measured with 16 heads and
# rows of 576: 8 sequences at 2,048 keys 30.8 us with 128, 32.8 with 256, 40.4 with 512; one sequence at 8,192 keys 55.9,
# 43.1, 45.2 (a partial result is 512 floats a head, and the merge reads them all).
LATENT_SPLIT_KEYS = 256


def attend_rows(ops, decode, qfull, mixed, n_seqs, max_q, n_heads, row, rank, scale, seq_qstart, seq_past, seq_slot, page_table,
                num_pages, pages, status, max_kv_len, buffer, tensor_cores=None) -> None:
    """Every head's query of ``row`` features (``qfull [n, n_heads * row]``) over the cached rows ``pages [pages, 1, 64, row]``
    as one kv head whose values are the rows' leading ``rank`` features; ``mixed [n, n_heads * rank]`` gets the weighted
    rows.  ``buffer(name, shape, dtype)`` hands out the step's scratch; ``max_kv_len``: the longest sequence of the step.
    ``tensor_cores``: None takes the tensor-core kernels where they take the shape (bfloat16, rows in steps of 64 up to
    576, values of 128, 256 or 512 features); False keeps the float32-arithmetic kernels."""
    if tensor_cores is None:
        tensor_cores = qfull.is_cuda and ops.attention_latent_supported(qfull.dtype, row, rank)
    if tensor_cores:
        scratch, split_keys, max_splits, floor = None, 0, 0, 0
        if decode:
            split_keys, max_splits, floor = ops.attention_latent_decode_ranges(qfull.device, n_seqs, n_heads, int(max_kv_len),
                                                                               LATENT_SPLIT_KEYS)
            scratch = buffer("attn.scratch", (ops.attention_generic_scratch_floats(n_seqs, n_heads, rank, max_splits),),
                             torch.float32)
        ops.attention_latent(decode, qfull, mixed, n_seqs, max_q, n_heads, row, rank, scale, seq_qstart, seq_past, seq_slot,
                             page_table, num_pages, pages, scratch, split_keys, max_splits, status, min_range_keys=floor)
        return
    scratch, max_splits = None, 0
    if decode:
        max_splits = max(1, -(-int(max_kv_len) // SPLIT_KEYS))
        scratch = buffer("attn.scratch", (ops.attention_generic_scratch_floats(n_seqs, n_heads, rank, max_splits),), torch.float32)
    ops.attention_generic_masked(decode, qfull, mixed, n_seqs, max_q, n_heads, 1, row, rank, scale, seq_qstart, seq_past, seq_slot,
                                 page_table, num_pages, pages, pages, scratch, SPLIT_KEYS, max_splits, status, v_ld=row)


@register("mixer", "latent_attention")
class LatentAttention:
    """params: ``hidden``, ``n_heads``, ``head_dim`` (features without position), ``rot_dim`` (rotated features, 0: none),
    ``v_head_dim``, ``kv_rank``, ``scale``, ``eps`` (of the latent row's norm), ``gate`` ("head": one gate a head;
    "feature": one a feature of the concatenated heads), ``position`` (name of a rotary encoding of the plan with
    interleaved pairs over at most ``rot_dim`` features, or None).  weights: ``q_proj [heads*(d+dr), hidden]``, ``dkv_proj
    [rank+dr, hidden]``, ``dkv_norm [rank]``, ``uk_proj [heads*d, rank]``, ``uv_proj [heads*dv, rank]``, ``g_proj [heads or
    heads*dv, hidden]``, ``o_proj [hidden, heads*dv]``."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    @classmethod
    def sizes(cls, params):
        return (int(params["hidden"]), int(params["n_heads"]), int(params["head_dim"]), int(params.get("rot_dim") or 0),
                int(params.get("v_head_dim") or params["head_dim"]), int(params["kv_rank"]))

    @classmethod
    def weight_decls(cls, params) -> Dict[str, WeightDecl]:
        h, nh, d, dr, dv, r = cls.sizes(params)
        gate_rows = nh if params.get("gate", "head") == "head" else nh * dv
        return {
            "q_proj": WeightDecl((nh * (d + dr), h)),
            "dkv_proj": WeightDecl((r + dr, h)),
            "dkv_norm": WeightDecl((r,), "norm"),
            "uk_proj": WeightDecl((nh * d, r)),
            "uv_proj": WeightDecl((nh * dv, r)),
            "g_proj": WeightDecl((gate_rows, h)),
            "o_proj": WeightDecl((h, nh * dv)),
        }

    @classmethod
    def cache_request(cls, params) -> Optional[CacheRequest]:
        _, _, _, dr, _, r = cls.sizes(params)
        return CacheRequest(kind="kv", kv_heads=1, head_dim=r + dr, v_head_dim=r, values_in_keys=True)

    def __init__(self, params, weights, runtime, positions=None) -> None:
        self.runtime = runtime
        self.hidden, self.n_heads, self.head_dim, self.rot_dim, self.v_dim, self.rank = self.sizes(params)
        self.row = self.rank + self.rot_dim
        if self.row > 1024 or self.rank > 512:
            raise ValueError(f"a latent row of {self.rank} + {self.rot_dim} features is beyond what the attention kernel takes "
                             "(rank <= 512, row <= 1024)")
        self.scale = float(params["scale"])
        self.eps = float(params.get("eps", 1e-6))
        self.gate = str(params.get("gate", "head"))
        if self.gate not in ("head", "feature"):
            raise ValueError(f"gate {self.gate!r} is not built ('head' and 'feature' are)")
        self.gate_rows = self.n_heads if self.gate == "head" else self.n_heads * self.v_dim
        nh, d, dr, dv, r = self.n_heads, self.head_dim, self.rot_dim, self.v_dim, self.rank
        # one product for everything that reads the block's input: q | low | gate
        self.qlg = fuse_rows(runtime, [weights["q_proj"], weights["dkv_proj"], weights["g_proj"]])
        self.q_cols = nh * (d + dr)
        self.low_col0 = self.q_cols
        self.gate_col0 = self.q_cols + r + dr
        self.norm_w = runtime.adopt(weights["dkv_norm"], torch.float32)
        dev, dt = runtime.device, runtime.dtype
        # per head: absorbed query = q_h [d] @ uk_h [d, rank];  head output = latent [rank] @ uv_h^T [rank, dv]
        self.uk = weights["uk_proj"].to(device=dev, dtype=dt).view(nh, d, r).contiguous()
        self.uv_t = weights["uv_proj"].to(device=dev, dtype=dt).view(nh, dv, r).transpose(1, 2).contiguous()
        self.o_proj = runtime.adopt(weights["o_proj"])
        self.position = None
        self.rot = 0
        name = params.get("position")
        if name is not None and dr:
            self.position = (positions or {})[name]
            if not (getattr(self.position, "fusable_rotary", False) and getattr(self.position, "interleaved", False)):
                raise ValueError(f"position {name!r} must be a rotary encoding with tables() over interleaved pairs")
            self.rot = int(self.position.tables()[2])
            if self.rot > dr:
                raise ValueError(f"position {name!r} turns {self.rot} features, the rotated part has {dr}")

    def forward(self, x: torch.Tensor, ctx, view, writes_cache: bool = True) -> torch.Tensor:
        rt = self.runtime
        n, nh, d, dr, dv, r, row = x.shape[0], self.n_heads, self.head_dim, self.rot_dim, self.v_dim, self.rank, self.row
        qlg = ctx.buffer("latent.qlg", (n, self.qlg.shape[0]), rt.dtype)
        rt.linear(x, self.qlg, out=qlg)
        qfull = ctx.buffer("latent.qfull", (n, nh, row), rt.dtype)
        cos = sin = None
        if self.rot:
            cos, sin, _ = self.position.tables()
        pages = view.k_pages
        # the absorbed queries, head by head: [heads, n, d] x [heads, d, rank]
        q_heads = qlg[:, :self.q_cols].view(n, nh, d + dr)[:, :, :d].transpose(0, 1)
        absorbed = ctx.buffer("latent.absorbed", (nh, n, r), rt.dtype)
        rt.batched_linear(q_heads, self.uk.transpose(1, 2), absorbed)
        # the cached rows into their pages; the queries' rows put together: [absorbed | turned part]
        ops.latent_prepare(qlg, 0, self.low_col0, nh, d, dr, r, self.norm_w, self.eps, cos, sin, self.rot, ctx.token_seq,
                           ctx.token_pos, ctx.seq_slot, view.page_table, view.num_pages, pages, qfull, writes_cache, rt.status,
                           absorbed=absorbed)
        mixed = ctx.buffer("latent.mixed", (n, nh, r), rt.dtype)
        attend_rows(ops, ctx.decode, qfull.view(n, nh * row), mixed.view(n, nh * r), ctx.n_seqs, ctx.max_q, nh, row, r, self.scale,
                    ctx.seq_qstart, ctx.seq_past, ctx.seq_slot, view.page_table, view.num_pages, pages, rt.status, ctx.max_kv_len,
                    ctx.buffer, tensor_cores=False if getattr(rt, "generic_attention", False) else None)
        # expand with W_uv head by head: [heads, n, rank] x [heads, rank, dv]
        heads_t = ctx.buffer("latent.heads_t", (nh, n, dv), rt.dtype)
        rt.batched_linear(mixed.transpose(0, 1), self.uv_t.transpose(1, 2), heads_t)
        heads = ctx.buffer("latent.heads", (n, nh * dv), rt.dtype)
        ops.sigmoid_gate(heads_t, qlg[:, self.gate_col0:self.gate_col0 + self.gate_rows], heads)
        delta = ctx.buffer("latent.delta", (n, self.hidden), rt.dtype)
        rt.linear(heads, self.o_proj, out=delta)
        return delta
