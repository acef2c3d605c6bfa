"""Differential attention: every head takes two softmax maps over the same values and subtracts the second.

For a token with input ``h`` (W stored [out, in]; q and k rows laid out head by head as [map 1 | map 2]):

    q = W_q h   heads x 2 x d        k = W_k h   kv_heads x 2 x d        v = W_v h   kv_heads x dv
    a_m   = softmax_j(scale * q_(head, m) . k_(head / group, m)(j)) v_(head / group)(j)        m = 1, 2, over visible j
    o     = a_1 - lambda * a_2 ;   o <- o / sqrt(mean(o^2) + eps) * (1 - diff)     per head, no weight
    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff                                one number for the layer
    out   = W_o o

Visible keys: j <= i, and with ``chunk`` only those of the query's own block of ``chunk`` positions (blocks counted from
the sequence's start).  A layer with ``shared_kv`` has no k and v projections: it reads the cache entry of another layer
(the plan's ``RunStep`` says which) with its own queries and mask.

The two maps run as one grouped-query attention: the projections' rows are reordered at load time to [map][head], so
the first map's heads come first, query head ``m * heads + h`` reads key head ``m * kv_heads + h / group`` (the usual
mapping), and key head g reads value head ``g % kv_heads``; the cache keeps ``2 * kv_heads`` key heads and ``kv_heads`` value
heads per position.  Scores, softmax, the subtraction and the norm are float32 in every run dtype.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..kernels import ops
from .attention import SPLIT_KEYS
from .linear import fuse_rows
from .registry import register
from .spec import CacheRequest, WeightDecl


def maps_first(w: torch.Tensor, heads: int, d: int) -> torch.Tensor:
    """Rows [head][map][d] of a projection reordered to [map][head][d]."""
    return w.view(heads, 2, d, w.shape[1]).transpose(0, 1).reshape(2 * heads * d, w.shape[1]).contiguous()


def attend_maps(ops, decode, q, maps, n_seqs, max_q, n_heads, n_kv_heads, d, dv, scale, chunk, seq_qstart, seq_past, seq_slot,
                page_table, num_pages, k_pages, v_pages, status, max_kv_len, buffer, tensor_cores=None) -> None:
    """Both softmax maps of every head as one grouped-query attention: ``q [n, 2 * n_heads * d]`` ([map][head][d]) over
    ``k_pages [pages, 2 * n_kv_heads, 64, d]`` and ``v_pages [pages, n_kv_heads, 64, dv]`` into ``maps [n, 2 * n_heads * dv]``
    float32.  ``buffer(name, shape, dtype)`` hands out the step's scratch; ``max_kv_len``: the longest sequence of the step.
    ``tensor_cores``: None takes the tensor-core kernels where they take the shape (bfloat16, keys and values of one size,
    64 or 128, groups up to 16); False keeps the float32-arithmetic kernels."""
    if tensor_cores is None:
        tensor_cores = q.is_cuda and d == dv and ops.attention_mma_supported(q.dtype, d, 2 * n_heads, 2 * n_kv_heads)
    if tensor_cores:
        scratch, split_keys, max_splits, floor = None, SPLIT_KEYS, 0, 0
        if decode:
            split_keys, max_splits, floor = ops.attention_mma_decode_ranges(q.device, d, n_seqs, 2 * n_kv_heads, int(max_kv_len),
                                                                            SPLIT_KEYS)
            scratch = buffer("attn.scratch", (ops.attention_generic_scratch_floats(n_seqs, 2 * n_heads, dv, max_splits),),
                             torch.float32)
        ops.attention_mma_masked(decode, q, maps, n_seqs, max_q, 2 * n_heads, 2 * n_kv_heads, d, scale, seq_qstart, seq_past,
                                 seq_slot, page_table, num_pages, k_pages, v_pages, scratch, split_keys, max_splits, status,
                                 min_range_keys=floor, chunk=chunk, v_heads=n_kv_heads, split_p=True)
        return
    scratch, max_splits = None, 0
    if decode:
        max_splits = max(1, -(-int(max_kv_len) // SPLIT_KEYS))
        scratch = buffer("attn.scratch", (ops.attention_generic_scratch_floats(n_seqs, 2 * n_heads, dv, max_splits),), torch.float32)
    ops.attention_generic_masked(decode, q, maps, n_seqs, max_q, 2 * n_heads, 2 * n_kv_heads, d, dv, scale, seq_qstart, seq_past,
                                 seq_slot, page_table, num_pages, k_pages, v_pages, scratch, SPLIT_KEYS, max_splits, status,
                                 chunk=chunk, v_heads=n_kv_heads)


@register("mixer", "diff_attention")
class DiffAttention:
    """params: ``hidden``, ``n_heads``, ``n_kv_heads``, ``head_dim``, ``v_head_dim``, ``scale``, ``diff``, ``eps``, ``chunk``
    (None: every earlier key), ``cache_chunk`` (what the cache may drop: the chunk that every reader of this layer's keys
    shares, or None), ``shared_kv`` (true: no k and v projections).  weights: ``q_proj [heads*2*d, hidden]``, ``k_proj
    [kv_heads*2*d, hidden]``, ``v_proj [kv_heads*dv, hidden]``, ``lq1, lk1, lq2, lk2 [d]``, ``o_proj [hidden, heads*dv]``."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    @classmethod
    def sizes(cls, params):
        return (int(params["hidden"]), int(params["n_heads"]), int(params["n_kv_heads"]), int(params["head_dim"]),
                int(params.get("v_head_dim") or params["head_dim"]))

    @classmethod
    def weight_decls(cls, params) -> Dict[str, WeightDecl]:
        h, nh, nkv, d, dv = cls.sizes(params)
        decls = {"q_proj": WeightDecl((nh * 2 * d, h)), "o_proj": WeightDecl((h, nh * dv))}
        if not params.get("shared_kv"):
            decls["k_proj"] = WeightDecl((nkv * 2 * d, h))
            decls["v_proj"] = WeightDecl((nkv * dv, h))
        for name in ("lq1", "lk1", "lq2", "lk2"):
            decls[name] = WeightDecl((d,))
        return decls

    @classmethod
    def cache_request(cls, params) -> Optional[CacheRequest]:
        _, _, nkv, d, dv = cls.sizes(params)
        return CacheRequest(kind="kv", kv_heads=2 * nkv, head_dim=d, v_head_dim=dv, value_heads=nkv,
                            chunk=params.get("cache_chunk") or None)

    def __init__(self, params, weights, runtime) -> None:
        self.runtime = runtime
        self.hidden, self.n_heads, self.n_kv_heads, self.head_dim, self.v_dim = self.sizes(params)
        nh, nkv, d, dv = self.n_heads, self.n_kv_heads, self.head_dim, self.v_dim
        if nh % nkv:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        if d > 512 or dv > 512:
            raise ValueError(f"head_dim {d} / v_head_dim {dv} is beyond what the attention kernels take (<= 512)")
        self.scale = float(params["scale"])
        self.diff = float(params["diff"])
        self.eps = float(params.get("eps", 1e-6))
        self.chunk = int(params["chunk"]) if params.get("chunk") else 0
        self.shared_kv = bool(params.get("shared_kv"))
        mats = [maps_first(weights["q_proj"], nh, d)]
        if not self.shared_kv:
            mats += [maps_first(weights["k_proj"], nkv, d), weights["v_proj"]]
        self.qkv = fuse_rows(runtime, mats)
        self.q_cols, self.k_cols, self.v_cols = 2 * nh * d, 2 * nkv * d, nkv * dv
        self.o_proj = runtime.adopt(weights["o_proj"])
        f = lambda name: weights[name].to(torch.float32)
        # one number for the layer, from float32 sums
        self.lam = (math.exp(float((f("lq1") * f("lk1")).sum())) - math.exp(float((f("lq2") * f("lk2")).sum())) + self.diff)

    def forward(self, x: torch.Tensor, ctx, view, writes_cache: bool = True) -> torch.Tensor:
        rt = self.runtime
        n, nh, nkv, d, dv = x.shape[0], self.n_heads, self.n_kv_heads, self.head_dim, self.v_dim
        if writes_cache and self.shared_kv:
            raise ValueError("a differential-attention layer without k and v projections reads another layer's cache entry")
        qkv = ctx.buffer("diff.qkv", (n, self.qkv.shape[0]), rt.dtype)
        rt.linear(x, self.qkv, out=qkv)
        where = (ctx.token_seq, ctx.token_pos, ctx.seq_slot, view.page_table, view.num_pages)
        if writes_cache:
            ops.rows_to_pages_pair(qkv, self.q_cols, 2 * nkv, d, view.k_pages, self.q_cols + self.k_cols, nkv, dv, view.v_pages,
                                   *where, rt.status)
        maps = ctx.buffer("diff.maps", (n, 2 * nh * dv), torch.float32)   # the two maps stay float32 up to their difference
        attend_maps(ops, ctx.decode, qkv, maps, ctx.n_seqs, ctx.max_q, nh, nkv, d, dv, self.scale, self.chunk, ctx.seq_qstart,
                    ctx.seq_past, ctx.seq_slot, view.page_table, view.num_pages, view.k_pages, view.v_pages, rt.status,
                    ctx.max_kv_len, ctx.buffer, tensor_cores=False if getattr(rt, "generic_attention", False) else None)
        heads = ctx.buffer("diff.heads", (n, nh * dv), rt.dtype)
        ops.diff_combine(maps, heads, nh, dv, self.lam, self.eps, 1.0 - self.diff)
        delta = ctx.buffer("diff.delta", (n, self.hidden), rt.dtype)
        rt.linear(heads, self.o_proj, out=delta)
        return delta
