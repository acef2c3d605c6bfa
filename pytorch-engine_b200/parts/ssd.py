"""The selective state-space mixer with one decay per head (the "state-space duality" form; the kernels and their formulas:
csrc/ssd.cu).

For a token with input ``h``, ``heads`` heads of ``dv`` features (``inner = heads * dv``), a state of ``n`` rows per head and
``groups`` groups of heads that share B and C:

    [z | x | B | C | dt] = W_in h                                   inner | inner | groups * n | groups * n | heads
    (x, B, C) = silu(conv(x | B | C) + conv_bias)                   one short causal convolution per channel
    dt = softplus(dt + dt_bias) ;  a = exp(-exp(A) dt)              per head, float32
    S <- a S + dt B x^T ;  y = S^T C + D x                          S [n, dv] per head, float32
    out = W_o (unit_parts(y * silu(z)) * norm)                      the gate first, then each of ``norm_groups`` equal parts
                                                                    of the row is divided by its own root mean square

What a sequence keeps between steps is of fixed size: every head's ``S`` and the last ``taps - 1`` inputs of the convolution,
float32 (a "state" entry of the cache, zero when a slot is taken).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from .registry import register
from .spec import CacheRequest, WeightDecl

# tokens per chunk when a prompt is cut into chunks that run side by side (the chain from chunk to chunk is one multiply-add
# per state element); steps whose longest sequence has at most two chunks walk each sequence in one go
CHUNK_TOKENS = 64


@register("mixer", "ssd")
class StateSpaceMixer:
    """params: ``hidden``, ``n_heads``, ``v_head_dim``, ``state`` (n), ``groups``, ``conv`` (taps), ``norm_groups``, ``eps``.
    weights: ``in_proj [2*inner + 2*groups*n + heads, hidden]``, ``conv [inner + 2*groups*n, taps]``, ``conv_bias``, ``dt_bias,
    A_log, D [heads]``, ``norm [inner]``, ``o_proj [hidden, inner]``."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    @classmethod
    def sizes(cls, params):
        h, nh, dv, n, g, taps = (int(params[k]) for k in ("hidden", "n_heads", "v_head_dim", "state", "groups", "conv"))
        return h, nh, dv, n, g, taps, nh * dv, nh * dv + 2 * g * n

    @classmethod
    def weight_decls(cls, params) -> Dict[str, WeightDecl]:
        h, nh, dv, n, g, taps, inner, ch = cls.sizes(params)
        return {"in_proj": WeightDecl((inner + ch + nh, h)), "conv": WeightDecl((ch, taps)), "conv_bias": WeightDecl((ch,)),
                "dt_bias": WeightDecl((nh,)), "A_log": WeightDecl((nh,)), "D": WeightDecl((nh,), "norm"),
                "norm": WeightDecl((inner,), "norm"), "o_proj": WeightDecl((h, inner))}

    @classmethod
    def cache_request(cls, params) -> Optional[CacheRequest]:
        h, nh, dv, n, g, taps, inner, ch = cls.sizes(params)
        shapes = [("S", (nh, n, dv), "float32")]
        if taps > 1:
            shapes.append(("conv", (taps - 1, ch), "float32"))
        return CacheRequest(kind="state", state_shapes=tuple(shapes))

    def __init__(self, params, weights, runtime) -> None:
        self.runtime = runtime
        (self.hidden, self.n_heads, self.v_dim, self.state, self.groups, self.taps, self.inner, self.channels) = self.sizes(params)
        if self.n_heads % self.groups:
            raise ValueError("n_heads must be a multiple of groups")
        self.norm_groups = int(params.get("norm_groups", 1))
        if self.inner % self.norm_groups:
            raise ValueError("heads * v_head_dim must be a multiple of norm_groups")
        self.eps = float(params.get("eps", 1e-5))
        if self.v_dim > 1024 or (self.state > 128 and (self.state * self.v_dim + 64 * self.state + 32 * self.v_dim) * 4 > 200 * 1024):
            raise ValueError(f"a head of {self.state} x {self.v_dim} is beyond what the recurrence kernel keeps on chip")
        f32 = torch.float32
        self.in_proj = runtime.adopt(weights["in_proj"])
        self.conv_w = runtime.adopt(weights["conv"], f32)
        self.conv_b = runtime.adopt(weights["conv_bias"], f32)
        self.dt_bias = runtime.adopt(weights["dt_bias"], f32)
        self.A_log = runtime.adopt(weights["A_log"], f32)
        self.D = runtime.adopt(weights["D"], f32)
        self.norm = runtime.adopt(weights["norm"], f32)
        self.o_proj = runtime.adopt(weights["o_proj"])
        self.no_tail = torch.zeros((1,), dtype=f32, device=runtime.device)

    def forward(self, x: torch.Tensor, ctx, view, writes_cache: bool = True) -> torch.Tensor:
        if not writes_cache:
            raise ValueError("a state-space mixer folds every token into its state; it cannot run without writing it")
        rt = self.runtime
        n = x.shape[0]
        inner, ch = self.inner, self.channels
        wide = ctx.buffer("ssd.wide", (n, inner + ch + self.n_heads), rt.dtype)
        rt.linear(x, self.in_proj, out=wide)
        xbc = ctx.buffer("ssd.xbc", (n, ch), rt.dtype)
        tail = view.state("conv") if self.taps > 1 else self.no_tail
        ops.short_conv_silu(wide, inner, self.conv_w, tail, ctx.token_seq, ctx.seq_slot, ctx.seq_qstart, xbc, ctx.n_seqs,
                            rt.status, bias=self.conv_b)
        y = ctx.buffer("ssd.y", (n, inner), torch.float32)
        chunk, max_chunks, scratch = 0, 1, None
        if ctx.max_q > 2 * CHUNK_TOKENS:
            chunk = CHUNK_TOKENS
            max_chunks = -(-ctx.max_q // chunk)
            scratch = ctx.buffer("ssd.scratch", (ops.ssd_scratch_floats(ctx.n_seqs, self.n_heads, self.state, self.v_dim, max_chunks),),
                                 torch.float32)
        ops.ssd_recurrence(xbc, wide[:, inner + ch:], self.dt_bias, self.A_log, self.D, y, view.state("S"), ctx.seq_slot,
                           ctx.seq_qstart, ctx.n_seqs, ctx.max_q, self.n_heads, self.groups, self.state, self.v_dim, rt.status,
                           chunk, max_chunks, scratch)
        normed = ctx.buffer("ssd.normed", (n, inner), rt.dtype)
        ops.gated_part_norm(y, wide[:, :inner], self.norm, self.eps, normed, self.norm_groups)
        delta = ctx.buffer("ssd.delta", (n, self.hidden), rt.dtype)
        rt.linear(normed, self.o_proj, out=delta)
        return delta
