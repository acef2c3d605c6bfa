"""The gated delta rule: a linear recurrence whose matrix state forgets per key channel and is corrected by every
token (the kernels and their formulas: csrc/delta_rule.cu).

For a token with input ``h``, ``kv_heads`` query/key heads of size ``d`` shared by groups of the ``heads`` value heads of
size ``dv``:

    q, k, v = silu(conv(W_q h)), silu(conv(W_k h)), silu(conv(W_v h))     short causal convolutions per channel
    q = q / |q| / sqrt(d) ;  k = k / |k|                                   |x| = sqrt(sum x^2 + 1e-6), per head
    beta = sigmoid(w_b . h) ;  g = exp(-exp(A) softplus(W_a2 W_a1 h + dt)) per head, g also per key channel
    S <- diag(g) S ;  u = beta (v - S^T k) ;  S <- S + k u^T ;  o = S^T q
    out = W_o (o / rms_per_head(o) * norm * sigmoid(W_g2 W_g1 h))

What a sequence keeps between steps is of fixed size: every head's ``S [d, dv]`` and the last ``taps - 1`` inputs of the
convolutions, float32 (a "state" entry of the cache, zero when a slot is taken).  State, decay, beta, the unit vectors
and the per-head norm are float32 in every run dtype; the decay's and beta's projections write float32.

A second form of the same mixer (``decay = "head"``, ``gate = "silu"``) has one decay per head and token from a projection
of full rank, ``g = exp(-exp(A) softplus(w_a . h + dt))`` with ``w_a [heads, hidden]``, and the output gate ``silu(W_g h)``
with ``W_g [heads * dv, hidden]``; everything else is the same, and so are the kernels.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from .linear import fuse_rows
from .registry import register
from .spec import CacheRequest, WeightDecl


# tokens per chunk when a prompt is cut into chunks that run side by side (the chain from chunk to chunk costs a product
# with a d x d matrix per chunk, so the chunks are longer than the mlstm's); steps whose longest sequence has no more
# tokens than one chunk walk each sequence in one go
CHUNK_TOKENS = 128


@register("mixer", "gated_delta")
class GatedDeltaMixer:
    """params: ``hidden``, ``n_heads``, ``n_kv_heads``, ``head_dim``, ``v_head_dim``, ``conv`` (taps), ``eps`` (of the
    per-head norm), ``rank`` (of the decay's and the gate's low-rank projections in a random model; a checkpoint's own
    tensors decide it).  weights: ``q_proj, k_proj [kv_heads*head_dim, hidden]``, ``v_proj [heads*v_head_dim, hidden]``,
    ``q_conv, k_conv, v_conv [channels, taps]``, ``b_proj [heads, hidden]``, ``A_log [heads]``, ``a1 [rank, hidden]``, ``a2
    [heads*head_dim, rank]``, ``dt_bias [heads*head_dim]``, ``g1 [rank, hidden]``, ``g2 [heads*v_head_dim, rank]``, ``norm
    [v_head_dim]``, ``o_proj [hidden, heads*v_head_dim]``.

    ``decay`` ("channel", the default, or "head": weights ``a_proj [heads, hidden]`` and ``dt_bias [heads]`` in place of ``a1,
    a2``) and ``gate`` ("sigmoid", the default, or "silu": weight ``g_proj [heads*v_head_dim, hidden]`` in place of ``g1, g2``)."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    @classmethod
    def weight_decls(cls, params) -> Dict[str, WeightDecl]:
        h, nh, nkv, d, dv, taps = (int(params[k]) for k in ("hidden", "n_heads", "n_kv_heads", "head_dim", "v_head_dim", "conv"))
        rank = int(params.get("rank", 16))
        decls = {"q_proj": WeightDecl((nkv * d, h)), "k_proj": WeightDecl((nkv * d, h)), "v_proj": WeightDecl((nh * dv, h)),
                 "q_conv": WeightDecl((nkv * d, taps)), "k_conv": WeightDecl((nkv * d, taps)), "v_conv": WeightDecl((nh * dv, taps)),
                 "b_proj": WeightDecl((nh, h)), "A_log": WeightDecl((nh,)),
                 "norm": WeightDecl((dv,), "norm"), "o_proj": WeightDecl((h, nh * dv))}
        if params.get("decay", "channel") == "head":
            decls.update({"a_proj": WeightDecl((nh, h)), "dt_bias": WeightDecl((nh,))})
        else:
            decls.update({"a1": WeightDecl((rank, h), any_dims=(0,)), "a2": WeightDecl((nh * d, rank), any_dims=(1,)),
                          "dt_bias": WeightDecl((nh * d,))})
        if params.get("gate", "sigmoid") == "silu":
            decls["g_proj"] = WeightDecl((nh * dv, h))
        else:
            decls.update({"g1": WeightDecl((rank, h), any_dims=(0,)), "g2": WeightDecl((nh * dv, rank), any_dims=(1,))})
        return decls

    @classmethod
    def cache_request(cls, params) -> Optional[CacheRequest]:
        nh, nkv, d, dv, taps = (int(params[k]) for k in ("n_heads", "n_kv_heads", "head_dim", "v_head_dim", "conv"))
        shapes = [("S", (nh, d, dv), "float32")]
        if taps > 1:
            shapes.append(("conv", (taps - 1, 2 * nkv * d + nh * dv), "float32"))
        return CacheRequest(kind="state", state_shapes=tuple(shapes))

    def __init__(self, params, weights, runtime) -> None:
        self.runtime = runtime
        self.hidden = int(params["hidden"])
        self.n_heads = int(params["n_heads"])
        self.n_kv_heads = int(params["n_kv_heads"])
        if self.n_heads % self.n_kv_heads:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        self.head_dim = int(params["head_dim"])
        self.v_dim = int(params["v_head_dim"])
        self.taps = int(params["conv"])
        self.eps = float(params.get("eps", 1e-5))
        d, dv = self.head_dim, self.v_dim
        in_registers = (d <= 32 and dv <= 512) or (d <= 128 and dv <= 256)
        if max(d, dv) > 1024 or (not in_registers and (d * max(d, dv) + 3 * d) * 4 > 200 * 1024) or (d * (d + 1) + 8 * d) * 4 > 200 * 1024:
            raise ValueError(f"a head of {d} x {dv} is beyond what the recurrence kernels keep on chip")
        f32 = torch.float32
        self.head_decay = params.get("decay", "channel") == "head"
        self.gate_silu = params.get("gate", "sigmoid") == "silu"
        if params.get("decay", "channel") not in ("channel", "head") or params.get("gate", "sigmoid") not in ("sigmoid", "silu"):
            raise ValueError("decay is 'channel' or 'head', gate is 'sigmoid' or 'silu'")
        self.rank_a = 0 if self.head_decay else int(weights["a1"].shape[0])
        self.rank_g = 0 if self.gate_silu else int(weights["g1"].shape[0])
        if (not self.head_decay and weights["a2"].shape[1] != self.rank_a) or (not self.gate_silu and weights["g2"].shape[1] != self.rank_g):
            raise ValueError("the two halves of a low-rank projection do not fit")
        self.channels = 2 * self.n_kv_heads * self.head_dim + self.n_heads * self.v_dim
        # q | k | v | the low ranks of decay and gate (or the gate itself): one product over the mixer's input
        fused = [weights["q_proj"], weights["k_proj"], weights["v_proj"]]
        if not self.head_decay:
            fused.append(weights["a1"])
        fused.append(weights["g_proj"] if self.gate_silu else weights["g1"])
        self.wide = fuse_rows(runtime, fused)
        self.conv_w = torch.cat([weights[f"{s}_conv"].to(device=runtime.device, dtype=f32) for s in "qkv"]).contiguous()
        # beta's projection, and with it the decay's when that is one number a head: float32 outputs of one product
        self.b_proj = (fuse_rows(runtime, [weights["b_proj"], weights["a_proj"]]) if self.head_decay
                       else runtime.adopt(weights["b_proj"]))
        self.a2 = None if self.head_decay else runtime.adopt(weights["a2"])
        self.g2 = None if self.gate_silu else runtime.adopt(weights["g2"])
        self.A_log = runtime.adopt(weights["A_log"], f32)
        self.dt_bias = runtime.adopt(weights["dt_bias"], f32)
        self.norm = runtime.adopt(weights["norm"], f32)
        self.o_proj = runtime.adopt(weights["o_proj"])
        self.no_tail = torch.zeros((1,), dtype=f32, device=runtime.device)

    def _f32_linear(self, x, w, buf):
        y = self.runtime.linear(x, w, out=buf, out_dtype=torch.float32)
        if y.data_ptr() != buf.data_ptr():
            buf.copy_(y)
        return buf

    def forward(self, x: torch.Tensor, ctx, view, writes_cache: bool = True) -> torch.Tensor:
        if not writes_cache:
            raise ValueError("a gated delta mixer folds every token into its state; it cannot run without writing it")
        rt = self.runtime
        n = x.shape[0]
        c, ra = self.channels, self.rank_a
        wide = ctx.buffer("delta.wide", (n, self.wide.shape[0]), rt.dtype)
        rt.linear(x, self.wide, out=wide)
        qkv = ctx.buffer("delta.qkv", (n, c), rt.dtype)
        tail = view.state("conv") if self.taps > 1 else self.no_tail
        ops.short_conv_silu(wide, 0, self.conv_w, tail, ctx.token_seq, ctx.seq_slot, ctx.seq_qstart, qkv, ctx.n_seqs, rt.status)
        if self.head_decay and self.gate_silu:
            return self.forward_full_rank(x, wide, qkv, ctx, view)
        if self.head_decay or self.gate_silu:
            raise ValueError("decay = 'head' and gate = 'silu' come together in this mixer")
        if n < rt.large_gemm_rows and c % 8 == 0 and ra % 8 == 0:
            # the low ranks as views of the wide product's rows (the products for few and for some rows take strided rows)
            low_a, low_g = wide[:, c:c + ra], wide[:, c + ra:]
        else:
            low_a = ctx.buffer("delta.low_a", (n, ra), rt.dtype)
            low_a.copy_(wide[:, c:c + ra])
            low_g = ctx.buffer("delta.low_g", (n, self.rank_g), rt.dtype)
            low_g.copy_(wide[:, c + ra:])
        decay = self._f32_linear(low_a, self.a2, ctx.buffer("delta.decay", (n, self.n_heads * self.head_dim), torch.float32))
        beta = self._f32_linear(x, self.b_proj, ctx.buffer("delta.beta", (n, self.n_heads), torch.float32))
        gate = ctx.buffer("delta.gate", (n, self.n_heads * self.v_dim), rt.dtype)
        rt.linear(low_g, self.g2, out=gate)
        out = ctx.buffer("delta.out", (n, self.n_heads * self.v_dim), rt.dtype)
        chunk, max_chunks, scratch = 0, 1, None
        if ctx.max_q > CHUNK_TOKENS:
            chunk = CHUNK_TOKENS
            max_chunks = -(-ctx.max_q // chunk)
            scratch = ctx.buffer("delta.scratch", (ops.delta_rule_scratch_floats(ctx.n_seqs, self.n_heads, self.head_dim, self.v_dim,
                                                                               max_chunks),), torch.float32)
        ops.delta_rule_recurrence(qkv, decay, self.dt_bias, self.A_log, beta, gate, self.norm, self.eps, self.head_dim ** -0.5,
                                  out, view.state("S"), ctx.seq_slot, ctx.seq_qstart, ctx.n_seqs, ctx.max_q, self.n_heads,
                                  self.n_kv_heads, self.head_dim, self.v_dim, rt.status, chunk, max_chunks, scratch)
        delta = ctx.buffer("delta.delta", (n, self.hidden), rt.dtype)
        rt.linear(out, self.o_proj, out=delta)
        return delta

    def forward_full_rank(self, x, wide, qkv, ctx, view) -> torch.Tensor:
        """The form with one decay per head and a silu gate of full rank: beta | decay are the float32 outputs of one product,
        the gate's rows are the last columns of the wide product."""
        rt = self.runtime
        n, nh = x.shape[0], self.n_heads
        ba = self._f32_linear(x, self.b_proj, ctx.buffer("delta.beta_decay", (n, 2 * nh), torch.float32))
        beta, decay = ba[:, :nh], ba[:, nh:]       # the kernel takes rows of any stride
        gate = wide[:, self.channels:]
        out = ctx.buffer("delta.out", (n, nh * self.v_dim), rt.dtype)
        chunk, max_chunks, scratch = 0, 1, None
        if ctx.max_q > CHUNK_TOKENS:
            chunk = CHUNK_TOKENS
            max_chunks = -(-ctx.max_q // chunk)
            scratch = ctx.buffer("delta.scratch", (ops.delta_rule_scratch_floats(ctx.n_seqs, nh, self.head_dim, self.v_dim,
                                                                               max_chunks),), torch.float32)
        ops.delta_rule_recurrence(qkv, decay, self.dt_bias, self.A_log, beta, gate, self.norm, self.eps, self.head_dim ** -0.5,
                                  out, view.state("S"), ctx.seq_slot, ctx.seq_qstart, ctx.n_seqs, ctx.max_q, nh,
                                  self.n_kv_heads, self.head_dim, self.v_dim, rt.status, chunk, max_chunks, scratch,
                                  head_decay=True, gate_silu=True)
        delta = ctx.buffer("delta.delta", (n, self.hidden), rt.dtype)
        rt.linear(out, self.o_proj, out=delta)
        return delta
