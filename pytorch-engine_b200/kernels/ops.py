"""Tensor-level wrappers of the CUDA entry points.  Every op requires CUDA tensors."""
from __future__ import annotations

from typing import Optional

import torch

from .lib import PE_BF16, PE_F32, KernelError, check, library


def dtype_tag(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return PE_F32
    if dtype == torch.bfloat16:
        return PE_BF16
    raise KernelError(f"unsupported dtype {dtype}: the kernels run in float32 or bfloat16")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("the kernels of this package run on CUDA tensors only; got a CPU tensor")
    return t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream's handle (the raw query is several times cheaper than building a
    ``torch.cuda.Stream`` object, and this runs once per launch)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


# How many kernels of this library were launched (a replayed CUDA graph counts its captured kernels
# through ``count_replay``); benchmarks report it.
_LAUNCHES = 0


def _count(n: int = 1) -> None:
    global _LAUNCHES
    _LAUNCHES += n


def launch_count() -> int:
    return _LAUNCHES


def count_replay(n: int) -> None:
    _count(n)


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, status: torch.Tensor, scale: float = 1.0,
                 copy: Optional[torch.Tensor] = None) -> None:
    """``out = table[ids] * scale`` (float32); ``copy`` (float32, the shape of ``out``) gets the same rows."""
    _need(ids.dtype == torch.int32 and out.dtype == torch.float32, "embed_gather: ids int32, out float32")
    _need(table.is_contiguous() and out.is_contiguous() and ids.is_contiguous(), "embed_gather: contiguous tensors")
    _need(copy is None or (copy.dtype == torch.float32 and copy.is_contiguous() and copy.shape == out.shape), "embed_gather: copy")
    n, hidden = out.shape
    check(library().pe_embed_gather_scaled(dtype_tag(table.dtype), _ptr(table), _ptr(ids), _ptr(out), n, hidden,
                                           table.shape[0], float(scale), _ptr(copy), _ptr(status), _stream()), "embed_gather")
    _count(1)


def rmsnorm_residual(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, out: torch.Tensor,
                     eps: float, rows: Optional[torch.Tensor] = None) -> None:
    """``out = rmsnorm(residual (+ delta)) * weight``; see csrc/rmsnorm.cu for the two modes."""
    _need(residual.dtype == torch.float32 and weight.dtype == torch.float32, "rmsnorm: stream and weight float32")
    _need(residual.is_contiguous() and out.is_contiguous(), "rmsnorm: contiguous tensors")
    if delta is not None:
        _need(delta.dtype == out.dtype and delta.is_contiguous() and delta.shape == residual.shape,
              "rmsnorm: delta must match the stream's shape and the output dtype")
    dim = residual.shape[-1]
    n_rows = out.shape[0]
    if rows is not None:
        _need(rows.dtype == torch.int32 and rows.numel() == n_rows, "rmsnorm: rows int32, one per output row")
    else:
        _need(n_rows == residual.shape[0], "rmsnorm: output rows must match the stream")
    check(library().pe_rmsnorm_residual(dtype_tag(out.dtype), _ptr(residual), _ptr(delta), _ptr(weight), _ptr(out),
                                        _ptr(rows), n_rows, dim, float(eps), _stream()), "rmsnorm_residual")
    _count(1)


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float) -> None:
    _need(x.is_contiguous() and out.is_contiguous() and weight.dtype == torch.float32, "rmsnorm: contiguous, weight f32")
    dim = x.shape[-1]
    check(library().pe_rmsnorm(dtype_tag(x.dtype), _ptr(x), _ptr(weight), _ptr(out), x.numel() // dim, dim, float(eps),
                               _stream()), "rmsnorm")
    _count(1)


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    _need(gate_up.is_contiguous() and out.is_contiguous(), "silu_mul: contiguous tensors")
    n, two_i = gate_up.shape
    _need(two_i == 2 * out.shape[1] and out.shape[0] == n and out.dtype == gate_up.dtype, "silu_mul: shapes")
    check(library().pe_silu_mul(dtype_tag(gate_up.dtype), _ptr(gate_up), _ptr(out), n, out.shape[1], _stream()), "silu_mul")
    _count(1)


def batch_expand(seq_qstart: torch.Tensor, seq_past: torch.Tensor, n_seqs: int, token_seq: torch.Tensor,
                 token_pos: torch.Tensor) -> None:
    check(library().pe_batch_expand(_ptr(seq_qstart), _ptr(seq_past), n_seqs, _ptr(token_seq), _ptr(token_pos),
                                    _stream()), "batch_expand")
    _count(1)


def qk_norm_rope_append(qkv: torch.Tensor, n_tokens: int, n_heads: int, n_kv_heads: int, head_dim: int,
                        q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], eps: float,
                        cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rotary_dim: int,
                        token_seq: torch.Tensor, token_pos: torch.Tensor, seq_slot: torch.Tensor,
                        seq_qstart: torch.Tensor, page_table: Optional[torch.Tensor], num_pages: int, k_pages: Optional[torch.Tensor],
                        v_pages: Optional[torch.Tensor], write_cache: bool, status: torch.Tensor) -> None:
    _need(qkv.stride(-1) == 1, "qk_norm_rope_append: rows of qkv must be contiguous")
    table_rows = 0 if cos is None else cos.shape[0]
    check(library().pe_qk_norm_rope_append(
        dtype_tag(qkv.dtype), _ptr(qkv), qkv.stride(0), n_tokens, n_heads, n_kv_heads, head_dim,
        _ptr(q_norm_w), _ptr(k_norm_w), float(eps), _ptr(cos), _ptr(sin), rotary_dim if cos is not None else 0,
        table_rows, _ptr(token_seq), _ptr(token_pos), _ptr(seq_slot), _ptr(seq_qstart), _ptr(page_table),
        0 if page_table is None else page_table.shape[1], num_pages, _ptr(k_pages), _ptr(v_pages),
        1 if write_cache else 0, _ptr(status), _stream()), "qk_norm_rope_append")
    _count(1)


def attention_generic_scratch_floats(n_seqs: int, n_heads: int, head_dim: int, max_splits: int) -> int:
    return int(library().pe_attention_generic_scratch_floats(n_seqs, n_heads, head_dim, max_splits))


def attention_generic(decode: bool, q: torch.Tensor, out: torch.Tensor, n_seqs: int, max_q: int, n_heads: int,
                      n_kv_heads: int, head_dim: int, scale: float, window: int, seq_qstart: torch.Tensor,
                      seq_past: torch.Tensor, seq_slot: torch.Tensor, page_table: torch.Tensor, num_pages: int,
                      k_pages: torch.Tensor, v_pages: torch.Tensor, scratch: Optional[torch.Tensor], split_keys: int,
                      max_splits: int, status: torch.Tensor) -> None:
    _need(q.stride(-1) == 1 and out.stride(-1) == 1, "attention: rows must be contiguous")
    _need(q.dtype == out.dtype == k_pages.dtype, "attention: q, out and the cache must share a dtype")
    check(library().pe_attention_generic(
        dtype_tag(q.dtype), 1 if decode else 0, _ptr(q), q.stride(0), _ptr(out), out.stride(0), n_seqs, max_q,
        n_heads, n_kv_heads, head_dim, float(scale), int(window), _ptr(seq_qstart), _ptr(seq_past), _ptr(seq_slot),
        _ptr(page_table), page_table.shape[1], num_pages, _ptr(k_pages), _ptr(v_pages), _ptr(scratch), split_keys,
        max_splits, _ptr(status), _stream()), "attention_generic")
    _count(2 if decode else 1)


def attention_generic_ex(decode: bool, q: torch.Tensor, out: torch.Tensor, n_seqs: int, max_q: int, n_heads: int,
                         n_kv_heads: int, head_dim: int, v_dim: int, scale: float, window: int, sink: bool,
                         out_cos: Optional[torch.Tensor], out_sin: Optional[torch.Tensor], out_rot: int,
                         out_interleaved: bool, seq_qstart: torch.Tensor, seq_past: torch.Tensor, seq_slot: torch.Tensor,
                         page_table: torch.Tensor, num_pages: int, k_pages: torch.Tensor, v_pages: torch.Tensor,
                         scratch: Optional[torch.Tensor], split_keys: int, max_splits: int, status: torch.Tensor) -> None:
    """``attention_generic`` with values of their own size ``v_dim`` (``out`` rows hold ``n_heads * v_dim``
    features; decode scratch: ``attention_generic_scratch_floats(.., v_dim, ..)``), optionally a sink in the
    softmax (one added to its denominator) and the output of each head turned back by the query's position
    (angle tables ``out_cos, out_sin [rows, out_rot / 2]``, pairs interleaved or split-half)."""
    _need(q.stride(-1) == 1 and out.stride(-1) == 1, "attention: rows must be contiguous")
    _need(q.dtype == out.dtype == k_pages.dtype == v_pages.dtype, "attention: q, out and the cache must share a dtype")
    _need(k_pages.is_contiguous() and v_pages.is_contiguous(), "attention: pages must be contiguous")
    if out_cos is not None:
        _need(out_cos.dtype == torch.float32 and out_sin.dtype == torch.float32 and out_cos.shape == out_sin.shape
              and out_cos.shape[1] * 2 == out_rot and out_cos.is_contiguous() and out_sin.is_contiguous(),
              "attention: the output's angle tables are float32 [rows, out_rot / 2]")
    check(library().pe_attention_generic_ex(
        dtype_tag(q.dtype), 1 if decode else 0, _ptr(q), q.stride(0), _ptr(out), out.stride(0), n_seqs, max_q,
        n_heads, n_kv_heads, head_dim, v_dim, float(scale), int(window), 1 if sink else 0, _ptr(out_cos), _ptr(out_sin),
        int(out_rot) if out_cos is not None else 0, 0 if out_cos is None else out_cos.shape[0],
        1 if out_interleaved else 0, _ptr(seq_qstart), _ptr(seq_past), _ptr(seq_slot), _ptr(page_table),
        page_table.shape[1], num_pages, _ptr(k_pages), _ptr(v_pages), _ptr(scratch), split_keys, max_splits,
        _ptr(status), _stream()), "attention_generic_ex")
    _count(2 if decode else 1)


def qkv_rotate_append(qkv: torch.Tensor, n_tokens: int, n_heads: int, n_kv_heads: int, head_dim: int, v_dim: int,
                      q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], eps: float,
                      cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rotary_dim: int, interleaved: bool,
                      v_unit_norm: bool, v_cos: Optional[torch.Tensor], v_sin: Optional[torch.Tensor], v_rotary_dim: int,
                      v_interleaved: bool, token_seq: torch.Tensor, token_pos: torch.Tensor, seq_slot: torch.Tensor,
                      seq_qstart: torch.Tensor, page_table: Optional[torch.Tensor], num_pages: int,
                      k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor], write_cache: bool,
                      status: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
    """The general form of ``qk_norm_rope_append`` (csrc/rope_append.cu): either layout of rotated pairs, values of
    their own size that may be divided by their root mean square and rotated by their position on the way to the
    cache.  ``qkv`` rows: q heads | k heads | v heads.  ``bias`` (float32, one per q|k|v feature) is added first."""
    _need(qkv.stride(-1) == 1, "qkv_rotate_append: rows of qkv must be contiguous")
    _need(bias is None or bias.numel() == (n_heads + n_kv_heads) * head_dim + n_kv_heads * v_dim, "qkv_rotate_append: bias size")
    for t in (cos, sin, v_cos, v_sin, q_norm_w, k_norm_w, bias):
        _need(t is None or (t.dtype == torch.float32 and t.is_contiguous()), "qkv_rotate_append: float32 tables and weights")
    check(library().pe_qkv_rotate_append(
        dtype_tag(qkv.dtype), _ptr(qkv), qkv.stride(0), n_tokens, n_heads, n_kv_heads, head_dim, v_dim,
        _ptr(q_norm_w), _ptr(k_norm_w), float(eps), _ptr(cos), _ptr(sin), rotary_dim if cos is not None else 0,
        0 if cos is None else cos.shape[0], 1 if interleaved else 0, 1 if v_unit_norm else 0, _ptr(v_cos), _ptr(v_sin),
        v_rotary_dim if v_cos is not None else 0, 0 if v_cos is None else v_cos.shape[0], 1 if v_interleaved else 0,
        _ptr(token_seq), _ptr(token_pos), _ptr(seq_slot), _ptr(seq_qstart), _ptr(page_table),
        0 if page_table is None else page_table.shape[1], num_pages, _ptr(k_pages), _ptr(v_pages),
        1 if write_cache else 0, _ptr(bias), _ptr(status), _stream()), "qkv_rotate_append")
    _count(1)


def rmsnorm_add(stream: torch.Tensor, delta: torch.Tensor, weight: torch.Tensor, eps: float,
                cast: Optional[torch.Tensor] = None) -> None:
    """``stream += delta / rms(delta) * weight`` (float32 stream, in place); ``cast``, if given, gets the new
    stream rows in the run dtype."""
    _need(stream.dtype == torch.float32 and weight.dtype == torch.float32, "rmsnorm_add: stream and weight float32")
    _need(stream.is_contiguous() and delta.is_contiguous() and delta.shape == stream.shape, "rmsnorm_add: shapes")
    if cast is not None:
        _need(cast.dtype == delta.dtype and cast.is_contiguous() and cast.shape == stream.shape, "rmsnorm_add: cast rows")
    n, dim = stream.shape
    check(library().pe_rmsnorm_add(dtype_tag(delta.dtype), _ptr(stream), _ptr(delta), _ptr(weight), _ptr(cast), n, dim,
                                   float(eps), _stream()), "rmsnorm_add")
    _count(1)


def token_gate(gx: torch.Tensor, table: torch.Tensor, col0: int, tokens: torch.Tensor, out: torch.Tensor,
               status: torch.Tensor) -> None:
    """``out[t] = gelu_tanh(gx[t]) * table[tokens[t], col0 : col0 + dim]``."""
    _need(gx.is_contiguous() and out.is_contiguous() and table.stride(1) == 1 and gx.shape == out.shape
          and gx.dtype == out.dtype == table.dtype and tokens.dtype == torch.int32, "token_gate: shapes and dtypes")
    n, dim = gx.shape
    check(library().pe_token_gate(dtype_tag(gx.dtype), _ptr(gx), _ptr(table), table.stride(0), int(col0), _ptr(tokens),
                                  _ptr(out), n, dim, table.shape[0], _ptr(status), _stream()), "token_gate")
    _count(1)


def token_shift_mix(x: torch.Tensor, mu: torch.Tensor, prev_state: torch.Tensor, token_seq: torch.Tensor,
                    seq_slot: torch.Tensor, seq_qstart: torch.Tensor, out: torch.Tensor, status: torch.Tensor) -> None:
    """``out[s, t] = x[t] + (x[t-1] - x[t]) * mu[s]``; a sequence's first token of the step takes
    ``prev_state[slot]`` (float32) for ``x[t-1]``."""
    n, width = x.shape
    _need(x.is_contiguous() and out.is_contiguous() and mu.dtype == torch.float32 and mu.is_contiguous()
          and mu.shape[1] == width and tuple(out.shape) == (mu.shape[0], n, width) and out.dtype == x.dtype
          and prev_state.dtype == torch.float32 and prev_state.is_contiguous() and prev_state.shape[1] == width,
          "token_shift_mix: shapes and dtypes")
    check(library().pe_token_shift_mix(dtype_tag(x.dtype), _ptr(x), _ptr(mu), mu.shape[0], _ptr(prev_state),
                                       _ptr(token_seq), _ptr(seq_slot), _ptr(seq_qstart), _ptr(out), n, width,
                                       prev_state.shape[0], _ptr(status), _stream()), "token_shift_mix")
    _count(1)


def tanh_(y: torch.Tensor) -> None:
    _need(y.is_contiguous(), "tanh_: contiguous")
    check(library().pe_tanh_inplace(dtype_tag(y.dtype), _ptr(y), y.numel(), _stream()), "tanh_")
    _count(1)


def wkv_scratch_floats(n_seqs: int, heads: int, d: int, max_chunks: int) -> int:
    return int(library().pe_wkv_scratch_floats(n_seqs, heads, d, max_chunks))


def wkv_recurrence(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, wlin: torch.Tensor,
                   w0: torch.Tensor, u: torch.Tensor, gnorm: torch.Tensor, eps: float, out: torch.Tensor,
                   state: torch.Tensor, prev_state: torch.Tensor, x: torch.Tensor, seq_slot: torch.Tensor,
                   seq_qstart: torch.Tensor, n_seqs: int, max_q: int, heads: int, d: int, chunk: int = 0,
                   max_chunks: int = 1, scratch: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None) -> None:
    """The recurrence of csrc/wkv.cu over each sequence's tokens of this step, from and to ``state [slots, heads, d,
    d]`` (float32); also leaves each sequence's last row of ``x`` in ``prev_state``.  ``r, k, v, g`` are views with
    one row stride; ``chunk`` > 0 cuts prompts into chunks that run side by side (``scratch``:
    ``wkv_scratch_floats``)."""
    ld = r.stride(0)
    _need(all(t.stride(-1) == 1 and t.stride(0) == ld and t.dtype == r.dtype for t in (r, k, v, g)),
          "wkv_recurrence: r, k, v, g share dtype and row stride")
    _need(wlin.dtype == torch.float32 and wlin.is_contiguous() and out.is_contiguous() and out.dtype == r.dtype
          and x.dtype == r.dtype and x.is_contiguous(), "wkv_recurrence: wlin float32, out and x in the run dtype")
    _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, d, d)
          and prev_state.dtype == torch.float32 and prev_state.is_contiguous(), "wkv_recurrence: state tensors")
    for t in (w0, u, gnorm):
        _need(t.dtype == torch.float32 and t.is_contiguous() and t.numel() == heads * d, "wkv_recurrence: per-channel constants")
    launches = 3 if chunk > 0 else 1
    check(library().pe_wkv_recurrence(
        dtype_tag(r.dtype), _ptr(r), _ptr(k), _ptr(v), _ptr(g), ld, _ptr(wlin), _ptr(w0), _ptr(u), _ptr(gnorm),
        float(eps), _ptr(out), _ptr(state), _ptr(prev_state), _ptr(x), x.shape[1], _ptr(seq_slot), _ptr(seq_qstart),
        n_seqs, max_q, heads, d, state.shape[0], int(chunk), int(max_chunks), _ptr(scratch), _ptr(status), _stream()),
        "wkv_recurrence")
    _count(launches)


def _check_out_tables(out_cos, out_sin, head_dim: int) -> None:
    if out_cos is None and out_sin is None:
        return
    _need(out_cos is not None and out_sin is not None and out_cos.dtype == out_sin.dtype == torch.float32
          and out_cos.is_contiguous() and out_sin.is_contiguous() and out_cos.shape == out_sin.shape
          and out_cos.shape[1] * 2 == head_dim and out_cos.data_ptr() % 16 == 0 and out_sin.data_ptr() % 16 == 0,
          "attention: the output's angle tables are float32 [rows, head_dim / 2], over the whole head")


def attention_mma_supported(dtype: torch.dtype, head_dim: int, n_heads: int, n_kv_heads: int) -> bool:
    """Whether the tensor-core attention kernels (csrc/attention_mma.cu) take this shape."""
    return dtype == torch.bfloat16 and bool(library().pe_attention_mma_supported(head_dim, n_heads, n_kv_heads))


def attention_mma(decode: bool, q: torch.Tensor, out: torch.Tensor, n_seqs: int, max_q: int, n_heads: int,
                  n_kv_heads: int, head_dim: int, scale: float, window: int, seq_qstart: torch.Tensor,
                  seq_past: torch.Tensor, seq_slot: torch.Tensor, page_table: torch.Tensor, num_pages: int,
                  k_pages: torch.Tensor, v_pages: torch.Tensor, scratch: Optional[torch.Tensor], split_keys: int,
                  max_splits: int, status: torch.Tensor, min_range_keys: int = 0, sink: bool = False,
                  out_cos: Optional[torch.Tensor] = None, out_sin: Optional[torch.Tensor] = None) -> None:
    """Same interface as ``attention_generic``, bfloat16 only, head sizes 64 and 128, groups up to 16.
    With ``split_keys`` 0 a sequence's keys are shared out evenly over ``max_splits`` ranges of whole pages,
    each of at least ``min_range_keys`` keys.  ``sink``: one added to the softmax's denominator.  ``out_cos,
    out_sin`` (float32 ``[rows, head_dim / 2]``): each head's output is turned back by the angle of the query's
    position, interleaved pairs over the whole head."""
    _need(q.stride(-1) == 1 and out.stride(-1) == 1, "attention: rows must be contiguous")
    _need(q.dtype == out.dtype == k_pages.dtype == torch.bfloat16, "attention_mma: bfloat16 tensors only")
    _check_out_tables(out_cos, out_sin, head_dim)
    check(library().pe_attention_mma_ex(
        1 if decode else 0, _ptr(q), q.stride(0), _ptr(out), out.stride(0), n_seqs, max_q, n_heads, n_kv_heads,
        head_dim, float(scale), int(window), 1 if sink else 0, _ptr(out_cos), _ptr(out_sin),
        0 if out_cos is None else out_cos.shape[0], _ptr(seq_qstart), _ptr(seq_past), _ptr(seq_slot), _ptr(page_table),
        page_table.shape[1], num_pages, _ptr(k_pages), _ptr(v_pages), _ptr(scratch), split_keys, max_splits,
        int(min_range_keys), _ptr(status), _stream()), "attention_mma")
    _count(2 if decode else 1)


def attention_mma_masked(decode: bool, q: torch.Tensor, out: torch.Tensor, n_seqs: int, max_q: int, n_heads: int,
                         n_kv_heads: int, head_dim: int, scale: float, seq_qstart: torch.Tensor, seq_past: torch.Tensor,
                         seq_slot: torch.Tensor, page_table: torch.Tensor, num_pages: int, k_pages: torch.Tensor,
                         v_pages: torch.Tensor, scratch: Optional[torch.Tensor], split_keys: int, max_splits: int,
                         status: torch.Tensor, min_range_keys: int = 0, window: int = 0, chunk: int = 0,
                         v_heads: Optional[int] = None, split_p: bool = False, keep_first: int = 0) -> None:
    """``attention_mma`` with a chunk mask (``chunk`` > 0: a query sees the keys of its own block of that many positions,
    blocks counted from position 0), kept first keys (``keep_first`` > 0 with a ``window``: positions below it stay visible to
    every later query), ``v_heads`` value heads in ``v_pages`` (kv head g reads value head g % v_heads: several
    key maps over one set of values), an output of bfloat16 or float32 (by ``out``'s dtype) and, with ``split_p``, every
    softmax weight as two bfloat16 terms in the product with the values (16 significant bits instead of 8)."""
    _need(q.stride(-1) == 1 and out.stride(-1) == 1, "attention: rows must be contiguous")
    _need(q.dtype == k_pages.dtype == v_pages.dtype == torch.bfloat16, "attention_mma: bfloat16 inputs only")
    _need(out.dtype in (torch.bfloat16, torch.float32), "attention_mma: out bfloat16 or float32")
    check(library().pe_attention_mma_masked(
        1 if decode else 0, _ptr(q), q.stride(0), _ptr(out), out.stride(0), n_seqs, max_q, n_heads, n_kv_heads, head_dim,
        float(scale), int(window), int(chunk), int(keep_first), int(n_kv_heads if v_heads is None else v_heads),
        1 if out.dtype == torch.float32 else 0, 1 if split_p else 0, 0, None, None, 0, _ptr(seq_qstart), _ptr(seq_past), _ptr(seq_slot),
        _ptr(page_table), page_table.shape[1], num_pages, _ptr(k_pages), _ptr(v_pages), _ptr(scratch), split_keys, max_splits,
        int(min_range_keys), _ptr(status), _stream()), "attention_mma_masked")
    _count(2 if decode else 1)


def attention_latent_supported(dtype: torch.dtype, row: int, rank: int) -> bool:
    """Whether the tensor-core kernels of csrc/attention_latent.cu take cached rows of ``row`` features whose leading
    ``rank`` are the values (bfloat16; rows in steps of 64 up to 576; values of 128, 256 or 512 features)."""
    return dtype == torch.bfloat16 and bool(library().pe_attention_latent_supported(int(row), int(rank)))


def attention_latent_decode_ranges(device: torch.device, n_seqs: int, n_heads: int, max_kv_len: int, split_keys: int) -> tuple:
    """``decode_ranges`` for csrc/attention_latent.cu on this device: one block an SM, a block for every 16 heads."""
    return decode_ranges(sm_count(device), n_seqs * ((n_heads + 15) // 16), max_kv_len, split_keys)


def attention_latent(decode: bool, q: torch.Tensor, out: torch.Tensor, n_seqs: int, max_q: int, n_heads: int, row: int,
                     rank: int, scale: float, seq_qstart: torch.Tensor, seq_past: torch.Tensor, seq_slot: torch.Tensor,
                     page_table: torch.Tensor, num_pages: int, pages: torch.Tensor, scratch: Optional[torch.Tensor],
                     split_keys: int, max_splits: int, status: torch.Tensor, min_range_keys: int = 0) -> None:
    """Causal attention of ``q [n, n_heads * row]`` over the cached rows ``pages [pages, 1, 64, row]`` taken as one kv head
    whose values are the rows' leading ``rank`` features; ``out [n, n_heads * rank]``.  bfloat16, on the tensor cores.
    Decode: ``scratch`` of ``attention_generic_scratch_floats(n_seqs, n_heads, rank, max_splits)`` floats; with
    ``split_keys`` 0 a sequence's keys are shared out evenly over ``max_splits`` ranges of at least ``min_range_keys``."""
    _need(q.stride(-1) == 1 and out.stride(-1) == 1 and pages.is_contiguous(), "attention: rows must be contiguous")
    _need(q.dtype == out.dtype == pages.dtype == torch.bfloat16, "attention_latent: bfloat16 tensors only")
    _need(pages.shape[-1] == row and pages.shape[-2] == 64, "attention_latent: pages of 64 rows of `row` features")
    check(library().pe_attention_latent(
        1 if decode else 0, _ptr(q), q.stride(0), _ptr(out), out.stride(0), n_seqs, max_q, n_heads, row, rank, float(scale),
        _ptr(seq_qstart), _ptr(seq_past), _ptr(seq_slot), _ptr(page_table), page_table.shape[1], num_pages, _ptr(pages),
        _ptr(scratch), split_keys, max_splits, int(min_range_keys), _ptr(status), _stream()), "attention_latent")
    _count(2 if decode else 1)


def gemm_smallm_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether csrc/gemm_smallm.cu takes ``x [M, K] @ weight [N, K]^T``: bfloat16, M <= 16, K % 8 == 0."""
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[0] <= 16
            and x.shape[1] % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and weight.is_contiguous()
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def gemm_smallm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, pair_offset: int = 0) -> None:
    """``out[M, N] = x @ weight^T`` (out bfloat16 or float32).  With ``pair_offset`` = I the weight holds
    gate rows then up rows and ``out[M, I] = silu(x @ gate^T) * (x @ up^T)``."""
    _need(gemm_smallm_supported(x, weight), "gemm_smallm: needs bfloat16, M <= 16, K % 8 == 0, contiguous rows")
    _need(out.stride(-1) == 1 and out.dtype in (torch.bfloat16, torch.float32), "gemm_smallm: out bfloat16 or float32")
    m, k = x.shape
    n = out.shape[1]
    _need(weight.shape[1] == k and weight.shape[0] == (2 * n if pair_offset else n) and out.shape[0] == m,
          "gemm_smallm: shapes do not match")
    _need(pair_offset in (0, n), "gemm_smallm: pair_offset must be 0 or the output width")
    check(library().pe_gemm_smallm(_ptr(x), x.stride(0), _ptr(weight), _ptr(out), out.stride(0), m, n, k,
                                   1 if out.dtype == torch.float32 else 0, pair_offset, sm_count(x.device), _stream()), "gemm_smallm")
    _count(1)


def gemm_smallm_grouped_supported(xs: torch.Tensor, weight: torch.Tensor, group_rows: int) -> bool:
    """Whether csrc/gemm_smallm.cu takes ``xs [G, M, K]`` (any strides of G and M that keep rows on 16-byte boundaries)
    times ``weight [G * group_rows, K]`` in one launch."""
    return (xs.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and xs.dim() == 3 and xs.stride(2) == 1
            and xs.stride(0) % 8 == 0 and xs.stride(1) % 8 == 0
            and weight.is_contiguous() and xs.shape[1] <= 16 and xs.shape[2] % 8 == 0 and group_rows % 16 == 0
            and weight.shape[0] == xs.shape[0] * group_rows and weight.shape[1] == xs.shape[2]
            and xs.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def gemm_smallm_grouped(xs: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, group_rows: int) -> None:
    """``out[:, i * group_rows : (i + 1) * group_rows] = xs[i] @ weight[i * group_rows : (i + 1) * group_rows]^T`` for every
    i, in one launch: several projections, each of an input of its own (bfloat16, at most 16 rows)."""
    _need(gemm_smallm_grouped_supported(xs, weight, group_rows), "gemm_smallm_grouped: shapes, dtypes or alignment")
    g, m, k = xs.shape
    _need(out.shape[0] == m and out.shape[1] == g * group_rows and out.stride(-1) == 1
          and out.dtype in (torch.bfloat16, torch.float32), "gemm_smallm_grouped: out [M, G * group_rows]")
    check(library().pe_gemm_smallm_grouped(_ptr(xs), xs.stride(1), xs.stride(0), g, group_rows, _ptr(weight), _ptr(out), out.stride(0),
                                           m, k, 1 if out.dtype == torch.float32 else 0, sm_count(xs.device), _stream()),
          "gemm_smallm_grouped")
    _count(1)


_SM_COUNT = {}


def sm_count(device) -> int:
    idx = torch.device(device).index or 0
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _SM_COUNT[idx]


def gemm_umma_supported(x: torch.Tensor, weight: torch.Tensor, pair_offset: int = 0) -> bool:
    """Whether csrc/gemm_umma.cu (tcgen05 + TMA) takes ``x [M, K] @ weight^T``: bfloat16, K % 8 == 0."""
    if not (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
            and x.stride(0) % 8 == 0 and weight.is_contiguous() and x.data_ptr() % 16 == 0):
        return False
    n = weight.shape[0] // 2 if pair_offset else weight.shape[0]
    return bool(library().pe_gemm_umma_supported(x.shape[0], n, x.shape[1], pair_offset))


def gemm_umma(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, status: torch.Tensor, pair_offset: int = 0) -> None:
    """``out[M, N] = x @ weight^T`` on the tcgen05 tensor cores (out bfloat16 or float32); with
    ``pair_offset`` = I: ``out[M, I] = silu(x @ gate^T) * (x @ up^T)`` for weight = [gate; up]."""
    _need(gemm_umma_supported(x, weight, pair_offset), "gemm_umma: needs bfloat16, K % 8 == 0, dense weight rows")
    _need(out.stride(-1) == 1 and out.dtype in (torch.bfloat16, torch.float32), "gemm_umma: out bfloat16 or float32")
    m, k = x.shape
    n = out.shape[1]
    _need(weight.shape[1] == k and weight.shape[0] == (2 * n if pair_offset else n) and out.shape[0] == m,
          "gemm_umma: shapes do not match")
    _need(not pair_offset or out.dtype == torch.bfloat16, "gemm_umma: the fused gate writes bfloat16")
    check(library().pe_gemm_umma(_ptr(x), x.stride(0), _ptr(weight), _ptr(out), out.stride(0), m, n, k,
                                 1 if out.dtype == torch.float32 else 0, pair_offset, sm_count(x.device), _ptr(status),
                                 _stream()), "gemm_umma")
    _count(1)


def gemm_umma2_supported(x: torch.Tensor, weight: torch.Tensor, pair_offset: int = 0) -> bool:
    """Whether csrc/gemm_umma2.cu takes the product: as ``gemm_umma_supported``, and K % 64 == 0."""
    if not gemm_umma_supported(x, weight, pair_offset):
        return False
    n = weight.shape[0] // 2 if pair_offset else weight.shape[0]
    return bool(library().pe_gemm_umma2_supported(x.shape[0], n, x.shape[1], pair_offset))


def gemm_umma2(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, status: torch.Tensor, pair_offset: int = 0) -> None:
    """``gemm_umma`` with two SMs per 256 x 256 output tile (csrc/gemm_umma2.cu, tcgen05 cta_group::2)."""
    _need(gemm_umma2_supported(x, weight, pair_offset), "gemm_umma2: needs bfloat16, K % 64 == 0, dense weight rows")
    _need(out.stride(-1) == 1 and out.dtype in (torch.bfloat16, torch.float32), "gemm_umma2: out bfloat16 or float32")
    m, k = x.shape
    n = out.shape[1]
    _need(weight.shape[1] == k and weight.shape[0] == (2 * n if pair_offset else n) and out.shape[0] == m,
          "gemm_umma2: shapes do not match")
    _need(not pair_offset or out.dtype == torch.bfloat16, "gemm_umma2: the fused gate writes bfloat16")
    check(library().pe_gemm_umma2(_ptr(x), x.stride(0), _ptr(weight), _ptr(out), out.stride(0), m, n, k,
                                  1 if out.dtype == torch.float32 else 0, pair_offset, sm_count(x.device), _ptr(status),
                                  _stream()), "gemm_umma2")
    _count(1)


def gemm_umma2_qkv_rope_supported(x: torch.Tensor, weight: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                                  rotary_dim: int) -> bool:
    """Whether the q|k|v projection of this layer can run with q/k-norm, rotation and cache append in its epilogue
    (csrc/gemm_umma2.cu, mode 3): bfloat16, head size 128, the whole head rotated or none of it, K % 64 == 0."""
    if not gemm_umma2_supported(x, weight):
        return False
    return bool(library().pe_gemm_umma2_qkv_rope_supported(x.shape[0], x.shape[1], n_heads, n_kv_heads, head_dim, rotary_dim))


def gemm_umma2_qkv_rope(x: torch.Tensor, weight: torch.Tensor, qkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                        q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], eps: float,
                        cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rotary_dim: int, token_seq: torch.Tensor,
                        token_pos: torch.Tensor, seq_slot: torch.Tensor, seq_qstart: torch.Tensor,
                        page_table: Optional[torch.Tensor], num_pages: int, k_pages: Optional[torch.Tensor],
                        v_pages: Optional[torch.Tensor], write_cache: bool, status: torch.Tensor) -> None:
    """``x @ weight^T`` (the fused q|k|v projection) with what ``qk_norm_rope_append`` does in the product's epilogue:
    ``qkv[:, :n_heads * head_dim]`` gets the normalised, rotated queries; keys and values go to the cache only."""
    _need(gemm_umma2_qkv_rope_supported(x, weight, n_heads, n_kv_heads, head_dim, rotary_dim if cos is not None else 0),
          "gemm_umma2_qkv_rope: needs bfloat16, head size 128, whole-head rotation, K % 64 == 0")
    _need(qkv.dtype == torch.bfloat16 and qkv.stride(-1) == 1 and qkv.shape[0] == x.shape[0], "gemm_umma2_qkv_rope: qkv rows")
    _need(weight.shape[0] == (n_heads + 2 * n_kv_heads) * head_dim, "gemm_umma2_qkv_rope: weight rows")
    m, k = x.shape
    check(library().pe_gemm_umma2_qkv_rope(
        _ptr(x), x.stride(0), _ptr(weight), _ptr(qkv), qkv.stride(0), m, k, n_heads, n_kv_heads, head_dim,
        _ptr(q_norm_w), _ptr(k_norm_w), float(eps), _ptr(cos), _ptr(sin), rotary_dim if cos is not None else 0,
        0 if cos is None else cos.shape[0], _ptr(token_seq), _ptr(token_pos), _ptr(seq_slot), _ptr(seq_qstart),
        _ptr(page_table), 0 if page_table is None else page_table.shape[1], num_pages, _ptr(k_pages), _ptr(v_pages),
        1 if write_cache else 0, sm_count(x.device), _ptr(status), _stream()), "gemm_umma2_qkv_rope")
    _count(1)


def decode_ranges(slots: int, pairs: int, max_kv_len: int, split_keys: int) -> tuple:
    """(split_keys, max_splits, min_range_keys) for a decode attention whose SMs hold ``slots`` blocks at a
    time and that has ``pairs`` (sequence, kv head) pairs; split_keys 0 means that each sequence's keys
    are shared out evenly over max_splits ranges (in whole pages, of at least min_range_keys keys).
    When one wave of blocks can hold at least two ranges per pair, that many ranges are used, but not
    more than ranges of ``split_keys`` keys would give (measured: the blocks of a second, partly filled
    wave cost more than longer ranges do, and more, shorter ranges only add merge work).  With more
    pairs than that there are several waves anyway, and ranges of about four times ``split_keys`` keys
    were measured best (batch 64 at 4,096 keys: 169 us with two ranges, 179 us with eight).  The same
    two sizes are the least a range may have: ``max_kv_len`` is the longest sequence the cache allows,
    and a sequence far shorter than that is not to be cut into as many ranges."""
    pairs = max(1, pairs)
    fixed = max(1, -(-max_kv_len // split_keys))
    per_pair = slots // pairs
    if per_pair < 2:
        return 0, max(1, min(fixed, -(-max_kv_len // (4 * split_keys)))), 4 * split_keys
    return 0, min(per_pair, fixed), split_keys


def attention_mma_decode_ranges(device: torch.device, head_dim: int, n_seqs: int, n_kv_heads: int, max_kv_len: int,
                                split_keys: int) -> tuple:
    """``decode_ranges`` for csrc/attention_mma.cu on this device."""
    slots = sm_count(device) * int(library().pe_attention_mma_decode_blocks_per_sm(head_dim))
    return decode_ranges(slots, n_seqs * n_kv_heads, max_kv_len, split_keys)


def attention_umma_supported(dtype: torch.dtype, head_dim: int, n_heads: int, n_kv_heads: int) -> bool:
    """Whether the tcgen05 prefill attention (csrc/attention_umma.cu) takes this shape."""
    return dtype == torch.bfloat16 and bool(library().pe_attention_umma_supported(head_dim, n_heads, n_kv_heads))


_WORK_COUNTERS = {}


def _work_counter(device: torch.device) -> torch.Tensor:
    """Two zero ints per (device, stream) for kernels that hand out work through a counter; the kernels
    leave them zero.  Launches on one stream run one after the other, so they may share a counter."""
    key = (device.index or 0, _stream())
    t = _WORK_COUNTERS.get(key)
    if t is None:
        t = torch.zeros(2, dtype=torch.int32, device=device)
        _WORK_COUNTERS[key] = t
    return t


def attention_umma_prefill(q: torch.Tensor, out: torch.Tensor, n_seqs: int, max_q: int, n_heads: int, n_kv_heads: int,
                           head_dim: int, scale: float, window: int, seq_qstart: torch.Tensor, seq_past: torch.Tensor,
                           seq_slot: torch.Tensor, page_table: torch.Tensor, num_pages: int, k_pages: torch.Tensor,
                           v_pages: torch.Tensor, status: torch.Tensor, sink: bool = False,
                           out_cos: Optional[torch.Tensor] = None, out_sin: Optional[torch.Tensor] = None) -> None:
    """Prefill attention on tcgen05 (bfloat16, head size 128, groups up to 32); ``q`` holds the step's
    query rows (the first ``n_heads * head_dim`` features of each row of the fused q|k|v buffer).  ``sink``,
    ``out_cos``, ``out_sin``: as for ``attention_mma``."""
    _need(q.stride(-1) == 1 and out.stride(-1) == 1, "attention: rows must be contiguous")
    _need(q.dtype == out.dtype == k_pages.dtype == torch.bfloat16, "attention_umma: bfloat16 tensors only")
    _check_out_tables(out_cos, out_sin, head_dim)
    check(library().pe_attention_umma_prefill_ex(
        _ptr(q), q.stride(0), q.shape[0], _ptr(out), out.stride(0), n_seqs, max_q, n_heads, n_kv_heads, head_dim,
        float(scale), int(window), 1 if sink else 0, _ptr(out_cos), _ptr(out_sin),
        0 if out_cos is None else out_cos.shape[0], _ptr(seq_qstart), _ptr(seq_past), _ptr(seq_slot), _ptr(page_table),
        page_table.shape[1], num_pages, _ptr(k_pages), _ptr(v_pages), sm_count(q.device), _ptr(_work_counter(q.device)), _ptr(status), _stream()),
        "attention_umma_prefill")
    _count(1)


def sample_scratch_bytes(n_rows: int, vocab: int, temperature: float, top_k: int, top_p: float = 1.0,
                         min_p: float = 0.0) -> int:
    """Bytes of scratch with which ``sample`` runs as two kernels (many blocks per row) for these
    settings: greedy, no filter at all, or a small top-k; 0 if it has no such path for them."""
    return int(library().pe_sample_scratch_bytes(int(n_rows), int(vocab), float(temperature), int(top_k),
                                                 float(top_p), float(min_p)))


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, min_p: float, seed: int,
           row_request: torch.Tensor, row_step: torch.Tensor, out_tokens: torch.Tensor,
           scratch: Optional[torch.Tensor] = None) -> None:
    """One token per row.  ``scratch`` (uint8, at least ``sample_scratch_bytes``) lets greedy and small
    top-k draws cut each row into chunks first; the drawn tokens are the same either way except
    where float32 sums in another order move an entry across a top-p threshold."""
    _need(logits.dtype == torch.float32 and logits.stride(-1) == 1, "sample: float32 logits with contiguous rows")
    n, vocab = logits.shape
    two = scratch is not None and scratch.numel() * scratch.element_size() >= max(1, sample_scratch_bytes(n, vocab, temperature, top_k, top_p, min_p))
    check(library().pe_sample(_ptr(logits), logits.stride(0), n, vocab, float(temperature), int(top_k), float(top_p),
                              float(min_p), int(seed) & ((1 << 64) - 1), _ptr(row_request), _ptr(row_step),
                              _ptr(out_tokens), _ptr(scratch) if two else None,
                              scratch.numel() * scratch.element_size() if two else 0, _stream()), "sample")
    _count(2 if two and sample_scratch_bytes(n, vocab, temperature, top_k, top_p, min_p) > 0 else 1)


def repetition_penalty(logits: torch.Tensor, recent: torch.Tensor, recent_count: torch.Tensor, penalty: float) -> None:
    n, vocab = logits.shape
    check(library().pe_repetition_penalty(_ptr(logits), logits.stride(0), n, vocab, _ptr(recent), recent.shape[1],
                                          _ptr(recent_count), float(penalty), _stream()), "repetition_penalty")
    _count(1)


def wait_poll_seconds(device, polls: int = 20000) -> float:
    """Seconds that one poll of an mbarrier takes when the phase it asks for is not complete (csrc/wait_probe.cu):
    ``polls`` polls of a barrier on which nothing arrives, timed on the device."""
    out = torch.zeros(2, dtype=torch.int64, device=device)
    check(library().pe_wait_probe(_ptr(out), int(polls), _stream()), "wait_probe")
    _count(1)
    ns, passed = out.tolist()
    _need(passed == 0, "wait_probe: a poll of a barrier that nothing arrives on passed")
    return ns * 1e-9 / polls


def wait_limit_seconds(device) -> float:
    """The longest that a bounded wait inside a kernel of this library lasts before it gives up."""
    return int(library().pe_wait_limit_polls()) * wait_poll_seconds(device)


# ---- pair embedding, sum of scaled deltas -------------------------------------------------------------------------
def embed_pair_gather(table: torch.Tensor, pairs: torch.Tensor, ids: torch.Tensor, token_seq: torch.Tensor,
                      token_pos: torch.Tensor, seq_slot: torch.Tensor, seq_qstart: torch.Tensor, last: torch.Tensor,
                      out: torch.Tensor, buckets: int, mul_prev: int, mul_cur: int, status: torch.Tensor) -> None:
    """``out[t] = table[tok] + pairs[(prev * mul_prev + tok * mul_cur) % buckets]`` (row ``buckets`` at position 0);
    ``last [slots]`` int32 holds every sequence's last token between steps (csrc/embedding.cu)."""
    _need(ids.dtype == torch.int32 and out.dtype == torch.float32 and last.dtype == torch.int32, "embed_pair_gather: dtypes")
    _need(table.is_contiguous() and pairs.is_contiguous() and out.is_contiguous() and last.is_contiguous(),
          "embed_pair_gather: contiguous tensors")
    _need(pairs.dtype == table.dtype and pairs.shape == (buckets + 1, table.shape[1]), "embed_pair_gather: pair table shape")
    n, hidden = out.shape
    check(library().pe_embed_pair_gather(dtype_tag(table.dtype), _ptr(table), _ptr(pairs), _ptr(ids), _ptr(token_seq),
                                         _ptr(token_pos), _ptr(seq_slot), _ptr(seq_qstart), _ptr(last), _ptr(out), n, hidden,
                                         table.shape[0], int(buckets), int(mul_prev), int(mul_cur), last.numel(),
                                         _ptr(status), _stream()), "embed_pair_gather")
    _count(1)


def rmsnorm_residual_sum(residual: torch.Tensor, deltas, scales, weight: torch.Tensor, out: Optional[torch.Tensor], eps: float,
                         rows: Optional[torch.Tensor] = None) -> None:
    """``h = residual + sum_i scales[i] * deltas[i]``; ``out = rmsnorm(h) * weight`` (``out`` None: the add alone).
    Without ``rows`` the sum is written back to the stream; with ``rows`` only those rows are read and nothing is."""
    import ctypes
    _need(residual.dtype == torch.float32 and weight.dtype == torch.float32 and residual.is_contiguous(), "rmsnorm_sum: stream f32")
    _need(0 <= len(deltas) <= 4 and len(deltas) == len(scales), "rmsnorm_sum: at most four deltas, a scale for each")
    dt = out.dtype if out is not None else (deltas[0].dtype if deltas else torch.float32)
    for d in deltas:
        _need(d.dtype == dt and d.is_contiguous() and d.shape == residual.shape, "rmsnorm_sum: deltas like the stream, in the run dtype")
    dim = residual.shape[-1]
    n_rows = residual.shape[0] if rows is None else rows.numel()
    if out is not None:
        _need(out.is_contiguous() and out.shape[0] == n_rows, "rmsnorm_sum: output rows")
    ptrs = (ctypes.c_void_p * 4)(*[_ptr(d) for d in deltas], *([None] * (4 - len(deltas))))
    sc = (ctypes.c_float * 4)(*[float(x) for x in scales], *([0.0] * (4 - len(scales))))
    check(library().pe_rmsnorm_residual_sum(dtype_tag(dt), _ptr(residual), ptrs, sc, len(deltas), _ptr(weight), _ptr(out),
                                            _ptr(rows), n_rows, dim, float(eps), _stream()), "rmsnorm_residual_sum")
    _count(1)


# ---- recurrences ------------------------------------------------------------------------------------------------------
def mlstm_recurrence(q, k, v, g, gates: torch.Tensor, gate_bias: torch.Tensor, norm_w: torch.Tensor, cap: float, eps: float,
                     q_scale: float, out: torch.Tensor, S: torch.Tensor, n: torch.Tensor, m: torch.Tensor,
                     seq_slot: torch.Tensor, seq_qstart: torch.Tensor, n_seqs: int, max_q: int, heads: int, d: int, dv: int,
                     status: torch.Tensor, chunk: int = 0, max_chunks: int = 1, scratch: Optional[torch.Tensor] = None) -> None:
    """csrc/mlstm.cu.  ``q, k, v, g``: views of one row stride in the run dtype; ``gates [N, 2 * heads]`` float32.
    ``chunk`` > 0: prompts cut into chunks of that many tokens that run side by side (``scratch``: float32,
    ``mlstm_scratch_floats`` of them)."""
    ld = q.stride(0)
    _need(all(t.stride(0) == ld and t.stride(1) == 1 and t.dtype == q.dtype for t in (k, v, g)), "mlstm: q, k, v, g share a row stride")
    _need(gates.dtype == torch.float32 and gates.is_contiguous() and S.dtype == torch.float32 and S.is_contiguous()
          and n.is_contiguous() and m.is_contiguous() and out.is_contiguous() and out.dtype == q.dtype, "mlstm: layouts")
    check(library().pe_mlstm_recurrence(dtype_tag(q.dtype), _ptr(q), _ptr(k), _ptr(v), _ptr(g), ld, _ptr(gates), _ptr(gate_bias),
                                        _ptr(norm_w), float(cap), float(eps), float(q_scale), _ptr(out), _ptr(S), _ptr(n), _ptr(m),
                                        _ptr(seq_slot), _ptr(seq_qstart), n_seqs, int(max_q), heads, d, dv, S.shape[0], int(chunk),
                                        int(max_chunks), _ptr(scratch), _ptr(status), _stream()), "mlstm_recurrence")
    _count(3 if chunk > 0 else 1)


def mlstm_scratch_floats(n_seqs: int, heads: int, d: int, dv: int, max_chunks: int) -> int:
    return int(library().pe_mlstm_scratch_floats(n_seqs, heads, d, dv, max_chunks))


def short_conv_silu(x: torch.Tensor, col0: int, w: torch.Tensor, tail: torch.Tensor, token_seq: torch.Tensor,
                    seq_slot: torch.Tensor, seq_qstart: torch.Tensor, out: torch.Tensor, n_seqs: int, status: torch.Tensor,
                    bias: Optional[torch.Tensor] = None) -> None:
    """Causal convolution over time per channel (plus ``bias``, float32 per channel), then silu; ``tail [slots, taps - 1,
    channels]`` float32 carries every sequence's last inputs between steps and is brought up to date (csrc/delta_rule.cu)."""
    channels, taps = w.shape
    _need(bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == channels), "short_conv: bias")
    _need(w.dtype == torch.float32 and w.is_contiguous() and tail.dtype == torch.float32 and tail.is_contiguous(), "short_conv: w, tail f32")
    _need(x.stride(1) == 1 and out.is_contiguous() and out.shape == (x.shape[0], channels) and out.dtype == x.dtype, "short_conv: shapes")
    _need(taps == 1 or tuple(tail.shape[1:]) == (taps - 1, channels), "short_conv: tail shape")
    check(library().pe_short_conv_silu(dtype_tag(x.dtype), _ptr(x), x.stride(0), int(col0), _ptr(w), _ptr(bias), taps, _ptr(tail),
                                       _ptr(token_seq), _ptr(seq_slot), _ptr(seq_qstart), _ptr(out), x.shape[0], n_seqs, channels,
                                       tail.shape[0] if taps > 1 else (1 << 30), _ptr(status), _stream()), "short_conv_silu")
    _count(2 if taps > 1 else 1)


def delta_rule_recurrence(qkv: torch.Tensor, a: torch.Tensor, dt_bias: torch.Tensor, A_log: torch.Tensor, b: torch.Tensor,
                          gate: torch.Tensor, norm_w: torch.Tensor, eps: float, q_scale: float, out: torch.Tensor,
                          S: torch.Tensor, seq_slot: torch.Tensor, seq_qstart: torch.Tensor, n_seqs: int, max_q: int, heads: int,
                          kv_heads: int, d: int, dv: int, status: torch.Tensor, chunk: int = 0, max_chunks: int = 1,
                          scratch: Optional[torch.Tensor] = None, head_decay: bool = False, gate_silu: bool = False) -> None:
    """csrc/delta_rule.cu.  ``qkv [N, 2 * kv_heads * d + heads * dv]`` after the convolutions; ``a [N, heads * d]`` and
    ``b [N, heads]`` float32 (any row strides); ``gate [N, heads * dv]`` in the run dtype (any row stride).  ``chunk`` > 0: prompts cut into
    chunks of that many tokens that run side by side (``scratch``: float32, ``delta_rule_scratch_floats`` of them).
    ``head_decay``: one decay per head (``a [N, heads]``, ``dt_bias [heads]``); ``gate_silu``: silu instead of sigmoid."""
    _need(a.shape[1] == (heads if head_decay else heads * d) and dt_bias.numel() == a.shape[1], "delta_rule: the decay's layout")
    _need(qkv.is_contiguous() and qkv.shape[1] == 2 * kv_heads * d + heads * dv, "delta_rule: q|k|v layout")
    _need(a.dtype == torch.float32 and a.stride(1) == 1 and b.dtype == torch.float32 and b.stride(1) == 1, "delta_rule: a, b f32")
    _need(gate.stride(1) == 1 and gate.dtype == qkv.dtype and out.is_contiguous() and S.is_contiguous(), "delta_rule: layouts")
    check(library().pe_delta_rule_recurrence(dtype_tag(qkv.dtype), _ptr(qkv), _ptr(a), _ptr(dt_bias), _ptr(A_log), _ptr(b),
                                             _ptr(gate), gate.stride(0), _ptr(norm_w), float(eps), float(q_scale), _ptr(out),
                                             _ptr(S), _ptr(seq_slot), _ptr(seq_qstart), n_seqs, int(max_q), heads, kv_heads, d, dv,
                                             S.shape[0], int(chunk), int(max_chunks), _ptr(scratch), 1 if head_decay else 0,
                                             1 if gate_silu else 0, a.stride(0), b.stride(0), _ptr(status), _stream()),
          "delta_rule_recurrence")
    _count(3 if chunk > 0 else 1)


def delta_rule_scratch_floats(n_seqs: int, heads: int, d: int, dv: int, max_chunks: int) -> int:
    return int(library().pe_delta_rule_scratch_floats(n_seqs, heads, d, dv, max_chunks))


# ---- routed experts ---------------------------------------------------------------------------------------------------
GLU_KINDS = {"silu": 1, "relu": 2, "clamped_swish": 3}


def moe_route(logits: torch.Tensor, correction: torch.Tensor, top: int, chosen: torch.Tensor, weight: torch.Tensor,
              dense_rows: Optional[torch.Tensor] = None, n_real: int = 0) -> None:
    """The router's choice (csrc/moe.cu).  ``dense_rows [N, top]`` int32, if given, gets ``token * n_real + expert`` for a
    chosen real expert and -1 for an identity expert: the row of the pair where every expert ran on every token."""
    _need(logits.dtype == torch.float32 and logits.is_contiguous() and correction.dtype == torch.float32, "moe_route: float32 logits")
    n, n_all = logits.shape
    _need(chosen.dtype == torch.int32 and weight.dtype == torch.float32 and chosen.numel() == n * top == weight.numel(), "moe_route: outputs")
    _need(dense_rows is None or (dense_rows.dtype == torch.int32 and dense_rows.numel() == n * top), "moe_route: dense_rows")
    check(library().pe_moe_route(_ptr(logits), _ptr(correction), n, n_all, int(top), _ptr(chosen), _ptr(weight), _ptr(dense_rows),
                                 int(n_real), _stream()), "moe_route")
    _count(1)


def moe_group(chosen: torch.Tensor, n_tokens: int, top: int, n_real: int, offsets: torch.Tensor, row_token: torch.Tensor,
              pair_row: torch.Tensor) -> None:
    _need(offsets.numel() == n_real + 1 and row_token.numel() >= n_tokens * top and pair_row.numel() == n_tokens * top, "moe_group: sizes")
    check(library().pe_moe_group(_ptr(chosen), n_tokens, int(top), int(n_real), _ptr(offsets), _ptr(row_token), _ptr(pair_row),
                                 _stream()), "moe_group")
    _count(1)


def moe_rows_gemm(x: torch.Tensor, row_map: Optional[torch.Tensor], offsets: torch.Tensor, n_groups: int, max_rows: int,
                  w: torch.Tensor, out: torch.Tensor, glu: int = 0, limit: float = 0.0, alpha: float = 1.0) -> None:
    """``out[r] = w[group of r] @ x[row_map[r]]`` for the rows ``offsets[g] .. offsets[g + 1]`` of every group; ``w [groups,
    n_out (twice with glu), k]``; with ``glu`` the output is act(gate rows, up rows) (csrc/moe.cu)."""
    _need(w.dim() == 3 and w.is_contiguous() and w.dtype == x.dtype and x.stride(1) == 1 and out.stride(1) == 1, "moe_rows_gemm: layouts")
    n_out = w.shape[1] // 2 if glu else w.shape[1]
    _need(out.shape[1] == n_out and x.shape[1] == w.shape[2], "moe_rows_gemm: shapes")
    check(library().pe_moe_rows_gemm(dtype_tag(x.dtype), dtype_tag(out.dtype), _ptr(x), x.stride(0), _ptr(row_map), _ptr(offsets),
                                     int(n_groups), int(max_rows), _ptr(w), w.stride(0), _ptr(out), out.stride(0), n_out, w.shape[2],
                                     int(glu), float(limit), float(alpha), _stream()), "moe_rows_gemm")
    _count(1)


def moe_gather_rows(x: torch.Tensor, row_token: torch.Tensor, offsets: torch.Tensor, n_groups: int, xs: torch.Tensor) -> None:
    """``xs[r] = x[row_token[r]]`` for the rows below ``offsets[n_groups]`` (the rest of ``xs`` is left as it is)."""
    _need(x.is_contiguous() and xs.is_contiguous() and xs.dtype == x.dtype and xs.shape[1] == x.shape[1], "moe_gather_rows: layouts")
    check(library().pe_moe_gather_rows(dtype_tag(x.dtype), _ptr(x), _ptr(row_token), _ptr(offsets), int(n_groups), _ptr(xs),
                                       xs.shape[0], x.shape[1], _stream()), "moe_gather_rows")
    _count(1)


def moe_combine(rows: torch.Tensor, x: torch.Tensor, shared: Optional[torch.Tensor], pair_row: torch.Tensor, weight: torch.Tensor,
                top: int, out: torch.Tensor) -> None:
    _need(x.is_contiguous() and out.is_contiguous() and rows.is_contiguous() and rows.shape[1] == x.shape[1], "moe_combine: layouts")
    _need(shared is None or (shared.is_contiguous() and shared.shape == x.shape), "moe_combine: shared like x")
    check(library().pe_moe_combine(dtype_tag(x.dtype), _ptr(rows), _ptr(x), _ptr(shared), _ptr(pair_row), _ptr(weight), int(top),
                                   _ptr(out), x.shape[0], x.shape[1], _stream()), "moe_combine")
    _count(1)


def glu_act(gate_up: torch.Tensor, out: torch.Tensor, kind: str, limit: float = 0.0, alpha: float = 1.0) -> None:
    """``out = act(gate, up)`` over the halves of ``gate_up [N, 2 * I]``: "silu", "relu", or "clamped_swish"
    (``g' sigmoid(alpha g') (u' + 1)`` with ``g' = min(g, limit)``, ``u' = clamp(u, -limit, limit)``)."""
    _need(gate_up.is_contiguous() and out.is_contiguous() and gate_up.shape[1] == 2 * out.shape[1], "glu_act: shapes")
    check(library().pe_glu_act(dtype_tag(gate_up.dtype), _ptr(gate_up), _ptr(out), out.shape[0], out.shape[1], GLU_KINDS[kind],
                               float(limit), float(alpha), _stream()), "glu_act")
    _count(1)


# ---- parts around the stream, and the other attentions (csrc/stream_parts.cu) ---------------------------------------------
def moe_route_logits(logits: torch.Tensor, bias: Optional[torch.Tensor], top: int, chosen: torch.Tensor, weight: torch.Tensor,
                     dense_rows: Optional[torch.Tensor] = None, n_real: int = 0) -> None:
    """The ``top`` largest of ``logits + bias`` per row, weighted by a softmax over the chosen ones alone (csrc/moe.cu)."""
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "moe_route_logits: float32 logits")
    n, n_all = logits.shape
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == n_all), "moe_route_logits: float32 bias, one per output")
    _need(chosen.dtype == torch.int32 and weight.dtype == torch.float32 and chosen.numel() == n * top == weight.numel(),
          "moe_route_logits: outputs")
    _need(dense_rows is None or (dense_rows.dtype == torch.int32 and dense_rows.numel() == n * top), "moe_route_logits: dense_rows")
    check(library().pe_moe_route_logits(_ptr(logits), _ptr(bias), n, n_all, int(top), _ptr(chosen), _ptr(weight),
                                        _ptr(dense_rows), int(n_real), _stream()), "moe_route_logits")
    _count(1)


def attention_generic_masked(decode: bool, q: torch.Tensor, out: torch.Tensor, n_seqs: int, max_q: int, n_heads: int,
                             n_kv_heads: int, head_dim: int, v_dim: int, scale: float, seq_qstart: torch.Tensor,
                             seq_past: torch.Tensor, seq_slot: torch.Tensor, page_table: torch.Tensor, num_pages: int,
                             k_pages: torch.Tensor, v_pages: torch.Tensor, scratch: Optional[torch.Tensor], split_keys: int,
                             max_splits: int, status: torch.Tensor, *, window: int = 0, chunk: int = 0,
                             v_ld: Optional[int] = None, v_heads: Optional[int] = None, keep_first: int = 0) -> None:
    """``attention_generic_ex`` with a chunk mask (``chunk`` > 0: a query sees the keys of its own block of that many
    positions, blocks counted from the sequence's start), kept first keys (``keep_first`` > 0 with a ``window``: positions
    below it stay visible to every later query), value rows ``v_ld`` elements apart (values that are the leading
    ``v_dim`` features of wider rows) and ``v_heads`` value heads a page (kv head g reads value head ``g % v_heads``)."""
    _need(q.stride(-1) == 1 and out.stride(-1) == 1, "attention: rows must be contiguous")
    _need(q.dtype == k_pages.dtype == v_pages.dtype and out.dtype in (q.dtype, torch.float32),
          "attention: q and the cache must share a dtype; out has it too, or is float32")
    v_ld = v_dim if v_ld is None else int(v_ld)
    v_heads = n_kv_heads if v_heads is None else int(v_heads)
    check(library().pe_attention_generic_masked(
        dtype_tag(q.dtype), 1 if decode else 0, _ptr(q), q.stride(0), _ptr(out), out.stride(0), n_seqs, max_q, n_heads,
        n_kv_heads, head_dim, v_dim, float(scale), int(window), int(chunk), int(keep_first), v_ld, v_heads,
        1 if (out.dtype == torch.float32 and q.dtype != torch.float32) else 0, 0, None, None, 0, 0, 0,
        _ptr(seq_qstart), _ptr(seq_past), _ptr(seq_slot), _ptr(page_table), page_table.shape[1], num_pages, _ptr(k_pages),
        _ptr(v_pages), _ptr(scratch), split_keys, max_splits, _ptr(status), _stream()), "attention_generic_masked")
    _count(2 if decode else 1)


def norm_token_shift(x: torch.Tensor, weight: torch.Tensor, eps: float, mix: torch.Tensor, state: torch.Tensor,
                     token_seq: torch.Tensor, seq_slot: torch.Tensor, seq_qstart: torch.Tensor, out: torch.Tensor,
                     status: torch.Tensor) -> None:
    """``h = rmsnorm(x) * weight`` in float32, ``out[t] = h[t] + (h[t-1] - h[t]) * mix``; a sequence's first token of the
    step takes ``state[slot]`` for ``h[t-1]``, and ``state[slot]`` then keeps the sequence's last ``h`` of the step."""
    n, width = x.shape
    _need(x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and tuple(out.shape) == (n, width)
          and weight.dtype == mix.dtype == state.dtype == torch.float32 and weight.numel() == width == mix.numel()
          and state.is_contiguous() and state.shape[1] == width, "norm_token_shift: shapes and dtypes")
    check(library().pe_norm_token_shift(dtype_tag(out.dtype), _ptr(x), _ptr(weight), float(eps), _ptr(mix), _ptr(state),
                                        _ptr(token_seq), _ptr(seq_slot), _ptr(seq_qstart), _ptr(out), n, width, state.shape[0],
                                        _ptr(status), _stream()), "norm_token_shift")
    _count(1)


def depth_average(results: torch.Tensor, coeff: torch.Tensor, n_terms: int, out: torch.Tensor,
                  copy: Optional[torch.Tensor] = None) -> None:
    """``out = sum_{j < n_terms} coeff[j] * results[j]`` (float32, terms added in order); ``copy`` gets the same rows."""
    _need(results.dtype == torch.float32 and results.is_contiguous() and out.dtype == torch.float32 and out.is_contiguous()
          and coeff.dtype == torch.float32 and coeff.numel() >= n_terms and results.shape[0] >= n_terms
          and results[0].numel() == out.numel(), "depth_average: shapes and dtypes")
    _need(copy is None or (copy.dtype == torch.float32 and copy.is_contiguous() and copy.numel() == out.numel()), "depth_average: copy")
    check(library().pe_depth_average(_ptr(results), results.stride(0), _ptr(coeff), int(n_terms), _ptr(out), _ptr(copy),
                                     out.numel(), _stream()), "depth_average")
    _count(1)


def polynorm(z: torch.Tensor, coeff: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """``coeff[0] N(z) + coeff[1] N(z^2) + coeff[2] N(z^3) + coeff[3]`` with ``N`` the division by a row's root mean square."""
    _need(z.is_contiguous() and out.is_contiguous() and z.shape == out.shape and z.dtype == out.dtype
          and coeff.dtype == torch.float32 and coeff.numel() == 4, "polynorm: shapes and dtypes")
    check(library().pe_polynorm(dtype_tag(z.dtype), _ptr(z), _ptr(coeff), float(eps), _ptr(out), z.shape[0], z.shape[1],
                                _stream()), "polynorm")
    _count(1)


def sigmoid_gate(x: torch.Tensor, g: torch.Tensor, out: torch.Tensor) -> None:
    """``out[t, h, :] = x[h, t, :] * sigmoid(g[t, h])`` when ``g`` has one column a head, ``* sigmoid(g[t, h, :])`` when it has
    one a feature.  ``x [heads, n, dv]`` with any head and token strides (a product over heads leaves one matrix a head; a
    transposed view of packed rows works too); ``out [n, heads * dv]``."""
    heads, n, dv = x.shape
    _need(x.stride(-1) == 1 and g.stride(-1) == 1 and out.stride(-1) == 1 and x.dtype == g.dtype == out.dtype
          and tuple(out.shape) == (n, heads * dv) and g.shape[1] in (heads, heads * dv) and g.shape[0] == n,
          "sigmoid_gate: shapes and dtypes")
    check(library().pe_sigmoid_gate(dtype_tag(x.dtype), _ptr(x), x.stride(0), x.stride(1), _ptr(g), g.stride(0), _ptr(out),
                                    out.stride(0), n, heads, dv, 1 if g.shape[1] == heads and dv != 1 else 0, _stream()),
          "sigmoid_gate")
    _count(1)


def diff_combine(a: torch.Tensor, out: torch.Tensor, heads: int, dv: int, lam: float, eps: float, post: float) -> None:
    """``o = a[:, h] - lam * a[:, heads + h]``; ``out[:, h] = o / sqrt(mean(o^2) + eps) * post``."""
    _need(a.is_contiguous() and out.is_contiguous() and a.dtype == torch.float32 and a.shape[1] == 2 * heads * dv
          and out.shape[1] == heads * dv and a.shape[0] == out.shape[0], "diff_combine: shapes and dtypes")
    check(library().pe_diff_combine(dtype_tag(out.dtype), _ptr(a), _ptr(out), a.shape[0], heads, dv, float(lam), float(eps),
                                    float(post), _stream()), "diff_combine")
    _count(1)


def rows_to_pages(src: torch.Tensor, col0: int, heads: int, dim: int, token_seq: torch.Tensor, token_pos: torch.Tensor,
                  seq_slot: torch.Tensor, page_table: torch.Tensor, num_pages: int, pages: torch.Tensor,
                  status: torch.Tensor) -> None:
    """Columns ``col0 .. col0 + heads * dim`` of every token's row into ``pages [num_pages, heads, 64, dim]`` at the
    token's position in its sequence."""
    _need(src.stride(-1) == 1 and pages.is_contiguous() and src.dtype == pages.dtype and col0 + heads * dim <= src.shape[1],
          "rows_to_pages: shapes and dtypes")
    check(library().pe_rows_to_pages(dtype_tag(src.dtype), _ptr(src), src.stride(0), int(col0), heads, dim, src.shape[0],
                                     _ptr(token_seq), _ptr(token_pos), _ptr(seq_slot), _ptr(page_table), page_table.shape[1],
                                     num_pages, _ptr(pages), _ptr(status), _stream()), "rows_to_pages")
    _count(1)


def rows_to_pages_pair(src: torch.Tensor, col0: int, heads: int, dim: int, pages: torch.Tensor, col0_b: int, heads_b: int,
                        dim_b: int, pages_b: torch.Tensor, token_seq: torch.Tensor, token_pos: torch.Tensor,
                        seq_slot: torch.Tensor, page_table: torch.Tensor, num_pages: int, status: torch.Tensor) -> None:
    """``rows_to_pages`` for two column ranges of the same rows at once (keys and values): the second range goes into
    ``pages_b [num_pages, heads_b, 64, dim_b]``, a pool with the same page numbers."""
    _need(src.stride(-1) == 1 and pages.is_contiguous() and pages_b.is_contiguous()
          and src.dtype == pages.dtype == pages_b.dtype and col0 + heads * dim <= src.shape[1]
          and col0_b + heads_b * dim_b <= src.shape[1] and pages.shape[0] == pages_b.shape[0] == num_pages,
          "rows_to_pages_pair: shapes and dtypes")
    check(library().pe_rows_to_pages_pair(dtype_tag(src.dtype), _ptr(src), src.stride(0), int(col0), heads, dim, int(col0_b),
                                          heads_b, dim_b, src.shape[0], _ptr(token_seq), _ptr(token_pos), _ptr(seq_slot),
                                          _ptr(page_table), page_table.shape[1], num_pages, _ptr(pages), _ptr(pages_b),
                                          _ptr(status), _stream()), "rows_to_pages_pair")
    _count(1)


def latent_prepare(x: torch.Tensor, q_col0: int, low_col0: int, heads: int, d: int, dr: int, rank: int, norm_w: torch.Tensor,
                   eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rot: int, token_seq: torch.Tensor,
                   token_pos: torch.Tensor, seq_slot: torch.Tensor, page_table: torch.Tensor, num_pages: int,
                   pages: torch.Tensor, qfull: torch.Tensor, write_cache: bool, status: torch.Tensor,
                   absorbed: Optional[torch.Tensor] = None) -> None:
    """A latent-attention layer's cached rows ``[normed low-rank row | turned shared key part]`` into their pages, and the
    turned part of every head's query into ``qfull [n, heads, rank + dr]``; ``absorbed [heads, n, rank]``, if given, fills
    the leading features of ``qfull``'s rows (csrc/stream_parts.cu)."""
    _need(absorbed is None or (absorbed.is_contiguous() and absorbed.dtype == x.dtype
                               and tuple(absorbed.shape) == (heads, x.shape[0], rank)), "latent_prepare: absorbed [heads, n, rank]")
    _need(x.stride(-1) == 1 and pages.is_contiguous() and qfull.is_contiguous() and x.dtype == pages.dtype == qfull.dtype
          and norm_w.dtype == torch.float32 and norm_w.numel() == rank, "latent_prepare: shapes and dtypes")
    if rot:
        _need(cos is not None and cos.dtype == torch.float32 and cos.is_contiguous() and cos.shape == sin.shape
              and cos.shape[1] * 2 == rot, "latent_prepare: angle tables float32 [rows, rot / 2]")
    check(library().pe_latent_prepare(dtype_tag(x.dtype), _ptr(x), x.stride(0), int(q_col0), int(low_col0), heads, d, dr, rank,
                                      _ptr(norm_w), float(eps), _ptr(cos) if rot else None, _ptr(sin) if rot else None, int(rot),
                                      cos.shape[0] if rot else 0, x.shape[0], _ptr(token_seq), _ptr(token_pos), _ptr(seq_slot),
                                      _ptr(page_table), page_table.shape[1], num_pages, _ptr(pages), _ptr(qfull), _ptr(absorbed),
                                      1 if write_cache else 0, _ptr(status), _stream()), "latent_prepare")
    _count(1)


def moe_route_sigmoid_groups(logits: torch.Tensor, top: int, n_groups: int, keep: int, chosen: torch.Tensor, weight: torch.Tensor,
                             dense_rows: Optional[torch.Tensor] = None, n_real: int = 0) -> None:
    """Scores ``sigmoid(logits)``; the outputs form ``n_groups`` equal groups of neighbours, a group scores the sum of its two
    largest, only the ``keep`` best groups may be chosen from; the ``top`` largest scores among them, weighted with the score
    itself (csrc/moe.cu).  ``n_groups`` <= 1: no groups."""
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "moe_route_sigmoid_groups: float32 logits")
    n, n_all = logits.shape
    _need(chosen.dtype == torch.int32 and weight.dtype == torch.float32 and chosen.numel() == n * top == weight.numel(),
          "moe_route_sigmoid_groups: outputs")
    _need(dense_rows is None or (dense_rows.dtype == torch.int32 and dense_rows.numel() == n * top), "moe_route_sigmoid_groups: dense_rows")
    check(library().pe_moe_route_sigmoid_groups(_ptr(logits), n, n_all, int(top), int(n_groups), int(keep), _ptr(chosen), _ptr(weight),
                                                _ptr(dense_rows), int(n_real), _stream()), "moe_route_sigmoid_groups")
    _count(1)


# ---- state-space recurrence ---------------------------------------------------------------------------------------------
def ssd_scratch_floats(n_seqs: int, heads: int, n: int, dv: int, max_chunks: int) -> int:
    return int(library().pe_ssd_scratch_floats(n_seqs, heads, n, dv, max_chunks))


def ssd_recurrence(xbc: torch.Tensor, dt: torch.Tensor, dt_bias: torch.Tensor, A_log: torch.Tensor, D: torch.Tensor, y: torch.Tensor,
                   S: torch.Tensor, seq_slot: torch.Tensor, seq_qstart: torch.Tensor, n_seqs: int, max_q: int, heads: int,
                   groups: int, n: int, dv: int, status: torch.Tensor, chunk: int = 0, max_chunks: int = 1,
                   scratch: Optional[torch.Tensor] = None) -> None:
    """csrc/ssd.cu.  ``xbc [N, heads * dv + 2 * groups * n]`` after the convolution (x | B | C, any row stride), ``dt [N, heads]``
    in the run dtype (any row stride), ``y [N, heads * dv]`` float32, ``S [slots, heads, n, dv]`` float32."""
    _need(xbc.stride(1) == 1 and dt.stride(1) == 1 and xbc.dtype == dt.dtype, "ssd: rows of xbc and dt contiguous, one dtype")
    _need(xbc.shape[1] == heads * dv + 2 * groups * n and dt.shape[1] == heads, "ssd: x|B|C and dt layout")
    _need(y.dtype == torch.float32 and y.is_contiguous() and S.dtype == torch.float32 and S.is_contiguous(), "ssd: y, S f32")
    for t in (dt_bias, A_log, D):
        _need(t.dtype == torch.float32 and t.numel() == heads, "ssd: dt_bias, A_log, D float32, one per head")
    check(library().pe_ssd_recurrence(dtype_tag(xbc.dtype), _ptr(xbc), xbc.stride(0), _ptr(dt), dt.stride(0), _ptr(dt_bias),
                                      _ptr(A_log), _ptr(D), _ptr(y), _ptr(S), _ptr(seq_slot), _ptr(seq_qstart), n_seqs, int(max_q),
                                      heads, groups, n, dv, S.shape[0], int(chunk), int(max_chunks), _ptr(scratch), _ptr(status),
                                      _stream()), "ssd_recurrence")
    _count(3 if chunk > 0 else 1)


def gated_part_norm(y: torch.Tensor, z: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor, parts: int) -> None:
    """``v = y * silu(z)``; each of ``parts`` equal parts of a row divided by its root mean square, times ``w`` (csrc/ssd.cu).
    ``y`` float32, ``z`` and ``out`` in the run dtype (``z`` with any row stride)."""
    n, width = y.shape
    _need(y.dtype == torch.float32 and y.is_contiguous() and out.is_contiguous() and z.stride(1) == 1 and z.dtype == out.dtype
          and tuple(out.shape) == (n, width) and tuple(z.shape) == (n, width), "gated_part_norm: shapes and dtypes")
    _need(w.dtype == torch.float32 and w.numel() == width and width % parts == 0, "gated_part_norm: weight, parts")
    check(library().pe_gated_part_norm(dtype_tag(out.dtype), _ptr(y), _ptr(z), z.stride(0), _ptr(w), float(eps), _ptr(out), n,
                                       width, int(parts), _stream()), "gated_part_norm")
    _count(1)


# ---- the norm without statistics ----------------------------------------------------------------------------------------
def dyt(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, alpha: float, out: torch.Tensor,
        rows: Optional[torch.Tensor] = None) -> None:
    """``out = tanh(alpha * x) * w + b`` (csrc/dyt.cu); ``x`` float32 or of ``out``'s dtype; ``rows``: gather those rows of x."""
    n, dim = out.shape
    _need(x.is_contiguous() and out.is_contiguous() and x.shape[1] == dim and x.dtype in (torch.float32, out.dtype), "dyt: shapes")
    _need(w.dtype == torch.float32 and b.dtype == torch.float32 and w.numel() == dim == b.numel(), "dyt: weight and bias float32")
    _need(rows is None or (rows.dtype == torch.int32 and rows.numel() >= n), "dyt: rows int32")
    check(library().pe_dyt(dtype_tag(out.dtype), 1 if x.dtype == torch.float32 else 0, _ptr(x), _ptr(rows), _ptr(w), _ptr(b),
                           float(alpha), _ptr(out), n, dim, _stream()), "dyt")
    _count(1)


def dyt_add(stream: torch.Tensor, delta: torch.Tensor, w: torch.Tensor, b: torch.Tensor, alpha: float,
            next_norm=None, out: Optional[torch.Tensor] = None) -> None:
    """``stream += tanh(alpha * delta) * w + b``; with ``next_norm = (w2, b2, alpha2)`` and ``out``: ``out = tanh(alpha2 *
    stream) * w2 + b2`` of the new rows in the same pass (csrc/dyt.cu)."""
    n, dim = stream.shape
    _need(stream.dtype == torch.float32 and stream.is_contiguous() and delta.is_contiguous() and tuple(delta.shape) == (n, dim),
          "dyt_add: shapes")
    w2 = b2 = None
    a2 = 0.0
    if out is not None:
        w2, b2, a2 = next_norm
        _need(out.dtype == delta.dtype and out.is_contiguous() and tuple(out.shape) == (n, dim), "dyt_add: out")
    check(library().pe_dyt_add(dtype_tag(delta.dtype), _ptr(stream), _ptr(delta), _ptr(w), _ptr(b), float(alpha), _ptr(w2), _ptr(b2),
                               float(a2), _ptr(out), n, dim, _stream()), "dyt_add")
    _count(1)


def rmsnorm_pair_mix(a: torch.Tensor, b: torch.Tensor, wa: torch.Tensor, wb: torch.Tensor, eps: float, sa: float, sb: float,
                     out: torch.Tensor) -> None:
    """``out = sa * unit(a) * wa + sb * unit(b) * wb`` row by row (csrc/dyt.cu)."""
    n, dim = a.shape
    _need(a.is_contiguous() and b.is_contiguous() and out.is_contiguous() and a.shape == b.shape == out.shape
          and a.dtype == b.dtype == out.dtype, "rmsnorm_pair_mix: shapes and dtypes")
    _need(wa.dtype == torch.float32 and wb.dtype == torch.float32 and wa.numel() == dim == wb.numel(), "rmsnorm_pair_mix: weights")
    check(library().pe_rmsnorm_pair_mix(dtype_tag(a.dtype), _ptr(a), _ptr(b), _ptr(wa), _ptr(wb), float(eps), float(sa), float(sb),
                                        _ptr(out), n, dim, _stream()), "rmsnorm_pair_mix")
    _count(1)


def concat_split(a: torch.Tensor, b: torch.Tensor, hi: torch.Tensor, lo: Optional[torch.Tensor]) -> None:
    """``hi = [a | b]`` (two float32 matrices side by side) in ``hi``'s dtype; ``lo``: what that rounding left over, rounded
    likewise, so that ``hi + lo`` holds 16 significant bits of every value (csrc/dyt.cu)."""
    n, dim = a.shape
    _need(a.dtype == torch.float32 and b.dtype == torch.float32 and a.is_contiguous() and b.is_contiguous() and a.shape == b.shape,
          "concat_split: two float32 matrices of one shape")
    _need(hi.is_contiguous() and tuple(hi.shape) == (n, 2 * dim) and (lo is None or (lo.is_contiguous() and lo.shape == hi.shape
                                                                                   and lo.dtype == hi.dtype)), "concat_split: outputs")
    check(library().pe_concat_split(dtype_tag(hi.dtype), _ptr(a), _ptr(b), _ptr(hi), _ptr(lo), n, dim, _stream()), "concat_split")
    _count(1)


def rmsnorm_pair_mix_dyt_add(a: torch.Tensor, b: torch.Tensor, wa: torch.Tensor, wb: torch.Tensor, eps: float, sa: float, sb: float,
                             stream: torch.Tensor, post, next_norm=None, out: Optional[torch.Tensor] = None) -> None:
    """``m = sa * unit(a) * wa + sb * unit(b) * wb``; ``stream += tanh(alpha * m) * w + b`` with ``post = (w, b, alpha)``; with
    ``next_norm = (w2, b2, alpha2)`` and ``out``: ``out = tanh(alpha2 * stream) * w2 + b2`` of the new rows, all in one pass
    (csrc/dyt.cu)."""
    n, dim = a.shape
    _need(a.is_contiguous() and b.is_contiguous() and a.shape == b.shape and a.dtype == b.dtype, "pair_mix_dyt_add: inputs")
    _need(stream.dtype == torch.float32 and stream.is_contiguous() and tuple(stream.shape) == (n, dim), "pair_mix_dyt_add: stream")
    w1, b1, a1 = post
    w2 = b2 = None
    a2 = 0.0
    if out is not None:
        w2, b2, a2 = next_norm
        _need(out.dtype == a.dtype and out.is_contiguous() and tuple(out.shape) == (n, dim), "pair_mix_dyt_add: out")
    check(library().pe_rmsnorm_pair_mix_dyt_add(dtype_tag(a.dtype), _ptr(a), _ptr(b), _ptr(wa), _ptr(wb), float(eps), float(sa),
                                                float(sb), _ptr(stream), _ptr(w1), _ptr(b1), float(a1), _ptr(w2), _ptr(b2), float(a2),
                                                _ptr(out), n, dim, _stream()), "rmsnorm_pair_mix_dyt_add")
    _count(1)
