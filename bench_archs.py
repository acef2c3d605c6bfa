"""``python bench.py --archs``: the Vabelorn, Lunadra and Vemepel architectures beside the Qwen3 dense decoder at equal layer
sizes (``--arch-names`` picks among them; Lunadra's own kernels stand beside the like kernels of the Vabelorn path, Vemepel's
beside those of the Qwen3 path).

Random weights, bfloat16, one B200.  For each size: tokens/s of a 2,048-token prompt and of decode steps at batch 8
(context 2,048) through ``ModelRunner.step``, for both architectures; then the kernels that only the new
architecture has, each beside the like kernel of the Qwen3 path at the same shape, with the bytes each must move
over its time as a fraction of the measured copy bandwidth (MEASURED_PEAKS.json).  Every timed loop works on
weights or buffers larger than L2 or flushes L2 between iterations (``flush`` in the output says which).  One JSON
line at the end; a table on standard error on the way.
"""
import importlib
import json
import math
import sys

SIZES = {
    # width, heads, kv heads, head size, feed-forward, layers, vocabulary, wkv heads x size
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=128, ff=6144, layers=4, vocab=32768, wkv_heads=32, wkv_dim=64),
    "w4096": dict(width=4096, heads=32, kv_heads=8, dim=128, ff=12288, layers=4, vocab=65536, wkv_heads=64, wkv_dim=64),
}
YARN = {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}


def vabelorn_config(pe, s):
    att = {"type": "attention", "mixer": {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"],
                                          "scale": 1.0 / math.sqrt(s["dim"]),
                                          "rot": {"base": 1e6, "dims": s["dim"] // 2, "scaling": YARN}},
           "mlp": {"kind": "dense", "ff": s["ff"]}}
    wkv = {"type": "wkv", "mixer": {"heads": s["wkv_heads"], "dim": s["wkv_dim"], "decay_rank": 64},
           "mlp": {"kind": "dense", "ff": s["ff"]}}
    return pe.VabelornConfig.from_dict({"architecture": "Vabelorn", "vocab": s["vocab"], "width": s["width"], "logit_scale": 1.0,
                                        "norm": {"eps": 1e-6}, "token_side": {"dim": 64},
                                        "layers": [att if i % 2 == 0 else wkv for i in range(s["layers"])]})


def lunadra_config(pe, s):
    """Lunadra at the same width, attention heads, feed-forward and vocabulary: window attention beside a gated delta rule
    (its state as large as the wkv layer's), mlstm layers, a dense feed-forward and routed experts whose two chosen
    experts and shared expert together are as wide as the dense one."""
    side = {"type": "parallel",
            "mixer": {"left": {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"],
                               "scale": 1.0 / math.sqrt(s["dim"]), "mask": {"size": 1024}, "rot": {"base": 1e6, "dims": s["dim"] // 2}},
                      "right": {"heads": s["wkv_heads"] // 4, "kv_heads": s["wkv_heads"] // 8, "dim": 128, "vdim": 128, "conv": 4, "rank": 64},
                      "left_scale": 1.0, "right_scale": 1.0},
            "mlp": {"kind": "dense", "ff": s["ff"]}}
    mem = {"type": "mlstm", "mixer": {"heads": s["width"] // 256, "dim": 128, "vdim": 256, "gate_cap": 15.0},
           "mlp": {"kind": "moe", "router": {"experts": 8, "identity": 2, "top": 2}, "expert": {"ff": s["ff"] // 4, "limit": 7.0},
                   "shared": {"ff": s["ff"] // 2, "limit": 7.0}}}
    return pe.LunadraConfig.from_dict({"architecture": "Lunadra", "vocab": s["vocab"], "width": s["width"], "residual_mult": 1.0,
                                       "norm": {"eps": 1e-6}, "embedding": {"bigram": {"buckets": 65521, "mul_prev": 31, "mul_cur": 7}},
                                       "layers": [side if i % 2 == 0 else mem for i in range(s["layers"])]})


def qwen3_config(pe, s):
    return pe.Qwen3Config.from_dict(dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=s["layers"], hidden_size=s["width"],
                                         num_attention_heads=s["heads"], num_key_value_heads=s["kv_heads"], head_dim=s["dim"],
                                         intermediate_size=s["ff"], vocab_size=s["vocab"], rope_theta=1e6, rms_norm_eps=1e-6,
                                         tie_word_embeddings=True, max_position_embeddings=8192))


def timed(torch, fn, steps, warmup, flush=None, graph=False):
    """Milliseconds per call of ``fn``, CUDA events around each call.  ``graph``: the call is recorded once into a CUDA
    graph and the replays are timed, which leaves the host's time to prepare a launch out of a kernel of a few
    microseconds.  ``flush``: a buffer larger than L2 that is written before every timed call."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    run = fn
    if graph:
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.graph(g, stream=side):
            fn()
        torch.cuda.synchronize()
        run = g.replay
        run()
    total = 0.0
    for _ in range(steps):
        if flush is not None:
            flush.add_(1.0)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / steps


def model_speeds(pe, torch, cfg, prompt, batch, context, steps, warmup):
    """(prompt tokens/s, decode tokens/s, kernels per decode step) through the step function."""
    vocab = cfg.vocab_size
    eng = pe.Engine.from_random(cfg, seed=0, dtype="bfloat16", max_context_len=context + 64,
                                max_cache_tokens=(batch + 1) * (context + 64), max_batch=batch)
    for g in eng.cache.groups:
        for t in (g.storage, g.v_storage):
            if t is not None:
                t.normal_(0.0, 0.5)
    gen = torch.Generator().manual_seed(1)
    toks = torch.randint(0, vocab, (prompt,), generator=gen).tolist()

    def one_prompt():
        s = eng.alloc_slot()
        eng.runner.step([pe.StepEntry(s, toks, (prompt - 1,))], check=False)
        eng.free_slot(s)

    ms_prompt = timed(torch, one_prompt, max(3, steps // 8), 3)
    slots = [eng.alloc_slot() for _ in range(batch)]
    start = context - steps - warmup - 1
    for s in slots:
        eng.cache.reserve(s, start)
        eng.cache.commit(s, start)
    dec = torch.randint(0, vocab, (steps + warmup + 1, batch), generator=gen).tolist()
    it = iter(range(steps + warmup + 1))

    def one_step():
        i = next(it)
        eng.runner.step([pe.StepEntry(s, (dec[i][j],), (0,)) for j, s in enumerate(slots)], check=False)

    one_step()
    ops = pe.kernels.ops
    for _ in range(warmup - 1):
        one_step()
    torch.cuda.synchronize()
    n0 = ops.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        one_step()
    e1.record()
    torch.cuda.synchronize()
    ms_step = e0.elapsed_time(e1) / steps
    launches = (ops.launch_count() - n0) / steps
    eng.runtime.raise_on_status()
    weights = eng.model.weight_bytes()
    del eng
    torch.cuda.empty_cache()
    return {"prompt_tokens_per_s": round(prompt / ms_prompt * 1e3), "prompt_ms": round(ms_prompt, 3),
            "decode_tokens_per_s": round(batch / ms_step * 1e3), "decode_ms_per_step": round(ms_step, 4),
            "kernels_per_decode_step": round(launches, 1), "weight_mib": round(weights / 2 ** 20)}


def kernel_pairs(pe, torch, s, hbm_gbs, prompt, batch, context):
    """The new kernels beside the like kernels of the Qwen3 path at the same shape: microseconds, and the bytes
    each must move over its time as a fraction of the copy bandwidth."""
    ops = pe.kernels.ops
    dev = torch.device("cuda:0")
    bf = torch.bfloat16
    H, G, d, width = s["heads"], s["kv_heads"], s["dim"], s["width"]
    flush = torch.zeros(96 * 2 ** 20, device=dev)            # 384 MB written between iterations: three times L2
    rt = pe.parts.Runtime(dev, bf)
    rope = pe.parts.lookup("position", "rope")
    pos_q = rope({"rotary_dim": d, "theta": 1e6, "max_positions": context + 64}, {}, rt)
    pos_qi = rope({"rotary_dim": d // 2, "theta": 1e6, "max_positions": context + 64, "style": "interleaved", "scaling": YARN}, {}, rt)
    pos_v = rope({"rotary_dim": d, "theta": 1e6, "max_positions": context + 64, "style": "interleaved"}, {}, rt)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    out = {}

    def us_of(fn):
        return 1e3 * timed(torch, fn, 20, 5, flush, graph=True)

    def frac(nbytes, us):
        return round(nbytes / (us * 1e-6) / (hbm_gbs * 1e9), 3)

    def entry(name, us_new, us_like, nbytes, like):
        out[name] = {"us": round(us_new, 2), "of_copy_peak": frac(nbytes, us_new), "like_kernel": like,
                     "like_us": round(us_like, 2), "like_of_copy_peak": frac(nbytes, us_like),
                     "times_as_far_from_roofline": round(us_new / us_like, 2)}

    for what, n_seqs, q_len, past in (("prompt", 1, prompt, 0), ("decode", batch, 1, context - 1)):
        n = n_seqs * q_len
        length = past + q_len
        pages_per = -(-length // 64)
        n_pages = n_seqs * pages_per
        table = torch.arange(n_pages, dtype=torch.int32, device=dev).view(n_seqs, pages_per).contiguous()
        kp = torch.randn(n_pages, G, 64, d, device=dev).to(bf)
        vp = torch.randn(n_pages, G, 64, d, device=dev).to(bf)
        qstart = torch.arange(0, n + 1, q_len, dtype=torch.int32, device=dev)
        pasts = torch.full((n_seqs,), past, dtype=torch.int32, device=dev)
        slots = torch.arange(n_seqs, dtype=torch.int32, device=dev)
        token_seq = torch.arange(n_seqs, dtype=torch.int32, device=dev).repeat_interleave(q_len).contiguous()
        token_pos = (torch.arange(q_len, dtype=torch.int32, device=dev)[None] + past).repeat(n_seqs, 1).view(-1).contiguous()
        qkv = torch.randn(n, (H + 2 * G) * d, device=dev).to(bf)
        qw, kw = torch.ones(d, device=dev), torch.ones(d, device=dev)
        where = (token_seq, token_pos, slots, qstart, table, n_pages, kp, vp)
        cq, sq, _ = pos_q.tables()
        ci, si, ri = pos_qi.tables()
        cv, sv, rv = pos_v.tables()
        # norm + rotation + append
        new = lambda: ops.qkv_rotate_append(qkv, n, H, G, d, d, qw, kw, 1e-6, ci, si, ri, True, True, cv, sv, rv, True, *where, True, status)
        like = lambda: ops.qk_norm_rope_append(qkv, n, H, G, d, qw, kw, 1e-6, cq, sq, d, *where, True, status)
        nbytes = n * (H + 2 * G) * d * 2 + n * (H + G) * d * 2 + n * 2 * G * d * 2        # rows in, q and k back, k and v to the cache
        entry(f"{what}: q/k/v norm, rotation, append", us_of(new), us_of(like), nbytes,
              "qk_norm_rope_append")
        # attention
        o = torch.empty(n, H * d, dtype=bf, device=dev)
        nbytes = n * H * d * 2 * 2 + n_seqs * length * 2 * G * d * 2
        if what == "prompt":
            new = lambda: ops.attention_umma_prefill(qkv, o, n_seqs, q_len, H, G, d, 0.088, 0, qstart, pasts, slots, table, n_pages, kp, vp,
                                                     status, sink=True, out_cos=cv, out_sin=sv)
            like = lambda: ops.attention_umma_prefill(qkv, o, n_seqs, q_len, H, G, d, 0.088, 0, qstart, pasts, slots, table, n_pages, kp, vp, status)
            name = "attention_umma_prefill"
        else:
            sk, ms, fl = ops.attention_mma_decode_ranges(dev, d, n_seqs, G, context + 64, 512)
            scratch = torch.empty(ops.attention_generic_scratch_floats(n_seqs, H, d, ms), device=dev)
            new = lambda: ops.attention_mma(True, qkv, o, n_seqs, 1, H, G, d, 0.088, 0, qstart, pasts, slots, table, n_pages, kp, vp, scratch,
                                            sk, ms, status, min_range_keys=fl, sink=True, out_cos=cv, out_sin=sv)
            like = lambda: ops.attention_mma(True, qkv, o, n_seqs, 1, H, G, d, 0.088, 0, qstart, pasts, slots, table, n_pages, kp, vp, scratch,
                                             sk, ms, status, min_range_keys=fl)
            name = "attention_mma (split + merge)"
        entry(f"{what}: attention with sink, outputs turned back", us_of(new), us_of(like), nbytes, name)
        # norm on the sublayer's output, then the add
        stream = torch.randn(n, width, device=dev)
        delta = torch.randn(n, width, device=dev).to(bf)
        w = torch.ones(width, device=dev)
        cast = torch.empty(n, width, dtype=bf, device=dev)
        new = lambda: ops.rmsnorm_add(stream, delta, w, 1e-6, cast)
        like = lambda: ops.rmsnorm_residual(stream, delta, w, cast, 1e-6)
        entry(f"{what}: norm of the output, add, copy in bfloat16", us_of(new), us_of(like),
              n * width * (4 + 4 + 2 + 2), "rmsnorm_residual")
        # the recurrence: no like kernel in the Qwen3 path; held against the bytes it must move
        WH, wd = s["wkv_heads"], s["wkv_dim"]
        hd = WH * wd
        r, k, v, g = (torch.randn(n, hd, device=dev).to(bf) for _ in range(4))
        k.mul_(0.3)
        wlin = torch.randn(n, hd, device=dev)
        w0, u, gn = torch.zeros(hd, device=dev), torch.zeros(hd, device=dev), torch.ones(hd, device=dev)
        res = torch.empty(n, hd, dtype=bf, device=dev)
        state = torch.zeros(n_seqs, WH, wd, wd, device=dev)
        prev = torch.zeros(n_seqs, width, device=dev)
        x = torch.randn(n, width, device=dev).to(bf)
        chunk, max_chunks, scratch = 0, 1, None
        if q_len > 128:
            chunk, max_chunks = 64, -(-q_len // 64)
            scratch = torch.empty(ops.wkv_scratch_floats(n_seqs, WH, wd, max_chunks), device=dev)
        new = lambda: ops.wkv_recurrence(r, k, v, g, wlin, w0, u, gn, 1e-6, res, state, prev, x, slots, qstart, n_seqs, q_len, WH, wd,
                                         chunk, max_chunks, scratch, status)
        us = us_of(new)
        nbytes = n * hd * (4 * 2 + 4 + 2) + n_seqs * WH * wd * wd * 4 * 2
        flops = n * WH * wd * wd * 5 * (2 if chunk else 1)
        out[f"{what}: wkv recurrence, head norm, gate"] = {"us": round(us, 2), "of_copy_peak": frac(nbytes, us), "like_kernel": None,
                                                           "float32_gflops": round(flops / us / 1e3, 1)}
        mixes = torch.empty(5, n, width, dtype=bf, device=dev)
        mu = torch.rand(5, width, device=dev)
        new = lambda: ops.token_shift_mix(x, mu, prev, token_seq, slots, qstart, mixes, status)
        us = us_of(new)
        out[f"{what}: token shift, five mixes"] = {"us": round(us, 2), "of_copy_peak": frac(n * width * 2 * 6, us), "like_kernel": None}
    return out


FP32_TFLOPS = 148 * 128 * 2 * 1.9e9 / 1e12      # float32 multiply-adds of the CUDA cores, for the recurrences' rooflines


def lunadra_kernel_pairs(pe, torch, s, hbm_gbs, prompt, batch, context):
    """The kernels that only Lunadra has, each beside the like kernel of the Vabelorn path at the same shape.  A kernel's
    roofline time is the larger of its bytes over the copy bandwidth and its float32 operations over the CUDA cores'
    rate; ``times_as_far_from_roofline`` divides the new kernel's distance from its roofline by the like kernel's."""
    ops = pe.kernels.ops
    dev = torch.device("cuda:0")
    bf = torch.bfloat16
    width = s["width"]
    flush = torch.zeros(96 * 2 ** 20, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    out = {}

    def us_of(fn):
        return 1e3 * timed(torch, fn, 20, 5, flush, graph=True)

    def roof_us(nbytes, flops=0.0):
        return max(nbytes / (hbm_gbs * 1e9), flops / (FP32_TFLOPS * 1e12)) * 1e6

    def entry(name, us_new, roof_new, like, us_like, roof_like):
        out[name] = {"us": round(us_new, 2), "roofline_us": round(roof_new, 2), "of_roofline": round(roof_new / us_new, 3)}
        if like:
            out[name].update({"like_kernel": like, "like_us": round(us_like, 2), "like_of_roofline": round(roof_like / us_like, 3),
                              "times_as_far_from_roofline": round((us_new / roof_new) / (us_like / roof_like), 2)})

    for what, n_seqs, q_len in (("prompt", 1, prompt), ("decode", batch, 1)):
        n = n_seqs * q_len
        qstart = torch.arange(0, n + 1, q_len, dtype=torch.int32, device=dev)
        slots = torch.arange(n_seqs, dtype=torch.int32, device=dev)
        token_seq = torch.arange(n_seqs, dtype=torch.int32, device=dev).repeat_interleave(q_len).contiguous()
        token_pos = torch.arange(q_len, dtype=torch.int32, device=dev).repeat(n_seqs).contiguous() + (0 if q_len > 1 else 5)
        chunked = q_len > 128
        dchunk = 128 if chunked else 0
        max_chunks = -(-q_len // 64) if chunked else 1
        # the like kernel: the wkv recurrence at its own shape (state heads x 64 x 64)
        WH, wd = s["wkv_heads"], s["wkv_dim"]
        hd = WH * wd
        r, k, v, g = (torch.randn(n, hd, device=dev).to(bf) for _ in range(4))
        k.mul_(0.3)
        wlin = torch.randn(n, hd, device=dev)
        w0, u, gn = torch.zeros(hd, device=dev), torch.zeros(hd, device=dev), torch.ones(hd, device=dev)
        res = torch.empty(n, hd, dtype=bf, device=dev)
        state = torch.zeros(n_seqs, WH, wd, wd, device=dev)
        prev = torch.zeros(n_seqs, width, device=dev)
        x = torch.randn(n, width, device=dev).to(bf)
        scratch = torch.empty(ops.wkv_scratch_floats(n_seqs, WH, wd, max_chunks), device=dev) if chunked else None
        us_wkv = us_of(lambda: ops.wkv_recurrence(r, k, v, g, wlin, w0, u, gn, 1e-6, res, state, prev, x, slots, qstart, n_seqs, q_len,
                                                  WH, wd, 64 if chunked else 0, max_chunks, scratch, status))
        roof_wkv = roof_us(n * hd * (4 * 2 + 4 + 2) + n_seqs * WH * wd * wd * 8, n * WH * wd * wd * 5.0)
        # mlstm
        H, d, dv = width // 256, 128, 256
        qk, vv = H * d, H * dv
        qkvg = (torch.randn(n, 2 * qk + 2 * vv, device=dev) * 0.5).to(bf)
        gates = torch.randn(n, 2 * H, device=dev)
        gbias, nw = torch.zeros(2 * H, device=dev), torch.ones(vv, device=dev)
        o = torch.empty(n, vv, dtype=bf, device=dev)
        S, nn, mm = torch.zeros(n_seqs, H, d, dv, device=dev), torch.zeros(n_seqs, H, d, device=dev), torch.zeros(n_seqs, H, device=dev)
        scratch_m = torch.empty(ops.mlstm_scratch_floats(n_seqs, H, d, dv, max_chunks), device=dev) if chunked else None
        us = us_of(lambda: ops.mlstm_recurrence(qkvg[:, :qk], qkvg[:, qk:2 * qk], qkvg[:, 2 * qk:2 * qk + vv], qkvg[:, 2 * qk + vv:], gates,
                                                gbias, nw, 15.0, 1e-6, d ** -0.5, o, S, nn, mm, slots, qstart, n_seqs, q_len, H, d, dv,
                                                status, 64 if chunked else 0, max_chunks, scratch_m))
        entry(f"{what}: mlstm recurrence, head norm, gate", us, roof_us(n * (2 * qk + 3 * vv) * 2 + n_seqs * H * d * dv * 8, n * H * d * dv * 5.0),
              "wkv_recurrence", us_wkv, roof_wkv)
        # gated delta rule
        DH, DG, dd, ddv = s["wkv_heads"] // 4, s["wkv_heads"] // 8, 128, 128
        ch = 2 * DG * dd + DH * ddv
        qkv = (torch.randn(n, ch, device=dev) * 0.5).to(bf)
        a_lin, beta = torch.randn(n, DH * dd, device=dev), torch.randn(n, DH, device=dev)
        dtb, alog, nw2 = torch.zeros(DH * dd, device=dev), torch.zeros(DH, device=dev), torch.ones(ddv, device=dev)
        gate = torch.randn(n, DH * ddv, device=dev).to(bf)
        o2 = torch.empty(n, DH * ddv, dtype=bf, device=dev)
        S2 = torch.zeros(n_seqs, DH, dd, ddv, device=dev)
        dmax = -(-q_len // 128) if chunked else 1
        scratch_d = torch.empty(ops.delta_rule_scratch_floats(n_seqs, DH, dd, ddv, dmax), device=dev) if chunked else None
        us = us_of(lambda: ops.delta_rule_recurrence(qkv, a_lin, dtb, alog, beta, gate, nw2, 1e-6, dd ** -0.5, o2, S2, slots, qstart, n_seqs,
                                                     q_len, DH, DG, dd, ddv, status, dchunk, dmax, scratch_d))
        entry(f"{what}: gated delta recurrence, head norm, gate", us,
              roof_us(n * (ch * 2 + DH * dd * 4 + DH * ddv * 4) + n_seqs * DH * dd * ddv * 8, n * DH * dd * ddv * 7.0),
              "wkv_recurrence", us_wkv, roof_wkv)
        # short convolutions beside the token shift (both: a token's row with the rows before it, kept inputs at the start)
        wide = torch.randn(n, ch + 128, device=dev).to(bf)
        cw = torch.randn(ch, 4, device=dev)
        tail = torch.zeros(n_seqs, 3, ch, device=dev)
        co = torch.empty(n, ch, dtype=bf, device=dev)
        us = us_of(lambda: ops.short_conv_silu(wide, 0, cw, tail, token_seq, slots, qstart, co, n_seqs, status))
        mixes = torch.empty(5, n, width, dtype=bf, device=dev)
        mu = torch.rand(5, width, device=dev)
        us_like = us_of(lambda: ops.token_shift_mix(x, mu, prev, token_seq, slots, qstart, mixes, status))
        entry(f"{what}: short convolutions, silu, kept inputs", us, roof_us(n * ch * 4), "token_shift_mix", us_like, roof_us(n * width * 12))
        # the add of three scaled outputs in the norm beside the add of one
        stream = torch.randn(n, width, device=dev)
        deltas = [torch.randn(n, width, device=dev).to(bf) for _ in range(3)]
        w = torch.ones(width, device=dev)
        normed = torch.empty(n, width, dtype=bf, device=dev)
        us = us_of(lambda: ops.rmsnorm_residual_sum(stream, deltas, [1.0, 0.5, 0.7], w, normed, 1e-6))
        us_like = us_of(lambda: ops.rmsnorm_residual(stream, deltas[0], w, normed, 1e-6))
        entry(f"{what}: add of three scaled outputs, norm", us, roof_us(n * width * (8 + 6 + 2)), "rmsnorm_residual", us_like,
              roof_us(n * width * (8 + 2 + 2)))
        # embedding with the pair table beside the plain gather
        table = torch.randn(s["vocab"], width, device=dev).to(bf)
        pairs = torch.randn(65522, width, device=dev).to(bf)
        ids = torch.randint(0, s["vocab"], (n,), dtype=torch.int32, device=dev)
        last = torch.zeros(n_seqs, dtype=torch.int32, device=dev)
        emb = torch.empty(n, width, device=dev)
        us = us_of(lambda: ops.embed_pair_gather(table, pairs, ids, token_seq, token_pos, slots, qstart, last, emb, 65521, 31, 7, status))
        us_like = us_of(lambda: ops.embed_gather(table, ids, emb, status))
        entry(f"{what}: token and pair embedding", us, roof_us(n * width * 8), "embed_gather", us_like, roof_us(n * width * 6))
        # routed experts: routing and grouping, then the experts' products
        E, top, ff = 8, 2, s["ff"] // 4
        logits = torch.randn(n, E + 2, device=dev)
        corr = torch.zeros(E + 2, device=dev)
        chosen = torch.empty(n, top, dtype=torch.int32, device=dev)
        weight = torch.empty(n, top, device=dev)
        offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
        row_token = torch.empty(n * top, dtype=torch.int32, device=dev)
        pair_row = torch.empty(n, top, dtype=torch.int32, device=dev)

        def route():
            ops.moe_route(logits, corr, top, chosen, weight)
            ops.moe_group(chosen, n, top, E, offsets, row_token, pair_row)
        entry(f"{what}: router softmax, choice, grouping (2 kernels)", us_of(route), roof_us(n * (E + 2) * 4 + n * top * 16), None, 0, 0)
        gate_up = (torch.randn(E, 2 * ff, width, device=dev) * 0.02).to(bf)
        act = torch.empty(n * top, ff, dtype=bf, device=dev)
        route()
        if what == "decode":
            # what a decode step runs: every expert on every row through the weight-streaming product, then the activation
            stacked = gate_up.view(E * 2 * ff, width)
            gu = torch.empty(n, E * 2 * ff, dtype=bf, device=dev)
            act_all = torch.empty(n * E, ff, dtype=bf, device=dev)

            def every_expert():
                ops.gemm_smallm(x, stacked, gu)
                ops.glu_act(gu.view(n * E, 2 * ff), act_all, "clamped_swish", 7.0, 1.702)
            us = us_of(every_expert)
            act2 = torch.empty(n, E * ff, dtype=bf, device=dev)
            us_like = us_of(lambda: ops.gemm_smallm(x, stacked, act2, pair_offset=E * ff))
            nbytes = E * 2 * ff * width * 2
            entry("decode: experts' gate|up product, then the activation (2 kernels; every expert's weights once)", us, roof_us(nbytes),
                  "gemm_smallm with SiLU epilogue, same matrix", us_like, roof_us(nbytes))
            # the row-group kernel, which runs instead where the pairs are far fewer than the experts and in float32
            us = us_of(lambda: ops.moe_rows_gemm(x, row_token, offsets, E, n * top, gate_up, act, 3, 7.0, 1.702))
            entry("decode: the same through the row-group kernel (not what a step of this size runs)", us, roof_us(nbytes),
                  "gemm_smallm with SiLU epilogue, same matrix", us_like, roof_us(nbytes))
        else:
            xs = torch.empty(n * top, width, dtype=bf, device=dev)

            def experts():
                ops.moe_gather_rows(x, row_token, offsets, E, xs)
                gu = torch._grouped_mm(xs, gate_up.transpose(1, 2), offs=offsets[1:], out_dtype=bf)
                ops.glu_act(gu, act, "clamped_swish", 7.0, 1.702)
            us = us_of(experts)
            out["prompt: experts' rows gathered, library product over row groups, activation"] = {
                "us": round(us, 2), "tflops": round(2.0 * n * top * 0.8 * 2 * ff * width / us / 1e6, 1), "like_kernel": "library product"}
        rows = torch.randn(n * top, width, device=dev).to(bf)
        shared = torch.randn(n, width, device=dev).to(bf)
        y = torch.empty(n, width, dtype=bf, device=dev)
        us = us_of(lambda: ops.moe_combine(rows, x, shared, pair_row, weight, top, y))
        entry(f"{what}: weighted sum of the chosen experts and the shared one", us, roof_us(n * width * 2 * (top + 3)), None, 0, 0)
    return out


def vemepel_config(pe, s):
    """Vemepel at the same width, heads and vocabulary: latent attention (a cached row of 512 + 64 features) and
    differential attention (two maps of the head size over shared values, a chunk of 1,024 positions, the second such
    layer reading the first one's keys), a PolyNorm feed-forward of two matrices as large as the gated one's three, and
    routed experts whose two chosen ones together are as wide as the dense one."""
    d = s["dim"]
    lat = lambda kind: {"type": kind, "mixer": dict({"heads": s["heads"], "dim": d, "vdim": d, "kv_rank": 4 * d, "scale": (1.5 * d) ** -0.5},
                                                   **({"rot_dim": d // 2, "rot": {"base": 1e6, "dims": d // 2}} if kind.endswith("_2") else {}))}
    dif = lambda src: {"type": "attention", "mixer": dict({"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": d, "vdim": d,
                                                           "scale": d ** -0.5, "diff": 0.5, "mask": {"size": 1024}},
                                                          **({"kv_from": src} if src is not None else {}))}
    dense = {"kind": "dense", "ff": s["ff"] * 3 // 2}
    moe = {"kind": "moe", "router": {"experts": 8, "top": 2}, "expert": {"ff": s["ff"] // 2}}
    pattern = [dict(lat("latent_attention_2"), mlp=dense), dict(dif(None), mlp=moe), dict(lat("latent_attention"), mlp=dense),
               dict(dif(1), mlp=moe)]
    layers = []
    for i in range(s["layers"]):
        layer = dict(pattern[i % 4])
        if "kv_from" in layer["mixer"]:
            layer["mixer"] = dict(layer["mixer"], kv_from=i - 2)
        layers.append(layer)
    return pe.VemepelConfig.from_dict({"architecture": "Vemepel", "vocab": s["vocab"], "width": s["width"], "logit_scale": 1.0,
                                       "norm": {"eps": 1e-6}, "layers": layers})


def vemepel_kernel_pairs(pe, torch, s, peaks, prompt, batch, context):
    """The kernels that only Vemepel has, each beside the like kernel of the Qwen3 path at the same shape.  A kernel's
    roofline time is the larger of its bytes over the copy bandwidth and, for the attentions, its tensor-core operations
    over the library product's rate; ``times_as_far_from_roofline`` divides the new kernel's distance from its roofline by
    the like kernel's."""
    ops = pe.kernels.ops
    dev = torch.device("cuda:0")
    bf = torch.bfloat16
    hbm_gbs, tflops = peaks["hbm_gbs"], peaks.get("bf16_tflops") or 1590.0
    H, G, d, width, ff = s["heads"], s["kv_heads"], s["dim"], s["width"], s["ff"]
    rank, dr = 4 * d, d // 2
    row = rank + dr
    flush = torch.zeros(96 * 2 ** 20, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    out = {}

    held = {}

    def buffer(name, shape, dtype):
        key = (name, tuple(shape), dtype)
        if key not in held:
            held[key] = torch.empty(shape, dtype=dtype, device=dev)
        return held[key]

    def us_of(fn):
        return 1e3 * timed(torch, fn, 20, 5, flush, graph=True)

    def roof_us(nbytes, flops=0.0):
        return max(nbytes / (hbm_gbs * 1e9), flops / (tflops * 1e12)) * 1e6

    def entry(name, us_new, roof_new, like, us_like, roof_like):
        out[name] = {"us": round(us_new, 2), "roofline_us": round(roof_new, 2), "of_roofline": round(roof_new / us_new, 3)}
        if like:
            out[name].update({"like_kernel": like, "like_us": round(us_like, 2), "like_of_roofline": round(roof_like / us_like, 3),
                              "times_as_far_from_roofline": round((us_new / roof_new) / (us_like / roof_like), 2)})

    for what, n_seqs, q_len, past in (("prompt", 1, prompt, 0), ("decode", batch, 1, context - 1)):
        n = n_seqs * q_len
        decode = q_len == 1
        length = past + q_len
        pages_per = -(-length // 64)
        n_pages = n_seqs * pages_per
        table = torch.arange(n_pages, dtype=torch.int32, device=dev).view(n_seqs, pages_per).contiguous()
        qstart = torch.arange(0, n + 1, q_len, dtype=torch.int32, device=dev)
        pasts = torch.full((n_seqs,), past, dtype=torch.int32, device=dev)
        slots = torch.arange(n_seqs, dtype=torch.int32, device=dev)
        token_seq = torch.arange(n_seqs, dtype=torch.int32, device=dev).repeat_interleave(q_len).contiguous()
        token_pos = (torch.arange(q_len, dtype=torch.int32, device=dev)[None] + past).repeat(n_seqs, 1).view(-1).contiguous()
        where = (qstart, pasts, slots, table, n_pages)
        pairs = n_seqs * (q_len * (q_len + 1) / 2 + q_len * past)        # (query, visible key) pairs without a chunk mask
        # ---- the like kernels: the Qwen3 path's attention at its own shape
        kp = torch.randn(n_pages, G, 64, d, device=dev).to(bf)
        vp = torch.randn(n_pages, G, 64, d, device=dev).to(bf)
        qkv = torch.randn(n, (H + 2 * G) * d, device=dev).to(bf)
        o = torch.empty(n, H * d, dtype=bf, device=dev)
        if decode:
            sk, ms, fl = ops.attention_mma_decode_ranges(dev, d, n_seqs, G, context + 64, 512)
            scratch = torch.empty(ops.attention_generic_scratch_floats(n_seqs, H, d, ms), device=dev)
            like_att = "attention_mma (split + merge)"
            us_att = us_of(lambda: ops.attention_mma(True, qkv, o, n_seqs, 1, H, G, d, 0.088, 0, *where, kp, vp, scratch, sk, ms, status,
                                                     min_range_keys=fl))
        else:
            like_att = "attention_umma_prefill"
            us_att = us_of(lambda: ops.attention_umma_prefill(qkv, o, n_seqs, q_len, H, G, d, 0.088, 0, *where, kp, vp, status))
        roof_att = roof_us(n * H * d * 4 + n_seqs * length * 2 * G * d * 2, pairs * H * d * 4.0)
        # ---- differential attention: 2H query maps over 2G key heads and G value heads, a chunk of 1,024 positions
        chunk = 1024
        kp2 = torch.randn(n_pages, 2 * G, 64, d, device=dev).to(bf)
        q2 = torch.randn(n, 2 * H * d, device=dev).to(bf)
        maps = torch.empty(n, 2 * H * d, device=dev)
        new = pe.parts.diff_attention.attend_maps
        seen = min(length, chunk) if decode else None
        dpairs = n_seqs * seen if decode else sum(min(chunk, q_len - c) * (min(chunk, q_len - c) + 1) / 2 for c in range(0, q_len, chunk))
        keys_read = n_seqs * (seen if decode else length)
        us = us_of(lambda: new(ops, decode, q2, maps, n_seqs, q_len, H, G, d, d, d ** -0.5, chunk, *where, kp2, vp, status,
                               context + 64, buffer))
        entry(f"{what}: differential attention, two maps, chunk mask", us,
              roof_us(n * 2 * H * d * (2 + 4) + keys_read * 3 * G * d * 2, dpairs * 2 * H * d * 4.0), like_att, us_att, roof_att)
        heads_o = torch.empty(n, H * d, dtype=bf, device=dev)
        us = us_of(lambda: ops.diff_combine(maps, heads_o, H, d, 0.4, 1e-6, 0.5))
        w = torch.ones(H * d, device=dev)
        xin = torch.randn(n, H * d, device=dev).to(bf)
        us_like = us_of(lambda: ops.rmsnorm(xin, w, heads_o, 1e-6))
        entry(f"{what}: difference of the maps, head norm", us, roof_us(n * H * d * (8 + 2)), "rmsnorm", us_like, roof_us(n * H * d * 4))
        # ---- latent attention: H query heads of rank + dr features over one cached row a position
        lp = torch.randn(n_pages, 1, 64, row, device=dev).to(bf)
        qf = (torch.randn(n, H * row, device=dev) * 0.3).to(bf)
        mixed = torch.empty(n, H * rank, dtype=bf, device=dev)
        lat = pe.parts.latent_attention.attend_rows
        us = us_of(lambda: lat(ops, decode, qf, mixed, n_seqs, q_len, H, row, rank, 0.07, *where, lp, status, context + 64, buffer))
        entry(f"{what}: latent attention over the cached rows ({rank} + {dr} features)", us,
              roof_us(n * H * (row + rank) * 2 + n_seqs * length * row * 2, pairs * H * (row + rank) * 2.0), like_att, us_att, roof_att)
        # ---- the latent rows' norm, rotation and append beside q/k-norm, rotation and append
        rope = pe.parts.lookup("position", "rope")
        rt = pe.parts.Runtime(dev, bf)
        pos_i = rope({"rotary_dim": dr, "theta": 1e6, "max_positions": context + 64, "style": "interleaved", "exact": True}, {}, rt)
        pos_q = rope({"rotary_dim": d, "theta": 1e6, "max_positions": context + 64}, {}, rt)
        ci, si, ri = pos_i.tables()
        cq, sq, _ = pos_q.tables()
        cols = H * (d + dr) + row + H
        qlg = torch.randn(n, cols, device=dev).to(bf)
        absorbed = torch.randn(H, n, rank, device=dev).to(bf)
        qfull = torch.empty(n, H, row, dtype=bf, device=dev)
        nw = torch.ones(rank, device=dev)
        us = us_of(lambda: ops.latent_prepare(qlg, 0, H * (d + dr), H, d, dr, rank, nw, 1e-6, ci, si, ri, token_seq, token_pos, slots,
                                              table, n_pages, lp, qfull, True, status, absorbed=absorbed))
        qw, kw = torch.ones(d, device=dev), torch.ones(d, device=dev)
        us_like = us_of(lambda: ops.qk_norm_rope_append(qkv, n, H, G, d, qw, kw, 1e-6, cq, sq, d, token_seq, token_pos, slots, qstart, table,
                                                        n_pages, kp, vp, True, status))
        entry(f"{what}: latent row's norm, rotation, append, queries put together", us,
              roof_us(n * (H * dr + row) * 2 + n * H * rank * 2 + n * H * row * 2 + n * row * 2), "qk_norm_rope_append", us_like,
              roof_us(n * (H + 2 * G) * d * 2 + n * (H + G) * d * 2 + n * 2 * G * d * 2))
        kv_rows = torch.randn(n, 3 * G * d, device=dev).to(bf)

        def append():
            ops.rows_to_pages_pair(kv_rows, 0, 2 * G, d, kp2, 2 * G * d, G, d, vp, token_seq, token_pos, slots, table, n_pages, status)
        entry(f"{what}: two key maps and the values into their pages", us_of(append), roof_us(n * 3 * G * d * 4),
              "qk_norm_rope_append", us_like, roof_us(n * (H + 2 * G) * d * 2 + n * (H + G) * d * 2 + n * 2 * G * d * 2))
        # ---- gates, norms and the stream
        heads_t = torch.randn(H, n, d, device=dev).to(bf)
        gate = torch.randn(n, H * d, device=dev).to(bf)
        us = us_of(lambda: ops.sigmoid_gate(heads_t, gate, heads_o))
        gu = torch.randn(n, 2 * ff, device=dev).to(bf)
        act = torch.empty(n, ff, dtype=bf, device=dev)
        us_silu = us_of(lambda: ops.silu_mul(gu, act))
        entry(f"{what}: sigmoid gate a feature on the heads' outputs", us, roof_us(n * H * d * 6), "silu_mul", us_silu, roof_us(n * ff * 6))
        z = torch.randn(n, ff * 3 // 2, device=dev).to(bf)
        pz = torch.empty_like(z)
        coeff = torch.tensor([0.5, 0.3, 0.2, 0.1], device=dev)
        us = us_of(lambda: ops.polynorm(z, coeff, 1e-6, pz))
        entry(f"{what}: PolyNorm activation", us, roof_us(n * (ff * 3 // 2) * 4), "silu_mul", us_silu, roof_us(n * ff * 6))
        stream = torch.randn(n, width, device=dev)
        delta = torch.randn(n, width, device=dev).to(bf)
        wn = torch.ones(width, device=dev)
        normed = torch.empty(n, width, dtype=bf, device=dev)
        mix = torch.rand(width, device=dev)
        prev = torch.zeros(n_seqs, width, device=dev)
        us = us_of(lambda: ops.norm_token_shift(stream, wn, 1e-6, mix, prev, token_seq, slots, qstart, normed, status))
        us_like = us_of(lambda: ops.rmsnorm_residual(stream, delta, wn, normed, 1e-6))
        entry(f"{what}: norm and token shift", us, roof_us(n * width * (4 + 2)), "rmsnorm_residual", us_like, roof_us(n * width * (8 + 2 + 2)))
        depth = s["layers"]
        results = torch.randn(depth + 1, n, width, device=dev)
        co = torch.rand(depth + 1, device=dev)
        avg = torch.empty(n, width, device=dev)
        us = us_of(lambda: ops.depth_average(results, co, depth + 1, avg, None))
        entry(f"{what}: average over {depth + 1} results of the depth", us, roof_us(n * width * 4 * (depth + 2)), "rmsnorm_residual", us_like,
              roof_us(n * width * (8 + 2 + 2)))
        # ---- the router by logits beside the router by probabilities
        E, top = 8, 2
        logits = torch.randn(n, E, device=dev)
        bias = torch.zeros(E, device=dev)
        chosen = torch.empty(n, top, dtype=torch.int32, device=dev)
        weight = torch.empty(n, top, device=dev)
        us = us_of(lambda: ops.moe_route_logits(logits, bias, top, chosen, weight))
        us_like = us_of(lambda: ops.moe_route(logits, bias, top, chosen, weight))
        entry(f"{what}: experts chosen by their logits", us, roof_us(n * (E * 4 + top * 8)), "moe_route", us_like, roof_us(n * (E * 4 + top * 8)))
    return out


def zonevik_config(pe, s):
    """Zonevik at the same width, attention heads, feed-forward and vocabulary: window attention that keeps the first positions
    beside a state-space mixer (inner width twice the model's, heads of 64, 128 state rows), the gated delta rule (its state as
    large as Lunadra's), gated attention with scaled rotation; routed experts (8, two chosen among the two best of four groups)
    whose chosen experts together are half as wide as the dense feed-forward; the two middle layers run twice."""
    moe = {"kind": "moe", "router": {"experts": 8, "top": 2, "groups": {"count": 4, "keep": 2}}, "expert": {"ff": s["ff"] // 4}}
    side = {"type": "parallel",
            "mixer": {"left": {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"],
                               "scale": 1.0 / math.sqrt(s["dim"]), "mask": {"size": 1024, "keep_first": 4}},
                      "right": {"heads": 2 * s["width"] // 64, "vdim": 64, "state": 128, "groups": 8, "conv": 4, "norm_groups": 8}},
            "mlp": moe}
    delta = {"type": "delta", "mixer": {"heads": s["wkv_heads"] // 4, "kv_heads": s["wkv_heads"] // 8, "dim": 128, "vdim": 128, "conv": 4},
             "mlp": moe}
    att = {"type": "attention", "mixer": {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"],
                                          "scale": 1.0 / math.sqrt(s["dim"]),
                                          "rot": {"base": 1e6, "dims": s["dim"] // 2, "scaling": YARN}}, "mlp": moe}
    layers = [side, delta, att, att][:s["layers"]] + [att] * max(0, s["layers"] - 4)
    return pe.ZonevikConfig.from_dict({"architecture": "Zonevik", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6},
                                       "embedding": {"scale": math.sqrt(s["width"])}, "loop": {"start": 1, "stop": 3, "times": 2},
                                       "layers": layers})


def zonevik_kernel_pairs(pe, torch, s, peaks, prompt, batch, context):
    """The kernels that only Zonevik has, each beside the like kernel of the Lunadra path (the closest model: window attention
    beside a recurrence, the gated delta rule, routed experts) at the same shape.  A kernel's roofline time is the larger of
    its bytes over the copy bandwidth and its float32 operations over the CUDA cores' rate; ``times_as_far_from_roofline``
    divides the new kernel's distance from its roofline by the like kernel's."""
    ops = pe.kernels.ops
    dev = torch.device("cuda:0")
    bf = torch.bfloat16
    width = s["width"]
    hbm_gbs, BF16_TFLOPS = peaks["hbm_gbs"], peaks.get("bf16_tflops") or 1590.0
    flush = torch.zeros(96 * 2 ** 20, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    out = {}

    def us_of(fn):
        return 1e3 * timed(torch, fn, 20, 5, flush, graph=True)

    def roof_us(nbytes, flops=0.0):
        return max(nbytes / (hbm_gbs * 1e9), flops / (FP32_TFLOPS * 1e12)) * 1e6

    def entry(name, us_new, roof_new, like, us_like, roof_like):
        out[name] = {"us": round(us_new, 2), "roofline_us": round(roof_new, 2), "of_roofline": round(roof_new / us_new, 3)}
        if like:
            out[name].update({"like_kernel": like, "like_us": round(us_like, 2), "like_of_roofline": round(roof_like / us_like, 3),
                              "times_as_far_from_roofline": round((us_new / roof_new) / (us_like / roof_like), 2)})

    for what, n_seqs, q_len in (("prompt", 1, prompt), ("decode", batch, 1)):
        n = n_seqs * q_len
        qstart = torch.arange(0, n + 1, q_len, dtype=torch.int32, device=dev)
        slots = torch.arange(n_seqs, dtype=torch.int32, device=dev)
        chunked = q_len > 128
        # the like kernel of the recurrence: the gated delta rule at Lunadra's shape
        DH, DG, dd, ddv = s["wkv_heads"] // 4, s["wkv_heads"] // 8, 128, 128
        ch = 2 * DG * dd + DH * ddv
        qkv = (torch.randn(n, ch, device=dev) * 0.5).to(bf)
        a_lin, beta = torch.randn(n, DH * dd, device=dev), torch.randn(n, DH, device=dev)
        dtb, alog, nw2 = torch.zeros(DH * dd, device=dev), torch.zeros(DH, device=dev), torch.ones(ddv, device=dev)
        gate = torch.randn(n, DH * ddv, device=dev).to(bf)
        o2 = torch.empty(n, DH * ddv, dtype=bf, device=dev)
        S2 = torch.zeros(n_seqs, DH, dd, ddv, device=dev)
        dmax = -(-q_len // 128) if chunked else 1
        scratch_d = torch.empty(ops.delta_rule_scratch_floats(n_seqs, DH, dd, ddv, dmax), device=dev) if chunked else None
        us_delta = us_of(lambda: ops.delta_rule_recurrence(qkv, a_lin, dtb, alog, beta, gate, nw2, 1e-6, dd ** -0.5, o2, S2, slots, qstart,
                                                           n_seqs, q_len, DH, DG, dd, ddv, status, 128 if chunked else 0, dmax, scratch_d))
        roof_delta = roof_us(n * (ch * 2 + DH * dd * 4 + DH * ddv * 4) + n_seqs * DH * dd * ddv * 8, n * DH * dd * ddv * 7.0)
        # the same kernel with one decay a head and the silu gate (what Zonevik's delta layers run)
        a_head, dtb_h = torch.randn(n, DH, device=dev), torch.zeros(DH, device=dev)
        us = us_of(lambda: ops.delta_rule_recurrence(qkv, a_head, dtb_h, alog, beta, gate, nw2, 1e-6, dd ** -0.5, o2, S2, slots, qstart,
                                                     n_seqs, q_len, DH, DG, dd, ddv, status, 128 if chunked else 0, dmax, scratch_d,
                                                     head_decay=True, gate_silu=True))
        entry(f"{what}: gated delta recurrence with one decay a head, silu gate", us,
              roof_us(n * (ch * 2 + DH * 8 + DH * ddv * 4) + n_seqs * DH * dd * ddv * 8, n * DH * dd * ddv * 7.0),
              "delta_rule_recurrence (decay per channel)", us_delta, roof_delta)
        # the state-space recurrence
        H, dv, N, G = 2 * width // 64, 64, 128, 8
        xbc = (torch.randn(n, H * dv + 2 * G * N, device=dev) * 0.5).to(bf)
        dt = torch.randn(n, H, device=dev).to(bf)
        dtb2, alog2, D = torch.zeros(H, device=dev), torch.zeros(H, device=dev), torch.ones(H, device=dev)
        y = torch.empty(n, H * dv, device=dev)
        S = torch.zeros(n_seqs, H, N, dv, device=dev)
        smax = -(-q_len // 64) if chunked else 1
        scratch_s = torch.empty(ops.ssd_scratch_floats(n_seqs, H, N, dv, smax), device=dev) if chunked else None
        us = us_of(lambda: ops.ssd_recurrence(xbc, dt, dtb2, alog2, D, y, S, slots, qstart, n_seqs, q_len, H, G, N, dv, status,
                                              64 if chunked else 0, smax, scratch_s))
        passes = 2.0 if chunked else 1.0     # the chunked form walks every token twice (fold, then outputs)
        entry(f"{what}: state-space recurrence", us,
              roof_us(n * ((H * dv + 2 * G * N) * 2 + H * 2 + H * dv * 4) + n_seqs * H * N * dv * 8, n * H * N * dv * 4.0),
              "delta_rule_recurrence", us_delta, roof_delta)
        out[f"{what}: state-space recurrence"]["fp32_tflops"] = round(passes * n * H * N * dv * 4.0 / us / 1e6, 1)
        # gate, then the norm over parts of the row, beside the plain norm of a row of the same size
        z = torch.randn(n, H * dv, device=dev).to(bf)
        nw = torch.ones(H * dv, device=dev)
        yo = torch.empty(n, H * dv, dtype=bf, device=dev)
        us = us_of(lambda: ops.gated_part_norm(y, z, nw, 1e-6, yo, 8))
        us_like = us_of(lambda: ops.rmsnorm(z, nw, yo, 1e-6))
        entry(f"{what}: silu gate, norm over parts of the row", us, roof_us(n * H * dv * 8), "rmsnorm", us_like, roof_us(n * H * dv * 4))
        # the norms around a sublayer
        stream = torch.randn(n, width, device=dev)
        delta = torch.randn(n, width, device=dev).to(bf)
        delta2 = torch.randn(n, width, device=dev).to(bf)
        w, b0 = torch.ones(width, device=dev), torch.zeros(width, device=dev)
        normed = torch.empty(n, width, dtype=bf, device=dev)
        us_like = us_of(lambda: ops.rmsnorm_residual(stream, delta, w, normed, 1e-6))
        roof_like = roof_us(n * width * (8 + 2 + 2))
        us = us_of(lambda: ops.dyt(stream, w, b0, 0.8, normed))
        entry(f"{what}: tanh norm of the stream", us, roof_us(n * width * 6), "rmsnorm_residual", us_like, roof_like)
        us = us_of(lambda: ops.dyt_add(stream, delta, w, b0, 0.8, (w, b0, 0.7), normed))
        entry(f"{what}: tanh norm of a sublayer's output, add, tanh norm of the new stream", us, roof_us(n * width * 12),
              "rmsnorm_residual", us_like, roof_like)
        us = us_of(lambda: ops.rmsnorm_pair_mix_dyt_add(delta, delta2, w, w, 1e-6, 0.5, 0.5, stream, (w, b0, 0.8), (w, b0, 0.7), normed))
        us_sum = us_of(lambda: ops.rmsnorm_residual_sum(stream, [delta, delta2], [1.0, 1.0], w, normed, 1e-6))
        entry(f"{what}: two outputs over their root mean squares, half their sum, tanh norm, add, next tanh norm", us,
              roof_us(n * width * (8 + 4 + 2)), "rmsnorm_residual_sum of two", us_sum, roof_us(n * width * (8 + 4 + 2)))
        # the router
        E, top = 8, 2
        logits = torch.randn(n, E, device=dev)
        corr = torch.zeros(E, device=dev)
        chosen = torch.empty(n, top, dtype=torch.int32, device=dev)
        weight = torch.empty(n, top, device=dev)
        us = us_of(lambda: ops.moe_route_sigmoid_groups(logits, top, 4, 2, chosen, weight))
        us_like = us_of(lambda: ops.moe_route(logits, corr, top, chosen, weight))
        entry(f"{what}: experts chosen among the best groups", us, roof_us(n * (E * 4 + top * 8)), "moe_route", us_like, roof_us(n * (E * 4 + top * 8)))
        # window attention that keeps the first positions, beside the window attention of the Lunadra path
        nh, nkv, d = s["heads"], s["kv_heads"], s["dim"]
        length = context if what == "decode" else prompt
        pages = -(-length // 64)
        kp = (torch.randn(n_seqs * pages + 1, nkv, 64, d, device=dev) * 0.5).to(bf)
        vp = (torch.randn(n_seqs * pages + 1, nkv, 64, d, device=dev) * 0.5).to(bf)
        table = torch.arange(n_seqs * pages, dtype=torch.int32, device=dev).view(n_seqs, pages).contiguous()
        past = torch.full((n_seqs,), length - q_len, dtype=torch.int32, device=dev)
        q = (torch.randn(n, nh * d, device=dev) * 0.5).to(bf)
        ao = torch.empty(n, nh * d, dtype=bf, device=dev)
        decode = what == "decode"
        sk, ms, floor = ops.attention_mma_decode_ranges(dev, d, n_seqs, nkv, length, 512) if decode else (512, 0, 0)
        scr2 = torch.empty(ops.attention_generic_scratch_floats(n_seqs, nh, d, max(ms, 1)), device=dev) if decode else None
        us = us_of(lambda: ops.attention_mma_masked(decode, q, ao, n_seqs, q_len, nh, nkv, d, d ** -0.5, qstart, past, slots, table,
                                                    kp.shape[0], kp, vp, scr2, sk, ms, status, min_range_keys=floor, window=1024,
                                                    keep_first=4))
        us_like = us_of(lambda: ops.attention_mma(decode, q, ao, n_seqs, q_len, nh, nkv, d, d ** -0.5, 1024, qstart, past, slots, table,
                                                  kp.shape[0], kp, vp, scr2, sk, ms, status, min_range_keys=floor))
        keys = min(length, 1024 + 4)
        att_bytes = n_seqs * keys * nkv * d * 4 + n * nh * d * 4 if decode else n * (nh + nkv) * d * 4
        att_flops = 4.0 * n * nh * d * (keys if decode else min(1024, length) * 0.75)
        roof = max(att_bytes / (hbm_gbs * 1e9), att_flops / (BF16_TFLOPS * 1e12)) * 1e6
        entry(f"{what}: window attention with kept first positions", us, roof, "attention_mma (window)", us_like, roof)
    return out


def main(args):
    import torch

    sys.path.insert(0, __file__.rsplit("/", 1)[0])
    import bench

    pe = importlib.import_module("pytorch-engine_b200")
    peaks = bench.load_peaks()
    prompt, batch, context = args.prefill_tokens, args.batch, min(args.context, 2048)
    result = {"metric": "architectures_beside_qwen3", "dtype": "bf16", "data": "synthetic (random weights)", "peaks": peaks,
              "prompt_tokens": prompt, "decode_batch": batch, "decode_context": context,
              "flush": "model runs: weights larger than L2; kernel pairs: 384 MB written between iterations", "sizes": {}}
    names = [n for n in SIZES if not args.arch_sizes or n in args.arch_sizes.split(",")]
    for name in names:
        s = SIZES[name]
        row = {"shape": s}
        wanted = [a for a in (args.arch_names or "vabelorn,qwen3,lunadra,vemepel,zonevik").split(",") if a]
        for arch, make in (("vabelorn", vabelorn_config), ("qwen3", qwen3_config), ("lunadra", lunadra_config),
                           ("vemepel", vemepel_config), ("zonevik", zonevik_config)):
            if arch not in wanted:
                continue
            row[arch] = model_speeds(pe, torch, make(pe, s), prompt, batch, context, args.steps, max(args.warmup, 3))
            print(f"[{name}] {arch}: {row[arch]}", file=sys.stderr, flush=True)
        if "vabelorn" in wanted:
            row["kernels"] = kernel_pairs(pe, torch, s, peaks["hbm_gbs"], prompt, batch, context)
            for k, v in row["kernels"].items():
                print(f"[{name}] {k}: {v}", file=sys.stderr, flush=True)
        if "lunadra" in wanted:
            row["lunadra_kernels"] = lunadra_kernel_pairs(pe, torch, s, peaks["hbm_gbs"], prompt, batch, context)
            for k, v in row["lunadra_kernels"].items():
                print(f"[{name}] {k}: {v}", file=sys.stderr, flush=True)
        if "vemepel" in wanted:
            row["vemepel_kernels"] = vemepel_kernel_pairs(pe, torch, s, peaks, prompt, batch, context)
            for k, v in row["vemepel_kernels"].items():
                print(f"[{name}] {k}: {v}", file=sys.stderr, flush=True)
        if "zonevik" in wanted:
            row["zonevik_kernels"] = zonevik_kernel_pairs(pe, torch, s, peaks, prompt, batch, context)
            for k, v in row["zonevik_kernels"].items():
                print(f"[{name}] {k}: {v}", file=sys.stderr, flush=True)
        result["sizes"][name] = row
    result["gpu_launches"] = pe.kernels.ops.launch_count()
    print(json.dumps(result))
    return 0
