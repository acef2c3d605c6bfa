"""The Zonevik decoder written out plainly and slowly in PyTorch, one function per mechanism, for the tests.

It shares no code with the package: it reads a configuration as a plain dict (the keys of ``config.json``) and weights
as a dict of tensors by checkpoint name, and computes everything in the dtype it is given (float64 by default), one
whole sequence at a time, with no cache and no state carried from call to call.

Notation: ``x`` is the residual stream ``[T, width]``; ``unit(x) = x / sqrt(mean(x^2) + eps)``.

    embedding:  x = E[tok] * c ;  x0 = x
    order:      layers [0, a), then layers [a, b) ``times`` times over (same weights), then layers [b, L);
                in front of every pass over [a, b):  x <- W_in [x ; x0]
    layer:      x += n1b(mixer(n1(x))) ;  x += n2b(ff(n2(x)))        n(x) = tanh(alpha x) * w + b   (no statistics)
    attention:  grouped heads; interleaved rotary pairs on the first ``dims`` features with YaRN-scaled frequencies;
                causal softmax; the joined heads times sigmoid(W_g h); W_o
    parallel:   (unit(left(h)) * w_l + unit(right(h)) * w_r) / 2
      left:       grouped heads with biases on q, k, v, no positions; key j is visible to query i if j <= i and
                  (i - j < size or j < keep_first); softmax; W_o
      right:      [z | x | B | C | dt] = W_in h ; (x, B, C) through a causal convolution with bias and silu ;
                  dt = softplus(dt + dt_bias) ; per head S <- exp(-exp(A) dt) S + dt B x^T ; y = S^T C + D x ;
                  y * silu(z), unit() over each of ``norm_groups`` equal parts, weight, W_o
    delta:      short causal convolutions and silu on q, k, v; q, k of length one, q / sqrt(dim); per head a matrix S:
                  S <- g S ; u = beta (v - S^T k) ; S <- S + k u^T ; o = S^T q
                with g = exp(-exp(A) softplus(W_a h + dt)) one number per head; unit(o), weight, silu(W_g h), W_o
    ff:         s = sigmoid(R h) ; the experts form equal groups of neighbours, a group's score is the sum of its two
                largest s ; the ``top`` largest s inside the ``keep`` best groups are chosen, weighted with s itself
      expert:     D (silu(G h) * (U h))
    output:     logits = E n(x)
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F

# ``STORE``: None, or a 16-bit dtype in which the results of matrix products are rounded (and brought back), at about
# the places where an engine that runs in that dtype rounds: the measure against which a 16-bit run is judged.
STORE = None


class stored:
    def __init__(self, dtype):
        self.dtype = dtype

    def __enter__(self):
        global STORE
        self.before, STORE = STORE, self.dtype

    def __exit__(self, *exc):
        global STORE
        STORE = self.before


def st(x: torch.Tensor) -> torch.Tensor:
    return x if STORE is None else x.to(STORE).to(x.dtype)


def lin(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    y = x @ w.T
    return st(y if b is None else y + b)


def unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def tanh_norm(x: torch.Tensor, w: Dict[str, torch.Tensor], name: str) -> torch.Tensor:
    return torch.tanh(w[name + ".alpha"] * x) * w[name] + w[name + ".b"]


# ---- feed-forward ---------------------------------------------------------------------------------------------
def router_choice(scores: torch.Tensor, r: dict, margins: Optional[list] = None):
    """``scores [T, E]`` -> (chosen [T, top] indices, their scores).  ``margins`` (a list) gets one tensor ``[T]``: by how much
    the choice was decided, in units of the router's logits: the smaller of the gap between the last kept and the first dropped
    group and the gap between the last chosen expert and the best one left out, each divided by how far the scores involved
    move per unit of their logits, ``s (1 - s)`` (an error of that size in the logits would have chosen otherwise)."""
    T, E = scores.shape
    top = int(r["top"])
    allowed = torch.ones_like(scores, dtype=torch.bool)
    margin = torch.full((T,), float("inf"), dtype=scores.dtype)
    groups = r.get("groups")
    if groups:
        count, keep = int(groups["count"]), int(groups["keep"])
        per = E // count
        g = scores.view(T, count, per)
        gtop = g.topk(min(2, per), dim=-1).values
        gscore = gtop.sum(-1)
        ranked = gscore.topk(count, dim=-1)
        if keep < count:
            moves = (gtop * (1 - gtop)).sum(-1).gather(1, ranked.indices[:, keep - 1:keep + 1]).sum(-1)
            margin = (ranked.values[:, keep - 1] - ranked.values[:, keep]) / (moves + 1e-12)
        gmask = torch.zeros(T, count, dtype=torch.bool)
        gmask.scatter_(1, ranked.indices[:, :keep], True)
        allowed = gmask[:, :, None].expand(T, count, per).reshape(T, E)
    masked = torch.where(allowed, scores, torch.full_like(scores, -1.0))
    ranked = masked.topk(min(top + 1, E), dim=-1)
    if top < E:
        last, left_out = ranked.values[:, top - 1], ranked.values[:, top]
        gap = (last - left_out) / (last * (1 - last) + left_out * (1 - left_out) + 1e-12)
        margin = torch.minimum(margin, torch.where(left_out >= 0, gap, margin))
    if margins is not None:
        margins.append(margin)
    chosen = ranked.indices[:, :top]
    return chosen, scores.gather(1, chosen)


def moe_ff(h: torch.Tensor, mlp: dict, w: Dict[str, torch.Tensor], p: str, margins: Optional[list] = None) -> torch.Tensor:
    r = mlp["router"]
    scores = torch.sigmoid(h @ w[f"{p}.router"].T)
    chosen, weight = router_choice(scores, r, margins)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(chosen[t].tolist(), weight[t]):
            q = f"{p}.e{e}"
            y = lin(st(F.silu(lin(h[t], w[f"{q}.gate"])) * lin(h[t], w[f"{q}.up"])), w[f"{q}.down"])
            out[t] += s * y
    return st(out)


# ---- rotary positions -------------------------------------------------------------------------------------------
def rotary_tables(rot: dict, positions: torch.Tensor):
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    mult = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, original = float(sc["factor"]), float(sc["original"])

        def where(t):
            return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))

        lo = max(math.floor(where(float(sc["fast"]))), 0)
        hi = min(math.ceil(where(float(sc["slow"]))), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mult = 0.1 * math.log(factor) + 1.0
    ang = positions.to(torch.float64)[:, None] * f[None, :]
    return torch.cos(ang) * mult, torch.sin(ang) * mult


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: Optional[dict]) -> torch.Tensor:
    """``x [T, heads, d]``: pairs (2i, 2i + 1) of the first ``dims`` features turn with the position."""
    if not rot or not int(rot.get("dims", 0)):
        return x
    dims = int(rot["dims"])
    cos, sin = rotary_tables(rot, positions)
    cos, sin = cos.to(x.dtype)[:, None, :], sin.to(x.dtype)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


# ---- softmax attention ------------------------------------------------------------------------------------------
def softmax_attention(q, k, v, scale: float, visible: torch.Tensor) -> torch.Tensor:
    """``q [T, H, d]``, ``k [T, G, d]``, ``v [T, G, dv]``, ``visible [T, T]`` bool -> ``[T, H * dv]``."""
    T, H, _ = q.shape
    G = k.shape[1]
    outs = []
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * scale
        s = s.masked_fill(~visible, float("-inf"))
        outs.append(torch.softmax(s, dim=-1) @ v[:, g])
    return torch.cat(outs, dim=-1)


def attention(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(T)
    q = st(rotate(lin(h, w[f"{p}.q"]).view(T, H, d), pos, m.get("rot")))
    k = st(rotate(lin(h, w[f"{p}.k"]).view(T, G, d), pos, m.get("rot")))
    v = lin(h, w[f"{p}.v"]).view(T, G, dv)
    visible = pos[None, :] <= pos[:, None]
    o = st(softmax_attention(q, k, v, float(m["scale"]), visible))
    o = st(o * torch.sigmoid(lin(h, w[f"{p}.g"])))
    return lin(o, w[f"{p}.o"])


def window_attention(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(T)
    q = lin(h, w[f"{p}.q"], w[f"{p}.q.b"]).view(T, H, d)
    k = lin(h, w[f"{p}.k"], w[f"{p}.k.b"]).view(T, G, d)
    v = lin(h, w[f"{p}.v"], w[f"{p}.v.b"]).view(T, G, dv)
    i, j = pos[:, None], pos[None, :]
    visible = j <= i
    mask = m.get("mask")
    if mask:
        visible = visible & ((i - j < int(mask["size"])) | (j < int(mask.get("keep_first", 0))))
    o = st(softmax_attention(q, k, v, float(m["scale"]), visible))
    return lin(o, w[f"{p}.o"])


# ---- recurrences ----------------------------------------------------------------------------------------------
def short_conv(x: torch.Tensor, taps_w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal convolution per channel: ``x [T, C]``, ``taps_w [C, taps]`` whose last column meets the current token."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x])
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + padded[j:j + T] * taps_w[:, j]
    if bias is not None:
        y = y + bias
    return st(F.silu(y))


def state_space(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, dv, N, G = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"])
    inner = H * dv
    proj = lin(h, w[f"{p}.in"])
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = short_conv(xbc, w[f"{p}.conv"], w[f"{p}.conv.b"])
    x = xbc[:, :inner].view(T, H, dv)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = F.softplus(dt + w[f"{p}.dt_bias"])
    rate = torch.exp(w[f"{p}.A_log"])
    y = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(N, dv, dtype=h.dtype)
        for t in range(T):
            S = torch.exp(-rate[hd] * dt[t, hd]) * S + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ C[t, g] + w[f"{p}.D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * F.silu(z)
    parts = int(m["norm_groups"])
    y = unit(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[f"{p}.norm"]
    return lin(st(y), w[f"{p}.o"])


def delta(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = short_conv(lin(h, w[f"{p}.q"]), w[f"{p}.q.conv"]).view(T, G, d)
    k = short_conv(lin(h, w[f"{p}.k"]), w[f"{p}.k.conv"]).view(T, G, d)
    v = short_conv(lin(h, w[f"{p}.v"]), w[f"{p}.v.conv"]).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[f"{p}.b"].T)
    g = torch.exp(-torch.exp(w[f"{p}.A_log"]) * F.softplus(h @ w[f"{p}.a"].T + w[f"{p}.dt_bias"]))
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        kv = hd // (H // G)
        S = torch.zeros(d, dv, dtype=h.dtype)
        for t in range(T):
            S = g[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, kv])
            S = S + torch.outer(k[t, kv], u)
            o[t, hd] = S.T @ q[t, kv]
    o = unit(o, eps) * w[f"{p}.norm"]
    o = o.reshape(T, H * dv) * F.silu(lin(h, w[f"{p}.g"]))
    return lin(st(o), w[f"{p}.o"])


def parallel(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    a = window_attention(h, m["left"], w, f"{p}.left")
    b = state_space(h, m["right"], w, f"{p}.right", eps)
    return 0.5 * (unit(a, eps) * w[f"{p}.left.out"] + unit(b, eps) * w[f"{p}.right.out"])


# ---- the model --------------------------------------------------------------------------------------------------
def run_order(cfg: dict) -> List[tuple]:
    """(layer, first of a pass) in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, False) for i in range(a)]
    for _ in range(times):
        order += [(i, i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, n)]


def layer(x: torch.Tensor, spec: dict, w: Dict[str, torch.Tensor], p: str, eps: float, margins: Optional[list] = None) -> torch.Tensor:
    h = st(tanh_norm(x, w, f"{p}.norm1"))
    kind = spec["type"]
    if kind == "attention":
        y = attention(h, spec["mixer"], w, f"{p}.mix")
    elif kind == "delta":
        y = delta(h, spec["mixer"], w, f"{p}.mix", eps)
    elif kind == "parallel":
        y = st(parallel(h, spec["mixer"], w, f"{p}.mix", eps))
    else:
        raise ValueError(kind)
    x = x + tanh_norm(y, w, f"{p}.norm1b")
    if spec.get("mlp") is not None:
        h = st(tanh_norm(x, w, f"{p}.norm2"))
        x = x + tanh_norm(moe_ff(h, spec["mlp"], w, f"{p}.mlp", margins), w, f"{p}.norm2b")
    return x


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64, streams: Optional[list] = None,
            margins: Optional[list] = None):
    """Logits ``[T, vocab]`` of one sequence; ``streams`` (a list) collects the stream after every layer that ran, ``margins``
    (a list) one tensor ``[T]`` per routed feed-forward that ran: by how much its choice of experts was decided."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][tokens] * float(cfg.get("embedding", {}).get("scale", 1.0))
    x0 = x
    for i, first in run_order(cfg):
        if first:
            x = torch.cat([x, x0], dim=-1) @ w["loop.in"].T
        x = layer(x, cfg["layers"][i], w, f"l{i}", eps, margins)
        if streams is not None:
            streams.append(x.clone())
    return st(tanh_norm(x, w, "final.norm")) @ w["embed"].T


def random_weights(cfg: dict, seed: int, std: float = 0.08) -> Dict[str, torch.Tensor]:
    """Weights by checkpoint name for any configuration of this design, as bfloat16-representable float32 values."""
    gen = torch.Generator().manual_seed(seed)
    W = int(cfg["width"])
    out: Dict[str, torch.Tensor] = {}

    def mat(name, *shape, s=std):
        out[name] = (torch.randn(*shape, generator=gen) * s).to(torch.bfloat16).to(torch.float32)

    def norm(name, n=W):
        out[name] = (1.0 + 0.2 * torch.randn(n, generator=gen)).to(torch.bfloat16).to(torch.float32)
        mat(name + ".b", n, s=0.05)
        out[name + ".alpha"] = torch.tensor(0.5 + 0.4 * torch.rand((), generator=gen).item()).to(torch.bfloat16).to(torch.float32)

    mat("embed", int(cfg["vocab"]), W, s=0.1)
    if cfg.get("loop"):
        mat("loop.in", W, 2 * W, s=0.7 / math.sqrt(W))
    for i, spec in enumerate(cfg["layers"]):
        p = f"l{i}"
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if spec.get("mlp") is not None else ()):
            norm(f"{p}.{n}")
        m = spec["mixer"]
        s_in = 1.0 / math.sqrt(W)
        if spec["type"] == "attention":
            H, G, d, dv = (int(m[k]) for k in ("heads", "kv_heads", "dim", "vdim"))
            mat(f"{p}.mix.q", H * d, W, s=s_in)
            mat(f"{p}.mix.k", G * d, W, s=s_in)
            mat(f"{p}.mix.v", G * dv, W, s=s_in)
            mat(f"{p}.mix.g", H * dv, W, s=s_in)
            mat(f"{p}.mix.o", W, H * dv, s=1.0 / math.sqrt(H * dv))
        elif spec["type"] == "delta":
            H, G, d, dv, taps = (int(m[k]) for k in ("heads", "kv_heads", "dim", "vdim", "conv"))
            for n, rows in (("q", G * d), ("k", G * d), ("v", H * dv)):
                mat(f"{p}.mix.{n}", rows, W, s=s_in)
                mat(f"{p}.mix.{n}.conv", rows, taps, s=0.5)
            mat(f"{p}.mix.b", H, W, s=s_in)
            mat(f"{p}.mix.a", H, W, s=s_in)
            mat(f"{p}.mix.A_log", H, s=0.5)
            mat(f"{p}.mix.dt_bias", H, s=0.5)
            out[f"{p}.mix.norm"] = (1.0 + 0.2 * torch.randn(dv, generator=gen)).to(torch.bfloat16).to(torch.float32)
            mat(f"{p}.mix.g", H * dv, W, s=s_in)
            mat(f"{p}.mix.o", W, H * dv, s=1.0 / math.sqrt(H * dv))
        else:
            a, b = m["left"], m["right"]
            H, G, d, dv = (int(a[k]) for k in ("heads", "kv_heads", "dim", "vdim"))
            for n, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
                mat(f"{p}.mix.left.{n}", rows, W, s=s_in)
                mat(f"{p}.mix.left.{n}.b", rows, s=0.1)
            mat(f"{p}.mix.left.o", W, H * dv, s=1.0 / math.sqrt(H * dv))
            H, dv, N, Gr, taps = (int(b[k]) for k in ("heads", "vdim", "state", "groups", "conv"))
            inner, ch = H * dv, H * dv + 2 * Gr * N
            mat(f"{p}.mix.right.in", 2 * inner + 2 * Gr * N + H, W, s=s_in)
            mat(f"{p}.mix.right.conv", ch, taps, s=0.5)
            mat(f"{p}.mix.right.conv.b", ch, s=0.1)
            mat(f"{p}.mix.right.dt_bias", H, s=0.5)
            mat(f"{p}.mix.right.A_log", H, s=0.5)
            out[f"{p}.mix.right.D"] = (1.0 + 0.2 * torch.randn(H, generator=gen)).to(torch.bfloat16).to(torch.float32)
            out[f"{p}.mix.right.norm"] = (1.0 + 0.2 * torch.randn(inner, generator=gen)).to(torch.bfloat16).to(torch.float32)
            mat(f"{p}.mix.right.o", W, inner, s=1.0 / math.sqrt(inner))
            for side in ("left", "right"):
                out[f"{p}.mix.{side}.out"] = (1.0 + 0.2 * torch.randn(W, generator=gen)).to(torch.bfloat16).to(torch.float32)
        mlp = spec.get("mlp")
        if mlp is not None:
            ff, E = int(mlp["expert"]["ff"]), int(mlp["router"]["experts"])
            mat(f"{p}.mlp.router", E, W, s=4.0 * s_in)      # decisive scores: few close calls between experts
            for e in range(E):
                mat(f"{p}.mlp.e{e}.gate", ff, W, s=s_in)
                mat(f"{p}.mlp.e{e}.up", ff, W, s=s_in)
                mat(f"{p}.mlp.e{e}.down", W, ff, s=1.0 / math.sqrt(ff))
    norm("final.norm")
    return out
