"""The Vemepel decoder written out plainly: one function per mechanism, float64, no kernels, no cache manager.

The tests compare the engine with this file.  It shares no code with the package: it reads the same ``config.json``
dictionary and the same tensor names, and keeps what a sequence carries from one call to the next in a plain dict.
``stored`` (default: identity) is applied wherever a 16-bit engine writes a matrix product or a cached row, so that
``stored = bf16`` shows what rounding alone does.

Notation: ``h`` a block's normed input ``[T, width]``, ``pos`` the tokens' positions, ``W x`` for weights stored
``[out, in]``.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional

import torch

F64 = torch.float64
Round = Callable[[torch.Tensor], torch.Tensor]


def same(x: torch.Tensor) -> torch.Tensor:
    return x


def bf16(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.float32).to(torch.bfloat16).to(F64)


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_around_zero(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose stored weight is the distance from one."""
    return unit_rms(x, eps) * (1.0 + w)


def norm_plain(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * w


def token_shift(h: torch.Tensor, before: torch.Tensor, mix: torch.Tensor):
    """Each token's input moves towards the previous token's (unmoved) input: h + (h_prev - h) * mix.
    ``before``: the input of the token before this portion (zeros at a sequence's start).  Returns the moved rows and
    the row to keep for the next portion."""
    prev = torch.cat([before[None], h[:-1]], 0)
    return h + (prev - h) * mix, h[-1].clone()


def depth_average(results: List[torch.Tensor], coeff: torch.Tensor) -> torch.Tensor:
    """sum_j coeff[j] * results[j] over the embedding output and every layer result so far."""
    assert len(results) == coeff.numel()
    return sum(c * r for c, r in zip(coeff, results))


def rotate_pairs(x: torch.Tensor, pos: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """Rotary encoding of adjacent pairs (2i, 2i+1) of the first ``dims`` features of ``x [T, ..., d]``; angle
    pos * base^(-2i/dims)."""
    i = torch.arange(dims // 2, dtype=F64)
    ang = pos.to(F64)[:, None] * base ** (-2.0 * i / dims)
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def softmax_attend(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, visible: torch.Tensor) -> torch.Tensor:
    """q [T, d], k [S, d], v [S, dv], visible [T, S] bool -> [T, dv]."""
    s = (q @ k.T) * scale
    s = s.masked_fill(~visible, -math.inf)
    return torch.softmax(s, -1) @ v


def latent_attention(h, pos, w: Dict[str, torch.Tensor], m: dict, eps: float, kept: dict, stored: Round = same):
    """Attention whose keys and values are expanded from a cached low-rank row.  ``w``: q, dkv, dkv.norm, uk, uv, g, o.
    With ``rot_dim`` in ``m`` a rotated part rides beside every head's keys (one shared rotated key part per token),
    and the output gate is per feature; without it the gate is one number per head."""
    H, d, dv, r = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
    dr = int(m.get("rot_dim", 0) or 0)
    T = h.shape[0]
    q = stored(h @ w["q"].T).view(T, H, d + dr)
    low = stored(h @ w["dkv"].T)
    c = stored(norm_plain(low[:, :r], w["dkv.norm"], eps))
    row = c
    if dr:
        rot = m["rot"]
        q = torch.cat([q[..., :d], rotate_pairs(q[..., d:], pos, float(rot["base"]), int(rot["dims"]))], -1)
        row = torch.cat([c, stored(rotate_pairs(low[:, r:], pos, float(rot["base"]), int(rot["dims"])))], -1)
    kept["rows"] = row if "rows" not in kept else torch.cat([kept["rows"], row], 0)
    rows = kept["rows"]
    S = rows.shape[0]
    kpos = torch.arange(S)
    visible = kpos[None, :] <= pos[:, None]
    keys = stored(rows[:, :r] @ w["uk"].T).view(S, H, d)
    vals = stored(rows[:, :r] @ w["uv"].T).view(S, H, dv)
    gate = torch.sigmoid(stored(h @ w["g"].T))
    heads = []
    for i in range(H):
        k_i = torch.cat([keys[:, i], rows[:, r:]], -1) if dr else keys[:, i]
        heads.append(softmax_attend(q[:, i], k_i, vals[:, i], m["scale"], visible))
    o = torch.stack(heads, 1)                                   # [T, H, dv]
    o = o * (gate.view(T, H, dv) if gate.shape[1] == H * dv else gate[:, :, None])
    return stored(stored(o.reshape(T, H * dv)) @ w["o"].T)


def differential_attention(h, pos, w: Dict[str, torch.Tensor], m: dict, eps: float, kept: dict, stored: Round = same,
                           borrowed: Optional[dict] = None):
    """Two softmax maps per head over the same values, the second subtracted with a weight lambda; keys visible inside
    the query's own block of ``mask.size`` positions only.  ``borrowed``: another layer's kept keys and values (this
    layer then has none of its own)."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = stored(h @ w["q"].T).view(T, H, 2, d)
    if borrowed is None:
        k = stored(h @ w["k"].T).view(T, G, 2, d)
        v = stored(h @ w["v"].T).view(T, G, dv)
        kept["k"] = k if "k" not in kept else torch.cat([kept["k"], k], 0)
        kept["v"] = v if "v" not in kept else torch.cat([kept["v"], v], 0)
        borrowed = kept
    K, V = borrowed["k"], borrowed["v"]
    S = K.shape[0]
    kpos = torch.arange(S)
    visible = kpos[None, :] <= pos[:, None]
    size = (m.get("mask") or {}).get("size")
    if size:
        visible = visible & (torch.div(kpos, size, rounding_mode="floor")[None, :]
                             == torch.div(pos, size, rounding_mode="floor")[:, None])
    diff = float(m["diff"])
    lam = torch.exp((w["lq1"] * w["lk1"]).sum()) - torch.exp((w["lq2"] * w["lk2"]).sum()) + diff
    heads = []
    for i in range(H):
        g = i // (H // G)
        a1 = softmax_attend(q[:, i, 0], K[:, g, 0], V[:, g], m["scale"], visible)
        a2 = softmax_attend(q[:, i, 1], K[:, g, 1], V[:, g], m["scale"], visible)
        heads.append(unit_rms(a1 - lam * a2, eps) * (1.0 - diff))
    o = torch.stack(heads, 1).reshape(T, H * dv)
    return stored(stored(o) @ w["o"].T)


def polynorm(z: torch.Tensor, coeff: torch.Tensor, eps: float) -> torch.Tensor:
    """a N(z) + b N(z^2) + c N(z^3) + e with N the division by a row's root mean square."""
    a, b, c, e = (float(x) for x in coeff)
    return a * unit_rms(z, eps) + b * unit_rms(z * z, eps) + c * unit_rms(z * z * z, eps) + e


def dense_ff(h, w: Dict[str, torch.Tensor], eps: float, stored: Round = same):
    return stored(stored(polynorm(stored(h @ w["up"].T), w["act"], eps)) @ w["down"].T)


def choose_experts(h, router: torch.Tensor, bias: torch.Tensor, top: int):
    """Logits W h + b; the ``top`` largest are chosen (ties: the lower index) and weighted by a softmax over the chosen
    logits alone."""
    z = h @ router.T + bias
    order = torch.sort(z, dim=-1, descending=True, stable=True).indices[:, :top]
    chosen = torch.gather(z, 1, order)
    return order, torch.softmax(chosen, -1)


def expert_ff(h, w: Dict[str, torch.Tensor], m: dict, stored: Round = same, router_input: Round = same):
    n, top = int(m["router"]["experts"]), int(m["router"]["top"])
    which, weight = choose_experts(router_input(h), w["router"], w["router.b"], top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(which[t, j])
            g = stored(h[t] @ w[f"e{e}.gate"].T)
            u = stored(h[t] @ w[f"e{e}.up"].T)
            y = stored(stored(g * torch.sigmoid(g) * u) @ w[f"e{e}.down"].T)
            out[t] += weight[t, j] * y
    assert n >= top
    return stored(out)


class PlainVemepel:
    """The whole model over one sequence at a time.  ``feed(state, tokens)`` runs the next tokens of a sequence whose
    ``state`` (a dict, empty at the start) holds what earlier calls left; returns logits ``[T, vocab]`` and, with
    ``trace=True``, also the stream after every layer."""

    def __init__(self, config: dict, weights: Dict[str, torch.Tensor], stored: Round = same) -> None:
        self.cfg = config
        self.w = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in weights.items()}
        self.eps = float(config["norm"]["eps"])
        self.stored = stored

    def sub(self, prefix: str) -> Dict[str, torch.Tensor]:
        return {k[len(prefix):]: v for k, v in self.w.items() if k.startswith(prefix)}

    def feed(self, state: dict, tokens, trace: bool = False):
        w, eps, st = self.w, self.eps, self.stored
        past = state.get("length", 0)
        T = len(tokens)
        pos = torch.arange(past, past + T)
        x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
        results = [x]
        after = []
        layers = self.cfg["layers"]
        for i, layer in enumerate(layers):
            p = f"l{i}."
            kept = state.setdefault(i, {})
            h = norm_around_zero(x, w[p + "norm1"], eps)
            before = kept.get("before", torch.zeros(x.shape[1], dtype=F64))
            h, kept["before"] = token_shift(h, before, w[p + "shift"])
            h = st(h)
            m = layer["mixer"]
            mw = self.sub(p + "mix.")
            if layer["type"] == "attention":
                borrowed = state[int(m["kv_from"])] if m.get("kv_from") is not None else None
                y = differential_attention(h, pos, mw, m, eps, kept, st, borrowed)
            else:
                y = latent_attention(h, pos, mw, m, eps, kept, st)
            x = x + norm_around_zero(y, w[p + "norm1b"], eps)
            mlp = layer.get("mlp")
            if mlp is not None:
                h2 = st(norm_around_zero(x, w[p + "norm2"], eps))
                fw = self.sub(p + "mlp.")
                y = dense_ff(h2, fw, eps, st) if mlp.get("kind", "dense") == "dense" else expert_ff(h2, fw, mlp, st)
                x = x + norm_around_zero(y, w[p + "norm2b"], eps)
            results.append(x)
            x = depth_average(results, w[p + "dwa"])
            after.append(x)
        state["length"] = past + T
        logits = st(norm_around_zero(x, w["final.norm"], eps)) @ w["head"].T * float(self.cfg["logit_scale"])
        return (logits, torch.stack(after)) if trace else logits


# ---- helpers of the tests: tensor shapes from the configuration, random weights, whole runs ----------------------------
def tensor_shapes(config: dict) -> Dict[str, tuple]:
    """Name -> shape of every tensor that a model of ``config`` holds."""
    W, V = int(config["width"]), int(config["vocab"])
    out = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        for n in ("norm1", "norm1b", "shift"):
            out[p + n] = (W,)
        out[p + "dwa"] = (i + 2,)
        H, d, dv = int(m["heads"]), int(m["dim"]), int(m.get("vdim", m["dim"]))
        if layer["type"] == "attention":
            G = int(m.get("kv_heads", H))
            out[p + "mix.q"] = (H * 2 * d, W)
            if m.get("kv_from") is None:
                out[p + "mix.k"] = (G * 2 * d, W)
                out[p + "mix.v"] = (G * dv, W)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                out[p + "mix." + n] = (d,)
        else:
            r, dr = int(m["kv_rank"]), int(m.get("rot_dim", 0) or 0)
            out[p + "mix.q"] = (H * (d + dr), W)
            out[p + "mix.dkv"] = (r + dr, W)
            out[p + "mix.dkv.norm"] = (r,)
            out[p + "mix.uk"] = (H * d, r)
            out[p + "mix.uv"] = (H * dv, r)
            out[p + "mix.g"] = (H * dv if dr else H, W)
        out[p + "mix.o"] = (W, H * dv)
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        out[p + "norm2"] = (W,)
        out[p + "norm2b"] = (W,)
        if mlp.get("kind", "dense") == "dense":
            F = int(mlp["ff"])
            out.update({p + "mlp.up": (F, W), p + "mlp.down": (W, F), p + "mlp.act": (4,)})
        else:
            E, F = int(mlp["router"]["experts"]), int(mlp["expert"]["ff"])
            out.update({p + "mlp.router": (E, W), p + "mlp.router.b": (E,)})
            for e in range(E):
                out.update({p + f"mlp.e{e}.gate": (F, W), p + f"mlp.e{e}.up": (F, W), p + f"mlp.e{e}.down": (W, F)})
    return out


def random_weights(config: dict, seed: int, sharpen: float = 3.0) -> Dict[str, torch.Tensor]:
    """Weights that make every mechanism matter: projections of unit gain, queries scaled by ``sharpen`` so that the
    softmax is peaked, norm weights, shifts, averaging coefficients and router biases well away from 0 and 1."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        last = name.rsplit(".", 1)[-1]
        if len(shape) == 2:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
            if name.endswith("mix.q"):
                t = t * sharpen
            if name == "embed":
                t = torch.randn(shape, generator=g)
        elif last == "shift":
            t = torch.rand(shape, generator=g) * 0.8 + 0.1
        elif last == "dwa":
            t = torch.softmax(torch.randn(shape, generator=g), 0) * 1.3
        elif last == "act":
            t = torch.tensor([0.8, 0.5, 0.3, 0.1]) + 0.2 * torch.randn(4, generator=g)
        elif last == "b":
            t = 0.5 * torch.randn(shape, generator=g)
        elif last in ("lq1", "lk1", "lq2", "lk2"):
            t = 0.4 * torch.randn(shape, generator=g)
        elif name.endswith("dkv.norm"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        else:                       # norms stored as their distance from one
            t = 0.2 * torch.randn(shape, generator=g)
        out[name] = t.to(torch.float32)
    return out


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens, stored: Round = same, portions=None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one sequence, fed whole or in the given portions."""
    model = PlainVemepel(config, weights, stored)
    state: dict = {}
    if not portions:
        return model.feed(state, list(tokens))
    out, at = [], 0
    for n in portions:
        out.append(model.feed(state, list(tokens[at:at + n])))
        at += n
    assert at == len(tokens)
    return torch.cat(out, 0)
