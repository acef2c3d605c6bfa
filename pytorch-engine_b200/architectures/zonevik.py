"""The Zonevik decoder as a plan of parts.

The embedding's rows are multiplied by ``embedding.scale``.  Every block is a ``sandwich`` arrangement (``parts/block.py``)
whose four norms are Dynamic Tanh (``tanh(alpha x) * w + b``, no statistics).  A range of layers may run several times in a
row with the same weights (``loop``): every run is an entry of the plan's order with a cache entry of its own, and the
first block of the range carries an ``input_mix`` part that replaces the stream by ``W [x ; x0]`` (``x0`` the embedding's
output) in front of every pass.  Layer by layer ``config.json`` chooses the mixer

* ``attention``: grouped-query softmax attention, interleaved rotary pairs on the first ``rot.dims`` features with YaRN-scaled
  frequencies, and a sigmoid output gate per feature (``parts/attention.py``);
* ``delta``: the gated delta rule behind short convolutions, one decay per head, silu output gate (``parts/delta_rule.py``);
* ``parallel``: two mixers on the same input, each output divided by its root mean square over the width and weighted,
  half their sum: softmax attention with biases, no positions, a sliding window that keeps the sequence's first positions
  visible (``parts/attention.py``), beside a selective state-space mixer (``parts/ssd.py``);

and the feed-forward: none, or routed experts with sigmoid scores chosen among the best groups of neighbouring experts
(``parts/moe.py``).  Final Dynamic Tanh norm; the output head is the embedding table itself (without the scale).

Tensor names: ``embed``, ``loop.in``, ``final.norm{,.b,.alpha}``; layer i: ``l<i>.norm1, norm1b, norm2, norm2b`` each with
``.b`` and ``.alpha``; ``l<i>.mix.{q,k,v,g,o}`` (attention); ``l<i>.mix.{q,k,v,b,a,g,o,norm,A_log,dt_bias}`` and
``l<i>.mix.{q,k,v}.conv`` (delta); ``l<i>.mix.left.{q,k,v,o,out}``, ``l<i>.mix.left.{q,k,v}.b``,
``l<i>.mix.right.{in,conv,conv.b,dt_bias,A_log,D,norm,o,out}`` (parallel); ``l<i>.mlp.router``, ``l<i>.mlp.e<j>.{gate,up,down}``.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.zonevik import ZonevikConfig
from ..parts.spec import BlockSpec, ModelPlan, PartSpec, RunStep


def zonevik_plan(cfg: ZonevikConfig) -> ModelPlan:
    h, eps = cfg.width, cfg.norm_eps
    norm = lambda name: PartSpec("dynamic_tanh", {"dim": h}, {"weight": name, "bias": f"{name}.b", "alpha": f"{name}.alpha"})
    positions = {}

    def position(spec: PartSpec) -> str:
        """One position encoding per distinct set of constants, shared by the layers that use it."""
        key = repr(sorted((k, repr(v)) for k, v in spec.params.items()))
        for name, have in positions.items():
            if repr(sorted((k, repr(v)) for k, v in have.params.items())) == key:
                return name
        name = f"rot{len(positions)}"
        positions[name] = spec
        return name

    blocks = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}"
        m = layer.mixer
        q = f"{p}.mix"
        parts = {}
        if cfg.loop is not None and i == cfg.loop.start:
            parts["inject"] = ("stream", PartSpec("input_mix", {"dim": h}, {"weight": "loop.in"}))
        parts["mixer_norm"] = ("norm", norm(f"{p}.norm1"))
        if layer.type == "attention":
            pos = None
            if m.rot_dims > 0:
                sc = m.rot_scaling
                scaling = None if sc is None else {"factor": sc.factor, "original": sc.original, "fast": sc.fast, "slow": sc.slow}
                pos = position(PartSpec("rope", {"rotary_dim": m.rot_dims, "theta": m.rot_base, "style": "interleaved",
                                                 "scaling": scaling, "max_positions": cfg.max_positions, "exact": True}))
            parts["mixer"] = ("mixer", PartSpec(
                "attention",
                {"hidden": h, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "v_head_dim": m.vdim,
                 "qk_norm": False, "eps": eps, "scale": m.scale, "window": None, "position": pos, "output_gate": "sigmoid"},
                {"q_proj": f"{q}.q", "k_proj": f"{q}.k", "v_proj": f"{q}.v", "g_proj": f"{q}.g", "o_proj": f"{q}.o"}))
        elif layer.type == "delta":
            parts["mixer"] = ("mixer", PartSpec(
                "gated_delta",
                {"hidden": h, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "v_head_dim": m.vdim,
                 "conv": m.conv, "eps": eps, "decay": "head", "gate": "silu"},
                {"q_proj": f"{q}.q", "k_proj": f"{q}.k", "v_proj": f"{q}.v", "q_conv": f"{q}.q.conv", "k_conv": f"{q}.k.conv",
                 "v_conv": f"{q}.v.conv", "b_proj": f"{q}.b", "a_proj": f"{q}.a", "A_log": f"{q}.A_log", "dt_bias": f"{q}.dt_bias",
                 "g_proj": f"{q}.g", "norm": f"{q}.norm", "o_proj": f"{q}.o"}))
        else:
            a, b = m.left, m.right
            lq, rq = f"{q}.left", f"{q}.right"
            parts["left"] = ("mixer", PartSpec(
                "attention",
                {"hidden": h, "n_heads": a.heads, "n_kv_heads": a.kv_heads, "head_dim": a.dim, "v_head_dim": a.vdim,
                 "qk_norm": False, "eps": eps, "scale": a.scale, "window": a.window, "keep_first": a.keep_first, "position": None,
                 "bias": True},
                {"q_proj": f"{lq}.q", "k_proj": f"{lq}.k", "v_proj": f"{lq}.v", "q_bias": f"{lq}.q.b", "k_bias": f"{lq}.k.b",
                 "v_bias": f"{lq}.v.b", "o_proj": f"{lq}.o"}))
            parts["right"] = ("mixer", PartSpec(
                "ssd",
                {"hidden": h, "n_heads": b.heads, "v_head_dim": b.vdim, "state": b.state, "groups": b.groups, "conv": b.conv,
                 "norm_groups": b.norm_groups, "eps": eps},
                {"in_proj": f"{rq}.in", "conv": f"{rq}.conv", "conv_bias": f"{rq}.conv.b", "dt_bias": f"{rq}.dt_bias",
                 "A_log": f"{rq}.A_log", "D": f"{rq}.D", "norm": f"{rq}.norm", "o_proj": f"{rq}.o"}))
            parts["combine"] = ("stream", PartSpec("normed_mean", {"dim": h, "eps": eps, "scale": 0.5},
                                                   {"weight_a": f"{lq}.out", "weight_b": f"{rq}.out"}))
        parts["post_mixer_norm"] = ("norm", norm(f"{p}.norm1b"))
        mlp = layer.mlp
        if mlp is not None:
            q = f"{p}.mlp"
            parts["ffn_norm"] = ("norm", norm(f"{p}.norm2"))
            names = {"router": f"{q}.router"}
            for e in range(mlp.experts):
                names.update({f"e{e}.{s}": f"{q}.e{e}.{s}" for s in ("gate", "up", "down")})
            parts["ffn"] = ("feed_forward", PartSpec(
                "routed_experts",
                {"hidden": h, "n_experts": mlp.experts, "n_identity": 0, "top": mlp.top, "intermediate": mlp.ff,
                 "activation": "silu", "choice": "sigmoid_groups", "groups": mlp.groups, "keep_groups": mlp.keep_groups,
                 "shared": None}, names))
            parts["post_ffn_norm"] = ("norm", norm(f"{p}.norm2b"))
        blocks.append(BlockSpec("sandwich", parts, name=f"layer {i}"))
    # the order: a looped range runs `times` times over; every run beyond the first keeps cache entries of its own
    n = len(cfg.layers)
    order = []
    if cfg.loop is None:
        order = [RunStep(block=i) for i in range(n)]
    else:
        a, b, times = cfg.loop.start, cfg.loop.stop, cfg.loop.times
        order = [RunStep(block=i) for i in range(a)]
        for t in range(times):
            order += [RunStep(block=i, cache=i if t == 0 else n + (t - 1) * (b - a) + (i - a)) for i in range(a, b)]
        order += [RunStep(block=i) for i in range(b, n)]
    # a layer without a feed-forward may still carry the two norms around it in its file
    ignored = tuple(f"l{i}.{nm}{suffix}" for i, layer in enumerate(cfg.layers) if layer.mlp is None
                    for nm in ("norm2", "norm2b") for suffix in ("", ".b", ".alpha"))
    return ModelPlan(
        hidden_size=h,
        vocab_size=cfg.vocab,
        max_positions=cfg.max_positions,
        embedding=PartSpec("token_embedding", {"vocab": cfg.vocab, "hidden": h, "scale": cfg.embedding_scale}, {"weight": "embed"}),
        blocks=tuple(blocks),
        order=tuple(order),
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab": cfg.vocab, "hidden": h}, {"weight": "embed"}),
        positions=positions,
        ignored=ignored,
        keep_embedding_output=cfg.loop is not None,
    )


register_architecture("Zonevik", ZonevikConfig, zonevik_plan, replace=True)
