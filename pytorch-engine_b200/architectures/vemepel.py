"""The Vemepel decoder as a plan of parts.

Every block is a ``sandwich_depth`` arrangement (``parts/block.py``): an RMS norm before and after each sublayer (weights
stored as their distance from one), a token shift on what the mixer reads, and behind the block a weighted sum over the
embedding's output and every block's result so far.  Layer by layer ``config.json`` chooses the mixer

* ``latent_attention``: keys and values expanded from a cached low-rank row, no positions, one output gate a head;
* ``latent_attention_2``: the same with a rotated part beside every head's keys (interleaved rotary pairs) and one
  output gate a feature (both ``parts/latent_attention.py``);
* ``attention``: differential attention (two softmax maps per head, the second subtracted) with a chunk mask; a layer
  with ``kv_from`` reads the keys and values that an earlier layer cached (``parts/diff_attention.py``);

and the feed-forward: none, a dense one with the PolyNorm activation (``parts/dense_ff.py``), or routed experts chosen by
their logits and weighted by a softmax over the chosen (``parts/moe.py``).  Final RMS norm, an output head of its own,
logits times ``logit_scale``.

Tensor names: ``embed``, ``final.norm``, ``head``; layer i: ``l<i>.norm1, norm1b, norm2, norm2b, shift, dwa``;
``l<i>.mix.{q,dkv,dkv.norm,uk,uv,g,o}`` (latent) or ``l<i>.mix.{q,k,v,lq1,lk1,lq2,lk2,o}`` (differential; no k, v with
``kv_from``); ``l<i>.mlp.{up,down,act}`` (dense) or ``l<i>.mlp.{router,router.b}``, ``l<i>.mlp.e<j>.{gate,up,down}`` (routed).
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.vemepel import DenseFf, VemepelConfig
from ..parts.spec import BlockSpec, ModelPlan, PartSpec, RunStep


def vemepel_plan(cfg: VemepelConfig) -> ModelPlan:
    h, eps = cfg.width, cfg.norm_eps
    norm = lambda name: PartSpec("rmsnorm", {"dim": h, "eps": eps, "offset": 1.0}, {"weight": name})
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

    depth = len(cfg.layers)
    # what the cache may drop of a layer's keys: the chunk that the layer and every layer that reads its keys share
    readers = {}
    for i, layer in enumerate(cfg.layers):
        if layer.type == "attention":
            owner = i if layer.mixer.kv_from is None else layer.mixer.kv_from
            readers.setdefault(owner, set()).add(layer.mixer.chunk)
    blocks, order = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}"
        m = layer.mixer
        q = f"{p}.mix"
        parts = {"mixer_norm": ("norm", norm(f"{p}.norm1")),
                 "shift": ("stream", PartSpec("token_shift", {"dim": h}, {"mix": f"{p}.shift"}))}
        run = RunStep(block=i)
        if layer.type == "attention":
            shared = m.kv_from is not None
            chunks = readers[m.kv_from if shared else i]
            names = {"q_proj": f"{q}.q", "o_proj": f"{q}.o", "lq1": f"{q}.lq1", "lk1": f"{q}.lk1", "lq2": f"{q}.lq2",
                     "lk2": f"{q}.lk2"}
            if not shared:
                names.update({"k_proj": f"{q}.k", "v_proj": f"{q}.v"})
            parts["mixer"] = ("mixer", PartSpec(
                "diff_attention",
                {"hidden": h, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "v_head_dim": m.vdim,
                 "scale": m.scale, "diff": m.diff, "eps": eps, "chunk": m.chunk, "shared_kv": shared,
                 "cache_chunk": next(iter(chunks)) if len(chunks) == 1 else None}, names))
            if shared:
                run = RunStep(block=i, cache=m.kv_from, writes_cache=False, shared=("mixer",))
        else:
            pos = None
            if m.rot_dim and m.rot_dims:
                pos = position(PartSpec("rope", {"rotary_dim": m.rot_dims, "theta": m.rot_base, "style": "interleaved",
                                                 "scaling": None, "max_positions": cfg.max_positions, "exact": True}))
            parts["mixer"] = ("mixer", PartSpec(
                "latent_attention",
                {"hidden": h, "n_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "v_head_dim": m.vdim,
                 "kv_rank": m.kv_rank, "scale": m.scale, "eps": eps, "position": pos,
                 "gate": "feature" if layer.type == "latent_attention_2" else "head"},
                {"q_proj": f"{q}.q", "dkv_proj": f"{q}.dkv", "dkv_norm": f"{q}.dkv.norm", "uk_proj": f"{q}.uk",
                 "uv_proj": f"{q}.uv", "g_proj": f"{q}.g", "o_proj": f"{q}.o"}))
        parts["post_mixer_norm"] = ("norm", norm(f"{p}.norm1b"))
        mlp = layer.mlp
        q = f"{p}.mlp"
        if mlp is not None:
            parts["ffn_norm"] = ("norm", norm(f"{p}.norm2"))
            if isinstance(mlp, DenseFf):
                parts["ffn"] = ("feed_forward", PartSpec(
                    "dense_act", {"hidden": h, "intermediate": mlp.ff, "activation": "polynorm", "eps": eps},
                    {"up_proj": f"{q}.up", "down_proj": f"{q}.down", "act": f"{q}.act"}))
            else:
                names = {"router": f"{q}.router", "router_bias": f"{q}.router.b"}
                for e in range(mlp.experts):
                    names.update({f"e{e}.{s}": f"{q}.e{e}.{s}" for s in ("gate", "up", "down")})
                parts["ffn"] = ("feed_forward", PartSpec(
                    "routed_experts",
                    {"hidden": h, "n_experts": mlp.experts, "n_identity": 0, "top": mlp.top, "intermediate": mlp.ff,
                     "activation": "silu", "choice": "top_logits", "shared": None}, names))
            parts["post_ffn_norm"] = ("norm", norm(f"{p}.norm2b"))
        parts["average"] = ("stream", PartSpec("depth_average", {"terms": i + 2}, {"coeff": f"{p}.dwa"}))
        blocks.append(BlockSpec("sandwich_depth", parts, name=f"layer {i}", params={"index": i, "depth": depth}))
        order.append(run)
    # a layer without a feed-forward may still carry the two norms around it in its file
    ignored = tuple(f"l{i}.{n}" for i, layer in enumerate(cfg.layers) if layer.mlp is None for n in ("norm2", "norm2b"))
    return ModelPlan(
        hidden_size=h,
        vocab_size=cfg.vocab,
        max_positions=cfg.max_positions,
        embedding=PartSpec("token_embedding", {"vocab": cfg.vocab, "hidden": h}, {"weight": "embed"}),
        blocks=tuple(blocks),
        order=tuple(order),
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab": cfg.vocab, "hidden": h, "scale": cfg.logit_scale}, {"weight": "head"}),
        positions=positions,
        ignored=ignored,
    )


register_architecture("Vemepel", VemepelConfig, vemepel_plan, replace=True)
