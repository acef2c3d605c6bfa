"""Typed configuration of the Zonevik decoder, read from its own ``config.json`` keys.

    {"architecture": "Zonevik", "vocab": V, "width": W, "norm": {"eps": e}, "embedding": {"scale": c},
     "loop": {"start": a, "stop": b, "times": n},
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale",
                           "rot": {"base", "dims", "scaling": {"factor", "original", "fast", "slow"}}},
                 "mlp": {"kind": "moe", "router": {"experts", "top", "groups": {"count", "keep"}}, "expert": {"ff"}}},
                {"type": "delta", "mixer": {"heads", "kv_heads", "dim", "vdim", "conv"}, "mlp": ...},
                {"type": "parallel",
                 "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size", "keep_first"}},
                           "right": {"heads", "vdim", "state", "groups", "conv", "norm_groups"}}, "mlp": null}, ...]}

Every size and constant is read from there, layer by layer; nothing is the same for two layers unless the file says so.
``loop`` (optional): layers ``start .. stop - 1`` run ``times`` times in a row with the same weights.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig, require_float, require_int
from .registry import register_preset_folder
from .vabelorn import _obj, _sub

# The file gives no longest sequence; position tables are made for what the engine is asked to hold, up to this.
MAX_POSITIONS = 1 << 17


@dataclass(frozen=True)
class RotaryScaling:
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class GatedAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_base: float
    rot_dims: int
    rot_scaling: Optional[RotaryScaling]


@dataclass(frozen=True)
class WindowAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]
    keep_first: int


@dataclass(frozen=True)
class StateSpace:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int


@dataclass(frozen=True)
class SideBySide:
    left: WindowAttention
    right: StateSpace


@dataclass(frozen=True)
class GatedDelta:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class RoutedFf:
    experts: int
    top: int
    ff: int
    groups: int        # 1: the experts are not grouped
    keep_groups: int


@dataclass(frozen=True)
class ZonevikLayer:
    type: str                       # "attention" | "delta" | "parallel"
    mixer: Any                      # GatedAttention | GatedDelta | SideBySide
    mlp: Optional[RoutedFf]


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int


def _heads(d: Dict[str, Any], where: str):
    whole, num = _sub(d, where)
    heads, kv = whole("heads"), whole("kv_heads", default=d.get("heads"))
    if heads % kv:
        raise ConfigError(f"config.json: {where}: 'heads' ({heads}) must be a multiple of 'kv_heads' ({kv})")
    dim = whole("dim")
    return whole, num, heads, kv, dim


def _mlp(d: Any, where: str) -> Optional[RoutedFf]:
    if d is None:
        return None
    d = _obj(d, where)
    kind = d.get("kind", "moe")
    if kind != "moe":
        raise ConfigError(f"config.json: {where}: 'kind' must be 'moe', got {kind!r}")
    r = _obj(d.get("router"), where + ".router")
    whole, _ = _sub(r, where + ".router")
    experts, top = whole("experts"), whole("top")
    groups, keep = 1, 1
    if r.get("groups"):
        gwhole, _ = _sub(_obj(r["groups"], where + ".router.groups"), where + ".router.groups")
        groups = gwhole("count")
        keep = gwhole("keep", default=groups)
        if experts % groups or keep > groups:
            raise ConfigError(f"config.json: {where}.router.groups: {experts} experts do not form {groups} equal groups of which "
                              f"{keep} are kept")
    if top > keep * (experts // groups):
        raise ConfigError(f"config.json: {where}.router: 'top' ({top}) exceeds the {keep * (experts // groups)} experts that can be chosen")
    ewhole, _ = _sub(_obj(d.get("expert"), where + ".expert"), where + ".expert")
    return RoutedFf(experts=experts, top=top, ff=ewhole("ff"), groups=groups, keep_groups=keep)


@dataclass(frozen=True)
class ZonevikConfig(ModelConfig):
    vocab: int
    width: int
    layers: Tuple[ZonevikLayer, ...]
    norm_eps: float
    embedding_scale: float = 1.0
    loop: Optional[Loop] = None
    eos_token_id: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    architecture: str = field(default="Zonevik")

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ZonevikConfig":
        vocab = require_int(d, "vocab")
        width = require_int(d, "width")
        _, nnum = _sub(_obj(d.get("norm"), "'norm'"), "'norm'")
        eps = nnum("eps")
        scale = 1.0
        if isinstance(d.get("embedding"), dict) and d["embedding"].get("scale") is not None:
            _, enum = _sub(d["embedding"], "'embedding'")
            scale = enum("scale")
        raw = d.get("layers")
        if not isinstance(raw, (list, tuple)) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw):
            where = f"layers[{i}]"
            entry = _obj(entry, where)
            kind = entry.get("type")
            m = _obj(entry.get("mixer"), where + ".mixer")
            mw = where + ".mixer"
            if kind == "attention":
                whole, num, heads, kv, dim = _heads(m, mw)
                rot = m.get("rot")
                base, dims, scaling = 10000.0, 0, None
                if rot:
                    rwhole, rnum = _sub(_obj(rot, mw + ".rot"), mw + ".rot")
                    dims = rwhole("dims", minimum=0)
                    if dims % 2 or dims > dim:
                        raise ConfigError(f"config.json: {mw}.rot: 'dims' must be even and at most the head size {dim}, got {dims}")
                    base = rnum("base")
                    if rot.get("scaling"):
                        _, snum = _sub(_obj(rot["scaling"], mw + ".rot.scaling"), mw + ".rot.scaling")
                        scaling = RotaryScaling(factor=snum("factor"), original=snum("original"), fast=snum("fast"), slow=snum("slow"))
                mixer = GatedAttention(heads=heads, kv_heads=kv, dim=dim, vdim=whole("vdim", default=dim), scale=num("scale"),
                                       rot_base=base, rot_dims=dims, rot_scaling=scaling)
            elif kind == "delta":
                whole, _, heads, kv, dim = _heads(m, mw)
                mixer = GatedDelta(heads=heads, kv_heads=kv, dim=dim, vdim=whole("vdim", default=dim), conv=whole("conv"))
            elif kind == "parallel":
                lw = mw + ".left"
                left = _obj(m.get("left"), lw)
                whole, num, heads, kv, dim = _heads(left, lw)
                window, keep_first = None, 0
                if left.get("mask"):
                    mwhole, _ = _sub(_obj(left["mask"], lw + ".mask"), lw + ".mask")
                    window = mwhole("size")
                    keep_first = mwhole("keep_first", minimum=0, default=0)
                att = WindowAttention(heads=heads, kv_heads=kv, dim=dim, vdim=whole("vdim", default=dim), scale=num("scale"),
                                      window=window, keep_first=keep_first)
                rw = mw + ".right"
                right = _obj(m.get("right"), rw)
                whole, _ = _sub(right, rw)
                heads, groups, vdim = whole("heads"), whole("groups", default=1), whole("vdim")
                norm_groups = whole("norm_groups", default=1)
                if heads % groups:
                    raise ConfigError(f"config.json: {rw}: 'heads' ({heads}) must be a multiple of 'groups' ({groups})")
                if (heads * vdim) % norm_groups:
                    raise ConfigError(f"config.json: {rw}: heads * vdim ({heads * vdim}) must be a multiple of 'norm_groups' ({norm_groups})")
                mixer = SideBySide(left=att, right=StateSpace(heads=heads, vdim=vdim, state=whole("state"), groups=groups,
                                                              conv=whole("conv"), norm_groups=norm_groups))
            else:
                raise ConfigError(f"config.json: {where}: 'type' must be 'attention', 'delta' or 'parallel', got {kind!r}")
            layers.append(ZonevikLayer(type=kind, mixer=mixer, mlp=_mlp(entry.get("mlp"), where + ".mlp")))
        loop = None
        if d.get("loop"):
            lwhole, _ = _sub(_obj(d["loop"], "'loop'"), "'loop'")
            loop = Loop(start=lwhole("start", minimum=0), stop=lwhole("stop"), times=lwhole("times"))
            if not loop.start < loop.stop <= len(layers):
                raise ConfigError(f"config.json: 'loop': layers {loop.start} .. {loop.stop - 1} are not layers of this model "
                                  f"({len(layers)} layers)")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else (eos,)))
        for e in eos_ids:
            if not 0 <= e < vocab:
                raise ConfigError(f"config.json: 'eos_token_id' {e} is outside the vocabulary (0..{vocab - 1})")
        bos = d.get("bos_token_id")
        return cls(vocab=vocab, width=width, layers=tuple(layers), norm_eps=eps, embedding_scale=scale, loop=loop,
                   eos_token_id=eos_ids, bos_token_id=None if bos is None else int(bos),
                   architecture=str(d.get("architecture") or "Zonevik"))

    def to_dict(self) -> Dict[str, Any]:
        layers = []
        for layer in self.layers:
            m = layer.mixer
            if layer.type == "attention":
                mixer: Dict[str, Any] = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}
                if m.rot_dims:
                    mixer["rot"] = {"base": m.rot_base, "dims": m.rot_dims}
                    if m.rot_scaling is not None:
                        s = m.rot_scaling
                        mixer["rot"]["scaling"] = {"factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}
            elif layer.type == "delta":
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "conv": m.conv}
            else:
                a, b = m.left, m.right
                left: Dict[str, Any] = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale}
                if a.window:
                    left["mask"] = {"size": a.window, "keep_first": a.keep_first}
                mixer = {"left": left, "right": {"heads": b.heads, "vdim": b.vdim, "state": b.state, "groups": b.groups,
                                                 "conv": b.conv, "norm_groups": b.norm_groups}}
            mlp = None
            if layer.mlp is not None:
                f = layer.mlp
                router: Dict[str, Any] = {"experts": f.experts, "top": f.top}
                if f.groups > 1:
                    router["groups"] = {"count": f.groups, "keep": f.keep_groups}
                mlp = {"kind": "moe", "router": router, "expert": {"ff": f.ff}}
            layers.append({"type": layer.type, "mixer": mixer, "mlp": mlp})
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                             "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale}, "layers": layers}
        if self.loop is not None:
            d["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        return d

    @property
    def max_positions(self) -> int:
        return MAX_POSITIONS

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def stop_token_ids(self) -> Tuple[int, ...]:
        return self.eos_token_id

    @property
    def bos_token(self) -> int:
        return self.bos_token_id if self.bos_token_id is not None else 0


register_preset_folder(os.path.join(os.path.dirname(os.path.abspath(__file__)), "presets"))
