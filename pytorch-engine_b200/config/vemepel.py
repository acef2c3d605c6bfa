"""Typed configuration of the Vemepel decoder, read from its own ``config.json`` keys.

    {"architecture": "Vemepel", "vocab": V, "width": W, "logit_scale": s, "norm": {"eps": e},
     "layers": [{"type": "latent_attention",   "mixer": {"heads", "dim", "vdim", "kv_rank", "scale"}, "mlp": ...},
                {"type": "latent_attention_2", "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "scale",
                                                         "rot": {"base", "dims"}}, "mlp": ...},
                {"type": "attention", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "diff", "mask": {"size"},
                                                "kv_from": j}, "mlp": ...}, ...]}

with ``mlp`` one of ``null``, ``{"kind": "dense", "ff": F}`` and ``{"kind": "moe", "router": {"experts", "top"},
"expert": {"ff"}}``.  Every size and constant is read from there; nothing is the same for two layers unless the file
says so.
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
class LatentMixer:
    """Keys and values expanded from a cached row of ``kv_rank`` features; with ``rot_dim`` > 0 a rotated part of
    that many features rides beside every head's keys (``rot_dims`` of them turn, with base ``rot_base``)."""

    heads: int
    dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_dim: int = 0
    rot_base: float = 10000.0
    rot_dims: int = 0


@dataclass(frozen=True)
class DiffMixer:
    """Two softmax maps per head; ``chunk``: keys are visible inside the query's own block of that many positions
    (None: every earlier key); ``kv_from``: the layer whose keys and values this one reads (None: its own)."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    chunk: Optional[int] = None
    kv_from: Optional[int] = None


@dataclass(frozen=True)
class DenseFf:
    ff: int


@dataclass(frozen=True)
class RoutedFf:
    experts: int
    top: int
    ff: int


@dataclass(frozen=True)
class VemepelLayer:
    type: str                       # "latent_attention" | "latent_attention_2" | "attention"
    mixer: Any                      # LatentMixer | DiffMixer
    mlp: Any                        # None | DenseFf | RoutedFf


def _mlp(d: Any, where: str):
    if d is None:
        return None
    d = _obj(d, where)
    kind = d.get("kind", "dense")
    if kind == "dense":
        whole, _ = _sub(d, where)
        return DenseFf(ff=whole("ff"))
    if kind == "moe":
        whole, _ = _sub(_obj(d.get("router"), where + ".router"), where + ".router")
        experts, top = whole("experts"), whole("top")
        if top > experts:
            raise ConfigError(f"config.json: {where}.router: 'top' ({top}) exceeds the {experts} experts")
        ewhole, _ = _sub(_obj(d.get("expert"), where + ".expert"), where + ".expert")
        return RoutedFf(experts=experts, top=top, ff=ewhole("ff"))
    raise ConfigError(f"config.json: {where}: 'kind' must be 'dense' or 'moe', got {kind!r}")


def _latent(m: Dict[str, Any], where: str, rotated: bool) -> LatentMixer:
    whole, num = _sub(m, where)
    dim = whole("dim")
    rot_dim, base, dims = 0, 10000.0, 0
    if rotated:
        rot_dim = whole("rot_dim")
        rwhole, rnum = _sub(_obj(m.get("rot"), where + ".rot"), where + ".rot")
        base, dims = rnum("base"), rwhole("dims", minimum=0)
        if dims % 2 or dims > rot_dim:
            raise ConfigError(f"config.json: {where}.rot: 'dims' must be even and at most 'rot_dim' ({rot_dim}), got {dims}")
    return LatentMixer(heads=whole("heads"), dim=dim, vdim=whole("vdim", default=dim), kv_rank=whole("kv_rank"),
                       scale=num("scale"), rot_dim=rot_dim, rot_base=base, rot_dims=dims)


def _diff(m: Dict[str, Any], where: str, index: int) -> DiffMixer:
    whole, num = _sub(m, where)
    heads = whole("heads")
    kv = whole("kv_heads", default=heads)
    if heads % kv:
        raise ConfigError(f"config.json: {where}: 'heads' ({heads}) must be a multiple of 'kv_heads' ({kv})")
    dim = whole("dim")
    chunk = None
    if m.get("mask"):
        mwhole, _ = _sub(_obj(m["mask"], where + ".mask"), where + ".mask")
        chunk = mwhole("size")
    src = m.get("kv_from")
    if src is not None:
        src = whole("kv_from", minimum=0)
        if src >= index:
            raise ConfigError(f"config.json: {where}: 'kv_from' ({src}) must name an earlier layer than {index}")
    return DiffMixer(heads=heads, kv_heads=kv, dim=dim, vdim=whole("vdim", default=dim), scale=num("scale"),
                     diff=num("diff", positive=False), chunk=chunk, kv_from=src)


@dataclass(frozen=True)
class VemepelConfig(ModelConfig):
    vocab: int
    width: int
    layers: Tuple[VemepelLayer, ...]
    norm_eps: float
    logit_scale: float = 1.0
    eos_token_id: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    architecture: str = field(default="Vemepel")

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "VemepelConfig":
        vocab = require_int(d, "vocab")
        width = require_int(d, "width")
        _, nnum = _sub(_obj(d.get("norm"), "'norm'"), "'norm'")
        eps = nnum("eps")
        raw = d.get("layers")
        if not isinstance(raw, (list, tuple)) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw):
            where = f"layers[{i}]"
            entry = _obj(entry, where)
            kind = entry.get("type")
            m = _obj(entry.get("mixer"), where + ".mixer")
            if kind == "latent_attention":
                mixer = _latent(m, where + ".mixer", rotated=False)
            elif kind == "latent_attention_2":
                mixer = _latent(m, where + ".mixer", rotated=True)
            elif kind == "attention":
                mixer = _diff(m, where + ".mixer", i)
            else:
                raise ConfigError(f"config.json: {where}: 'type' must be 'latent_attention', 'latent_attention_2' or "
                                  f"'attention', got {kind!r}")
            layers.append(VemepelLayer(type=kind, mixer=mixer, mlp=_mlp(entry.get("mlp"), where + ".mlp")))
        for i, layer in enumerate(layers):
            m = layer.mixer
            if layer.type == "attention" and m.kv_from is not None:
                src = layers[m.kv_from]
                s = src.mixer
                if src.type != "attention" or s.kv_from is not None:
                    raise ConfigError(f"config.json: layers[{i}].mixer: 'kv_from' must name an attention layer with keys "
                                      f"and values of its own, layers[{m.kv_from}] is not one")
                if (s.kv_heads, s.dim, s.vdim) != (m.kv_heads, m.dim, m.vdim):
                    raise ConfigError(f"config.json: layers[{i}].mixer: kv_heads, dim and vdim must equal those of "
                                      f"layers[{m.kv_from}], whose keys and values it reads")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else (eos,)))
        for e in eos_ids:
            if not 0 <= e < vocab:
                raise ConfigError(f"config.json: 'eos_token_id' {e} is outside the vocabulary (0..{vocab - 1})")
        bos = d.get("bos_token_id")
        return cls(vocab=vocab, width=width, layers=tuple(layers), norm_eps=eps,
                   logit_scale=require_float(d, "logit_scale", default=1.0), eos_token_id=eos_ids,
                   bos_token_id=None if bos is None else int(bos), architecture=str(d.get("architecture") or "Vemepel"))

    def to_dict(self) -> Dict[str, Any]:
        layers = []
        for layer in self.layers:
            m = layer.mixer
            if layer.type == "attention":
                mixer: Dict[str, Any] = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim,
                                         "scale": m.scale, "diff": m.diff}
                if m.chunk:
                    mixer["mask"] = {"size": m.chunk}
                if m.kv_from is not None:
                    mixer["kv_from"] = m.kv_from
            else:
                mixer = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "kv_rank": m.kv_rank, "scale": m.scale}
                if layer.type == "latent_attention_2":
                    mixer.update({"rot_dim": m.rot_dim, "rot": {"base": m.rot_base, "dims": m.rot_dims}})
            mlp = layer.mlp
            if isinstance(mlp, DenseFf):
                mlp_d: Any = {"kind": "dense", "ff": mlp.ff}
            elif mlp is not None:
                mlp_d = {"kind": "moe", "router": {"experts": mlp.experts, "top": mlp.top}, "expert": {"ff": mlp.ff}}
            else:
                mlp_d = None
            layers.append({"type": layer.type, "mixer": mixer, "mlp": mlp_d})
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                             "logit_scale": self.logit_scale, "norm": {"eps": self.norm_eps}, "layers": layers}
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
