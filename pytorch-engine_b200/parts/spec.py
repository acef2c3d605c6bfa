"""The data that describes a model: which parts, with which constants, in which order.

An architecture turns its typed configuration into a ``ModelPlan``.  The plan is plain data:
every part is a ``PartSpec`` (a registry key, the part's sizes and constants, and the checkpoint
tensor name of each of its weights); a block is an arrangement and the named parts it wires (usually
two norms, a mixer and a feed-forward); and the order in which blocks run is a list of ``RunStep`` entries, which may name
a block twice or let a block use the cache entry of another one.  Nothing in ``parts/`` knows
which model it is part of: the generic decoder (``engine/model.py``) builds whatever the plan
says by looking the kinds up in ``parts/registry.py``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: ``kind`` is the key in its registry, ``params`` its sizes and constants,
    ``weights`` maps the part's own weight names to checkpoint tensor names."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    weights: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class BlockSpec:
    """A residual block: an ``arrangement`` (registry of block arrangements: how the parts are wired
    around the residual stream) and the parts themselves, by name: ``parts[name] = (role, PartSpec)``
    with ``role`` one of "norm", "mixer", "feed_forward".  The arrangement decides which names it
    wants; a block may carry four norms, two mixers or no feed-forward.  Every part is chosen
    independently, so two blocks of one model may differ in any of them.

    ``BlockSpec.standard`` builds the usual block of two norms, a mixer and a feed-forward under
    the names ``mixer_norm, mixer, ffn_norm, ffn``."""

    arrangement: str
    parts: Mapping[str, Tuple[str, PartSpec]]
    name: str = ""
    # constants of the arrangement itself (a factor on what the block adds, a weight per mixer)
    params: Mapping[str, Any] = field(default_factory=dict)

    @classmethod
    def standard(cls, arrangement: str, mixer_norm: PartSpec, mixer: PartSpec, ffn_norm: PartSpec, ffn: PartSpec,
                 name: str = "") -> "BlockSpec":
        return cls(arrangement, {"mixer_norm": ("norm", mixer_norm), "mixer": ("mixer", mixer),
                                 "ffn_norm": ("norm", ffn_norm), "ffn": ("feed_forward", ffn)}, name)

    def part(self, name: str) -> PartSpec:
        return self.parts[name][1]

    def mixer_names(self) -> Tuple[str, ...]:
        """Names of the parts that are mixers, in the order the block lists them."""
        return tuple(n for n, (role, _) in self.parts.items() if role == "mixer")

    def keeper_names(self) -> Tuple[str, ...]:
        """Names of the parts that may keep something per sequence: the mixers, and the parts of role "stream" (a
        token shift keeps the previous token's input), in the order the block lists them."""
        return tuple(n for n, (role, _) in self.parts.items() if role in ("mixer", "stream"))


@dataclass(frozen=True)
class RunStep:
    """One entry of the execution order: run ``block``; its mixer uses cache entry ``cache``
    (default: the block's own).  ``writes_cache`` False makes the mixer read that entry without
    appending to it (a block that attends over another block's keys and values)."""

    block: int
    cache: Optional[int] = None
    writes_cache: bool = True
    # the names of the block's parts that ``cache`` and ``writes_cache`` apply to; empty: all of them.  A part that is
    # not named keeps an entry of its own and writes it (a block that reads another block's keys and values while its
    # token shift keeps a row of its own).
    shared: Tuple[str, ...] = ()

    @property
    def cache_entry(self) -> int:
        return self.block if self.cache is None else self.cache

    def entry_of(self, part_name: str) -> int:
        """The cache entry that the block's part ``part_name`` uses in this run."""
        return self.cache_entry if (not self.shared or part_name in self.shared) else self.block

    def writes(self, part_name: str) -> bool:
        return self.writes_cache or bool(self.shared and part_name not in self.shared)


@dataclass(frozen=True)
class ModelPlan:
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    blocks: Tuple[BlockSpec, ...]
    order: Tuple[RunStep, ...]
    final_norm: PartSpec
    head: PartSpec
    # position encodings by name; a mixer names the one it uses in params["position"]
    positions: Mapping[str, PartSpec] = field(default_factory=dict)
    # checkpoint names that a file may hold beside the plan's own: ``duplicates[name] = other`` accepts
    # ``name`` if it equals tensor ``other`` (a tied head stored twice); ``ignored`` are name patterns
    # (``fnmatch``) of stored buffers that carry no weights
    duplicates: Mapping[str, str] = field(default_factory=dict)
    ignored: Tuple[str, ...] = ()
    # true: the decoder keeps a float32 copy of the embedding's output for the length of a step (``ctx.embedding_output``),
    # for a part that reads it again further down (an input that is mixed back into the stream)
    keep_embedding_output: bool = False

    def part_specs(self):
        """Every PartSpec of the plan as (label, role, spec), for the weight loader and error texts."""
        yield "embedding", "embedding", self.embedding
        for name, spec in self.positions.items():
            yield f"position {name}", "position", spec
        for i, b in enumerate(self.blocks):
            label = b.name or f"block {i}"
            for name, (role, spec) in b.parts.items():
                yield f"{label} {name}", role, spec
        yield "final_norm", "norm", self.final_norm
        yield "head", "head", self.head


@dataclass(frozen=True)
class WeightDecl:
    """What a part expects of one of its weights: shape, and the ``role`` that decides how a
    random model fills it and what the part converts it to (``matrix``/``embedding``: normal
    with the given std, run dtype; ``norm``: one plus normal, float32; ``table_int``: int32;
    ``unit``: uniform in (0, 1), a mixing coefficient).  ``any_dims`` lists the dimensions whose size the
    checkpoint decides (a projection's rank that no configuration key names): the loader accepts any size
    there, ``shape`` holds the size that random weights get, and the part reads the tensor's own shape."""

    shape: Tuple[int, ...]
    role: str = "matrix"
    any_dims: Tuple[int, ...] = ()

    def fits(self, got) -> bool:
        got = tuple(got)
        return len(got) == len(self.shape) and all(
            i in self.any_dims or int(g) == int(w) for i, (g, w) in enumerate(zip(got, self.shape)))


@dataclass(frozen=True)
class CacheRequest:
    """What a mixer needs the cache to hold per sequence.

    ``kind`` "kv": keys and values of every position, ``kv_heads x head_dim`` each (values
    ``kv_heads x v_head_dim`` when that is given and differs), and with ``window`` only the last
    ``window`` positions need to stay (and, with ``keep_first``, the first that many positions); with ``chunk`` only the positions of the block of ``chunk`` positions that
    the next query falls into.  ``value_heads``: the values have that many heads instead of ``kv_heads`` (several
    key maps over one set of values).  ``values_in_keys``: no values are stored; the mixer reads them out of the key
    rows (a latent cache whose row is both).  ``kind`` "state": tensors of fixed
    shape per sequence (``state_shapes``: name -> (shape, torch dtype name)), zero when a
    sequence starts.  Entries with equal requests share one group of storage.
    """

    kind: str
    kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    state_shapes: Tuple[Tuple[str, Tuple[int, ...], str], ...] = ()
    v_head_dim: Optional[int] = None
    chunk: Optional[int] = None
    value_heads: Optional[int] = None
    values_in_keys: bool = False
    # with ``window``: the first ``keep_first`` positions stay visible to every later query, so their pages stay too
    keep_first: int = 0

    @property
    def value_dim(self) -> int:
        return self.head_dim if self.v_head_dim is None else self.v_head_dim

    @property
    def n_value_heads(self) -> int:
        return self.kv_heads if self.value_heads is None else self.value_heads

    def group_key(self):
        return (self.kind, self.kv_heads, self.head_dim, self.window, self.state_shapes, self.value_dim, self.chunk,
                self.n_value_heads, self.values_in_keys, self.keep_first if self.window else 0)
