"""Architecture-neutral description of a decoder: what each layer is made of.

A model is data: a list of :class:`LayerSpec` (mixer x feed-forward x norm, arranged by
a block kind) and a *run order* that says which layer runs when and whose cache it
reads.  The reference describes a model the same way, as one `Mixer` per layer, one
`FeedForward` and a `PositionSpec` (crates/foundation/ir/src/model.rs:45-141), lowered
to a per-token op list (crates/model/recipes/src/decoder.rs:93-154).

Every spec carries only sizes and constants; the `kind` string selects the class that
implements it from the part registries in :mod:`inferloop_b200.parts.registry`.  Specs
are plain frozen dataclasses so they can be compared, hashed and printed.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


def _freeze(params: Mapping[str, Any]) -> Tuple[Tuple[str, Any], ...]:
    return tuple(sorted(params.items()))


@dataclass(frozen=True)
class PartSpec:
    """`kind` names a registered part; `params` are its sizes and constants."""

    kind: str
    items: Tuple[Tuple[str, Any], ...] = ()

    @classmethod
    def make(cls, kind: str, **params: Any) -> "PartSpec":
        return cls(kind, _freeze(params))

    @property
    def params(self) -> dict:
        return dict(self.items)

    def __getitem__(self, key: str) -> Any:
        for k, v in self.items:
            if k == key:
                return v
        raise KeyError(f"{self.kind} spec has no parameter {key!r}")

    def get(self, key: str, default: Any = None) -> Any:
        for k, v in self.items:
            if k == key:
                return v
        return default


@dataclass(frozen=True)
class LayerSpec:
    """One decoder layer: tensor-name prefix, the block arrangement and its parts."""

    prefix: str                 # e.g. "model.layers.3."
    block: PartSpec             # arrangement of the parts, e.g. kind "pre_norm"
    mixer: PartSpec             # token mixer, e.g. kind "gqa_attention"
    feed_forward: PartSpec      # e.g. kind "swiglu"
    norm: PartSpec              # norm used by the block, e.g. kind "rms"


@dataclass(frozen=True)
class RunEntry:
    """One position of the run order.

    `layer` indexes :attr:`ModelSpec.layers`.  `cache_of` is the layer whose cache the
    mixer reads and writes; it equals `layer` unless this entry borrows another
    layer's cache.  `writes_cache` is False for an entry that only reads it.
    """

    layer: int
    cache_of: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding_name: str                 # token table, relative to the weight prefix
    head_name: Optional[str]            # output matrix, at the file's root; None = tied
    final_norm_name: str                # relative to the weight prefix
    final_norm: PartSpec
    layers: Tuple[LayerSpec, ...]
    run_order: Tuple[RunEntry, ...] = field(default=())
    # Prefixes tried in order for every prefix-relative name; the first one under which
    # `embedding_name` exists is used (crates/model/package/src/storage/package.rs:231-237).
    weight_prefixes: Tuple[str, ...] = ("",)
    # What some architectures put around the layers: a multiplier on the embedding rows, and
    # a part of role "logits" that maps the logits in place (a soft cap, a scale).
    embedding_scale: Optional[float] = None
    logits_post: Optional[PartSpec] = None
    # Integer inputs per token beside its id and position (name, width): a position encoding
    # with several axes, say.  Steps carry them (StepEntry.extras); parts read
    # step.extras[name] as an int32 [tokens, width] device tensor.
    token_extras: Tuple[Tuple[str, int], ...] = ()

    def __post_init__(self) -> None:
        if not self.run_order:
            object.__setattr__(
                self, "run_order",
                tuple(RunEntry(i, i) for i in range(len(self.layers))))
        n = len(self.layers)
        owners_written = set()
        for e in self.run_order:
            if not (0 <= e.layer < n and 0 <= e.cache_of < n):
                raise ValueError(f"run order entry {e} names a layer outside 0..{n - 1}")
            if e.writes_cache:
                owners_written.add(e.cache_of)
        for e in self.run_order:
            if not e.writes_cache and e.cache_of not in owners_written:
                raise ValueError(
                    f"run order entry {e} reads the cache of layer {e.cache_of}, "
                    "which no entry writes")
