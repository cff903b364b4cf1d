"""What a model is made of, as data.

An architecture's builder (see ``registry.register_architecture``) turns its
typed configuration into a :class:`ModelSpec`: a list of layers, each naming
its mixer, feed-forward, norms and position encoding by *kind* with every size
and constant as a parameter, and a run order.  Nothing below this file knows
which model it is in.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Sequence


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: ``kind`` selects the class from the part registry,
    ``params`` are its constructor arguments (sizes, constants, switches) and
    ``prefix`` is the tensor-name prefix its weights live under."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    prefix: str = ""


@dataclass(frozen=True)
class LayerSpec:
    """A pre-norm residual block: x += mixer(norm1(x)); x += ff(norm2(x)).
    The position encoding belongs to the layer and is handed to the mixer."""
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    position: Optional[PartSpec] = None


@dataclass(frozen=True)
class RunEntry:
    """One line of the run order.  ``layer`` indexes ``ModelSpec.layers`` (a
    layer may be named more than once: its weights are shared).  ``cache`` names
    the cache the mixer uses; entries with the same ``cache`` share it, and only
    the entry with ``writes_cache`` appends to it (the others read it)."""
    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    layers: Sequence[LayerSpec]
    run_order: Sequence[RunEntry]
    embedding: PartSpec
    final_norm: PartSpec
    lm_head: PartSpec
    bos_token_id: int = -1
    eos_token_id: int = -1

    def __post_init__(self):
        owners = {}
        for i, e in enumerate(self.run_order):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"run order entry {i} names layer {e.layer}, but there are {len(self.layers)} layers")
            if e.writes_cache:
                if e.cache in owners:
                    raise ValueError(f"cache {e.cache} is written by run entries {owners[e.cache]} and {i}")
                owners[e.cache] = i
        for i, e in enumerate(self.run_order):
            if e.cache not in owners:
                raise ValueError(f"run entry {i} reads cache {e.cache}, which no entry writes")
            if owners[e.cache] > i:
                raise ValueError(f"run entry {i} reads cache {e.cache} before entry {owners[e.cache]} has written it")
