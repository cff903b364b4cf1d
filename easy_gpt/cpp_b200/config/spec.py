"""What a model is made of, as data.

An architecture's builder (see ``registry.register_architecture``) turns its
typed configuration into a :class:`ModelSpec`: a list of layers, each naming
its sub-layers (mixer, feed-forward, their norms and where these stand) and its
position encoding by *kind* with every size and constant as a parameter, and a
run order.  Nothing below this file knows
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
class SubLayerSpec:
    """One residual sub-layer of a layer: a part (``role`` "mixer" or "feed_forward") and where its
    norms stand.  With x the residual stream and f the part:

    * ``norm`` given, ``norm_placement`` "pre" (the default):  x = x + f(norm(x))
    * ``norm`` given, ``norm_placement`` "post":               x = norm(x + f(x))
    * ``norm`` None:                                           x = x + f(x)
    * ``output_norm`` given as well (a "sandwich"):            the part's output is normalised by it before
      it is added: x = x + output_norm(f(norm(x)))
    """
    role: str
    part: PartSpec
    norm: Optional[PartSpec] = None
    norm_placement: str = "pre"
    output_norm: Optional[PartSpec] = None

    def __post_init__(self):
        if self.role not in ("mixer", "feed_forward"):
            raise ValueError(f"a sub-layer's role is 'mixer' or 'feed_forward', not {self.role!r}")
        if self.norm_placement not in ("pre", "post"):
            raise ValueError(f"norm_placement is 'pre' or 'post', not {self.norm_placement!r}")


@dataclass(frozen=True)
class LayerSpec:
    """A layer: residual sub-layers in the order they run (``sublayers``), and the position encoding
    that is handed to its mixer.  The common pre-norm block x += mixer(norm1(x)); x += ff(norm2(x))
    can be written with the four fields ``mixer``, ``feed_forward``, ``mixer_norm`` and
    ``feed_forward_norm`` instead; ``sublayers`` is then derived from them.  A layer has at most one
    mixer (the run order gives a layer one cache); it may have no feed-forward, or several."""
    mixer: Optional[PartSpec] = None
    feed_forward: Optional[PartSpec] = None
    mixer_norm: Optional[PartSpec] = None
    feed_forward_norm: Optional[PartSpec] = None
    position: Optional[PartSpec] = None
    sublayers: Sequence[SubLayerSpec] = ()

    def __post_init__(self):
        if not self.sublayers:
            subs = []
            if self.mixer is not None:
                subs.append(SubLayerSpec("mixer", self.mixer, self.mixer_norm))
            if self.feed_forward is not None:
                subs.append(SubLayerSpec("feed_forward", self.feed_forward, self.feed_forward_norm))
            object.__setattr__(self, "sublayers", tuple(subs))
        elif self.mixer is not None or self.feed_forward is not None:
            raise ValueError("give a layer either sublayers or mixer/feed_forward, not both")
        if not self.sublayers:
            raise ValueError("a layer needs at least one sub-layer")
        if sum(s.role == "mixer" for s in self.sublayers) > 1:
            raise ValueError("a layer has at most one mixer")


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
    # a position encoding that works on the residual stream right after the token embedding
    # (learned absolute positions, say); None: positions reach the model through the layers' own
    embedding_position: Optional[PartSpec] = None

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
