"""Interfaces of the parts a layer is put together from.

A *mixer* moves information between the tokens of a request (attention here);
a *feed-forward* works on each token alone; a *norm* normalises the residual
stream; a *position encoding* is handed to the mixer that wants one.  Every part
is built from ``PartSpec.params`` (its sizes and constants) and ``prefix`` (where
its tensors live) and never learns which model it sits in.

The residual stream is float32 in both precisions.  A block hands each part the
normalised input in the compute dtype and gets back a *delta* in the compute
dtype; the next norm adds the delta to the residual in float32 while it
normalises (one fused kernel).

To add a part: subclass the matching base, implement ``tensor_requests``,
``load`` and ``forward`` (and ``cache_need`` for a mixer that keeps something per
request), and ``register_part(role, kind, cls)``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from ..weights.loader import TensorRequest


# ---------------------------------------------------------------------------
# what a mixer needs the cache manager to keep for it
# ---------------------------------------------------------------------------

@dataclass(frozen=True)
class PagedKVNeed:
    """Keys and values of every token (or of the last ``window`` tokens) in pages."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """A tensor of fixed shape per live request, zeroed when a request starts.  ``dtype`` is the name of
    a torch dtype ("float32", "bfloat16", "int32", ...)."""
    shape: Tuple[int, ...]
    dtype: str = "float32"


# ---------------------------------------------------------------------------
# what a step hands to the parts
# ---------------------------------------------------------------------------

@dataclass
class GroupTables:
    """Cache addressing of one cache group for this step."""
    page_size: int
    block_table: torch.Tensor      # int32 [num_seqs, max_pages]: page id per logical page, -1 where none
    slot_map: torch.Tensor         # int32 [T]: page * page_size + offset where the token's key/value is stored


@dataclass
class StepContext:
    """Everything about one step's batch that a part may need.  All tensors are on
    the device; the ``host_*`` twins are Python lists for parts (and tests) that
    plan their launches on the host."""
    dtype: torch.dtype
    device: torch.device
    num_tokens: int
    num_seqs: int
    token_ids: torch.Tensor        # int32 [T]
    positions: torch.Tensor        # int32 [T] absolute position of each token in its request
    token_seq: torch.Tensor        # int32 [T] which entry of the batch the token belongs to
    seq_starts: torch.Tensor       # int32 [num_seqs + 1] prefix sums of the entries' token counts
    seq_context: torch.Tensor      # int32 [num_seqs] tokens of the request already cached before this step
    seq_slots: torch.Tensor        # int32 [num_seqs] state slot of each entry's request
    status: torch.Tensor           # int32 [1] device status word the kernels OR their complaints into
    groups: Dict[int, GroupTables] = field(default_factory=dict)
    host_seq_starts: List[int] = field(default_factory=list)
    host_seq_context: List[int] = field(default_factory=list)
    host_seq_slots: List[int] = field(default_factory=list)
    max_query_len: int = 0
    max_context_len: int = 0       # longest context + query of the batch
    all_decode: bool = False       # every entry brings exactly one token
    # runs of up to 128 consecutive tokens of the entries that bring more than SMALL_ENTRY_TOKENS tokens (prompt
    # portions): int32 [n, 3] = (entry, first token, count); None if there is no such entry
    query_tiles: Optional[torch.Tensor] = None
    # token indices of the entries too short for tiles (decoded tokens beside prompt portions); None if there are none
    small_tokens: Optional[torch.Tensor] = None
    # per-step data that parts share between layers (cleared at the start of every forward)
    scratch: Dict = field(default_factory=dict)


@dataclass
class CacheView:
    """What the cache manager gives a mixer for one run entry."""
    group: int = -1                           # key into StepContext.groups (paged) ...
    k: Optional[torch.Tensor] = None          # [pages, NKV, page_size, HD] slice of the pool for this cache
    v: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None      # [max_slots, *StateNeed.shape] for a mixer with fixed-size state
    writes: bool = True                       # False: read another entry's cache, store nothing


# ---------------------------------------------------------------------------
# the parts
# ---------------------------------------------------------------------------

class Part:
    # True if forward() only launches device work whose shape depends on the batch's size alone
    # (no host reads of the batch's contents, no .item()): then decode steps may be captured in a
    # CUDA graph.  A part that plans on the host (ctx.host_*) leaves this False and every step of
    # a model that contains it runs eagerly.
    capturable = False

    def __init__(self, params: Mapping, prefix: str):
        self.params = dict(params)
        self.prefix = prefix

    def tensor_requests(self) -> List[TensorRequest]:
        return []

    def load(self, tensors: Mapping[str, torch.Tensor], device: torch.device, dtype: torch.dtype) -> None:
        """Take this part's tensors (host, stored precision) to the device in the form its kernels want."""

    def weight_bytes(self) -> int:
        """Bytes of weights one forward reads (for roofline arithmetic)."""
        return 0

    def streamed_weights(self) -> List[torch.Tensor]:
        """The large weights this part's kernels stream, in the order they are used."""
        return []

    # Set by the model after loading: ``streamed_weights()`` of the part that runs next.
    # A part's decode kernels may ask the L2 to fetch these while they work (a hint only).
    prefetch_hints: Sequence[torch.Tensor] = ()

    def _hint(self, i: int) -> Optional[torch.Tensor]:
        return self.prefetch_hints[i] if i < len(self.prefetch_hints) else None


@dataclass(frozen=True)
class HalfRotation:
    """What a rotary encoding hands to a consumer whose kernels rotate by themselves: for k <
    rotary_dim / 2 the pair (x[k], x[k + rotary_dim / 2]) of every head turns by the angle
    float32(position) * inv_freq[k]; dimensions from rotary_dim on pass through."""
    inv_freq: torch.Tensor          # float32 [rotary_dim / 2] on the device
    rotary_dim: int
    key: tuple = ()                 # equal keys mean equal tables: consumers may share what they derive from one


class PositionEncoding(Part):
    """How positions reach the model.  A position encoding is built once per layer (or once for the
    embedding) and offers any of three things; a consumer asks for what it can use and every method has
    a default that does nothing, so an encoding implements only what it is:

    * ``half_rotation()``: a :class:`HalfRotation` if the encoding is a half rotation of queries and
      keys that attention kernels can apply themselves (fused with the cache write), else None;
    * ``apply_to_query_key(q, k, ctx)``: changes q [T, heads, head_dim] and k [T, kv heads, head_dim]
      (views into the step's buffers) in place, for encodings that are no half rotation; it is called
      only when ``half_rotation()`` returns None;
    * ``add_to_embedding(residual, ctx)``: adds to the float32 residual stream [T, hidden] right
      after the token embedding (learned absolute positions); called for the model's
      ``embedding_position``.

    Positions are ``ctx.positions`` (int32, absolute position of each token in its request)."""

    def half_rotation(self) -> Optional["HalfRotation"]:
        return None

    def apply_to_query_key(self, q: torch.Tensor, k: torch.Tensor, ctx: "StepContext") -> None:
        return None

    def add_to_embedding(self, residual: torch.Tensor, ctx: "StepContext") -> None:
        return None


class Norm(Part):
    def rms_parameters(self):
        """(gain float32 [size], eps) if this norm is a plain RMSNorm that a consumer's
        kernel may fold in; None otherwise."""
        return None

    def forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], out: torch.Tensor,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """residual += delta (float32, in place, unless rows is given); returns the
        normalised rows in ``out`` (compute dtype).  With ``rows`` only those rows
        are normalised, into out[:len(rows)], and the residual is left as it is."""
        raise NotImplementedError


class FollowingNorm:
    """The add and the norm that come right after a part: ``residual`` (float32 [T, hidden]) gets the
    part's output added, and ``norm`` (a plain RMSNorm: ``gain``, ``eps``) normalises the sum for the
    part that runs next.  A block offers this to a part that sets ``fuses_following_norm``; such a part
    may let its last kernel do both (it then updates ``residual`` in place and returns a ``PreNormed``
    instead of its delta) or ignore the offer and return the delta as ever."""

    def __init__(self, norm: "Norm", pending: "PendingNorm"):
        self.norm = norm
        self.gain, self.eps = norm.rms_parameters()
        self._pending = pending

    @property
    def residual(self) -> torch.Tensor:
        """The buffer that holds the residual stream once the part's own input norm has run."""
        assert self._pending.consumed
        return self._pending.residual_after


class PreNormed:
    """Returned by a part in place of its delta when it took a ``FollowingNorm`` over: the residual
    already holds the sum v; ``rows`` is bfloat16(gain * v) [T, hidden] and ``ss_parts`` float32
    [parts, padded T] the partial sums of v^2 per token, to be added up in their order."""

    def __init__(self, norm: "Norm", rows: torch.Tensor, ss_parts: torch.Tensor):
        self.norm, self.rows, self.ss_parts = norm, rows, ss_parts


class PendingNorm:
    """x = norm(residual + delta), not computed yet.

    A block hands this to a part that sets ``accepts_pending_norm``.  Such a part
    either folds the add and the norm into its own first kernel (``fused()``,
    possible when ``fusable``) or calls ``materialize`` and works on the tensor.
    Either way the sum residual + delta ends up in ``residual_after``: in place
    when materialised, in the spare buffer when fused (other CTAs of the fused
    kernel still read the old residual while one of them writes the new one).
    """

    def __init__(self, norm: "Norm", residual: torch.Tensor, delta: Optional[torch.Tensor], spare: torch.Tensor,
                 work: torch.Tensor, rows: Optional[torch.Tensor] = None, max_fused_rows: int = 0):
        self.norm, self.residual, self.delta, self.spare, self.work, self.rows = norm, residual, delta, spare, work, rows
        self.residual_after = residual
        self.spare_after = spare
        self.consumed = False
        rms = norm.rms_parameters()
        # the part in front has already added its output to the residual and prepared the rows for this norm
        self.prenormed = delta if isinstance(delta, PreNormed) else None
        if self.prenormed is not None:
            assert self.prenormed.norm is norm, "a PreNormed belongs to the norm it was prepared for"
            self.delta = None
        self.fusable = (rms is not None and rows is None and work.dtype == torch.bfloat16
                        and 0 < residual.shape[0] <= max_fused_rows
                        and (self.delta is None or self.delta.dtype == torch.bfloat16))
        self._rms = rms

    def materialize(self) -> torch.Tensor:
        assert not self.consumed
        self.consumed = True
        return self.norm.forward(self.residual, self.delta, self.work, self.rows)

    def fused(self) -> "NormInFront":
        """Hands the add and the norm over to the part, whose first kernel does both."""
        assert not self.consumed and self.fusable
        self.consumed = True
        gain, eps = self._rms
        if self.prenormed is not None:
            return NormInFront(eps=eps, prepared_rows=self.prenormed.rows, prepared_sums=self.prenormed.ss_parts)
        if self.delta is not None:
            self.residual_after, self.spare_after = self.spare, self.residual
        return NormInFront(eps=eps, gain=gain, residual=self.residual, delta=self.delta,
                           residual_out=self.spare if self.delta is not None else None)


@dataclass
class NormInFront:
    """An add and an RMSNorm that a part's first kernel is to do itself, in one of two forms.
    Either ``residual`` (float32 [T, hidden]), an optional ``delta`` to add to it first (the sum is
    then also to be written to ``residual_out``, another buffer: other CTAs still read the old one),
    ``gain`` and ``eps``.  Or ``prepared_rows`` (compute dtype [T, hidden], already gain * sum) and
    ``prepared_sums`` (float32 [parts, padded T], partial sums of squares per token, to be added up in
    their order) with ``eps``: only the scale 1/sqrt(mean + eps) is still missing."""
    eps: float
    gain: Optional[torch.Tensor] = None
    residual: Optional[torch.Tensor] = None
    delta: Optional[torch.Tensor] = None
    residual_out: Optional[torch.Tensor] = None
    prepared_rows: Optional[torch.Tensor] = None
    prepared_sums: Optional[torch.Tensor] = None


class Mixer(Part):
    accepts_pending_norm = False       # True: forward() takes a PendingNorm instead of a tensor
    fuses_following_norm = False       # True: forward() takes follow=FollowingNorm and may return a PreNormed

    def __init__(self, params: Mapping, prefix: str, position: Optional[PositionEncoding] = None):
        super().__init__(params, prefix)
        self.position = position

    def cache_need(self):
        """PagedKVNeed, StateNeed or None."""
        return None

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        """x [T, hidden] normalised input -> delta [T, hidden], both in ctx.dtype."""
        raise NotImplementedError


class FeedForward(Part):
    accepts_pending_norm = False
    fuses_following_norm = False

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError
