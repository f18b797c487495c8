"""Architecture-neutral descriptions of a decoder model.

A model is data: a list of block specifications (one per distinct layer), each
naming its norm, mixer, feed-forward and position encoding with all sizes and
constants, plus a schedule that says in which order layers run and which cache
entry each run uses.  Parts are built from these records and never see which
architecture produced them.

The reference keeps the same facts as predicates on one flat ``Config``
(model.go:204-319: usesLayerNorm, forcesParallelResidual,
sharesParallelBranchNorm, usesPlainMLP, layerUsesRoPE); here they are fields.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    """A normalisation over the last axis.

    kind: registered norm name ("layernorm": mean/variance with bias,
    bert.go:748-776; "rmsnorm": root-mean-square, model.go:2949-2981).
    """
    kind: str
    dim: int
    eps: float
    bias: bool = True
    # the file holds the weight minus this value (1.0: the norm multiplies by 1 + w)
    weight_offset: float = 0.0
    # the weight is a single number for all coordinates (the file holds a tensor without axes)
    single_weight: bool = False


@dataclass(frozen=True)
class PositionSpec:
    """Position encoding applied to queries and keys inside a mixer.

    kind "rope": rotary embedding over the first ``rotary_dim`` dims of each
    head; ``interleaved`` False pairs dim i with i+rotary_dim/2 (the NeoX
    split-half layout, model.go:3072-3080), True pairs 2i with 2i+1
    (model.go:3064-3071).  kind "none": nothing.
    """
    kind: str = "none"
    rotary_dim: int = 0
    theta: float = 10000.0
    interleaved: bool = False
    extra: Tuple[Tuple[str, object], ...] = ()   # free-form options for other encodings

    def option(self, key, default=None):
        return dict(self.extra).get(key, default)


@dataclass(frozen=True)
class MixerSpec:
    """Token mixer of a block.  kind "attention" is softmax attention over a
    key/value cache with ``num_kv_heads`` groups; ``window`` 0 means all keys,
    w > 0 means the last w keys (the query's own position included).  Other kinds (mixers that keep a
    state instead of a cache, a pair of mixers side by side) read the sizes they share with attention
    from the same fields and their own constants from ``extra``."""
    kind: str
    hidden: int
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    window: int = 0
    q_scale: float = 1.0          # multiplies q after position encoding
    bias: bool = True
    qk_norm: Optional[NormSpec] = None
    position: PositionSpec = PositionSpec()
    extra: Tuple[Tuple[str, object], ...] = ()   # free-form options for other mixers
    value_dim: int = 0            # size of a head's values where it differs from head_dim (0: the same)

    def option(self, key, default=None):
        return dict(self.extra).get(key, default)


@dataclass(frozen=True)
class FeedForwardSpec:
    """Feed-forward of a block.  kind "dense": act(x·W1ᵀ+b1)·W2ᵀ+b2."""
    kind: str
    hidden: int
    intermediate: int = 0
    activation: str = "gelu_new"
    bias: bool = True
    extra: Tuple[Tuple[str, object], ...] = ()

    def option(self, key, default=None):
        return dict(self.extra).get(key, default)


@dataclass(frozen=True)
class BlockSpec:
    """One layer.  arrangement "parallel": one norm feeds mixer and
    feed-forward, both are added to the residual (model.go:2732-2746,
    2812-2815).  arrangement "sequential": norm → mixer → add → norm2 →
    feed-forward → add."""
    arrangement: str
    norm: NormSpec
    mixer: MixerSpec
    ffn: Optional[FeedForwardSpec]           # None: a layer without a feed-forward (arrangements that allow it)
    norm2: Optional[NormSpec] = None
    extra: Tuple[Tuple[str, object], ...] = ()   # free-form options for other arrangements (further norms, branches)

    def option(self, key, default=None):
        return dict(self.extra).get(key, default)


@dataclass(frozen=True)
class HashedPairSpec:
    """A second embedding added to a token's own: row (token before * mul_prev + token * mul_cur) mod
    ``buckets`` of a table of buckets + 1 rows, whose last row serves a sequence's first token.  The token
    before a step's first token is kept per sequence, with the cache."""
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class PassEntry:
    """What happens to the residual stream right before a run that opens a pass over a looped range of
    layers: the stream as it left the embedding is added (``add_embedding``), then row ``index`` of the
    model's table of per-pass vectors (``ModelSpec.pass_vectors`` rows)."""
    index: int
    add_embedding: bool = False


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  ``layer`` indexes ModelSpec.layers; ``cache`` is
    the cache entry this run reads (None: the mixer keeps nothing);
    ``writes`` False lets a run read an entry another run filled; ``enter``
    marks the first run of a pass over a looped range."""
    layer: int
    cache: Optional[int]
    writes: bool = True
    enter: Optional[PassEntry] = None


@dataclass(frozen=True)
class ModelSpec:
    hidden: int
    vocab: int
    max_positions: int
    layers: Tuple[BlockSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: NormSpec
    tie_embeddings: bool = False
    head_bias: bool = True
    embedding_scale: float = 1.0
    stop_tokens: Tuple[int, ...] = ()
    # learned absolute positions: a table of this many rows added to the embeddings before the first
    # layer (model.go:2648-2651); 0: none
    position_table: int = 0
    # logits * logit_scale, then softcap * tanh(logits / softcap) when softcap > 0 (model.go:2555-2564)
    logit_scale: float = 1.0
    logit_softcap: float = 0.0
    # a norm between the embedding and the first layer; its output is "the embedding's output"
    embedding_norm: Optional[NormSpec] = None
    # rows of the table of learned vectors added at the start of each pass over a looped range; 0: none
    pass_vectors: int = 0
    # an embedding of the pair (token before, token) added to the token's own; None: none
    pair_embedding: Optional[HashedPairSpec] = None

    def __post_init__(self):
        if self.position_table and self.position_table < self.max_positions:
            raise ValueError(f"a position table of {self.position_table} rows does not cover "
                             f"{self.max_positions} positions")
        if self.logit_softcap < 0 or not self.logit_scale > 0:
            raise ValueError("logit_softcap must be >= 0 and logit_scale > 0")
        for e in self.schedule:
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule names layer {e.layer}, model has {len(self.layers)}")
        for e in self.schedule:
            if e.enter is not None and not 0 <= e.enter.index < max(self.pass_vectors, 1):
                raise ValueError(f"a run enters pass {e.enter.index}, the model has {self.pass_vectors} pass vectors")
        writers = {}
        for e in self.schedule:
            if e.cache is None:
                continue
            if e.writes:
                if e.cache in writers:
                    raise ValueError(f"cache entry {e.cache} is written by two runs")
                writers[e.cache] = e.layer
        for e in self.schedule:
            if e.cache is not None and not e.writes and e.cache not in writers:
                raise ValueError(f"cache entry {e.cache} is read but never written")

    @property
    def num_cache_entries(self) -> int:
        ids = [e.cache for e in self.schedule if e.cache is not None]
        return (max(ids) + 1) if ids else 0

    @property
    def embedding_cache_entry(self) -> Optional[int]:
        """The cache entry that holds what the embedding keeps per sequence (the token before), behind the
        entries of the schedule; None if the embedding keeps nothing."""
        return self.num_cache_entries if self.pair_embedding is not None else None


def default_schedule(num_layers: int) -> Tuple[ScheduleEntry, ...]:
    """Layer i runs once, in order, on cache entry i."""
    return tuple(ScheduleEntry(layer=i, cache=i) for i in range(num_layers))


def looped_schedule(num_layers: int, start: int, stop: int, times: int) -> Tuple[ScheduleEntry, ...]:
    """Layers 0..start-1 once, then layers start..stop-1 ``times`` times in a row with the same weights,
    then the rest once.  Every run has a cache entry of its own (a pass never sees another pass's keys or
    state).  The first run of each pass is marked: pass t adds the model's pass vector t, and every pass
    but the first adds the embedding's output before that."""
    if not (0 <= start <= stop <= num_layers) or times < 1:
        raise ValueError(f"loop over layers {start}..{stop} x {times} does not fit {num_layers} layers")
    runs = []
    for i in range(start):
        runs.append(ScheduleEntry(layer=i, cache=len(runs)))
    for t in range(times):
        for i in range(start, stop):
            enter = PassEntry(index=t, add_embedding=t > 0) if i == start else None
            runs.append(ScheduleEntry(layer=i, cache=len(runs), enter=enter))
    for i in range(stop, num_layers):
        runs.append(ScheduleEntry(layer=i, cache=len(runs)))
    return tuple(runs)
