"""Declarative description of a decoder: what each part is and how layers are arranged.

An architecture turns its typed configuration into one ``ModelSpec``. Every size
and constant a part needs is a field of its spec, so no part knows which model it
is in; ``kind`` selects the implementation from the part registries, layer by
layer, so one model may mix different mixers and feed-forwards. The order in
which layers run is data as well (``run_order``): an entry may name a layer twice
or let a layer read another layer's cache.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class TensorDecl:
    """One checkpoint tensor a part wants.

    role: 'matrix' and 'table' are kept in the engine dtype (bfloat16 or float32),
    'vector' is always float32 (biases, norm parameters), 'int' is int32.
    ``stored_in_out``: the checkpoint holds the matrix as [in, out] (GPT-2 Conv1D);
    the device copy is always [out, in], K-contiguous.
    ``pieces``: the checkpoint does not hold this tensor whole but as several tensors
    ((checkpoint name, shape as stored), ...) that are joined along the output axis, in
    this order, when they are placed (separate query, key and value projections that one
    fused product reads); ``name`` is then only the key under which the part finds the
    joined tensor, and ``shape`` its shape as if it had been stored whole.
    """
    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    stored_in_out: bool = False
    pieces: Tuple[Tuple[str, Tuple[int, ...]], ...] = ()


@dataclass(frozen=True)
class NormSpec:
    kind: str            # 'layernorm' | 'rmsnorm'
    width: int
    eps: float
    weight: str          # checkpoint names
    bias: Optional[str] = None
    weight_offset: float = 0.0   # 'rmsnorm': the factor is weight_offset + weight (1 for a weight stored around zero)


@dataclass(frozen=True)
class PositionSpec:
    kind: str            # 'learned'
    n_positions: int
    width: int
    table: Optional[str] = None


@dataclass(frozen=True)
class LongContextBlend:
    """Rotary frequencies blended for contexts beyond the one a model was trained at (the YaRN rule): pair i keeps
    its frequency f_i where its wavelength turns more than ``fast`` times over ``original`` tokens, gets f_i / factor
    where it turns fewer than ``slow`` times, a linear blend between; cosine and sine are scaled by
    0.1 ln(factor) + 1."""
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class RotarySpec:
    kind: str            # 'rotary'
    head_dim: int
    dims: int            # the first `dims` dimensions of a head are rotated, the rest pass unchanged
    base: float
    interleaved: bool = True     # pairs are neighbours (2i, 2i+1); False: halves (i, i + dims/2)
    blend: Optional[LongContextBlend] = None


@dataclass(frozen=True)
class AttentionSpec:
    kind: str            # 'attention'
    width: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    scale: float         # multiplies q.k (already includes any per-layer factor)
    window: Optional[int]  # None = all earlier keys; n = the query and the n-1 keys before it
    qkv_weight: object   # checkpoint name of the fused projection, or the three names (query, key, value) of separate ones
    qkv_bias: object     # None, one name, or three names
    out_weight: str
    out_bias: Optional[str]
    stored_in_out: bool = False
    value_dim: Optional[int] = None   # size of a value head where it differs from head_dim
    chunk: Optional[int] = None       # positions in chunks of this many from the start; nothing is seen across a border
    gate_weight: Optional[str] = None  # [n_heads, width]: a head's output is multiplied by sigmoid(gate . input)
    rotary: object = None             # a position-encoding spec of the mixer's own (applied to its queries and keys)


@dataclass(frozen=True)
class DenseFeedForwardSpec:
    kind: str            # 'dense'
    width: int
    inner: int
    activation: str      # 'gelu_new' | 'gelu' | 'relu2'
    up_weight: str
    up_bias: Optional[str]
    down_weight: str
    down_bias: Optional[str]
    stored_in_out: bool = False


@dataclass(frozen=True)
class GatedUnitSpec:
    """A small feed-forward with a clamped gate: g = min(W_gate y, limit), u = clamp(W_up y, -limit, limit),
    output W_down (g * sigmoid(alpha g) * (u + 1)). No biases."""
    inner: int
    limit: float
    gate_weight: str
    up_weight: str
    down_weight: str
    alpha: float = 1.702


@dataclass(frozen=True)
class TableRoutedExpertsSpec:
    kind: str            # 'experts_by_table'
    width: int
    vocab_size: int
    top: int             # experts per token; each weighs 1 / top
    table: str           # checkpoint name of the integer table [vocab, top]: a token id's experts
    experts: Tuple[GatedUnitSpec, ...]       # all of one size and limit
    shared: Optional[GatedUnitSpec] = None   # runs for every token and is added


@dataclass(frozen=True)
class NoFeedForwardSpec:
    kind: str = "none"


@dataclass(frozen=True)
class LayerSpec:
    """A layer: a mixer, a feed-forward, as many norms as its arrangement wants, and the arrangement that wires them
    ('pre_norm' takes two norms: before the mixer, before the feed-forward; 'pre_norm_mixer' one norm and no
    feed-forward)."""
    arrangement: str
    mixer: object
    feed_forward: object
    norms: Tuple[object, ...]

    @property
    def kind(self):
        return self.arrangement


@dataclass(frozen=True)
class EmbeddingSpec:
    kind: str            # 'tokens': a row of the table per token id (the position encoding may add its own table)
    vocab_size: int
    width: int
    table: str           # checkpoint name
    scale: float = 1.0   # multiplies the row


@dataclass(frozen=True)
class HeadSpec:
    kind: str            # 'linear': final norm on the wanted rows, then logits = y . W^T (+ bias)
    vocab_size: int
    width: int
    norm: object         # a norm spec
    weight: str          # checkpoint name of W [vocab, width]
    tied: bool = False   # W is the embedding's table (declared there, not again)
    bias: Optional[str] = None


@dataclass(frozen=True)
class RunEntry:
    """One stop of the forward pass: run ``layer`` (an index into ``ModelSpec.layers``).

    Every stop has a cache of its own, so a layer that is named twice keeps the keys and
    values of its two runs apart. ``cache_of`` = the index of an EARLIER STOP in
    ``run_order`` makes this stop read that stop's cache instead: it gets no pages of its
    own and does not write (its mixer sees ``cache.writable == False``).
    """
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    width: int
    max_positions: Optional[int]      # None: the architecture sets no limit (the engine's cache does)
    embedding: object                 # an embedding spec
    position: object                  # a position-encoding spec
    layers: Tuple[LayerSpec, ...]
    run_order: Tuple[RunEntry, ...]
    head: object                      # a head spec (with the final norm)
    eos_token_ids: Tuple[int, ...] = ()
    ignored_tensors: Tuple[str, ...] = field(default_factory=tuple)   # regexes of tensors to drop
    tied_duplicates: Tuple[Tuple[str, str], ...] = field(default_factory=tuple)  # (name, must equal)
    optional_prefix: str = ""          # e.g. 'transformer.': stripped from every name when present

    @property
    def prefix_probe(self):
        """The tensor whose presence under the optional prefix says that the checkpoint uses the prefix."""
        return self.embedding.table
