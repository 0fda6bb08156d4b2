"""Architecture-neutral description of a model as data.

A model is a list of layers; a layer is a block arrangement of a mixer, a
feed-forward and its norms; the order in which layers run is a list of its own.
Every size and constant lives in these records, none in the parts' code, and a
part never learns which architecture it belongs to.  An architecture module
(e.g. `reflex_b200.models.qwen3`) turns its typed config.json record into a
`ModelSpec`; everything below that (weights, cache, step) works from the
`ModelSpec` alone.

Each `*Spec` names its part by `kind`, the key under which the part's class is
registered (`reflex_b200.parts.registry`).  `names` maps the part's local
tensor roles to the checkpoint's tensor-name suffixes, so a rename in a
checkpoint format is one line in the architecture module.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    """A normalisation over the last dimension of `size` elements."""

    kind: str  # "rmsnorm"; "layernorm" (mean taken off, a weight and no bias)
    size: int
    eps: float
    # y = x * r * (weight_offset + w); 0.0 is the reference's plain weight
    # (src/kernels_cuda/rmsnorm.cu:44-52), 1.0 the "1 + w" variant.
    weight_offset: float = 0.0


@dataclass(frozen=True)
class PositionSpec:
    """A position encoding applied to query and key head vectors."""

    kind: str  # "rope_neox"; "rope_scaled" (params: factor, low, high, original)
    head_dim: int
    rotary_dim: int
    theta: float
    params: Tuple[Tuple[str, Any], ...] = ()


@dataclass(frozen=True)
class MixerSpec:
    """The sequence-mixing half of a layer.  For attention: sizes of the heads,
    the optional per-head q/k norm, the position encoding and the window."""

    kind: str  # "gqa_attention"
    hidden_size: int
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    scale: float = 0.0
    # query i sees key j iff 0 <= i - j < window (src/model/config.rs:1184-1185);
    # None = every earlier key.
    window: Optional[int] = None
    qk_norm: Optional[NormSpec] = None
    position: Optional[PositionSpec] = None
    names: Tuple[Tuple[str, str], ...] = ()
    # what only some kinds have, by name: "latent_attention" reads q_rank, kv_rank,
    # eps and sink; "mlstm" reads gate_cap and eps; "conv_attention" reads kv taps,
    # temp_coef, temp_every, sink and distance_slopes; "rglru" reads width, blocks,
    # taps and decay_scale; "pair" reads left and right (two `MixerSpec`s) and eps;
    # "gqa_attention" reads values_are_keys, output_gate and keep_first; "selective_scan"
    # reads inner, state, dt_rank and taps
    params: Tuple[Tuple[str, Any], ...] = ()
    # size of a head's value vector when it differs from `head_dim`; 0: the same
    v_head_dim: int = 0

    @property
    def value_dim(self) -> int:
        return self.v_head_dim or self.head_dim

    def param(self, name: str, default: Any = None) -> Any:
        return dict(self.params).get(name, default)


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str  # "swiglu"; "relu2"; "glu_clamped" (params: alpha, limit); "moe" (params: experts, top, activation,
    # router_bias, scores, weight_input, alpha, limit, shared_ff, shared_limit)
    hidden_size: int
    intermediate_size: int
    names: Tuple[Tuple[str, str], ...] = ()
    params: Tuple[Tuple[str, Any], ...] = ()

    def param(self, name: str, default: Any = None) -> Any:
        return dict(self.params).get(name, default)


@dataclass(frozen=True)
class EmbeddingTermSpec:
    """Something added to the token embedding before the first layer: a
    registered embedding term (`reflex_b200.parts.embedding`), e.g.
    "bigram_hash" (params: buckets, mul_prev, mul_cur) or "sinusoidal" (params:
    base)."""

    kind: str
    hidden_size: int
    names: Tuple[Tuple[str, str], ...] = ()
    params: Tuple[Tuple[str, Any], ...] = ()

    def param(self, name: str, default: Any = None) -> Any:
        return dict(self.params).get(name, default)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: which block arrangement, and the parts it arranges.

    `prefix` is prepended to every tensor name of the layer's parts."""

    block: str  # "prenorm"
    prefix: str
    mixer: MixerSpec
    feed_forward: Optional[FeedForwardSpec]  # None: the layer is its mixer alone
    mixer_norm: NormSpec
    feed_forward_norm: Optional[NormSpec]
    names: Tuple[Tuple[str, str], ...] = ()
    # further norms of the arrangement, by role (sandwich norms after the mixer and
    # after the feed-forward, before the residual add: src/model/dense.rs:72-83,
    # 928-930), and any other option of it: a block registered outside the
    # framework reads them, the framework only carries them
    extra_norms: Tuple[Tuple[str, NormSpec], ...] = ()
    params: Tuple[Tuple[str, Any], ...] = ()


@dataclass(frozen=True)
class RunEntry:
    """One position of the run order.

    `layer` indexes `ModelSpec.layers` (a layer may appear more than once: its
    weights are then shared).  `cache` names the cache entry this run uses; by
    default every run has an entry of its own.  With `writes_cache=False` the
    run reads the entry that an earlier run filled (key/value sharing between
    layers) and stores nothing."""

    layer: int
    cache: int
    writes_cache: bool = True
    # the run starts from a mix of the stream and the embedding output x0,
    # x <- W [x; x0] with the model's `stream_mix_name` matrix [hidden, 2 hidden]
    mixes_input: bool = False
    # the run is the first of a pass over a repeated stretch of layers: before it, row
    # `pass_vector` of the model's `pass_vectors_name` tensor [passes, hidden] is added to
    # the stream, and with `adds_input` the embedding output x0 as well
    pass_vector: Optional[int] = None
    adds_input: bool = False


@dataclass
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    layers: List[LayerSpec]
    final_norm: NormSpec
    tie_word_embeddings: bool
    max_positions: int
    embedding_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm.weight"
    head_name: str = "lm_head.weight"
    run_order: List[RunEntry] = field(default_factory=list)
    # y = embedding * embedding_scale (1.0 for the reference's dense path,
    # src/model/dense.rs:1959-1967 gathers rows with no scaling)
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    bos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    # terms added to the token embedding, in order
    embedding_terms: Tuple[EmbeddingTermSpec, ...] = ()
    # logits <- cap * tanh(logits / cap) after the scale; 0: no cap
    logit_softcap: float = 0.0
    # the matrix of the runs that start from a mix of the stream and the embedding
    # output (`RunEntry.mixes_input`); None: the model has none
    stream_mix_name: Optional[str] = None
    # the residual as this many parallel copies of the width (hyper-connections): the
    # embedding output goes into every copy, the layers' blocks read and rewrite all of
    # them ([rows, streams * hidden] 32-bit), and their sum meets the final norm
    residual_streams: int = 1
    # the vectors of the runs that start a pass (`RunEntry.pass_vector`), [passes, hidden];
    # None: the model has none
    pass_vectors_name: Optional[str] = None
    pass_vectors: int = 0

    def __post_init__(self) -> None:
        if not self.run_order:
            self.run_order = [RunEntry(i, i) for i in range(len(self.layers))]

    def cache_entries(self) -> Dict[int, int]:
        """cache entry -> the layer whose mixer defines its shape (the first
        run that writes it)."""
        out: Dict[int, int] = {}
        for run in self.run_order:
            if run.writes_cache and run.cache not in out:
                out[run.cache] = run.layer
        for run in self.run_order:
            if run.cache not in out:
                raise ValueError(
                    f"run order reads cache entry {run.cache} that no run writes"
                )
        return out


def names_dict(names: Tuple[Tuple[str, str], ...]) -> Dict[str, str]:
    return dict(names)
