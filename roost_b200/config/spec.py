"""What a model is made of, as data.

A ``ModelSpec`` lists blocks (one per distinct set of weights) and a run order. Each block names its mixer,
feed-forward, norms and arrangement by a spec object whose ``kind`` selects the part class from the part
registries (``roost_b200.parts``); every size and constant a part needs is a field of its spec. Nothing
here knows an architecture: an architecture module (``roost_b200.config.qwen3``) turns its config.json into
these objects, as the reference's model definition turns attributes into a node list whose ops take their
constants as arguments (src/Starlings.Roost.Models.Tiny/RoostTiny.cs:14-57).
"""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass(frozen=True)
class NormSpec:
    """``rms_norm``: x / sqrt(mean(x^2) + eps) * w. ``layer_norm``: (x - mean) / sqrt(var + eps) * w + b, var the mean squared
    deviation; it reads a 32-bit stream and writes the activation dtype."""
    size: int
    eps: float
    kind: str = "rms_norm"


@dataclass(frozen=True)
class PositionSpec:
    """Position encoding applied inside a mixer. ``rope_neox``: rotation of the first ``rotary_dim``
    elements of each head, pairs (i, i + rotary_dim/2), frequencies theta^(-2i/rotary_dim)."""
    kind: str = "rope_neox"
    rotary_dim: int = 0
    theta: float = 10000.0
    max_positions: int = 0


@dataclass(frozen=True)
class MixerSpec:
    kind: str = ""


@dataclass(frozen=True)
class AttentionSpec(MixerSpec):
    """Grouped-query causal attention over a paged cache. ``window`` counts the keys a query sees, its own
    included (Hugging Face ``sliding_window``); None means every earlier key."""
    kind: str = "paged_attention"
    hidden: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    scale: float = 0.0
    window: int | None = None
    qk_norm: NormSpec | None = None
    position: PositionSpec | None = None


@dataclass(frozen=True)
class LatentAttentionSpec(MixerSpec):
    """Causal attention whose keys and values are made per head from one latent vector a token: the cache keeps the
    latent (``kv_rank`` numbers, unit root mean square times a weight) and one rotated key part of ``rope_dim`` numbers
    that all heads share. A head's key is [W_uk c | shared part] against a query of ``nope_dim`` plain and ``rope_dim``
    rotated numbers, its value W_uv c of ``v_dim`` numbers. ``window`` counts the keys a query sees, its own included
    (None: all). ``own_latent`` False: the run makes no latent and reads another run's; ``cache_window`` is then the
    window the shared cache is kept for (the widest of the runs that read it; None: everything is kept)."""
    kind: str = "latent_attention"
    hidden: int = 0
    num_heads: int = 0
    nope_dim: int = 0
    rope_dim: int = 0
    v_dim: int = 0
    kv_rank: int = 0
    scale: float = 0.0
    window: int | None = None
    cache_window: int | None = None
    own_latent: bool = True
    latent_eps: float = 1e-6
    position: PositionSpec | None = None


@dataclass(frozen=True)
class Mamba2Spec(MixerSpec):
    """The Mamba-2 recurrence. The input projection gives [z | x | B | C | dt]; x, B and C pass a causal convolution of
    ``conv_taps`` taps a channel and SiLU; per head (``head_dim`` values, state ``state`` x ``head_dim``, B and C shared by
    the heads of one of ``groups`` groups) S <- exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x with dt = softplus(dt +
    dt_bias); y SiLU(z) is divided by its root mean square in ``norm_groups`` equal parts, times a weight, and projected
    out. The state and the last ``conv_taps`` - 1 inputs of the convolution are kept per request in 32-bit."""
    kind: str = "mamba2"
    hidden: int = 0
    num_heads: int = 0
    head_dim: int = 0
    state: int = 0
    groups: int = 1
    conv_taps: int = 4
    norm_groups: int = 1
    eps: float = 1e-6


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str = ""


@dataclass(frozen=True)
class GatedMlpSpec(FeedForwardSpec):
    """down(act(x Wg^T) * (x Wu^T)); ``activation`` is the gate's function."""
    kind: str = "gated_mlp"
    hidden: int = 0
    intermediate: int = 0
    activation: str = "silu"


@dataclass(frozen=True)
class RoutedMlpSpec(FeedForwardSpec):
    """``experts`` gated feed-forwards of ``expert_intermediate`` rows of which a token uses the ``top`` with the largest
    router scores, and a shared one of ``shared_intermediate`` rows (0: none) that every token uses. ``score``: the
    function that turns router logits into scores ("sigmoid"); ``renormalize``: whether the chosen scores are divided by
    their sum; ``weight_on``: "input" when a chosen expert is given score * x (the sum of expert(score x)), "output" when
    its output is multiplied."""
    kind: str = "routed_mlp"
    hidden: int = 0
    experts: int = 0
    top: int = 1
    expert_intermediate: int = 0
    shared_intermediate: int = 0
    activation: str = "silu"
    score: str = "sigmoid"
    renormalize: bool = False
    weight_on: str = "input"


@dataclass(frozen=True)
class EmbeddingSpec:
    """How token ids become the first hidden states. ``table``: a row copy, no scaling
    (src/Starlings.Roost.Ops/CpuOps.cs:441-458)."""
    kind: str = "table"
    vocab: int = 0
    hidden: int = 0


@dataclass(frozen=True)
class HeadSpec:
    """How the final hidden states of the wanted rows become logits. ``linear``: a product with a [vocab, hidden] matrix
    into 32-bit logits, no soft cap (src/Starlings.Roost.Ops/CpuOps.cs:465-495)."""
    kind: str = "linear"
    vocab: int = 0
    hidden: int = 0


@dataclass(frozen=True)
class ScaledEmbeddingSpec(EmbeddingSpec):
    """h0[t, :] = table[ids[t], :] * scale, formed and kept in 32-bit (the stream of a ``pre_norm_wide`` model)."""
    kind: str = "scaled_table"
    scale: float = 1.0


@dataclass(frozen=True)
class CappedHeadSpec(HeadSpec):
    """logits = cap * tanh((final W^T) / cap) in 32-bit."""
    kind: str = "capped_linear"
    cap: float = 0.0


@dataclass(frozen=True)
class BlockSpec:
    """One layer's parts and their arrangement. ``pre_norm``: h += mixer(norm1(h)); h += ff(norm2(h)), the stream in the
    activation dtype. ``pre_norm_wide``: the same with the stream kept and summed in 32-bit whatever the activation dtype
    is; its ``feed_forward`` and ``post_mixer_norm`` may be None (a layer that is its mixer only)."""
    mixer: MixerSpec
    feed_forward: FeedForwardSpec | None
    input_norm: NormSpec
    post_mixer_norm: NormSpec | None
    kind: str = "pre_norm"


@dataclass(frozen=True)
class RunEntry:
    """One run of a block. ``block`` indexes ``ModelSpec.blocks`` (the same block may run twice: it then has
    one set of weights and two caches). ``reads_cache_of`` is None when the run keeps a cache of its own, or
    the index of an earlier run whose cache it reads without writing."""
    block: int
    reads_cache_of: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden: int
    vocab: int
    blocks: tuple[BlockSpec, ...]
    schedule: tuple[RunEntry, ...]
    final_norm: NormSpec
    tie_embeddings: bool
    max_positions: int
    stop_token_ids: tuple[int, ...] = ()
    stored_dtype: str = "bfloat16"
    # the two ends of the model as parts of their own kinds (None: a table embedding and a linear head of the model's
    # vocabulary and width)
    embedding: EmbeddingSpec | None = None
    head: HeadSpec | None = None
    # checkpoint tensors the model does not use and a checkpoint may hold all the same (the loader passes over them)
    ignorable_tensors: tuple = ()
    # checkpoint tensor names: scope -> {part-local parameter name -> tuple of checkpoint names whose rows
    # are concatenated in order}. Scopes: "embed", "final_norm", "lm_head", "blocks.<i>.<part>".
    weight_names: dict = field(default_factory=dict, compare=False, hash=False)

    def __post_init__(self):
        if self.embedding is None:
            object.__setattr__(self, "embedding", EmbeddingSpec(vocab=self.vocab, hidden=self.hidden))
        if self.head is None:
            object.__setattr__(self, "head", HeadSpec(vocab=self.vocab, hidden=self.hidden))
        for n, e in enumerate(self.schedule):
            if not 0 <= e.block < len(self.blocks):
                raise ValueError(f"schedule entry {n} names block {e.block}; the model has {len(self.blocks)}")
            if e.reads_cache_of is not None:
                if not 0 <= e.reads_cache_of < n:
                    raise ValueError(f"schedule entry {n} reads the cache of entry {e.reads_cache_of}, which does not run before it")
                if self.schedule[e.reads_cache_of].reads_cache_of is not None:
                    raise ValueError(f"schedule entry {n} reads the cache of entry {e.reads_cache_of}, which keeps none of its own")
